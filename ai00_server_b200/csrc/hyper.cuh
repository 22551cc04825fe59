// Several copies of the residual ("streams") around pre-norm sublayers, with a layer norm on the read side.
//
// A sublayer reads one mix of the streams and writes its output back into all of them:
//     u = sum_s a[s] x_s;    y = Sublayer(LN(u));    x_t <- sum_s M[s, t] x_s + b[t] y           (every x_t from the old x_s)
//     LN(u) = (u - mean(u)) / sqrt(mean((u - mean(u))^2) + eps) * w + c
// One stream with a = b = M = 1 is the ordinary pre-norm residual  x <- x + Sublayer(LN(x)).
//
//   hc_step_kernel   one CTA per token: writes a finished sublayer's output into the streams (the output row is either a plain
//                    row or the weighted sum of a routed feed-forward's chosen expert rows: then this is also the experts'
//                    combine step), and / or forms the read of the NEXT sublayer and its layer norm, so that a sublayer boundary
//                    is one launch.  The last call of a model reads the plain sum of the streams, norms it with the model's
//                    last norm and writes only the rows that want logits, compactly.
//   hc_sum_kernel    the sum of the streams of every token (what a one-stream model would carry) -> [T, W]
// All f32: the streams are the residual sum, which stays in 32-bit.
#pragma once
#include <cuda_runtime.h>
#include "common.cuh"
#include "rmsnorm.cuh"

namespace b200 {

constexpr int HC_MAX_STREAMS = 16;                // kernel template: loops unrolled for up to 4, 8 or 16 streams
constexpr int HC_MAX_TOP = 8;

enum HcRead { HC_READ_NONE = 0, HC_READ_MIX = 1, HC_READ_SUM = 2 };

struct HcStepParams {
    float* x;                 // [T][S][W]
    int S, W;
    // write side (upd_out == nullptr: nothing to write)
    const float* upd_mix;     // [S][S], indexed [from][to]
    const float* upd_out;     // [S]
    const float* y;           // [T, W] sublayer output (nullptr with rows)
    const float* rows;        // [T * top, W] expert outputs in compact rows
    const int* row_of; const float* wgt; int top;
    // read side
    int read;                 // HcRead
    const float* rd_in;       // [S] (HC_READ_MIX)
    const float* ln_w; const float* ln_b;     // [W]
    float eps;
    float* h;                 // [T, W], or [R, W] with compact
    int compact;              // 1: only the tokens that want logits, at their logits row
    float* hidden;            // [T, W] copy of u (nullptr: none)
    MetaView meta;
};

constexpr int HC_THREADS_FEW_ROWS = 1024;       // block size for steps of few tokens (decode): a thread then owns one or two columns

template <int THREADS, int SMAX>
__global__ void __launch_bounds__(THREADS) hc_step_kernel(const HcStepParams p) {
    __shared__ float red[32];
    __shared__ float s_mix[SMAX * SMAX], s_out[SMAX], s_in[SMAX];
    extern __shared__ __align__(16) float hc_u[];      // [W] the read row
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int S = p.S, W = p.W;
    const bool upd = p.upd_out != nullptr;
    for (int i = threadIdx.x; i < S * S && upd; i += blockDim.x) s_mix[i] = p.upd_mix[i];
    if (threadIdx.x < S) {
        if (upd) s_out[threadIdx.x] = p.upd_out[threadIdx.x];
        s_in[threadIdx.x] = p.read == HC_READ_MIX ? p.rd_in[threadIdx.x] : 1.f;
    }
    int rw[HC_MAX_TOP]; float wg[HC_MAX_TOP];
    if (upd && p.rows) {
#pragma unroll
        for (int k = 0; k < HC_MAX_TOP; ++k)
            if (k < p.top) { rw[k] = p.row_of[(size_t)t * p.top + k]; wg[k] = p.wgt[(size_t)t * p.top + k]; }
    }
    __syncthreads();
    // a column of the token's streams is read and written by one thread only, and nothing else the loop reads is written here
    float* __restrict__ xt = p.x + (size_t)t * S * W;
    const float* __restrict__ yrow = p.y ? p.y + (size_t)t * W : nullptr;
    const float* __restrict__ erows = p.rows;
    float sum = 0.f;
#pragma unroll 2
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float xs[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) xs[s] = xt[(size_t)s * W + c];
        if (upd) {
            float yv;
            if (p.rows) {
                yv = 0.f;
#pragma unroll
                for (int k = 0; k < HC_MAX_TOP; ++k)
                    if (k < p.top) yv = fmaf(wg[k], erows[(size_t)rw[k] * W + c], yv);
            } else {
                yv = yrow[c];
            }
            float xn[SMAX];
#pragma unroll
            for (int to = 0; to < SMAX; ++to) {
                if (to >= S) break;
                float a = 0.f;
#pragma unroll
                for (int fr = 0; fr < SMAX; ++fr)
                    if (fr < S) a = fmaf(s_mix[fr * S + to], xs[fr], a);
                xn[to] = fmaf(s_out[to], yv, a);
            }
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) { xs[s] = xn[s]; xt[(size_t)s * W + c] = xn[s]; }
        }
        if (p.read != HC_READ_NONE) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) u = fmaf(s_in[s], xs[s], u);
            hc_u[c] = u;
            sum += u;
        }
    }
    if (p.read == HC_READ_NONE) return;
    const int row = p.compact ? p.meta.tok_outrow()[t] : t;
    if (p.hidden)
        for (int c = threadIdx.x; c < W; c += blockDim.x) p.hidden[(size_t)t * W + c] = hc_u[c];
    if (row < 0) return;
    const float mean = rms_block_sum(sum, red) / (float)W;
    float sq = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = hc_u[c] - mean; sq = fmaf(d, d, sq); }
    sq = rms_block_sum(sq, red);
    const float r = 1.f / sqrtf(sq / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) p.h[(size_t)row * W + c] = (hc_u[c] - mean) * r * p.ln_w[c] + p.ln_b[c];
}

struct HcSumParams { const float* x; float* out; int S, W; MetaView meta; };

__global__ void __launch_bounds__(NORM_THREADS) hc_sum_kernel(const HcSumParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    for (int c = threadIdx.x; c < p.W; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < p.S; ++s) a += p.x[((size_t)t * p.S + s) * p.W + c];
        p.out[(size_t)t * p.W + c] = a;
    }
}

}  // namespace b200
