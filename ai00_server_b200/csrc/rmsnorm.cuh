// Root-mean-square normalisation stages on f32 rows (every norm of this family is computed in 32-bit):
//   embed_rows_kernel      x[t] = table[token[t]] * scale, written to every copy of the residual   (bf16 table -> f32 residual)
//   norm_shift_kernel      h = x / rms(x) * g (one scalar gain);  hs = h + (h_prev - h) * mu  (token shift on the NORMED row;
//                          h_prev = the previous token's h: the row before it in this step, or the sequence's shift state);
//   shift_commit_kernel    the last token of every sequence in the step leaves its h as the new shift state
//   rms_rows_kernel        y[r, c*w .. c*w+w) = x / rms(x over the w-wide chunk) * weight[w]   (per-chunk norm with a weight vector)
//   final_norm_kernel      rows that want logits: x[out_tok[r]] / rms * g  -> compact [R, W] head operand (+ all hidden rows);
//                          g = one scalar gain or a weight vector
//   norm_add_kernel        x += y / rms(y) * w: the norm sits on a sublayer's output (optionally combining routed expert rows first)
//   pre_norm_kernel        the boundary in front of a pre-norm sublayer in one pass: the routed experts that just finished are
//                          combined into the residual, a looped run of layers that begins adds the embedding row and its pass
//                          vector, and the normed row (or, at the end of the stack, the compact rows that want logits) is written
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "common.cuh"

namespace b200 {

constexpr int NORM_THREADS = 256;

__device__ __forceinline__ float rms_block_sum(float v, float* red /* [32] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                       // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];      // same order in every thread
    return s;
}

struct EmbedRowsParams {
    const __nv_bfloat16* table;
    float* x;
    int W;
    MetaView meta;
    float scale = 1.f;       // factor on the row
    int copies = 1;          // the row is written `copies` times: x is [T][copies][W]
};

__global__ void __launch_bounds__(NORM_THREADS) embed_rows_kernel(const EmbedRowsParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const __nv_bfloat16* src = p.table + (size_t)p.meta.tok()[t] * p.W;
    float* dst = p.x + (size_t)t * p.copies * p.W;
    for (int c = threadIdx.x; c < p.W; c += blockDim.x) {
        const float v = __bfloat162float(src[c]) * p.scale;
        for (int s = 0; s < p.copies; ++s) dst[(size_t)s * p.W + c] = v;
    }
}

struct NormShiftParams {
    const float* x;          // [T, W] residual
    float* h;                // [T, W] normed row (feed-forward, gates)
    float* hs;               // [T, W] token-shifted normed row (mixer); nullptr: no shift
    const float* mu;         // [W]
    float* shift_state;      // [S, W] of this layer
    float gain, eps;
    int W;
    MetaView meta;
};

__global__ void __launch_bounds__(NORM_THREADS) norm_shift_kernel(const NormShiftParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    const float* xr = p.x + (size_t)t * W;
    const int prev = p.meta.tok_prev()[t];
    const int slot = p.meta.tok_slot()[t];
    float ss = 0.f, sp = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
        if (prev >= 0) { const float u = p.x[(size_t)prev * W + c]; sp = fmaf(u, u, sp); }
    }
    ss = rms_block_sum(ss, red);
    const float r = p.gain / sqrtf(ss / (float)W + p.eps);
    float rp = 0.f;
    if (prev >= 0) { sp = rms_block_sum(sp, red); rp = p.gain / sqrtf(sp / (float)W + p.eps); }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float hv = xr[c] * r;
        p.h[(size_t)t * W + c] = hv;
        if (p.hs) {
            const float hp = prev >= 0 ? p.x[(size_t)prev * W + c] * rp : p.shift_state[(size_t)slot * W + c];
            p.hs[(size_t)t * W + c] = hv + (hp - hv) * p.mu[c];
        }
    }
}

// shift-state commit, run after norm_shift_kernel of the same layer (a first token of the sequence may still be reading the
// old row while the last token's CTA would overwrite it, so the commit is its own launch)
__global__ void __launch_bounds__(NORM_THREADS) shift_commit_kernel(const NormShiftParams p) {
    const int i = blockIdx.x;
    if (i >= p.meta.nslots()) return;
    const int t = p.meta.slot_start()[i] + p.meta.slot_count()[i] - 1;
    const int slot = p.meta.slot_id()[i];
    for (int c = threadIdx.x; c < p.W; c += blockDim.x) p.shift_state[(size_t)slot * p.W + c] = p.h[(size_t)t * p.W + c];
}

struct RmsRowsParams {
    const float* x; int ldx;
    float* y; int ldy;
    const float* weight;     // [w]
    int w, chunks;           // `chunks` chunks of width w per row
    float eps;
    const int* nrows;
};

__global__ void __launch_bounds__(128) rms_rows_kernel(const RmsRowsParams p) {
    __shared__ float red[32];
    const int r = blockIdx.x, c = blockIdx.y;
    if (r >= *p.nrows) return;
    const float* x = p.x + (size_t)r * p.ldx + (size_t)c * p.w;
    float* y = p.y + (size_t)r * p.ldy + (size_t)c * p.w;
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.w; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = rms_block_sum(ss, red);
    const float s = 1.f / sqrtf(ss / (float)p.w + p.eps);
    for (int i = threadIdx.x; i < p.w; i += blockDim.x) y[i] = x[i] * s * p.weight[i];
}

struct FinalNormParams {
    const float* x;          // [T, W]
    float* y;                // [R, W]
    float* hidden;           // [T, W] copy of the residual (embeddings route); may be nullptr
    float gain, eps;
    int W;
    MetaView meta;
    const float* weight = nullptr;   // [W] per-channel weight instead of the scalar gain
};

__global__ void __launch_bounds__(NORM_THREADS) final_norm_kernel(const FinalNormParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    const float* xr = p.x + (size_t)t * W;
    const int row = p.meta.tok_outrow()[t];
    if (p.hidden)
        for (int c = threadIdx.x; c < W; c += blockDim.x) p.hidden[(size_t)t * W + c] = xr[c];
    if (row < 0) return;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = rms_block_sum(ss, red);
    const float r = (p.weight ? 1.f : p.gain) / sqrtf(ss / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) p.y[(size_t)row * W + c] = xr[c] * r * (p.weight ? p.weight[c] : 1.f);
}

// Norm on a sublayer's OUTPUT, added to the residual:  x[t] += y[t] / rms(y[t]) * w.  The sublayer's output row y is either a
// plain row, or the weighted sum of a routed feed-forward's chosen expert rows plus its shared expert (then this is also the
// experts' combine step).  All f32.
struct NormAddParams {
    float* x;                 // [T, W] residual, accumulated in place
    const float* y;           // [T, W] sublayer output (nullptr with rows)
    const float* rows;        // [T * top, W] expert outputs in compact rows (nullptr: y)
    const int* row_of; const float* wgt; int top;
    const float* shared;      // [T, W] added to the experts' sum (nullptr: none)
    const float* weight;      // [W]
    float eps;
    int W;
    MetaView meta;
};

constexpr int NORM_ADD_MAX_TOP = 8;

__global__ void __launch_bounds__(NORM_THREADS) norm_add_kernel(const NormAddParams p) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float norm_add_row[];      // [W] the combined row (expert form only)
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    float ss = 0.f;
    if (p.rows) {
        int rw[NORM_ADD_MAX_TOP]; float wg[NORM_ADD_MAX_TOP];
#pragma unroll
        for (int k = 0; k < NORM_ADD_MAX_TOP; ++k)
            if (k < p.top) { rw[k] = p.row_of[(size_t)t * p.top + k]; wg[k] = p.wgt[(size_t)t * p.top + k]; }
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            float f = 0.f;
#pragma unroll
            for (int k = 0; k < NORM_ADD_MAX_TOP; ++k)
                if (k < p.top) f = fmaf(wg[k], p.rows[(size_t)rw[k] * W + c], f);
            if (p.shared) f += p.shared[(size_t)t * W + c];
            norm_add_row[c] = f;
            ss = fmaf(f, f, ss);
        }
    } else {
        for (int c = threadIdx.x; c < W; c += blockDim.x) { const float f = p.y[(size_t)t * W + c]; ss = fmaf(f, f, ss); }
    }
    ss = rms_block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float f = p.rows ? norm_add_row[c] : p.y[(size_t)t * W + c];
        p.x[(size_t)t * W + c] += f * r * p.weight[c];
    }
}

// The boundary in front of a pre-norm sublayer.  In this order, each part optional:
//   x[t] += sum_k wgt[t, k] rows[row_of[t, k]] + shared[t]     the routed feed-forward that just finished (its combine step)
//   snap[t] = x[t]                                             the residual as the finished layer leaves it (bring-up aid)
//   x[t] += table[token[t]] + vec                              a pass of a looped run of layers begins
//   h[t] = x[t] / rms(x[t]) * weight                           the sublayer's input; `weight` holds the whole factor (a model
//                                                              that stores offsets from one uploads 1 + w)
// With `compact` only the rows that want logits are normed and land in h[row]; `hidden` gets a copy of every residual row.
// All f32.  Dynamic shared memory: W floats.
struct PreNormParams {
    float* x;                 // [T, W] residual, updated in place
    const float* rows;        // [T * top, W] expert outputs in compact rows (nullptr: nothing pending)
    const int* row_of; const float* wgt; int top;
    const float* shared;      // [T, W] (nullptr: none)
    float* snap;              // [T, W] (nullptr: none)
    const __nv_bfloat16* table;   // [vocab, W] (nullptr: none)
    const float* vec;         // [W] (nullptr: none)
    const float* weight;      // [W] (nullptr: no norm, x is only updated)
    float eps;
    float* h;                 // [T, W], or [R, W] with compact
    int compact;
    float* hidden;            // [T, W] (nullptr: none)
    int W;
    MetaView meta;
};

constexpr int PRE_NORM_THREADS_FEW_ROWS = 1024;    // block size for steps of few tokens (decode): a thread then owns one or two columns

template <int THREADS>
__global__ void __launch_bounds__(THREADS) pre_norm_kernel(const PreNormParams p) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float pre_norm_row[];      // [W]
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    float* xr = p.x + (size_t)t * W;
    int rw[NORM_ADD_MAX_TOP]; float wg[NORM_ADD_MAX_TOP];
    if (p.rows) {
#pragma unroll
        for (int k = 0; k < NORM_ADD_MAX_TOP; ++k)
            if (k < p.top) { rw[k] = p.row_of[(size_t)t * p.top + k]; wg[k] = p.wgt[(size_t)t * p.top + k]; }
    }
    const __nv_bfloat16* er = p.table ? p.table + (size_t)p.meta.tok()[t] * W : nullptr;
    const bool writes = p.rows || er || p.vec;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = xr[c];
        if (p.rows) {
            float f = 0.f;
#pragma unroll
            for (int k = 0; k < NORM_ADD_MAX_TOP; ++k)
                if (k < p.top) f = fmaf(wg[k], p.rows[(size_t)rw[k] * W + c], f);
            if (p.shared) f += p.shared[(size_t)t * W + c];
            v += f;
        }
        if (p.snap) p.snap[(size_t)t * W + c] = v;
        if (er) v += __bfloat162float(er[c]);
        if (p.vec) v += p.vec[c];
        if (writes) xr[c] = v;
        if (p.hidden) p.hidden[(size_t)t * W + c] = v;
        pre_norm_row[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (!p.weight) return;
    const int row = p.compact ? p.meta.tok_outrow()[t] : t;
    if (row < 0) return;
    ss = rms_block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) p.h[(size_t)row * W + c] = pre_norm_row[c] * r * p.weight[c];
}

}  // namespace b200
