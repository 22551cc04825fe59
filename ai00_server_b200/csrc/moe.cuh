// Routed mixture of experts around the grouped linear kernels (linear.cuh).
//   moe_route_kernel     one CTA per token: router logits (f32 products on the f32 row, in every precision), probabilities =
//                        softmax over all router outputs (real + identity experts);
//                        the `top` largest of (probability + selection bias) are chosen (ties: lower index), their weights
//                        are the un-biased probabilities, not renormalised
//   moe_group_kernel     one CTA: per-expert row counts, offsets and token lists in token order (deterministic), and for every
//                        (token, choice) its compact row, or -1 for an identity expert
//   moe_combine_kernel   x[t] += gate2[t] * ( sum_k w_k * (expert row | h[t] for an identity expert)
//                                              + sigmoid(sg . h[t]) * shared[t] )                     (residual accumulate, f32)
// The experts' matrices are stacked [E][...] so that one grouped launch covers all of them; rows are gathered by list.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"

namespace b200 {

constexpr int MOE_MAX_TOP = 8;

struct MoeRouteParams {
    const float* h; int ldh;                  // [T, K] router input (f32)
    const __nv_bfloat16* Wr;                  // [NE, K] router matrix
    int K;
    const float* bias;                        // [NE] selection bias (nullptr: none)
    int NE, top;
    int* sel;                                 // [T][top] expert index
    float* wgt;                               // [T][top]
    MetaView meta;
    int mode = 0;                             // MOE_SOFTMAX_ALL | MOE_TOP_LOGITS | MOE_SIGMOID_GROUPS
    int groups = 0, keep = 0;                 // MOE_SIGMOID_GROUPS: equal groups of neighbouring experts, groups that stay eligible (0: no groups)
};

// MOE_SOFTMAX_ALL: probabilities over all outputs, choice by probability + bias, weights = the chosen probabilities as they are.
// MOE_TOP_LOGITS:  bias is part of the logits; the `top` largest logits are chosen, weights = softmax over the chosen logits only.
// MOE_SIGMOID_GROUPS: scores = sigmoid(logit); a group of neighbouring experts is judged by the sum of its two largest scores and
//                  only experts of the `keep` best groups are eligible; the `top` largest eligible scores are chosen, weights =
//                  the chosen scores over their sum.
enum MoeRouteMode { MOE_SOFTMAX_ALL = 0, MOE_TOP_LOGITS = 1, MOE_SIGMOID_GROUPS = 2 };

constexpr int MOE_ROUTE_THREADS = 256;
__host__ __device__ inline size_t moe_route_smem(int K, int NE) { return ((size_t)K + 3 * (size_t)NE) * sizeof(float); }

// warp-wide arg-max over a[0 .. n) in shared memory (ties: lower index); the winner's entry becomes -inf so that the next call
// finds the runner-up.  Every lane returns the same (index, value).
__device__ __forceinline__ int moe_warp_take_max(float* a, int n, float& val) {
    const int lane = threadIdx.x & 31;
    float best = -CUDART_INF_F; int bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
        const float c = a[e];
        if (c > best || (c == best && e < bi)) { best = c; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    __syncwarp();
    if (lane == 0 && bi < n) a[bi] = -CUDART_INF_F;
    __syncwarp();
    val = best;
    return bi;
}

// One CTA per token: router logits in f32 on the f32 row (every warp takes outputs warp, warp + 8, ...), then warp 0 turns them
// into the choice: softmax, + selection bias, `top` largest, weights = the unbiased probabilities.
__global__ void __launch_bounds__(MOE_ROUTE_THREADS) moe_route_kernel(const MoeRouteParams p) {
    extern __shared__ __align__(16) float moe_route_sm[];
    float* sh = moe_route_sm;                 // [K]
    float* z = sh + p.K;                      // [NE]
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, K = p.K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) sh[k] = p.h[(size_t)t * p.ldh + k];
    __syncthreads();
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.Wr) & 15) == 0);
    for (int e = warp; e < p.NE; e += MOE_ROUTE_THREADS / 32) {
        const __nv_bfloat16* w = p.Wr + (size_t)e * K;
        float acc = 0.f;
        if (vec) {
            for (int k = lane * 8; k < K; k += 256) {
                const uint4 q = __ldg(reinterpret_cast<const uint4*>(w + k));
                const __nv_bfloat162* hq = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(hq[j]);
                    acc = fmaf(f.x, sh[k + 2 * j], acc);
                    acc = fmaf(f.y, sh[k + 2 * j + 1], acc);
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(w[k]), sh[k], acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) z[e] = acc + (p.mode == MOE_TOP_LOGITS && p.bias ? p.bias[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    if (p.mode == MOE_SIGMOID_GROUPS) {
        float* ms = z + p.NE;                 // [NE] scores still eligible (-inf: not, or already chosen)
        float* gs = ms + p.NE;                // [groups] group scores; a kept group's entry ends as -inf
        for (int e = lane; e < p.NE; e += 32) { const float s = 1.f / (1.f + expf(-z[e])); z[e] = s; ms[e] = s; }
        __syncwarp();
        if (p.groups > 0) {
            const int per = p.NE / p.groups;
            for (int g = lane; g < p.groups; g += 32) {
                float a = -CUDART_INF_F, b = -CUDART_INF_F;          // the two largest of the group
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    const float s = z[e];
                    if (s > a) { b = a; a = s; } else if (s > b) b = s;
                }
                gs[g] = per > 1 ? a + b : a;
            }
            __syncwarp();
            for (int k = 0; k < p.keep; ++k) {             // taking a maximum leaves -inf in its place (every score is finite)
                float v;
                (void)moe_warp_take_max(gs, p.groups, v);
            }
            for (int e = lane; e < p.NE; e += 32)
                if (gs[e / per] != -CUDART_INF_F) ms[e] = -CUDART_INF_F;   // its group was not kept
            __syncwarp();
        }
        int idx[MOE_MAX_TOP];
        float sc[MOE_MAX_TOP], sum = 0.f;
        for (int k = 0; k < p.top; ++k) {
            float v;
            idx[k] = moe_warp_take_max(ms, p.NE, v);
            sc[k] = z[min(idx[k], p.NE - 1)];
            sum += sc[k];
        }
        if (lane == 0)
            for (int k = 0; k < p.top; ++k) {
                p.sel[(size_t)t * p.top + k] = idx[k];
                p.wgt[(size_t)t * p.top + k] = sc[k] / (sum + 1e-20f);
            }
        return;
    }
    if (p.mode == MOE_TOP_LOGITS) {
        unsigned long long taken = 0ull;
        float zs[MOE_MAX_TOP];
        float top_max = -CUDART_INF_F;
        for (int k = 0; k < p.top; ++k) {
            float best = -CUDART_INF_F; int bi = 0x7fffffff;
            for (int e = lane, i = 0; e < p.NE; e += 32, ++i) {
                if ((taken >> i) & 1ull) continue;
                const float c = z[e];
                if (c > best || (c == best && e < bi)) { best = c; bi = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
            }
            if ((bi & 31) == lane) taken |= 1ull << (bi >> 5);
            if (lane == 0) p.sel[(size_t)t * p.top + k] = bi;
            zs[k] = best;
            if (k == 0) top_max = best;
        }
        float sum = 0.f;
        for (int k = 0; k < p.top; ++k) sum += expf(zs[k] - top_max);
        if (lane == 0)
            for (int k = 0; k < p.top; ++k) p.wgt[(size_t)t * p.top + k] = expf(zs[k] - top_max) / sum;
        return;
    }
    float mx = -CUDART_INF_F;
    for (int e = lane; e < p.NE; e += 32) mx = fmaxf(mx, z[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < p.NE; e += 32) sum += expf(z[e] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    unsigned long long taken_lo = 0ull;       // lanes keep their own "already chosen" marks: expert e = lane + 32 * i -> bit i
    for (int k = 0; k < p.top; ++k) {
        float best = -CUDART_INF_F; int bi = 0x7fffffff;
        for (int e = lane, i = 0; e < p.NE; e += 32, ++i) {
            if ((taken_lo >> i) & 1ull) continue;
            const float c = expf(z[e] - mx) * inv + (p.bias ? p.bias[e] : 0.f);
            if (c > best || (c == best && e < bi)) { best = c; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if ((bi & 31) == lane) taken_lo |= 1ull << (bi >> 5);
        if (lane == 0) {
            p.sel[(size_t)t * p.top + k] = bi;
            p.wgt[(size_t)t * p.top + k] = expf(z[bi] - mx) * inv;
        }
    }
}

struct MoeGroupParams {
    const int* sel; int top, E;               // real experts are 0 .. E-1
    int* cnt; int* off; int* list;            // [E], [E], [T * top]
    int* row_of;                              // [T][top] compact row or -1
    MetaView meta;
};

__global__ void __launch_bounds__(256) moe_group_kernel(const MoeGroupParams p) {
    extern __shared__ int moe_smem[];         // [E] counts, [E] offsets, [T * top] choices
    int* s_cnt = moe_smem;
    int* s_off = s_cnt + p.E;
    int* s_sel = s_off + p.E;
    const int T = p.meta.T(), n = T * p.top;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s_sel[i] = p.sel[i];
    __syncthreads();
    // a warp per expert: ballots over 32 choices at a time keep the token order without a serial scan
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < p.E; e += nw) {
        int c = 0;
        for (int i0 = 0; i0 < n; i0 += 32) c += __popc(__ballot_sync(0xffffffffu, i0 + lane < n && s_sel[i0 + lane] == e));
        if (lane == 0) s_cnt[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < p.E; ++e) { s_off[e] = acc; acc += s_cnt[e]; }
    }
    __syncthreads();
    for (int e = warp; e < p.E; e += nw) {
        if (lane == 0) { p.cnt[e] = s_cnt[e]; p.off[e] = s_off[e]; }
        int w = s_off[e];
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < n && s_sel[i] == e;
            const unsigned mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int pos = w + __popc(mask & ((1u << lane) - 1u));
                p.list[pos] = i / p.top;
                p.row_of[i] = pos;
            }
            w += __popc(mask);
        }
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (s_sel[i] >= p.E) p.row_of[i] = -1;
}

struct MoeCombineParams {
    float* x;                                 // [T, W] residual, accumulated in place
    const float* h;                           // [T, W] the feed-forward's input
    const float* gate;  int ldg;              // [T, W] residual gate of the feed-forward
    const float* rows;                        // [T * top, W] expert outputs, compact rows
    const int* row_of; const float* wgt; int top;
    const float* shared;                      // [T, W] shared expert output (nullptr: none)
    const __nv_bfloat16* sg;                  // [W] shared-expert gate vector
    int W;
    MetaView meta;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombineParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    float sgate = 0.f;
    if (p.shared) {
        float d = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) d = fmaf(__bfloat162float(p.sg[c]), p.h[(size_t)t * W + c], d);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = d;
        __syncthreads();
        d = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) d += red[w];
        sgate = 1.f / (1.f + expf(-d));
    }
    int rows[MOE_MAX_TOP]; float wg[MOE_MAX_TOP];
#pragma unroll
    for (int k = 0; k < MOE_MAX_TOP; ++k)
        if (k < p.top) { rows[k] = p.row_of[(size_t)t * p.top + k]; wg[k] = p.wgt[(size_t)t * p.top + k]; }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float f = 0.f;
#pragma unroll
        for (int k = 0; k < MOE_MAX_TOP; ++k)
            if (k < p.top) f = fmaf(wg[k], rows[k] >= 0 ? p.rows[(size_t)rows[k] * W + c] : p.h[(size_t)t * W + c], f);
        if (p.shared) f = fmaf(sgate, p.shared[(size_t)t * W + c], f);
        p.x[(size_t)t * W + c] += p.gate[(size_t)t * p.ldg + c] * f;
    }
}

}  // namespace b200
