// Grouped linear layers over row-major f32 activations and bf16 weights stored [out, in]:  Y[r, n] = epi(sum_k X[r, k] W[n, k]).
//
// One launch covers `groups` independent problems that share N and K (blockIdx.z): the heads of a per-head projection (column
// offsets into X / Y), or the experts of a routed feed-forward (row lists built on the device).  Row counts come from device
// memory (the step metadata, the router's per-expert counts), so a captured step graph never changes.
//
//   lin_tile_kernel<EXACT>   steps of many rows.  EXACT = false: bf16 operands on the tensor cores (mma.sync m16n8k16, f32
//                            accumulate) behind a two-stage cp.async pipeline, activations rounded to bf16 when the fragments
//                            are built; EXACT = true: plain f32 FMA on the f32 activations (bf16 weights widen exactly), no
//                            reduced-precision product anywhere.
//   lin_mma16_kernel         serving precision, steps of up to 16 rows (decode): the same tensor-core product with the k range
//                            split over the warps of a CTA and every operand streamed straight from global memory; the launch
//                            is bound by the weight bytes.
//   lin_skinny_kernel        exact precision, a few rows: one warp per output pair, weight rows streamed as 16-byte loads, f32
//                            FMA.
//
// Epilogues (fused): bias, sigmoid / silu / erf-gelu / squared relu / capped tanh, a sigmoid gate on the output, accumulate-into-residual
// (plain or through a gate), and the gated units
// (clamped, or plain silu(g) * u) on interleaved (gate, up) output pairs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum LinEpi {
    LE_STORE = 0,       // Y = acc (+ bias)
    LE_SIGMOID = 1,     // Y = sigmoid(acc + bias)
    LE_GATED_ADD = 2,   // Y += gate[r, n] * acc          (residual accumulate; every element has one writer)
    LE_GLU_CLAMP = 3,   // outputs (2i, 2i+1) = (g, u): Y[r, i] = min(g, lim) * sigmoid(1.702 min(g, lim)) * (clamp(u, -lim, lim) + 1)
    LE_GLU_SILU = 4,    // outputs (2i, 2i+1) = (g, u): Y[r, i] = g * sigmoid(g) * u
    LE_GELU_ERF = 5,    // Y = a * Phi(a), a = acc + bias, Phi the normal distribution function (erf form)
    LE_RELU_SQ = 6,     // Y = max(acc + bias, 0)^2
    LE_ADD = 7,         // Y += acc + bias                 (residual accumulate; every element has one writer)
    LE_MUL_SIGMOID = 8, // Y = (acc + bias) * sigmoid(gate[r, n])   (group g reads gate + g * gate_gstride)
    LE_TANH_CAP = 9,    // Y = limit * tanh((acc + bias) / limit)
};

struct LinParams {
    const float* X; int ldx; long long x_gstride;      // X + g * x_gstride, row stride ldx (floats)
    const __nv_bfloat16* W; long long w_gstride;       // W + g * w_gstride, row n at n * K
    float* Y; int ldy; long long y_gstride;
    int N, K;
    const int* cnt; int cnt_gstride;                   // rows of group g = cnt[g * cnt_gstride]
    const int* off;                                    // first compact row of group g (nullptr: 0)
    const int* xlist;                                  // X row of compact row i (nullptr: i)
    const float* bias;                                 // [N] (nullptr: none); group g adds g * N
    const float* gate; int ldg;                        // LE_GATED_ADD, LE_MUL_SIGMOID
    long long gate_gstride;                            // LE_MUL_SIGMOID: gate + g * gate_gstride
    float limit;                                       // LE_GLU_CLAMP, LE_TANH_CAP
    int epi;
    int max_rows;                                      // upper bound of any group's rows (grid sizing)
    // split-k (tensor-core tile kernel, one group): blockIdx.x = split * n_tiles + n_tile, split s multiplies its own range of
    // k slabs and leaves raw sums in ws[s][max_rows][N]; lin_splitk_finish_kernel adds the splits in order and runs the epilogue.
    // Projections with few output tiles (low-rank stages) otherwise occupy a handful of SMs, each waiting on its own loads.
    int ksplit;                                        // 0 / 1: off
    float* ws;
};

__device__ __forceinline__ float lin_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ float lin_glu(float g, float u, float lim) {
    g = fminf(g, lim);
    u = fminf(fmaxf(u, -lim), lim);
    return g * lin_sigmoid(1.702f * g) * (u + 1.f);
}

// one finished output element (or pair) -> memory
__device__ __forceinline__ void lin_store(const LinParams& p, int g, int yrow, int n, float a0, float a1, bool has1) {
    float* Y = p.Y + g * p.y_gstride;
    if (p.epi == LE_GLU_CLAMP) {                       // n is even: (gate, up) pair -> column n / 2
        Y[(size_t)yrow * p.ldy + (n >> 1)] = lin_glu(a0, a1, p.limit);
        return;
    }
    if (p.epi == LE_GLU_SILU) {
        Y[(size_t)yrow * p.ldy + (n >> 1)] = a0 * lin_sigmoid(a0) * a1;
        return;
    }
    const float* b = p.bias ? p.bias + (size_t)g * p.N : nullptr;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        if (j == 1 && !has1) break;
        float a = j ? a1 : a0;
        const int nn = n + j;
        if (b) a += b[nn];
        float* y = Y + (size_t)yrow * p.ldy + nn;
        if (p.epi == LE_SIGMOID) *y = lin_sigmoid(a);
        else if (p.epi == LE_GELU_ERF) *y = 0.5f * a * (1.f + erff(a * 0.70710678118654752f));
        else if (p.epi == LE_RELU_SQ) { const float r = fmaxf(a, 0.f); *y = r * r; }
        else if (p.epi == LE_GATED_ADD) *y += p.gate[(size_t)yrow * p.ldg + nn] * a;
        else if (p.epi == LE_ADD) *y += a;
        else if (p.epi == LE_MUL_SIGMOID) *y = a * lin_sigmoid(p.gate[g * p.gate_gstride + (size_t)yrow * p.ldg + nn]);
        else if (p.epi == LE_TANH_CAP) *y = p.limit * tanhf(a / p.limit);
        else *y = a;
    }
}

// ------------------------------------------------------------------------------------------------------------------
// tiled kernel: 64 rows x 64 outputs per CTA, k in slabs of 32; 128 threads
// ------------------------------------------------------------------------------------------------------------------
constexpr int LIN_BM = 64, LIN_BN = 64, LIN_BK = 32, LIN_THREADS = 128;
constexpr int LIN_TC_BK = 64, LIN_TC_STAGES = 3;       // tensor-core path: k slab and pipeline depth
constexpr size_t LIN_TC_SMEM = (size_t)LIN_TC_STAGES * (LIN_BM * (LIN_TC_BK + 4) * sizeof(float) + LIN_BN * (LIN_TC_BK + 8) * 2);

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float2 v) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <bool EXACT>
__global__ void __launch_bounds__(LIN_THREADS) lin_tile_kernel(const LinParams p) {
    const int g = blockIdx.z;
    const int rows = p.cnt[(size_t)g * p.cnt_gstride];
    const int r0 = blockIdx.y * LIN_BM;
    if (r0 >= rows) return;
    const int n_tiles = (p.N + LIN_BN - 1) / LIN_BN;
    const int n0 = (blockIdx.x % n_tiles) * LIN_BN;
    const int split = blockIdx.x / n_tiles;            // 0 unless split-k
    const int base = p.off ? p.off[g] : 0;
    const float* X = p.X + g * p.x_gstride;
    const __nv_bfloat16* W = p.W + g * p.w_gstride;
    const int tid = threadIdx.x, K = p.K, N = p.N;

    __shared__ int s_xrow[LIN_BM];
    for (int i = tid; i < LIN_BM; i += LIN_THREADS) {
        const int r = r0 + i;
        s_xrow[i] = r < rows ? (p.xlist ? p.xlist[base + r] : base + r) : -1;
    }

    if constexpr (EXACT) {
        __shared__ float sA[LIN_BK][LIN_BM + 1];       // k-major: the inner product walks k, threads differ in row / column
        __shared__ float sB[LIN_BK][LIN_BN + 1];
        const int ty = tid >> 3, tx = tid & 7;         // 16 x 8 threads: 4 rows x 8 columns each
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        __syncthreads();
        for (int k0 = 0; k0 < K; k0 += LIN_BK) {
            for (int e = tid; e < LIN_BM * LIN_BK; e += LIN_THREADS) {
                const int r = e / LIN_BK, k = e % LIN_BK;
                const int xr = s_xrow[r];
                sA[k][r] = (xr >= 0 && k0 + k < K) ? X[(size_t)xr * p.ldx + k0 + k] : 0.f;
                const int n = n0 + r;
                sB[k][r] = (n < N && k0 + k < K) ? __bfloat162float(W[(size_t)n * K + k0 + k]) : 0.f;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = 0; k < LIN_BK; ++k) {
                float a[4], b[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = sA[k][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 8; ++j) b[j] = sB[k][tx * 8 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + ty * 4 + i;
            if (r >= rows) continue;
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const int n = n0 + tx * 8 + j;
                if (n < N) lin_store(p, g, base + r, n, acc[i][j], acc[i][j + 1], n + 1 < N);
            }
        }
    } else {
        // three-stage cp.async pipeline over k slabs of 64: two slabs stream in while one is multiplied.  Activations are
        // staged as f32 and rounded to bf16 when the fragments are built; weights are staged as stored.
        constexpr int LDA = LIN_TC_BK + 4;             // floats: 272-byte rows (16-byte aligned chunks, spread banks)
        constexpr int LDB = LIN_TC_BK + 8;             // bf16: 144-byte rows
        extern __shared__ __align__(16) unsigned char lin_dyn_smem[];
        float (*sA)[LIN_BM][LDA] = reinterpret_cast<float (*)[LIN_BM][LDA]>(lin_dyn_smem);
        __nv_bfloat16 (*sB)[LIN_BN][LDB] =
            reinterpret_cast<__nv_bfloat16 (*)[LIN_BN][LDB]>(lin_dyn_smem + sizeof(float) * LIN_TC_STAGES * LIN_BM * LDA);
        const int warp = tid >> 5, lane = tid & 31;
        const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;      // 2 x 2 warps, 32 x 32 each
        const int gq = lane >> 2, tq = lane & 3;
        float acc[2][4][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
        const bool vecW = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
        const bool vecX = (p.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
        __syncthreads();
        auto stage = [&](int buf, int k0) {
            for (int e = tid; e < LIN_BM * (LIN_TC_BK / 4); e += LIN_THREADS) {
                const int r = e / (LIN_TC_BK / 4), k = (e % (LIN_TC_BK / 4)) * 4;
                const int xr = s_xrow[r];
                float* dst = &sA[buf][r][k];
                if (xr >= 0 && vecX && k0 + k + 3 < K) {
                    cp_async16(dst, X + (size_t)xr * p.ldx + k0 + k);
                } else {
                    float v[4] = {0.f, 0.f, 0.f, 0.f};
                    if (xr >= 0) {
                        const float* src = X + (size_t)xr * p.ldx + k0 + k;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (k0 + k + j < K) v[j] = src[j];
                    }
                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                }
            }
            for (int e = tid; e < LIN_BN * (LIN_TC_BK / 8); e += LIN_THREADS) {
                const int r = e / (LIN_TC_BK / 8), k = (e % (LIN_TC_BK / 8)) * 8;
                const int n = n0 + r;
                __nv_bfloat16* dst = &sB[buf][r][k];
                if (n < N && vecW && k0 + k + 7 < K) {
                    cp_async16(dst, W + (size_t)n * K + k0 + k);
                } else {
                    __align__(16) __nv_bfloat16 t[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) t[j] = (n < N && k0 + k + j < K) ? W[(size_t)n * K + k0 + k + j] : __float2bfloat16(0.f);
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(t);
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };
        const int nslab_all = (K + LIN_TC_BK - 1) / LIN_TC_BK;
        const int nsp = p.ksplit > 1 ? p.ksplit : 1;
        const int per = (nslab_all + nsp - 1) / nsp;
        const int slab0 = split * per;
        const int nslab = max(0, min(nslab_all, slab0 + per) - slab0);
        // one commit group per slab, empty past the end, so that "all but the two newest groups" always means slab sl
        for (int i = 0; i < LIN_TC_STAGES - 1; ++i) {
            if (i < nslab) stage(i, (slab0 + i) * LIN_TC_BK);
            else asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        for (int sl = 0; sl < nslab; ++sl) {
            const int buf = sl % LIN_TC_STAGES;
            // the buffer refilled here was multiplied in iteration sl - 1, which ended with a barrier
            if (sl + LIN_TC_STAGES - 1 < nslab) stage((sl + LIN_TC_STAGES - 1) % LIN_TC_STAGES, (slab0 + sl + LIN_TC_STAGES - 1) * LIN_TC_BK);
            else asm volatile("cp.async.commit_group;\n" ::: "memory");
            asm volatile("cp.async.wait_group %0;\n" ::"n"(LIN_TC_STAGES - 1) : "memory");
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < LIN_TC_BK; kk += 16) {
                uint32_t a[2][4], b[4][2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int r = wm + i * 16 + gq;
                    a[i][0] = pack_bf16x2(*reinterpret_cast<const float2*>(&sA[buf][r][kk + tq * 2]));
                    a[i][1] = pack_bf16x2(*reinterpret_cast<const float2*>(&sA[buf][r + 8][kk + tq * 2]));
                    a[i][2] = pack_bf16x2(*reinterpret_cast<const float2*>(&sA[buf][r][kk + 8 + tq * 2]));
                    a[i][3] = pack_bf16x2(*reinterpret_cast<const float2*>(&sA[buf][r + 8][kk + 8 + tq * 2]));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = wn + j * 8 + gq;
                    b[j][0] = *reinterpret_cast<const uint32_t*>(&sB[buf][n][kk + tq * 2]);
                    b[j][1] = *reinterpret_cast<const uint32_t*>(&sB[buf][n][kk + 8 + tq * 2]);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], b[j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + tq * 2;
                if (n >= N) continue;
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int r = r0 + wm + i * 16 + gq + hrow * 8;
                    if (r >= rows) continue;
                    if (p.ksplit > 1) {
                        float* dst = p.ws + ((size_t)split * p.max_rows + r) * N + n;
                        dst[0] = acc[i][j][hrow * 2];
                        if (n + 1 < N) dst[1] = acc[i][j][hrow * 2 + 1];
                    } else {
                        lin_store(p, g, base + r, n, acc[i][j][hrow * 2], acc[i][j][hrow * 2 + 1], n + 1 < N);
                    }
                }
            }
    }
}

// sums the split-k partials in split order and runs the epilogue (one group, rows in place)
__global__ void __launch_bounds__(256) lin_splitk_finish_kernel(const LinParams p) {
    const int r = blockIdx.y;
    if (r >= p.cnt[0]) return;
    const int n = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (n >= p.N) return;
    const bool has1 = n + 1 < p.N;
    float s0 = 0.f, s1 = 0.f;
    for (int sp = 0; sp < p.ksplit; ++sp) {
        const float* src = p.ws + ((size_t)sp * p.max_rows + r) * p.N + n;
        s0 += src[0];
        if (has1) s1 += src[1];
    }
    lin_store(p, 0, r, n, s0, s1, has1);
}

// ------------------------------------------------------------------------------------------------------------------
// skinny kernel: up to LIN_SK_ROWS rows per pass, one warp per output pair
// ------------------------------------------------------------------------------------------------------------------
constexpr int LIN_SK_ROWS = 8, LIN_SK_WARPS = 8;

__global__ void __launch_bounds__(LIN_SK_WARPS * 32) lin_skinny_kernel(const LinParams p) {
    const int g = blockIdx.z;
    const int rows = p.cnt[(size_t)g * p.cnt_gstride];
    if (rows <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = (blockIdx.x * LIN_SK_WARPS + warp) * 2;
    if (n >= p.N) return;
    const bool has1 = n + 1 < p.N;
    const int base = p.off ? p.off[g] : 0;
    const float* X = p.X + g * p.x_gstride;
    const __nv_bfloat16* w0 = p.W + g * p.w_gstride + (size_t)n * p.K;
    const __nv_bfloat16* w1 = has1 ? w0 + p.K : w0;
    const int K = p.K;
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(w0) & 15) == 0) && (p.ldx % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
    for (int rb = 0; rb < rows; rb += LIN_SK_ROWS) {
        const int nr = min(LIN_SK_ROWS, rows - rb);
        const float* xr[LIN_SK_ROWS];
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) {
            const int r = rb + min(i, nr - 1);
            xr[i] = X + (size_t)(p.xlist ? p.xlist[base + r] : base + r) * p.ldx;
        }
        float a0[LIN_SK_ROWS], a1[LIN_SK_ROWS];
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) a0[i] = a1[i] = 0.f;
        if (vec) {
            for (int k = lane * 8; k < K; k += 256) {
                const uint4 q0 = *reinterpret_cast<const uint4*>(w0 + k);
                const uint4 q1 = *reinterpret_cast<const uint4*>(w1 + k);
                const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&q0);
                const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&q1);
                float f0[8], f1[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 u = __bfloat1622float2(h0[j]), v = __bfloat1622float2(h1[j]);
                    f0[2 * j] = u.x; f0[2 * j + 1] = u.y; f1[2 * j] = v.x; f1[2 * j + 1] = v.y;
                }
#pragma unroll
                for (int i = 0; i < LIN_SK_ROWS; ++i) {
                    if (i >= nr) break;
                    const float4 xa = *reinterpret_cast<const float4*>(xr[i] + k);
                    const float4 xb = *reinterpret_cast<const float4*>(xr[i] + k + 4);
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) { a0[i] = fmaf(xv[j], f0[j], a0[i]); a1[i] = fmaf(xv[j], f1[j], a1[i]); }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float f0 = __bfloat162float(w0[k]), f1 = __bfloat162float(w1[k]);
#pragma unroll
                for (int i = 0; i < LIN_SK_ROWS; ++i) {
                    if (i >= nr) break;
                    const float xv = xr[i][k];
                    a0[i] = fmaf(xv, f0, a0[i]); a1[i] = fmaf(xv, f1, a1[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a0[i] += __shfl_xor_sync(0xffffffffu, a0[i], o);
                a1[i] += __shfl_xor_sync(0xffffffffu, a1[i], o);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < LIN_SK_ROWS; ++i)
                if (i < nr) lin_store(p, g, base + rb + i, n, a0[i], a1[i], has1);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// steps of up to 16 rows on the tensor cores: 16 outputs per CTA, the k range split over 8 warps.  A lane streams 16 bytes of
// one weight row (8 consecutive k) and the matching 8 activations of rows g and g + 8 straight from global memory; those 8 k
// feed two m16n8k16 products (any fixed pairing of k between the A and B fragments is a valid sum order), so no operand
// passes through shared memory and every weight byte is read once, in full 32-byte sectors.
// ------------------------------------------------------------------------------------------------------------------
constexpr int LIN_M16_WARPS = 8;

__device__ __forceinline__ void lin_ld8(const float* p, bool vec, int valid, float v[8]) {
    if (vec && valid >= 8) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = j < valid ? p[j] : 0.f;
    }
}

constexpr int LIN_M16_BN = 16;                     // outputs per CTA: two n8 tiles share every activation fragment

__global__ void __launch_bounds__(LIN_M16_WARPS * 32, 3) lin_mma16_kernel(const LinParams p) {
    const int g = blockIdx.z;
    const int rows = p.cnt[(size_t)g * p.cnt_gstride];
    if (rows <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * LIN_M16_BN;
    const int base = p.off ? p.off[g] : 0;
    const float* X = p.X + g * p.x_gstride;
    const int K = p.K;
    const __nv_bfloat16* Wg = p.W + g * p.w_gstride;
    const __nv_bfloat16* wrow[2];
    bool nvalid[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int n = n0 + j * 8 + gq;
        nvalid[j] = n < p.N;
        wrow[j] = Wg + (size_t)min(n, p.N - 1) * K;
    }
    const bool vecW = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(Wg) & 15) == 0);
    const bool vecX = (p.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
    __shared__ float red[LIN_M16_WARPS][16][LIN_M16_BN];
    for (int rb = 0; rb < rows; rb += 16) {
        const int rlo = rb + gq, rhi = rb + gq + 8;
        const float* xlo = rlo < rows ? X + (size_t)(p.xlist ? p.xlist[base + rlo] : base + rlo) * p.ldx : nullptr;
        const float* xhi = rhi < rows ? X + (size_t)(p.xlist ? p.xlist[base + rhi] : base + rhi) * p.ldx : nullptr;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        constexpr int U = 2;                       // k blocks per batch: 4 weight loads in flight per lane
        for (int kb0 = warp * 32; kb0 < K; kb0 += LIN_M16_WARPS * 32 * U) {
            uint4 wq[U][2];
#pragma unroll
            for (int u = 0; u < U; ++u) {          // all weight loads of the batch first: they are the HBM stream
                const int k = kb0 + u * LIN_M16_WARPS * 32 + tq * 8;
                const int valid = max(0, min(8, K - k));
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    wq[u][j] = make_uint4(0, 0, 0, 0);
                    if (nvalid[j] && valid > 0) {
                        if (vecW) {
                            wq[u][j] = __ldg(reinterpret_cast<const uint4*>(wrow[j] + k));
                        } else {
                            __align__(16) __nv_bfloat16 t[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) t[e] = e < valid ? wrow[j][k + e] : __float2bfloat16(0.f);
                            wq[u][j] = *reinterpret_cast<const uint4*>(t);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = kb0 + u * LIN_M16_WARPS * 32 + tq * 8;
                const int valid = max(0, min(8, K - k));
                if (kb0 + u * LIN_M16_WARPS * 32 >= K) break;          // warp-uniform
                float lo[8], hi[8];
                if (xlo && valid > 0) lin_ld8(xlo + k, vecX, valid, lo);
                else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) lo[e] = 0.f;
                }
                if (xhi && valid > 0) lin_ld8(xhi + k, vecX, valid, hi);
                else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) hi[e] = 0.f;
                }
                uint32_t a0[4], a1[4];
                a0[0] = pack_bf16x2(make_float2(lo[0], lo[1])); a0[1] = pack_bf16x2(make_float2(hi[0], hi[1]));
                a0[2] = pack_bf16x2(make_float2(lo[2], lo[3])); a0[3] = pack_bf16x2(make_float2(hi[2], hi[3]));
                a1[0] = pack_bf16x2(make_float2(lo[4], lo[5])); a1[1] = pack_bf16x2(make_float2(hi[4], hi[5]));
                a1[2] = pack_bf16x2(make_float2(lo[6], lo[7])); a1[3] = pack_bf16x2(make_float2(hi[6], hi[7]));
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t b[2];
                    b[0] = wq[u][j].x; b[1] = wq[u][j].y;
                    mma_bf16_16816(acc[j], a0, b);
                    b[0] = wq[u][j].z; b[1] = wq[u][j].w;
                    mma_bf16_16816(acc[j], a1, b);
                }
            }
        }
        __syncthreads();                           // red of the previous row block has been read
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            red[warp][gq][j * 8 + tq * 2] = acc[j][0]; red[warp][gq][j * 8 + tq * 2 + 1] = acc[j][1];
            red[warp][gq + 8][j * 8 + tq * 2] = acc[j][2]; red[warp][gq + 8][j * 8 + tq * 2 + 1] = acc[j][3];
        }
        __syncthreads();
        if (threadIdx.x < 128) {
            const int r = threadIdx.x >> 3, c = (threadIdx.x & 7) * 2;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int w = 0; w < LIN_M16_WARPS; ++w) { s0 += red[w][r][c]; s1 += red[w][r][c + 1]; }
            if (rb + r < rows && n0 + c < p.N) lin_store(p, g, base + rb + r, n0 + c, s0, s1, n0 + c + 1 < p.N);
        }
    }
}

}  // namespace b200
