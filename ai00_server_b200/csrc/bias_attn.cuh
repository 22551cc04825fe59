// Causal softmax attention over a paged key / value cache with a learned bias per (distance, head) and no rotation: positions
// enter only through the bias.
//
// H query heads, G key / value heads (query head h reads head h / (H / G)).  Per layer and token the cache row holds the G keys
// (unit root-mean-square) followed by the G values: D = G (dk + dv) floats.  For query position i and key position j <= i
//     s_h(i, j) = (q_h(i) . k(j)) * scale + bias[min(i - j, nb)][h]
//     o_h(i) = sum_j softmax_j(s_h(i, .)) v(j)
// The table bias[0 .. nb][H] is built by the host from the model's bucket table (distances share buckets that are evenly
// spaced in the logarithm of the distance; everything from nb on shares the last one), so the kernel knows nothing of buckets
// and another bias law is another table.
// The values may be blended with those another layer computed for the same token before they are cached:
//     v <- (1 - lam) v + lam v_first
//
//   bias_attn_prep_kernel   per token: q heads / rms(q) * scale -> q buffer;  k heads / rms(k) and the (blended) v -> the cache
//                           row of (slot, position); the first blending layer also leaves its v in the step's v_first buffer.
//   bias_attn_kernel        a cluster of 1..8 CTAs per chunk of consecutive tokens of one sequence (SeqMeta chunks), all heads;
//                           the 32-key tiles up to the chunk's last position are dealt out among the cluster's CTAs; every CTA
//                           walks its tiles ONCE with a running maximum / sum per (token, head) row (online softmax) and the
//                           CTAs' partial results are merged through distributed shared memory in rank order.  A warp owns
//                           1, 2 or 4 rows of one key / value head (template): it scores them against a key per lane, then
//                           applies the tile's weights to the values, with no CTA barrier in between; the next tiles arrive by
//                           cp.async into a second buffer meanwhile.  Scores, weights and sums in f32.  Any head size.
//   bias_attn_reg_kernel    the same result for head sizes that are multiples of four up to 128, with nothing staged in shared
//                           memory: see the comment above it.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"
#include "latent_attn.cuh"
#include "linear.cuh"

namespace b200 {

enum BiasAttnVMode { BA_V_PLAIN = 0, BA_V_FIRST = 1, BA_V_BLEND = 2 };

struct BiasAttnPrepParams {
    const float* q; const float* k; const float* v; int ld;      // projection rows: q [H * dk], k [G * dk], v [G * dv]
    float* qo; int ldq;                           // [T, H * dk]
    float* cache;                                 // [pages][page][G * dk + G * dv]
    const int* table; int stride; int page;
    float* vfirst; int ldv;                       // [T, G * dv] values of the first blending layer (this step's tokens)
    int vmode; float lam;
    int H, G, dk, dv;
    float scale, eps;
    MetaView meta; SeqMeta sm;
};

__global__ void __launch_bounds__(128) bias_attn_prep_kernel(const BiasAttnPrepParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int slot = p.meta.tok_slot()[t], ipos = p.sm.tok_pos()[t];
    const int D = p.G * (p.dk + p.dv);
    float* row = p.cache + ((size_t)p.table[(size_t)slot * p.stride + ipos / p.page] * p.page + ipos % p.page) * D;
    for (int hh = warp; hh < p.H + p.G; hh += nw) {
        const bool isq = hh < p.H;
        const int h = isq ? hh : hh - p.H;
        const float* src = (isq ? p.q : p.k) + (size_t)t * p.ld + (size_t)h * p.dk;
        float* dst = isq ? p.qo + (size_t)t * p.ldq + (size_t)h * p.dk : row + (size_t)h * p.dk;
        float ss = 0.f;
        for (int i = lane; i < p.dk; i += 32) ss = fmaf(src[i], src[i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = (isq ? p.scale : 1.f) / sqrtf(ss / (float)p.dk + p.eps);
        for (int i = lane; i < p.dk; i += 32) dst[i] = src[i] * r;
    }
    float* vdst = row + (size_t)p.G * p.dk;
    const float* vsrc = p.v + (size_t)t * p.ld;
    float* vf = p.vfirst + (size_t)t * p.ldv;
    for (int i = threadIdx.x; i < p.G * p.dv; i += blockDim.x) {
        float val = vsrc[i];
        if (p.vmode == BA_V_FIRST) vf[i] = val;
        else if (p.vmode == BA_V_BLEND) val = (1.f - p.lam) * val + p.lam * vf[i];
        vdst[i] = val;
    }
}

struct BiasAttnParams {
    const float* q; int ldq;                      // [T, H * dk] prepared queries
    const float* cache;
    const int* table; int stride; int page;
    float* out; int ldo;                          // [T, H * dv]
    const float* bias; int nb;                    // [nb + 1][H]
    int H, G, dk, dv;
    int qb;                                       // tokens per chunk the shared memory was sized for
    int gt;                                       // key / value heads per tile load
    int cl;                                       // CTAs per chunk (cluster size)
    int ks;                                       // register form: warps of a CTA that share one item's key tiles
    MetaView meta; SeqMeta sm;
};

constexpr int BA_KT = 32;                          // keys per tile (one per lane in the score phase)
constexpr int BA_THREADS = 512;                    // most threads per CTA; the host launches 256 where fewer warps find work
constexpr int BA_RB = 4;                           // most rows of one key / value head a warp works on together (kernel template: 1, 2, 4)

__host__ __device__ inline size_t bias_attn_smem(int qb, int H, int dk, int dv, int gt) {
    const size_t R = (size_t)qb * H;
    return (R * dk + R * dv + R * BA_KT + 2 * (size_t)gt * BA_KT * (dk + 4 + dv + 4) + 3 * R + 8) * sizeof(float);      // two tile buffers
}

// `nk` cache rows from position j0 on: `wk` floats at offset `offk` and `wv` floats at offset `offv` of each of `gn` consecutive
// heads -> tk[head][key][tsk], tv[head][key][tsv]; value rows past nk are zero (their weights are zero too, and 0 * junk must
// stay 0).  vec: 16-byte cp.async copies, a warp per cache row, all copies of the tile in flight together.  Ends with a commit
// of the copies it issued (an empty group on the scalar path); the caller waits.
__device__ __forceinline__ void ba_load_tiles(const float* cache, const int* tbl, int page, int D, size_t offk, int wk, size_t offv, int wv,
                                              float* tk, int tsk, float* tv, int tsv, int gn, int nk, int j0, bool vec) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (int)(blockDim.x >> 5);
    for (int kt = warp; kt < BA_KT; kt += nw) {
        if (kt >= nk) {
            for (int c = 0; c < gn; ++c)
                for (int i = lane; i < wv; i += 32) tv[((size_t)c * BA_KT + kt) * tsv + i] = 0.f;
            continue;
        }
        const int j = j0 + kt, pg = j / page;
        const float* src = cache + ((size_t)tbl[pg] * page + (j - pg * page)) * D;
        if (vec) {
            for (int c = 0; c < gn; ++c) {
                for (int v4 = lane; v4 < (wk >> 2); v4 += 32) cp_async16(tk + ((size_t)c * BA_KT + kt) * tsk + v4 * 4, src + offk + (size_t)c * wk + v4 * 4);
                for (int v4 = lane; v4 < (wv >> 2); v4 += 32) cp_async16(tv + ((size_t)c * BA_KT + kt) * tsv + v4 * 4, src + offv + (size_t)c * wv + v4 * 4);
            }
        } else {
            for (int c = 0; c < gn; ++c) {
                for (int i = lane; i < wk; i += 32) tk[((size_t)c * BA_KT + kt) * tsk + i] = src[offk + (size_t)c * wk + i];
                for (int i = lane; i < wv; i += 32) tv[((size_t)c * BA_KT + kt) * tsv + i] = src[offv + (size_t)c * wv + i];
            }
        }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

template <int RBT>
__global__ void __launch_bounds__(BA_THREADS) bias_attn_kernel(const BiasAttnParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = p.cl, rank = blockIdx.x % CL, ch = blockIdx.x / CL;
    if (ch >= p.sm.n_chunks()) return;             // the same for every CTA of a cluster
    const int t0 = p.sm.chunk_start()[ch], nq = p.sm.chunk_count()[ch];
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, G = p.G, dk = p.dk, dv = p.dv, rep = H / G, R = nq * H;
    // head sizes that are multiples of four: tile rows start on 16 bytes (stride d + 4: a quarter warp's 16-byte reads of eight
    // different rows fall into different banks) and arrive by cp.async; otherwise stride d + 1 and scalar loads
    const bool vec = (dk % 4 == 0) && (dv % 4 == 0);
    const int tsk = dk + (vec ? 4 : 1), tsv = dv + (vec ? 4 : 1), D = G * (dk + dv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    extern __shared__ __align__(16) float ba_smem[];
    const int Rcap = p.qb * H;
    float* sP = ba_smem;                           // [R][KT] weights of the tile (rows start on 16 bytes for any head size)
    float* sK = sP + (size_t)Rcap * BA_KT;         // [2][gt][KT][tsk]
    float* sV = sK + 2 * (size_t)p.gt * BA_KT * (dk + 4);   // [gt][KT][tsv], two buffers each: a stage's tiles arrive while the
    float* sQ = sV + 2 * (size_t)p.gt * BA_KT * (dv + 4);   // [R][dk]                 previous stage is multiplied
    float* sO = sQ + (size_t)Rcap * dk;            // [R][dv] un-normalised outputs
    float* sMax = sO + (size_t)Rcap * dv;          // [R] running maximum / sum / last rescale of this CTA
    float* sSum = sMax + Rcap;
    float* sScl = sSum + Rcap;
    for (int e = threadIdx.x; e < R * dk; e += (int)blockDim.x) {
        const int r = e / dk, i = e % dk;
        sQ[e] = p.q[(size_t)(t0 + r / H) * p.ldq + (size_t)(r % H) * dk + i];
    }
    for (int e = threadIdx.x; e < R * dv; e += (int)blockDim.x) sO[e] = 0.f;
    for (int e = threadIdx.x; e < R; e += (int)blockDim.x) { sMax[e] = -CUDART_INF_F; sSum[e] = 0.f; sScl[e] = 1.f; }
    const int ntiles = (pos1 + BA_KT) / BA_KT;     // keys 0 .. pos1
    const int* tbl = p.table + (size_t)slot * p.stride;
    const int nrg = nq * rep;                      // rows of one key / value head
    constexpr int RB = RBT;                        // rows of one key / value head a warp takes together
    const int nblk = (nrg + RB - 1) / RB;          // row blocks of one head
    // a stage = one tile of keys x one group of `gt` heads; this CTA's stages in order, the next one's loads always in flight
    const int ngrp = (G + p.gt - 1) / p.gt;
    const int nstage = rank < ntiles ? ((ntiles - rank + CL - 1) / CL) * ngrp : 0;
    const size_t bufK = (size_t)p.gt * BA_KT * (dk + 4), bufV = (size_t)p.gt * BA_KT * (dv + 4);
    auto load_stage = [&](int rd) {
        const int ti = rank + (rd / ngrp) * CL, c0 = (rd % ngrp) * p.gt;
        const int j0 = ti * BA_KT;
        ba_load_tiles(p.cache, tbl, p.page, D, (size_t)c0 * dk, dk, (size_t)G * dk + (size_t)c0 * dv, dv, sK + (rd & 1) * bufK, tsk,
                      sV + (rd & 1) * bufV, tsv, min(p.gt, G - c0), min(BA_KT, pos1 + 1 - j0), j0, vec);
    };
    if (nstage > 0) load_stage(0);
    for (int rd = 0; rd < nstage; ++rd) {
        if (rd + 1 < nstage) {
            load_stage(rd + 1);                    // into the buffer that stage rd - 1 used: everyone left it at the barrier below
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();                           // stage rd's tiles are visible (and, the first time, the rows are initialised)
        {
            const int ti = rank + (rd / ngrp) * CL, c0 = (rd % ngrp) * p.gt;
            const int j0 = ti * BA_KT, nk = min(BA_KT, pos1 + 1 - j0), jl = j0 + lane;
            const int gn = min(p.gt, G - c0);
            const float* cK = sK + (rd & 1) * bufK;
            const float* cV = sV + (rd & 1) * bufV;
            for (int it = warp; it < gn * nblk; it += nw) {
                const int cl_ = it / nblk, c = c0 + cl_, rr0 = (it % nblk) * RB, nr = min(RB, nrg - rr0);
                int rows[RBT];
                const float* qv[RBT];
#pragma unroll
                for (int b = 0; b < RBT; ++b) {
                    const int rr = rr0 + min(b, nr - 1);
                    rows[b] = (rr / rep) * H + c * rep + rr % rep;
                    qv[b] = sQ + (size_t)rows[b] * dk;
                }
                // ---- scores of the warp's rows against key `lane` ----
                float sc[RBT];
#pragma unroll
                for (int b = 0; b < RBT; ++b) sc[b] = 0.f;
                if (lane < nk) {
                    const float* kv = cK + ((size_t)cl_ * BA_KT + lane) * tsk;
                    if (vec) {
                        const float4* k4 = reinterpret_cast<const float4*>(kv);
#pragma unroll 4
                        for (int i = 0; i < dk / 4; ++i) {
                            const float4 kx = k4[i];
#pragma unroll
                            for (int b = 0; b < RBT; ++b) {
                                const float4 qx = reinterpret_cast<const float4*>(qv[b])[i];
                                sc[b] = fmaf(qx.x, kx.x, sc[b]); sc[b] = fmaf(qx.y, kx.y, sc[b]);
                                sc[b] = fmaf(qx.z, kx.z, sc[b]); sc[b] = fmaf(qx.w, kx.w, sc[b]);
                            }
                        }
                    } else {
#pragma unroll 4
                        for (int i = 0; i < dk; ++i) {
                            const float kx = kv[i];
#pragma unroll
                            for (int b = 0; b < RBT; ++b) sc[b] = fmaf(qv[b][i], kx, sc[b]);
                        }
                    }
                }
                // ---- running maximum / sum of every row, the tile's weights ----
#pragma unroll
                for (int b = 0; b < RBT; ++b) {
                    if (b >= nr) break;
                    const int r = rows[b], pq = pos0 + r / H, h = r % H;
                    const bool vis = lane < nk && jl <= pq;
                    const float s = vis ? sc[b] + p.bias[(size_t)min(pq - jl, p.nb) * H + h] : -CUDART_INF_F;
                    float mx = s;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    const float mo = sMax[r], mn = fmaxf(mo, mx);
                    float e = vis ? expf(s - mn) : 0.f;        // mn is finite wherever a key is visible
                    sP[r * BA_KT + lane] = e;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
                    __syncwarp();                              // everyone has read the old maximum
                    if (lane == 0) {
                        const float scl = mo > -CUDART_INF_F ? expf(mo - mn) : 0.f;
                        sScl[r] = scl;
                        sSum[r] = sSum[r] * scl + e;
                        sMax[r] = mn;
                    }
                }
                __syncwarp();
                // ---- weights x values ----
                const float* vt = cV + (size_t)cl_ * BA_KT * tsv;
                for (int d = lane; d < dv; d += 32) {
                    float acc[RBT];
#pragma unroll
                    for (int b = 0; b < RBT; ++b) acc[b] = sO[(size_t)rows[b] * dv + d] * sScl[rows[b]];
#pragma unroll 2
                    for (int kt = 0; kt < BA_KT; kt += 4) {
                        const float v0 = vt[(kt + 0) * tsv + d], v1 = vt[(kt + 1) * tsv + d], v2 = vt[(kt + 2) * tsv + d], v3 = vt[(kt + 3) * tsv + d];
#pragma unroll
                        for (int b = 0; b < RBT; ++b) {
                            const float4 w4 = *reinterpret_cast<const float4*>(sP + rows[b] * BA_KT + kt);
                            acc[b] = fmaf(w4.x, v0, acc[b]); acc[b] = fmaf(w4.y, v1, acc[b]);
                            acc[b] = fmaf(w4.z, v2, acc[b]); acc[b] = fmaf(w4.w, v3, acc[b]);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < RBT; ++b)
                        if (b < nr) sO[(size_t)rows[b] * dv + d] = acc[b];
                }
                __syncwarp();
            }
        }
        __syncthreads();                           // everyone is done with stage rd's buffers
    }
    // the CTAs' partial results merged in rank order; every CTA finishes its share of the outputs
    cluster.sync();
    for (int e = rank * (int)blockDim.x + threadIdx.x; e < R * dv; e += CL * (int)blockDim.x) {
        const int r = e / dv, d = e % dv;
        float m = -CUDART_INF_F;
        for (int rk = 0; rk < CL; ++rk) m = fmaxf(m, cluster.map_shared_rank(sMax, rk)[r]);
        float num = 0.f, den = 0.f;
        for (int rk = 0; rk < CL; ++rk) {
            const float mr = cluster.map_shared_rank(sMax, rk)[r];
            if (mr > -CUDART_INF_F) {
                const float f = expf(mr - m);
                num = fmaf(cluster.map_shared_rank(sO, rk)[e], f, num);
                den = fmaf(cluster.map_shared_rank(sSum, rk)[r], f, den);
            }
        }
        p.out[(size_t)(t0 + r / H) * p.ldo + (size_t)(r % H) * dv + d] = num / den;
    }
    cluster.sync();                                // nobody leaves while its shared memory is still being read
}

// ------------------------------------------------------------------------------------------------------------------
// register form (head sizes that are multiples of four, at most 128): no tile passes through shared memory
// ------------------------------------------------------------------------------------------------------------------
// A warp owns RB rows of one key / value head and a share of the chunk's key tiles, and keeps everything it accumulates in
// registers: lane l holds entries 4l .. 4l + 3 of the RB query rows and of the RB un-normalised output rows, plus the rows'
// running maxima and sums.  Per tile of 32 keys:
//   scores   eight keys at a time: every lane loads its 16 bytes of each key row straight from the cache (a whole row per warp
//            load), multiplies them with its query entries, and a butterfly over the lanes (keep half of the keys, send the other
//            half: 4 + 2 + 1 exchanges, then two plain ones) leaves the finished score of key (l >> 2) of the batch in lane l;
//   softmax  bias, causal mask, running maximum / sum with three exchanges per row;
//   values   the weight of each key is broadcast from its lane, every lane loads its 16 bytes of the value row.
// With few (head, row block) items per chunk the key tiles are split over KS warps per item as well as over the cluster's
// CTAs; the partial (maximum, sum, output) triples meet in shared memory (within a CTA) and then through distributed shared
// memory (across the cluster), always in a fixed order.
constexpr int BAR_THREADS = 256;                   // 8 warps, two CTAs per SM (128 registers per thread)

__host__ __device__ inline size_t bias_attn_reg_smem(int qb, int H, int G, int dv, int rb, int ks) {
    const size_t nblk = ((size_t)qb * (H / G) + rb - 1) / rb, slots = (size_t)G * nblk * ks;
    return (slots * rb * (dv + 2) + 2 * (size_t)G * nblk * rb + 8) * sizeof(float);
}

template <int RB>
__global__ void __launch_bounds__(BAR_THREADS, 2) bias_attn_reg_kernel(const BiasAttnParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = p.cl, rank = blockIdx.x % CL, ch = blockIdx.x / CL;
    if (ch >= p.sm.n_chunks()) return;             // the same for every CTA of a cluster
    const int t0 = p.sm.chunk_start()[ch], nq = p.sm.chunk_count()[ch];
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, G = p.G, dk = p.dk, dv = p.dv, rep = H / G, R = nq * H, KS = p.ks;
    const int D = G * (dk + dv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, NW = blockDim.x >> 5;
    const int nblk_cap = (p.qb * rep + RB - 1) / RB;          // row blocks of one head the shared memory was sized for
    const int nrg = nq * rep, nblk = (nrg + RB - 1) / RB;     // rows / row blocks of one head in this chunk
    extern __shared__ __align__(16) float bar_smem[];
    float* sO = bar_smem;                                      // [G * nblk_cap][KS][RB][dv] partial outputs (slot 0 of an item: merged)
    float* sM = sO + (size_t)G * nblk_cap * KS * RB * dv;      // [G * nblk_cap][KS][RB]
    float* sL = sM + (size_t)G * nblk_cap * KS * RB;
    float* sM2 = sL + (size_t)G * nblk_cap * KS * RB;          // [G * nblk_cap][RB] merged over the CTA's key splits
    float* sL2 = sM2 + (size_t)G * nblk_cap * RB;
    const int* tbl = p.table + (size_t)slot * p.stride;
    const int ntiles = (pos1 + BA_KT) / BA_KT;                 // keys 0 .. pos1
    const int l4 = lane * 4, kq = lane >> 2;
    const bool kact = l4 < dk, vact = l4 < dv;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int it = warp; it < G * nblk * KS; it += NW) {
        const int item = it / KS, ks = it % KS;
        const int c = item / nblk, rr0 = (item % nblk) * RB, nr = min(RB, nrg - rr0);
        int qi[RB], hh[RB];
        float4 q[RB], acc[RB];
        float m[RB], l[RB];
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            const int rr = rr0 + min(b, nr - 1);
            qi[b] = rr / rep; hh[b] = c * rep + rr % rep;
            q[b] = kact ? *reinterpret_cast<const float4*>(p.q + (size_t)(t0 + qi[b]) * p.ldq + (size_t)hh[b] * dk + l4) : zero4;
            acc[b] = zero4; m[b] = -CUDART_INF_F; l[b] = 0.f;
        }
        const float* kbase = p.cache + (size_t)c * dk + l4;
        const float* vbase = p.cache + (size_t)G * dk + (size_t)c * dv + l4;
        for (int ti = rank * KS + ks; ti < ntiles; ti += CL * KS) {
            const int j0 = ti * BA_KT, nk = min(BA_KT, pos1 + 1 - j0);
            unsigned long long myoff = 0ull;                   // cache offset of key j0 + lane
            if (lane < nk) {
                const int j = j0 + lane, pg = j / p.page;
                myoff = ((unsigned long long)tbl[pg] * p.page + (unsigned)(j - pg * p.page)) * (unsigned)D;
            }
            float s[4][RB];
            // ---- scores: four batches of eight keys ----
#pragma unroll
            for (int bt = 0; bt < 4; ++bt) {
                float4 kx[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const unsigned long long off = __shfl_sync(0xffffffffu, myoff, bt * 8 + u);
                    kx[u] = (kact && bt * 8 + u < nk) ? __ldg(reinterpret_cast<const float4*>(kbase + off)) : zero4;
                }
#pragma unroll
                for (int b = 0; b < RB; ++b) {
                    float pt[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        pt[u] = fmaf(q[b].x, kx[u].x, fmaf(q[b].y, kx[u].y, fmaf(q[b].z, kx[u].z, q[b].w * kx[u].w)));
                    // butterfly: lanes with bit 4 set keep keys 4..7 and send 0..3, and so on; lane l ends with key (l >> 2) & 7
                    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
                    float a4[4], a2[2], a1;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float send = h16 ? pt[i] : pt[i + 4], keep = h16 ? pt[i + 4] : pt[i];
                        a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float send = h8 ? a4[i] : a4[i + 2], keep = h8 ? a4[i + 2] : a4[i];
                        a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                    {
                        const float send = h4 ? a2[0] : a2[1], keep = h4 ? a2[1] : a2[0];
                        a1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
                    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
                    s[bt][b] = a1;
                }
            }
            // ---- bias, causal mask, running maximum and sum of every row; s becomes the tile's weights ----
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                const int pq = pos0 + qi[b];
                float tmax = -CUDART_INF_F;
#pragma unroll
                for (int bt = 0; bt < 4; ++bt) {
                    const int kk = bt * 8 + kq, j = j0 + kk;
                    const bool vis = kk < nk && j <= pq;
                    s[bt][b] = vis ? s[bt][b] + p.bias[(size_t)min(pq - j, p.nb) * H + hh[b]] : -CUDART_INF_F;
                    tmax = fmaxf(tmax, s[bt][b]);
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
                const float mn = fmaxf(m[b], tmax);            // the same in every lane
                const bool any = mn > -CUDART_INF_F;
                const float scl = (any && m[b] > -CUDART_INF_F) ? expf(m[b] - mn) : 0.f;
                float tsum = 0.f;
#pragma unroll
                for (int bt = 0; bt < 4; ++bt) {
                    const float w = (any && s[bt][b] > -CUDART_INF_F) ? expf(s[bt][b] - mn) : 0.f;
                    s[bt][b] = w;
                    tsum += w;
                }
                tsum += __shfl_xor_sync(0xffffffffu, tsum, 16);
                tsum += __shfl_xor_sync(0xffffffffu, tsum, 8);
                tsum += __shfl_xor_sync(0xffffffffu, tsum, 4);   // lanes that differ in bits 0..1 hold the same keys
                l[b] = l[b] * scl + tsum;
                m[b] = mn;
                acc[b].x *= scl; acc[b].y *= scl; acc[b].z *= scl; acc[b].w *= scl;
            }
            // ---- weights x values ----
#pragma unroll
            for (int bt = 0; bt < 4; ++bt) {
                if (bt * 8 >= nk) break;                       // warp-uniform
                float4 vx[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const unsigned long long off = __shfl_sync(0xffffffffu, myoff, bt * 8 + u);
                    vx[u] = (vact && bt * 8 + u < nk) ? __ldg(reinterpret_cast<const float4*>(vbase + off)) : zero4;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int b = 0; b < RB; ++b) {
                        const float w = __shfl_sync(0xffffffffu, s[bt][b], u << 2);
                        acc[b].x = fmaf(w, vx[u].x, acc[b].x); acc[b].y = fmaf(w, vx[u].y, acc[b].y);
                        acc[b].z = fmaf(w, vx[u].z, acc[b].z); acc[b].w = fmaf(w, vx[u].w, acc[b].w);
                    }
            }
        }
        const size_t sl = (size_t)(c * nblk_cap + item % nblk) * KS + ks;
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            if (b >= nr) break;
            if (vact) *reinterpret_cast<float4*>(sO + (sl * RB + b) * dv + l4) = acc[b];
            if (lane == 0) { sM[sl * RB + b] = m[b]; sL[sl * RB + b] = l[b]; }
        }
    }
    __syncthreads();
    // the CTA's key splits of every row merged in split order (into split 0's place)
    for (int e = threadIdx.x; e < R * dv; e += (int)blockDim.x) {
        const int r = e / dv, d = e % dv, qi_ = r / H, h = r % H, c = h / rep, rr = qi_ * rep + h % rep;
        const size_t it0 = (size_t)(c * nblk_cap + rr / RB) * KS;
        const int b = rr % RB;
        float mx = -CUDART_INF_F;
        for (int k = 0; k < KS; ++k) mx = fmaxf(mx, sM[(it0 + k) * RB + b]);
        float num = 0.f, den = 0.f;
        for (int k = 0; k < KS; ++k) {
            const float mr = sM[(it0 + k) * RB + b];
            if (mr > -CUDART_INF_F) {
                const float f = expf(mr - mx);
                num = fmaf(sO[((it0 + k) * RB + b) * dv + d], f, num);
                den = fmaf(sL[(it0 + k) * RB + b], f, den);
            }
        }
        sO[(it0 * RB + b) * dv + d] = num;                     // only this thread touches column d of the row
        if (d == 0) { sM2[(it0 / KS) * RB + b] = mx; sL2[(it0 / KS) * RB + b] = den; }
    }
    // the CTAs' partial results merged in rank order; every CTA finishes its share of the outputs
    cluster.sync();
    for (int e = rank * (int)blockDim.x + threadIdx.x; e < R * dv; e += CL * (int)blockDim.x) {
        const int r = e / dv, d = e % dv, qi_ = r / H, h = r % H, c = h / rep, rr = qi_ * rep + h % rep;
        const size_t ib = (size_t)(c * nblk_cap + rr / RB);
        const int b = rr % RB;
        // all remote reads first (a cluster has at most 8 CTAs), then the arithmetic: the reads overlap instead of queueing up
        float mr[8], orr[8], lr[8];
#pragma unroll
        for (int rk = 0; rk < 8; ++rk) {
            mr[rk] = -CUDART_INF_F; orr[rk] = 0.f; lr[rk] = 0.f;
            if (rk < CL) {
                mr[rk] = cluster.map_shared_rank(sM2, rk)[ib * RB + b];
                orr[rk] = cluster.map_shared_rank(sO, rk)[(ib * KS * RB + b) * dv + d];
                lr[rk] = cluster.map_shared_rank(sL2, rk)[ib * RB + b];
            }
        }
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int rk = 0; rk < 8; ++rk) mx = fmaxf(mx, mr[rk]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int rk = 0; rk < 8; ++rk)
            if (mr[rk] > -CUDART_INF_F) {
                const float f = expf(mr[rk] - mx);
                num = fmaf(orr[rk], f, num);
                den = fmaf(lr[rk], f, den);
            }
        p.out[(size_t)(t0 + qi_) * p.ldo + (size_t)h * dv + d] = num / den;
    }
    cluster.sync();                                // nobody leaves while its shared memory is still being read
}

}  // namespace b200
