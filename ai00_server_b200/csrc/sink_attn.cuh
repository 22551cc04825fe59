// Softmax attention over a paged cache with a sliding window, a learned "sink" term per head in the softmax denominator, and
// (optionally) block means of the keys / values that have left the window.  No positions enter the scores here: a layer that
// rotates its queries and keys does so before it calls this.
//
// H query heads, G key / value heads (query head h reads head h / (H / G)).  A cache row of D floats holds, for every key /
// value head c, a key of dk floats at `koff + c dk` and a value of dv floats at `voff + c dv` (the two may be the same floats:
// a latent row that is scored against and summed, G = 1).  For query position i:
//     tokens   j with  i - win < j <= i
//     blocks   b with  (b + 1) pool <= i - win + 1      (pool > 0): the mean of the cache rows b pool .. b pool + pool - 1,
//              kept in a second pool of rows with the same layout (pool_write_kernel) so that a block costs one row to read
//     s_h(i, u) = (q_h(i) . k(u)) * scale           over the visible tokens and blocks u together
//     o_h(i) = sum_u exp(s_h(i, u)) v(u) / (exp(sink_h) + sum_u exp(s_h(i, u)))        * sigmoid(gate_h(i))  (gate optional)
//
//   pool_write_kernel     every token of the step that closes a block writes the block's mean row (sums in position order, f32)
//   pool_rebuild_kernel   the same for all closed blocks of one sequence (after a state import)
//   sink_attn_kernel      a cluster of 1..8 CTAs per (chunk of consecutive tokens of one sequence, group of HB query heads);
//                         the visible block rows and then the window's token rows form 32-key tiles that are dealt out among
//                         the cluster's CTAs; every CTA walks its tiles once with a running maximum / sum per (token, head) row
//                         and the partial results are merged through distributed shared memory in rank order, where the sink
//                         and the gate come in.  A warp owns 1, 2 or 4 rows of one key / value head (template).  Tiles arrive
//                         by cp.async into one or two buffers.  Scores, weights and sums in f32.  Any head size.
//   sink_attn_reg_kernel  the same result for key / value sizes that are multiples of four up to 128 NC (template), with nothing
//                         staged in shared memory: see the comment above it.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"
#include "latent_attn.cuh"
#include "linear.cuh"

namespace b200 {

// row of pooled block b of a sequence: the block lives in the page of its first position
__device__ __forceinline__ size_t sa_pool_row(const int* tbl, int page, int pool, int prow, int b) {
    const int p0 = b * pool, pg = p0 / page;
    return (size_t)tbl[pg] * prow + (size_t)((p0 - pg * page) / pool);
}
__device__ __forceinline__ size_t sa_token_row(const int* tbl, int page, int j) {
    const int pg = j / page;
    return (size_t)tbl[pg] * page + (size_t)(j - pg * page);
}

struct PoolWriteParams {
    const float* cache; float* pcache;             // [pages][page][D], [pages][prow][D]
    const int* table; int stride, page;
    int D, pool, prow;
    int slot, nblocks;                             // pool_rebuild_kernel: the sequence and its closed blocks
    MetaView meta; SeqMeta sm;
};

__device__ __forceinline__ void sa_pool_block(const PoolWriteParams& p, const int* tbl, int b) {
    float* dst = p.pcache + sa_pool_row(tbl, p.page, p.pool, p.prow, b) * p.D;
    const float inv = 1.f / (float)p.pool;
    for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < p.D; d += gridDim.y * blockDim.x) {
        float s = 0.f;
#pragma unroll 4
        for (int u = 0; u < p.pool; ++u) s += p.cache[sa_token_row(tbl, p.page, b * p.pool + u) * p.D + d];
        dst[d] = s * inv;
    }
}

__global__ void __launch_bounds__(128) pool_write_kernel(const PoolWriteParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int ipos = p.sm.tok_pos()[t];
    if ((ipos + 1) % p.pool != 0) return;
    sa_pool_block(p, p.table + (size_t)p.meta.tok_slot()[t] * p.stride, ipos / p.pool);
}

__global__ void __launch_bounds__(128) pool_rebuild_kernel(const PoolWriteParams p) {
    if ((int)blockIdx.x < p.nblocks) sa_pool_block(p, p.table + (size_t)p.slot * p.stride, blockIdx.x);
}

struct SinkAttnParams {
    const float* q; int ldq;                       // query of (t, h): q + t ldq + h dk
    const float* cache; const float* pcache;       // token rows; block-mean rows (nullptr / pool = 0: none)
    const int* table; int stride, page;
    int D, koff, voff;
    float* out; int ldo;                           // [T, H dv]
    const float* gate; int ldg;                    // out *= sigmoid(gate[t ldg + h dv + d])   (nullptr: no gate)
    const float* sink;                             // [H] (nullptr: no sink term)
    float scale;
    int H, G, dk, dv, HB;                          // HB query heads per CTA: a multiple of H / G, or a divisor of it
    int win, pool, prow;
    int qb;                                        // tokens per chunk the shared memory was sized for
    int gt;                                        // key / value heads per tile load
    int cl;                                        // CTAs per chunk (cluster size)
    int nbuf;                                      // tile buffers (2: the next tile loads while this one is multiplied)
    int valias;                                    // the value is the first dv floats of the key (one tile serves both)
    int nsub;                                      // the step's chunks hold nsub * qb tokens: a CTA group takes one part of a chunk
    int ks;                                        // register form: warps of a CTA that share one item's key tiles
    MetaView meta; SeqMeta sm;
};

// which part of which chunk this CTA group works on; false: nothing (the same answer in every CTA of a cluster)
__device__ __forceinline__ bool sa_chunk(const SinkAttnParams& p, int grp, int& t0, int& nq) {
    const int ch = grp / p.nsub, sb = grp % p.nsub;
    if (ch >= p.sm.n_chunks()) return false;
    nq = min(p.qb, p.sm.chunk_count()[ch] - sb * p.qb);
    t0 = p.sm.chunk_start()[ch] + sb * p.qb;
    return nq > 0;
}

constexpr int SA_KT = 32;                          // keys per tile (one per lane in the score phase)
constexpr int SA_THREADS = 512;                    // most threads per CTA; the host launches 256 where fewer warps find work
constexpr int SA_RB = 4;                           // most rows of one key / value head a warp works on together

__host__ __device__ inline size_t sink_attn_smem(int qb, int HB, int dk, int dv, int gt, int nbuf, bool valias) {
    const size_t R = (size_t)qb * HB;
    return (R * dk + R * dv + R * SA_KT + (size_t)nbuf * gt * SA_KT * ((dk + 4) + (valias ? 0 : dv + 4)) + 3 * R + 8) * sizeof(float);
}

template <int RBT>
__global__ void __launch_bounds__(SA_THREADS) sink_attn_kernel(const SinkAttnParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = p.cl, rank = blockIdx.x % CL;
    int t0, nq;
    if (!sa_chunk(p, blockIdx.x / CL, t0, nq)) return;
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, dk = p.dk, dv = p.dv, rep = H / p.G;
    const int h0 = blockIdx.y * p.HB, nh = min(p.HB, H - h0);       // query heads of this CTA
    const int c_first = h0 / rep, nhc = min(rep, nh), ncv = nh / nhc;   // first key head, query heads per key head, key heads
    const int R = nq * nh, D = p.D;
    const bool valias = p.valias != 0;
    // sizes that are multiples of four: tile rows start on 16 bytes (stride d + 4: a quarter warp's 16-byte reads of eight
    // different rows fall into different banks) and arrive by cp.async; otherwise stride d + 1 and scalar loads
    const bool vec = (dk % 4 == 0) && (dv % 4 == 0) && (D % 4 == 0) && (p.koff % 4 == 0) && (p.voff % 4 == 0);
    const int tsk = dk + (vec ? 4 : 1), tsv = valias ? tsk : dv + (vec ? 4 : 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    extern __shared__ __align__(16) float sa_smem[];
    const int Rcap = p.qb * p.HB;
    const size_t bufK = (size_t)p.gt * SA_KT * (dk + 4), bufV = valias ? 0 : (size_t)p.gt * SA_KT * (dv + 4);
    float* sP = sa_smem;                           // [R][KT] weights of the tile
    float* sK = sP + (size_t)Rcap * SA_KT;         // [nbuf][gt][KT][tsk]
    float* sV = sK + (size_t)p.nbuf * bufK;        // [nbuf][gt][KT][tsv]
    float* sQ = sV + (size_t)p.nbuf * bufV;        // [R][dk]
    float* sO = sQ + (size_t)Rcap * dk;            // [R][dv] un-normalised outputs
    float* sMax = sO + (size_t)Rcap * dv;          // [R] running maximum / sum / last rescale of this CTA
    float* sSum = sMax + Rcap;
    float* sScl = sSum + Rcap;
    for (int e = threadIdx.x; e < R * dk; e += (int)blockDim.x) {
        const int r = e / dk, i = e % dk;
        sQ[e] = p.q[(size_t)(t0 + r / nh) * p.ldq + (size_t)(h0 + r % nh) * dk + i];
    }
    for (int e = threadIdx.x; e < R * dv; e += (int)blockDim.x) sO[e] = 0.f;
    for (int e = threadIdx.x; e < R; e += (int)blockDim.x) { sMax[e] = -CUDART_INF_F; sSum[e] = 0.f; sScl[e] = 1.f; }
    // what the chunk can see: the blocks its last token sees, then the tokens from the first token's window edge on
    const int npb = p.pool > 0 ? max(0, pos1 - p.win + 1) / p.pool : 0;
    const int jlo = max(0, pos0 - p.win + 1), ntk = pos1 - jlo + 1;
    const int npt = (npb + SA_KT - 1) / SA_KT, ntiles = npt + (ntk + SA_KT - 1) / SA_KT;
    const int* tbl = p.table + (size_t)slot * p.stride;
    const int nrg = nq * nhc;                      // rows of one key / value head
    constexpr int RB = RBT;
    const int nblk = (nrg + RB - 1) / RB;          // row blocks of one head
    // a stage = one tile of keys x one group of `gt` heads; this CTA's stages in order
    const int ngrp = (ncv + p.gt - 1) / p.gt;
    const int nstage = rank < ntiles ? ((ntiles - rank + CL - 1) / CL) * ngrp : 0;
    auto load_stage = [&](int rd) {
        const int ti = rank + (rd / ngrp) * CL, g0 = (rd % ngrp) * p.gt, gn = min(p.gt, ncv - g0);
        const bool pooled = ti < npt;
        const int i0 = pooled ? ti * SA_KT : jlo + (ti - npt) * SA_KT;          // first block / position of the tile
        const int nk = pooled ? min(SA_KT, npb - i0) : min(SA_KT, pos1 + 1 - i0);
        float* tk = sK + (size_t)(rd % p.nbuf) * bufK;
        float* tv = sV + (size_t)(rd % p.nbuf) * bufV;
        const size_t offk = (size_t)p.koff + (size_t)(c_first + g0) * dk, offv = (size_t)p.voff + (size_t)(c_first + g0) * dv;
        for (int kt = warp; kt < SA_KT; kt += nw) {
            if (kt >= nk) {                        // rows past the tile's keys: their weights are zero and 0 * junk must stay 0
                for (int c = 0; c < gn; ++c) {
                    if (valias) for (int i = lane; i < dv; i += 32) tk[((size_t)c * SA_KT + kt) * tsk + i] = 0.f;
                    else for (int i = lane; i < dv; i += 32) tv[((size_t)c * SA_KT + kt) * tsv + i] = 0.f;
                }
                continue;
            }
            const float* src = pooled ? p.pcache + sa_pool_row(tbl, p.page, p.pool, p.prow, i0 + kt) * D
                                      : p.cache + sa_token_row(tbl, p.page, i0 + kt) * D;
            for (int c = 0; c < gn; ++c) {
                float* dk_ = tk + ((size_t)c * SA_KT + kt) * tsk;
                float* dv_ = tv + ((size_t)c * SA_KT + kt) * tsv;
                if (vec) {
                    for (int v4 = lane; v4 < (dk >> 2); v4 += 32) cp_async16(dk_ + v4 * 4, src + offk + (size_t)c * dk + v4 * 4);
                    if (!valias) for (int v4 = lane; v4 < (dv >> 2); v4 += 32) cp_async16(dv_ + v4 * 4, src + offv + (size_t)c * dv + v4 * 4);
                } else {
                    for (int i = lane; i < dk; i += 32) dk_[i] = src[offk + (size_t)c * dk + i];
                    if (!valias) for (int i = lane; i < dv; i += 32) dv_[i] = src[offv + (size_t)c * dv + i];
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    if (nstage > 0 && p.nbuf > 1) load_stage(0);
    for (int rd = 0; rd < nstage; ++rd) {
        if (p.nbuf > 1) {
            if (rd + 1 < nstage) {
                load_stage(rd + 1);                // into the buffer that stage rd - 1 used: everyone left it at the barrier below
                asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            }
        } else {
            load_stage(rd);
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();                           // stage rd's tiles are visible (and, the first time, the rows are initialised)
        {
            const int ti = rank + (rd / ngrp) * CL, g0 = (rd % ngrp) * p.gt, gn = min(p.gt, ncv - g0);
            const bool pooled = ti < npt;
            const int i0 = pooled ? ti * SA_KT : jlo + (ti - npt) * SA_KT;
            const int nk = pooled ? min(SA_KT, npb - i0) : min(SA_KT, pos1 + 1 - i0);
            const int il = i0 + lane;              // this lane's block or position
            const float* cK = sK + (size_t)(rd % p.nbuf) * bufK;
            const float* cV = valias ? cK : sV + (size_t)(rd % p.nbuf) * bufV;
            for (int it = warp; it < gn * nblk; it += nw) {
                const int cl_ = it / nblk, lc = g0 + cl_, rr0 = (it % nblk) * RB, nr = min(RB, nrg - rr0);
                int rows[RBT];
                const float* qv[RBT];
#pragma unroll
                for (int b = 0; b < RBT; ++b) {
                    const int rr = rr0 + min(b, nr - 1);
                    rows[b] = (rr / nhc) * nh + lc * nhc + rr % nhc;
                    qv[b] = sQ + (size_t)rows[b] * dk;
                }
                // ---- scores of the warp's rows against key `lane` ----
                float sc[RBT];
#pragma unroll
                for (int b = 0; b < RBT; ++b) sc[b] = 0.f;
                if (lane < nk) {
                    const float* kv = cK + ((size_t)cl_ * SA_KT + lane) * tsk;
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
                    const int r = rows[b], pq = pos0 + r / nh;
                    const bool vis = lane < nk && (pooled ? il < max(0, pq - p.win + 1) / p.pool : (il <= pq && il > pq - p.win));
                    const float s = vis ? sc[b] * p.scale : -CUDART_INF_F;
                    float mx = s;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    const float mo = sMax[r], mn = fmaxf(mo, mx);
                    float e = vis ? expf(s - mn) : 0.f;        // mn is finite wherever a key is visible
                    sP[r * SA_KT + lane] = e;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
                    __syncwarp();                              // everyone has read the old maximum
                    if (lane == 0) {
                        const float scl = mo > -CUDART_INF_F ? expf(mo - mn) : (mn > -CUDART_INF_F ? 0.f : 1.f);
                        sScl[r] = scl;
                        sSum[r] = sSum[r] * scl + e;
                        sMax[r] = mn;
                    }
                }
                __syncwarp();
                // ---- weights x values ----
                const float* vt = cV + (size_t)cl_ * SA_KT * tsv;
                if (vec) {                         // four neighbouring outputs per lane: a 16-byte value load feeds 4 RB products
                    for (int d = lane * 4; d < dv; d += 128) {
                        float4 acc[RBT];
#pragma unroll
                        for (int b = 0; b < RBT; ++b) {
                            const float f = sScl[rows[b]];
                            acc[b] = *reinterpret_cast<const float4*>(sO + (size_t)rows[b] * dv + d);
                            acc[b].x *= f; acc[b].y *= f; acc[b].z *= f; acc[b].w *= f;
                        }
#pragma unroll 2
                        for (int kt = 0; kt < SA_KT; kt += 4) {
                            const float4 v0 = *reinterpret_cast<const float4*>(vt + (kt + 0) * tsv + d);
                            const float4 v1 = *reinterpret_cast<const float4*>(vt + (kt + 1) * tsv + d);
                            const float4 v2 = *reinterpret_cast<const float4*>(vt + (kt + 2) * tsv + d);
                            const float4 v3 = *reinterpret_cast<const float4*>(vt + (kt + 3) * tsv + d);
#pragma unroll
                            for (int b = 0; b < RBT; ++b) {
                                const float4 w4 = *reinterpret_cast<const float4*>(sP + rows[b] * SA_KT + kt);
                                acc[b].x = fmaf(w4.x, v0.x, acc[b].x); acc[b].y = fmaf(w4.x, v0.y, acc[b].y);
                                acc[b].z = fmaf(w4.x, v0.z, acc[b].z); acc[b].w = fmaf(w4.x, v0.w, acc[b].w);
                                acc[b].x = fmaf(w4.y, v1.x, acc[b].x); acc[b].y = fmaf(w4.y, v1.y, acc[b].y);
                                acc[b].z = fmaf(w4.y, v1.z, acc[b].z); acc[b].w = fmaf(w4.y, v1.w, acc[b].w);
                                acc[b].x = fmaf(w4.z, v2.x, acc[b].x); acc[b].y = fmaf(w4.z, v2.y, acc[b].y);
                                acc[b].z = fmaf(w4.z, v2.z, acc[b].z); acc[b].w = fmaf(w4.z, v2.w, acc[b].w);
                                acc[b].x = fmaf(w4.w, v3.x, acc[b].x); acc[b].y = fmaf(w4.w, v3.y, acc[b].y);
                                acc[b].z = fmaf(w4.w, v3.z, acc[b].z); acc[b].w = fmaf(w4.w, v3.w, acc[b].w);
                            }
                        }
#pragma unroll
                        for (int b = 0; b < RBT; ++b)
                            if (b < nr) *reinterpret_cast<float4*>(sO + (size_t)rows[b] * dv + d) = acc[b];
                    }
                } else
                for (int d = lane; d < dv; d += 32) {
                    float acc[RBT];
#pragma unroll
                    for (int b = 0; b < RBT; ++b) acc[b] = sO[(size_t)rows[b] * dv + d] * sScl[rows[b]];
#pragma unroll 2
                    for (int kt = 0; kt < SA_KT; kt += 4) {
                        const float v0 = vt[(kt + 0) * tsv + d], v1 = vt[(kt + 1) * tsv + d], v2 = vt[(kt + 2) * tsv + d], v3 = vt[(kt + 3) * tsv + d];
#pragma unroll
                        for (int b = 0; b < RBT; ++b) {
                            const float4 w4 = *reinterpret_cast<const float4*>(sP + rows[b] * SA_KT + kt);
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
    // the CTAs' partial results merged in rank order, the sink joins the denominator; every CTA finishes its share of the outputs
    cluster.sync();
    for (int e = rank * (int)blockDim.x + threadIdx.x; e < R * dv; e += CL * (int)blockDim.x) {
        const int r = e / dv, d = e % dv, t = t0 + r / nh, h = h0 + r % nh;
        float m = p.sink ? p.sink[h] : -CUDART_INF_F;
        for (int rk = 0; rk < CL; ++rk) m = fmaxf(m, cluster.map_shared_rank(sMax, rk)[r]);
        float num = 0.f, den = p.sink ? expf(p.sink[h] - m) : 0.f;
        for (int rk = 0; rk < CL; ++rk) {
            const float mr = cluster.map_shared_rank(sMax, rk)[r];
            if (mr > -CUDART_INF_F) {
                const float f = expf(mr - m);
                num = fmaf(cluster.map_shared_rank(sO, rk)[e], f, num);
                den = fmaf(cluster.map_shared_rank(sSum, rk)[r], f, den);
            }
        }
        float o = num / den;
        if (p.gate) o *= lin_sigmoid(p.gate[(size_t)t * p.ldg + (size_t)h * dv + d]);
        p.out[(size_t)t * p.ldo + (size_t)h * dv + d] = o;
    }
    cluster.sync();                                // nobody leaves while its shared memory is still being read
}

// ------------------------------------------------------------------------------------------------------------------
// register form (key and value sizes that are multiples of four, at most 128 NC; the engine builds NC = 1): no tile passes
// through shared memory
// ------------------------------------------------------------------------------------------------------------------
// A warp owns RB rows of one key / value head and a share of the visible tiles, and keeps everything it accumulates in
// registers: lane l holds entries 128 c + 4 l .. + 3 (c < NC) of the RB query rows and of the RB un-normalised output rows,
// plus the rows' running maxima and sums.  Per tile of 32 keys:
//   scores   eight keys at a time: every lane loads its 16 bytes of each 512-byte piece of a key row straight from the cache,
//            multiplies them with its query entries, and a butterfly over the lanes (keep half of the keys, send the other
//            half: 4 + 2 + 1 exchanges, then two plain ones) leaves the finished score of key (l >> 2) of the batch in lane l;
//   softmax  window / block mask, running maximum / sum with three exchanges per row;
//   values   the weight of each key is broadcast from its lane, every lane loads its 16 bytes of each piece of the value row.
// With few (head, row block) items per chunk the tiles are split over KS warps per item as well as over the cluster's CTAs;
// the partial (maximum, sum, output) triples meet in shared memory (within a CTA) and then through distributed shared memory
// (across the cluster), always in a fixed order; the sink term and the gate come in at the end.
constexpr int SAR_THREADS = 256;

__host__ __device__ inline size_t sink_attn_reg_smem(int qb, int HB, int rep, int dv, int rb, int ks) {
    const int nhc = rep < HB ? rep : HB, ncv = HB / nhc;
    const size_t nblk = ((size_t)qb * nhc + rb - 1) / rb, slots = (size_t)ncv * nblk * ks;
    return (slots * rb * (dv + 2) + 2 * (size_t)ncv * nblk * rb + 8) * sizeof(float);
}

template <int RB, int NC>
__global__ void __launch_bounds__(SAR_THREADS, NC == 1 ? 2 : 1) sink_attn_reg_kernel(const SinkAttnParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = p.cl, rank = blockIdx.x % CL;
    int t0, nq;
    if (!sa_chunk(p, blockIdx.x / CL, t0, nq)) return;
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, dk = p.dk, dv = p.dv, rep = H / p.G, KS = p.ks, D = p.D;
    const int h0 = blockIdx.y * p.HB, nh = min(p.HB, H - h0);
    const int c_first = h0 / rep, nhc = min(rep, nh), ncv = nh / nhc;
    const int R = nq * nh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, NW = blockDim.x >> 5;
    const int ncv_cap = p.HB / min(rep, p.HB);
    const int nblk_cap = (p.qb * min(rep, p.HB) + RB - 1) / RB;   // row blocks of one head the shared memory was sized for
    const int nrg = nq * nhc, nblk = (nrg + RB - 1) / RB;         // rows / row blocks of one head in this chunk
    extern __shared__ __align__(16) float sar_smem[];
    float* sO = sar_smem;                                          // [ncv * nblk_cap][KS][RB][dv] partial outputs (slot 0 of an item: merged)
    float* sM = sO + (size_t)ncv_cap * nblk_cap * KS * RB * dv;    // [ncv * nblk_cap][KS][RB]
    float* sL = sM + (size_t)ncv_cap * nblk_cap * KS * RB;
    float* sM2 = sL + (size_t)ncv_cap * nblk_cap * KS * RB;        // [ncv * nblk_cap][RB] merged over the CTA's key splits
    float* sL2 = sM2 + (size_t)ncv_cap * nblk_cap * RB;
    const int* tbl = p.table + (size_t)slot * p.stride;
    const int npb = p.pool > 0 ? max(0, pos1 - p.win + 1) / p.pool : 0;
    const int jlo = max(0, pos0 - p.win + 1), ntk = pos1 - jlo + 1;
    const int npt = (npb + SA_KT - 1) / SA_KT, ntiles = npt + (ntk + SA_KT - 1) / SA_KT;
    const int l4 = lane * 4, kq = lane >> 2;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int it = warp; it < ncv * nblk * KS; it += NW) {
        const int item = it / KS, ks = it % KS;
        const int lc = item / nblk, c = c_first + lc, rr0 = (item % nblk) * RB, nr = min(RB, nrg - rr0);
        int qi[RB], hh[RB];
        float4 q[RB][NC], acc[RB][NC];
        float m[RB], l[RB];
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            const int rr = rr0 + min(b, nr - 1);
            qi[b] = rr / nhc; hh[b] = h0 + lc * nhc + rr % nhc;
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) {
                q[b][cc] = (l4 + 128 * cc < dk) ? *reinterpret_cast<const float4*>(p.q + (size_t)(t0 + qi[b]) * p.ldq + (size_t)hh[b] * dk + l4 + 128 * cc) : zero4;
                acc[b][cc] = zero4;
            }
            m[b] = -CUDART_INF_F; l[b] = 0.f;
        }
        const size_t koffs = (size_t)p.koff + (size_t)c * dk + l4, voffs = (size_t)p.voff + (size_t)c * dv + l4;
        for (int ti = rank * KS + ks; ti < ntiles; ti += CL * KS) {
            const bool pooled = ti < npt;
            const int i0 = pooled ? ti * SA_KT : jlo + (ti - npt) * SA_KT;
            const int nk = pooled ? min(SA_KT, npb - i0) : min(SA_KT, pos1 + 1 - i0);
            const float* base = pooled ? p.pcache : p.cache;
            unsigned long long myoff = 0ull;                       // row offset of key i0 + lane
            if (lane < nk) myoff = (unsigned long long)(pooled ? sa_pool_row(tbl, p.page, p.pool, p.prow, i0 + lane) : sa_token_row(tbl, p.page, i0 + lane)) * (unsigned)D;
            float s[4][RB];
            // ---- scores: four batches of eight keys ----
#pragma unroll
            for (int bt = 0; bt < 4; ++bt) {
                float pt[RB][8];
#pragma unroll
                for (int b = 0; b < RB; ++b)
#pragma unroll
                    for (int u = 0; u < 8; ++u) pt[b][u] = 0.f;
                unsigned long long off[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) off[u] = __shfl_sync(0xffffffffu, myoff, bt * 8 + u);
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) {
                    if (128 * cc >= dk) break;                     // warp-uniform
                    const bool kact = l4 + 128 * cc < dk;
                    float4 kx[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        kx[u] = (kact && bt * 8 + u < nk) ? __ldg(reinterpret_cast<const float4*>(base + off[u] + koffs + 128 * cc)) : zero4;
#pragma unroll
                    for (int b = 0; b < RB; ++b)
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            pt[b][u] = fmaf(q[b][cc].x, kx[u].x, fmaf(q[b][cc].y, kx[u].y, fmaf(q[b][cc].z, kx[u].z, fmaf(q[b][cc].w, kx[u].w, pt[b][u]))));
                }
#pragma unroll
                for (int b = 0; b < RB; ++b) {
                    // butterfly: lanes with bit 4 set keep keys 4..7 and send 0..3, and so on; lane l ends with key (l >> 2) & 7
                    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
                    float a4[4], a2[2], a1;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float send = h16 ? pt[b][i] : pt[b][i + 4], keep = h16 ? pt[b][i + 4] : pt[b][i];
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
            // ---- mask, running maximum and sum of every row; s becomes the tile's weights ----
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                const int pq = pos0 + qi[b];
                const int lim = pooled ? max(0, pq - p.win + 1) / p.pool : 0;      // blocks this row sees
                float tmax = -CUDART_INF_F;
#pragma unroll
                for (int bt = 0; bt < 4; ++bt) {
                    const int kk = bt * 8 + kq, i = i0 + kk;
                    const bool vis = kk < nk && (pooled ? i < lim : (i <= pq && i > pq - p.win));
                    s[bt][b] = vis ? s[bt][b] * p.scale : -CUDART_INF_F;
                    tmax = fmaxf(tmax, s[bt][b]);
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
                const float mn = fmaxf(m[b], tmax);                // the same in every lane
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
                tsum += __shfl_xor_sync(0xffffffffu, tsum, 4);     // lanes that differ in bits 0..1 hold the same keys
                l[b] = l[b] * scl + tsum;
                m[b] = mn;
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) { acc[b][cc].x *= scl; acc[b][cc].y *= scl; acc[b][cc].z *= scl; acc[b][cc].w *= scl; }
            }
            // ---- weights x values ----
#pragma unroll
            for (int bt = 0; bt < 4; ++bt) {
                if (bt * 8 >= nk) break;                           // warp-uniform
                float w[RB][8];
                unsigned long long off[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    off[u] = __shfl_sync(0xffffffffu, myoff, bt * 8 + u);
#pragma unroll
                    for (int b = 0; b < RB; ++b) w[b][u] = __shfl_sync(0xffffffffu, s[bt][b], u << 2);
                }
#pragma unroll
                for (int cc = 0; cc < NC; ++cc) {
                    if (128 * cc >= dv) break;                     // warp-uniform
                    const bool vact = l4 + 128 * cc < dv;
                    float4 vx[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        vx[u] = (vact && bt * 8 + u < nk) ? __ldg(reinterpret_cast<const float4*>(base + off[u] + voffs + 128 * cc)) : zero4;
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int b = 0; b < RB; ++b) {
                            acc[b][cc].x = fmaf(w[b][u], vx[u].x, acc[b][cc].x); acc[b][cc].y = fmaf(w[b][u], vx[u].y, acc[b][cc].y);
                            acc[b][cc].z = fmaf(w[b][u], vx[u].z, acc[b][cc].z); acc[b][cc].w = fmaf(w[b][u], vx[u].w, acc[b][cc].w);
                        }
                }
            }
        }
        const size_t sl = (size_t)(lc * nblk_cap + item % nblk) * KS + ks;
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            if (b >= nr) break;
#pragma unroll
            for (int cc = 0; cc < NC; ++cc)
                if (l4 + 128 * cc < dv) *reinterpret_cast<float4*>(sO + (sl * RB + b) * dv + l4 + 128 * cc) = acc[b][cc];
            if (lane == 0) { sM[sl * RB + b] = m[b]; sL[sl * RB + b] = l[b]; }
        }
    }
    __syncthreads();
    // the CTA's key splits of every row merged in split order (into split 0's place)
    for (int e = threadIdx.x; e < R * dv; e += (int)blockDim.x) {
        const int r = e / dv, d = e % dv, qi_ = r / nh, hl = r % nh, lc = hl / nhc, rr = qi_ * nhc + hl % nhc;
        const size_t it0 = (size_t)(lc * nblk_cap + rr / RB) * KS;
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
        sO[(it0 * RB + b) * dv + d] = num;                         // only this thread touches column d of the row
        if (d == 0) { sM2[(it0 / KS) * RB + b] = mx; sL2[(it0 / KS) * RB + b] = den; }
    }
    // the CTAs' partial results merged in rank order; every CTA finishes its share of the outputs
    cluster.sync();
    for (int e = rank * (int)blockDim.x + threadIdx.x; e < R * dv; e += CL * (int)blockDim.x) {
        const int r = e / dv, d = e % dv, qi_ = r / nh, hl = r % nh, lc = hl / nhc, rr = qi_ * nhc + hl % nhc;
        const int t = t0 + qi_, h = h0 + hl;
        const size_t ib = (size_t)(lc * nblk_cap + rr / RB);
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
        float mx = p.sink ? p.sink[h] : -CUDART_INF_F;
#pragma unroll
        for (int rk = 0; rk < 8; ++rk) mx = fmaxf(mx, mr[rk]);
        float num = 0.f, den = p.sink ? expf(p.sink[h] - mx) : 0.f;
#pragma unroll
        for (int rk = 0; rk < 8; ++rk)
            if (mr[rk] > -CUDART_INF_F) {
                const float f = expf(mr[rk] - mx);
                num = fmaf(orr[rk], f, num);
                den = fmaf(lr[rk], f, den);
            }
        float o = num / den;
        if (p.gate) o *= lin_sigmoid(p.gate[(size_t)t * p.ldg + (size_t)h * dv + d]);
        p.out[(size_t)t * p.ldo + (size_t)h * dv + d] = o;
    }
    cluster.sync();                                // nobody leaves while its shared memory is still being read
}

}  // namespace b200
