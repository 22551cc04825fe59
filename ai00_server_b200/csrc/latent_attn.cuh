// Latent ("compressed key/value") attention over a paged cache, in the absorbed form.
//
// A layer caches, per token, one latent row c [rk] (RMS-normed down-projection) and one rotated key part kr [dr] shared by
// all heads: D = rk + dr floats per token and layer.  Per head the key is [W_uk c ; kr] and the value W_uv c, so with
//     qa[h] = W_uk[h]^T q_plain[h]   (rk numbers)           -- a grouped linear over heads, W_uk stored transposed at load
// the score is (qa[h] . c_j + q_rot[h] . kr_j) * scale and the head's output is W_uv[h] (sum_j p_j c_j): the attention itself
// runs over the shared rows [c_j ; kr_j] for all heads (no per-head keys or values are ever materialised), and the two
// up-projections are grouped linears before and after it.  Scores, softmax and the weighted sums are f32.
//
// Paging: the cache of every layer is a pool of pages of `page` tokens; page_table[slot][i] names the page that holds the
// sequence's positions [i * page, (i + 1) * page).  Pages are handed out and taken back by the host (engine state manager);
// a step uploads the table entries it added (page_update_kernel).  A layer that borrows another layer's cache reads that
// layer's pool with the same table.
//
//   rope_rows_kernel     rotate-half rotary embedding on `dims` leading entries of a per-head chunk (positions and angles f32;
//                        frequency table with the long-context rescaling folded in at load, magnitude factor on cos and sin)
//   kv_write_kernel      c = rms(kv[:rk]) * w, kr = rope(kv[rk:]) -> cache row of (slot, position)
//   latent_attn_kernel   QB consecutive tokens of one sequence x HG heads per CTA share every key tile; online softmax; the
//                        context may be split over blockIdx.z (long contexts at small batch), partial (o, m, l) per split
//   latent_merge_kernel  combines the splits in fixed order and normalises
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"

namespace b200 {

// per-step sequence metadata that follows the MetaView block in the same upload
struct SeqMeta {
    const int* base;
    int maxT;
    __host__ __device__ int n_upd() const { return base[0]; }
    __host__ __device__ int n_chunks() const { return base[1]; }
    __host__ __device__ const int* tok_pos() const { return base + 8; }                     // [maxT] position of the token in its sequence
    __host__ __device__ const int* chunk_start() const { return base + 8 + maxT; }          // [maxT] first token of an attention chunk
    __host__ __device__ const int* chunk_count() const { return base + 8 + 2 * maxT; }      // [maxT] tokens of the chunk (one sequence)
    __host__ __device__ const int* upd() const { return base + 8 + 3 * maxT; }              // [maxT][3] (slot, index, page)
    __host__ __device__ static size_t ints(int maxT) { return 8 + 6 * (size_t)maxT; }
};

struct PageUpdateParams { SeqMeta sm; int* table; int stride; };

__global__ void page_update_kernel(const PageUpdateParams p) {
    const int n = p.sm.n_upd();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int* u = p.sm.upd() + 3 * i;
        p.table[(size_t)u[0] * p.stride + u[1]] = u[2];
    }
}

struct RopeParams {
    const float* src; int lds, s_head, s_off;      // element (t, h, i) at src[t * lds + h * s_head + s_off + i]
    float* dst; int ldd, d_head, d_off;
    int heads, dims, width;                        // rotate the first `dims` of `width` entries; the rest are copied
    const float* freq;                             // [dims / 2]
    float mag;
    MetaView meta; SeqMeta sm;
    const double* pair_freq = nullptr;             // set: neighbouring entries (2i, 2i + 1) turn together (angle reduced in double)
};

// the pair (2i, 2i + 1) of `s` turned by position * freq[i]; returns entry i of the result
__device__ __forceinline__ float rot_pair_entry(const float* s, int i, int pos, const double* freq) {
    float cs, sn;
    rot_cos_sin(pos, freq[i >> 1], cs, sn);
    const float u = s[i & ~1], v = s[i | 1];
    return (i & 1) ? v * cs + u * sn : u * cs - v * sn;
}

__global__ void __launch_bounds__(128) rope_rows_kernel(const RopeParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const float pos = (float)p.sm.tok_pos()[t];
    const int half = p.dims >> 1;
    for (int e = threadIdx.x; e < p.heads * p.width; e += blockDim.x) {
        const int h = e / p.width, i = e % p.width;
        const float* s = p.src + (size_t)t * p.lds + (size_t)h * p.s_head + p.s_off;
        float* d = p.dst + (size_t)t * p.ldd + (size_t)h * p.d_head + p.d_off;
        if (i >= p.dims) { d[i] = s[i]; continue; }
        if (p.pair_freq) { d[i] = rot_pair_entry(s, i, p.sm.tok_pos()[t], p.pair_freq); continue; }
        const int j = i < half ? i : i - half;
        const float a = pos * p.freq[j];
        const float cs = cosf(a) * p.mag, sn = sinf(a) * p.mag;
        const float u = s[j], v = s[j + half];
        d[i] = i < half ? u * cs - v * sn : v * cs + u * sn;
    }
}

struct KvWriteParams {
    const float* kv; int ld;                       // [T, rk + dr] down-projection rows
    float* cache;                                  // pool of this layer: [pages][page][D]
    const int* table; int stride; int page;
    const float* weight;                           // [rk]
    int rk, dr, dims;
    const float* freq; float mag, eps;
    MetaView meta; SeqMeta sm;
    const double* pair_freq = nullptr;             // as in RopeParams
};

__global__ void __launch_bounds__(128) kv_write_kernel(const KvWriteParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int slot = p.meta.tok_slot()[t], ipos = p.sm.tok_pos()[t];
    const float* src = p.kv + (size_t)t * p.ld;
    const int D = p.rk + p.dr;
    float* dst = p.cache + ((size_t)p.table[(size_t)slot * p.stride + ipos / p.page] * p.page + ipos % p.page) * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.rk; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        ss = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) ss += red[i];
    }
    const float r = 1.f / sqrtf(ss / (float)p.rk + p.eps);
    for (int i = threadIdx.x; i < p.rk; i += blockDim.x) dst[i] = src[i] * r * p.weight[i];
    const float pos = (float)ipos;
    const int half = p.dims >> 1;
    for (int i = threadIdx.x; i < p.dr; i += blockDim.x) {
        const float* s = src + p.rk;
        if (i >= p.dims) { dst[p.rk + i] = s[i]; continue; }
        if (p.pair_freq) { dst[p.rk + i] = rot_pair_entry(s, i, ipos, p.pair_freq); continue; }
        const int j = i < half ? i : i - half;
        const float a = pos * p.freq[j];
        const float cs = cosf(a) * p.mag, sn = sinf(a) * p.mag;
        const float u = s[j], v = s[j + half];
        dst[p.rk + i] = i < half ? u * cs - v * sn : v * cs + u * sn;
    }
}

struct LatentAttnParams {
    const float* q;                                // [T, H * D]: per head [qa (rk) ; q_rot (dr)]
    const float* cache;
    const int* table; int stride; int page;
    float* part;                                   // [T][H][nsplit][rk + 2]: unnormalised o, running max, running sum
    int H, rk, dr, nsplit;
    float scale;
    MetaView meta; SeqMeta sm;
};

constexpr int LA_KT = 32;                          // keys per tile (one per lane in the score phase)
constexpr int LA_THREADS = 128;
constexpr int LA_MAX_RK_CHUNKS = 16;               // rk <= 512

template <int QB, int HG>
__host__ __device__ constexpr size_t latent_attn_smem(int D) {
    return ((size_t)QB * HG * D + (size_t)LA_KT * (D + 1) + (size_t)QB * HG * LA_KT) * sizeof(float);
}

template <int QB, int HG>
__global__ void __launch_bounds__(LA_THREADS) latent_attn_kernel(const LatentAttnParams p) {
    constexpr int R = QB * HG;                     // (token, head) rows of this CTA
    constexpr int RPW = R / 4;                     // rows per warp
    static_assert(R % 4 == 0, "rows must split over four warps");
    const int ci = blockIdx.x;
    if (ci >= p.sm.n_chunks()) return;
    const int t0 = p.sm.chunk_start()[ci], nt = p.sm.chunk_count()[ci];
    const int h0 = blockIdx.y * HG;
    const int D = p.rk + p.dr, rk = p.rk;
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0];           // chunk tokens sit at consecutive positions pos0, pos0 + 1, ...
    const int nkeys = pos0 + nt;                   // keys 0 .. pos0 + nt - 1 are visible to the last token
    const int tiles = (nkeys + LA_KT - 1) / LA_KT;
    const int per = (tiles + p.nsplit - 1) / p.nsplit;
    const int tile_lo = blockIdx.z * per, tile_hi = min(tiles, tile_lo + per);

    extern __shared__ float la_smem[];
    float* sq = la_smem;                             // [R][D]
    float* sk = sq + (size_t)R * D;                // [LA_KT][D + 1]
    float* sp = sk + (size_t)LA_KT * (D + 1);      // [R][LA_KT]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int e = threadIdx.x; e < R * D; e += LA_THREADS) {
        const int r = e / D, d = e % D;
        const int qi = r / HG, h = h0 + r % HG;
        sq[e] = (qi < nt && h < p.H) ? p.q[(size_t)(t0 + qi) * p.H * D + (size_t)h * D + d] : 0.f;
    }
    float m[RPW], l[RPW], o[RPW][LA_MAX_RK_CHUNKS];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -CUDART_INF_F; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < LA_MAX_RK_CHUNKS; ++c) o[i][c] = 0.f;
    }
    const int* tab = p.table + (size_t)slot * p.stride;
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int kb = tile * LA_KT;
        __syncthreads();                           // previous tile fully consumed (and sq written, first time)
        for (int e = threadIdx.x; e < LA_KT * D; e += LA_THREADS) {
            const int j = e / D, d = e % D;
            const int kj = kb + j;
            float v = 0.f;
            if (kj < nkeys) v = p.cache[((size_t)tab[kj / p.page] * p.page + kj % p.page) * D + d];
            sk[(size_t)j * (D + 1) + d] = v;
        }
        __syncthreads();
        // scores: lane = key
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const float* kr = sk + (size_t)lane * (D + 1);
        for (int d = 0; d < D; ++d) {
            const float kv = kr[d];
#pragma unroll
            for (int i = 0; i < RPW; ++i) s[i] = fmaf(sq[(size_t)(warp * RPW + i) * D + d], kv, s[i]);
        }
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp * RPW + i;
            const int qi = r / HG;
            const bool live = qi < nt && (kb + lane) <= pos0 + qi;          // causal: key position <= query position
            const float sc = live ? s[i] * p.scale : -CUDART_INF_F;
            float mx = sc;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
            const float mn = fmaxf(m[i], mx);
            float pj = 0.f, corr = 1.f;
            if (mn > -CUDART_INF_F) {
                pj = live ? expf(sc - mn) : 0.f;
                corr = expf(m[i] - mn);            // m = -inf -> 0
            }
            float ps = pj;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, of);
            l[i] = l[i] * corr + ps;
            m[i] = mn;
#pragma unroll
            for (int c = 0; c < LA_MAX_RK_CHUNKS; ++c) o[i][c] *= corr;
            sp[(size_t)r * LA_KT + lane] = pj;
        }
        __syncwarp();
        // weighted sum of the latent rows: lane = latent channel (mod 32)
#pragma unroll
        for (int c = 0; c < LA_MAX_RK_CHUNKS; ++c) {
            const int d = c * 32 + lane;
            if (c * 32 >= rk) break;
            if (d < rk) {
                for (int j = 0; j < LA_KT; ++j) {
                    const float kv = sk[(size_t)j * (D + 1) + d];
#pragma unroll
                    for (int i = 0; i < RPW; ++i) o[i][c] = fmaf(sp[(size_t)(warp * RPW + i) * LA_KT + j], kv, o[i][c]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        const int qi = r / HG, h = h0 + r % HG;
        if (qi >= nt || h >= p.H) continue;
        float* dst = p.part + (((size_t)(t0 + qi) * p.H + h) * p.nsplit + blockIdx.z) * (rk + 2);
#pragma unroll
        for (int c = 0; c < LA_MAX_RK_CHUNKS; ++c) {
            const int d = c * 32 + lane;
            if (d < rk) dst[d] = o[i][c];
        }
        if (lane == 0) { dst[rk] = m[i]; dst[rk + 1] = l[i]; }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Tensor-core variant for the serving precision: the same CTA shape (16 (token, head) rows, 32-key tiles, online softmax in
// f32) with both products on mma.sync m16n8k8 TF32 (operands rounded to TF32 with cvt.rna, f32 accumulation):
//   scores  S[16 x 32]  = Q[16 x D] . K^T      warp w owns keys 8w .. 8w+7, D / 8 k-steps
//   output  O[16 x rk] += P[16 x 32] . C       warp w owns a quarter of the latent channels, 4 k-steps per 8 channels
// Scores go through shared memory between the two so that the softmax keeps the row-per-warp form of the f32 kernel.
// Row strides are = 4 (mod 32) floats: fragment loads of the score phase are bank-conflict free.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ void mma_tf32_1688(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__host__ __device__ inline int la_pad8(int n) { return (n + 7) & ~7; }
__host__ __device__ inline int la_stride(int D) { const int dp = la_pad8(D); return dp + ((4 - dp % 32) + 32) % 32; }
__host__ __device__ inline size_t latent_attn_tc_smem(int D) {
    return ((size_t)16 * la_stride(D) + (size_t)LA_KT * la_stride(D) + 16 * 36 + 64) * sizeof(float);
}
constexpr int LA_TC_MAX_NT = 16;                   // 8-channel tiles per warp: rk <= 512

template <int QB, int HG>
__global__ void __launch_bounds__(LA_THREADS) latent_attn_tc_kernel(const LatentAttnParams p) {
    static_assert(QB * HG == 16, "one m16 tile of (token, head) rows");
    const int ci = blockIdx.x;
    if (ci >= p.sm.n_chunks()) return;
    const int t0 = p.sm.chunk_start()[ci], nt = p.sm.chunk_count()[ci];
    const int h0 = blockIdx.y * HG;
    const int D = p.rk + p.dr, rk = p.rk, Dp = la_pad8(D), DS = la_stride(D);
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0];
    const int nkeys = pos0 + nt;
    const int tiles = (nkeys + LA_KT - 1) / LA_KT;
    const int per = (tiles + p.nsplit - 1) / p.nsplit;
    const int tile_lo = blockIdx.z * per, tile_hi = min(tiles, tile_lo + per);

    extern __shared__ __align__(16) float la_tc_smem[];
    float* sq = la_tc_smem;                        // [16][DS]
    float* sk = sq + (size_t)16 * DS;              // [LA_KT][DS]
    float* ss = sk + (size_t)LA_KT * DS;           // [16][36] scores, then probabilities
    float* scorr = ss + 16 * 36;                   // [16] rescale of the running output
    float* sml = scorr + 16;                       // [16][2] final (m, l)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;

    for (int e = threadIdx.x; e < 16 * DS; e += LA_THREADS) {
        const int r = e / DS, d = e % DS;
        const int qi = r / HG, h = h0 + r % HG;
        sq[e] = (d < D && qi < nt && h < p.H) ? p.q[(size_t)(t0 + qi) * p.H * D + (size_t)h * D + d] : 0.f;
    }
    for (int e = threadIdx.x; e < LA_KT * (DS - D); e += LA_THREADS) {       // pad columns of the key tile stay zero
        const int j = e / (DS - D), d = D + e % (DS - D);
        sk[(size_t)j * DS + d] = 0.f;
    }
    constexpr int RPW = 4;
    float m[RPW], l[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) { m[i] = -CUDART_INF_F; l[i] = 0.f; }
    const int cw = la_pad8((rk + 3) / 4);          // latent channels per warp, a multiple of 8
    float o[LA_TC_MAX_NT][4];
#pragma unroll
    for (int n = 0; n < LA_TC_MAX_NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int* tab = p.table + (size_t)slot * p.stride;
    const bool vec = (D % 4 == 0);
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int kb = tile * LA_KT;
        __syncthreads();                           // the previous tile is consumed; sq and the pad columns are written
        if (vec) {
            const int cpr = D / 4;                 // 16-byte chunks per row
            for (int e = threadIdx.x; e < LA_KT * cpr; e += LA_THREADS) {
                const int j = e / cpr, c = e % cpr;
                const int kj = kb + j;
                float* dst = sk + (size_t)j * DS + c * 4;
                if (kj < nkeys) {
                    const float* src = p.cache + ((size_t)tab[kj / p.page] * p.page + kj % p.page) * D + c * 4;
                    const uint32_t da = (uint32_t)__cvta_generic_to_shared(dst);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(da), "l"(src) : "memory");
                } else {
                    *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
        } else {
            for (int e = threadIdx.x; e < LA_KT * D; e += LA_THREADS) {
                const int j = e / D, d = e % D;
                const int kj = kb + j;
                sk[(size_t)j * DS + d] = kj < nkeys ? p.cache[((size_t)tab[kj / p.page] * p.page + kj % p.page) * D + d] : 0.f;
            }
        }
        __syncthreads();
        {   // scores of keys 8 * warp .. + 7
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const float* qa0 = sq + (size_t)gq * DS + tq;
            const float* qa1 = sq + (size_t)(gq + 8) * DS + tq;
            const float* kb0 = sk + (size_t)(warp * 8 + gq) * DS + tq;
#pragma unroll 4
            for (int ks = 0; ks < Dp; ks += 8) {
                uint32_t a[4], b[2];
                a[0] = to_tf32(qa0[ks]); a[1] = to_tf32(qa1[ks]); a[2] = to_tf32(qa0[ks + 4]); a[3] = to_tf32(qa1[ks + 4]);
                b[0] = to_tf32(kb0[ks]); b[1] = to_tf32(kb0[ks + 4]);
                mma_tf32_1688(acc, a, b);
            }
            ss[gq * 36 + warp * 8 + tq * 2] = acc[0]; ss[gq * 36 + warp * 8 + tq * 2 + 1] = acc[1];
            ss[(gq + 8) * 36 + warp * 8 + tq * 2] = acc[2]; ss[(gq + 8) * 36 + warp * 8 + tq * 2 + 1] = acc[3];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RPW; ++i) {            // softmax rows 4 * warp .. + 3, lane = key
            const int r = warp * RPW + i;
            const int qi = r / HG;
            const bool live = qi < nt && (kb + lane) <= pos0 + qi;
            const float sc = live ? ss[r * 36 + lane] * p.scale : -CUDART_INF_F;
            float mx = sc;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
            const float mn = fmaxf(m[i], mx);
            float pj = 0.f, corr = 1.f;
            if (mn > -CUDART_INF_F) {
                pj = live ? expf(sc - mn) : 0.f;
                corr = expf(m[i] - mn);
            }
            float ps = pj;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, of);
            l[i] = l[i] * corr + ps;
            m[i] = mn;
            ss[r * 36 + lane] = pj;
            if (lane == 0) scorr[r] = corr;
        }
        __syncthreads();
        {   // output: this warp's latent channels
            uint32_t a[4][4];
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                a[ks][0] = to_tf32(ss[gq * 36 + ks * 8 + tq]); a[ks][1] = to_tf32(ss[(gq + 8) * 36 + ks * 8 + tq]);
                a[ks][2] = to_tf32(ss[gq * 36 + ks * 8 + tq + 4]); a[ks][3] = to_tf32(ss[(gq + 8) * 36 + ks * 8 + tq + 4]);
            }
            const float c0 = scorr[gq], c1 = scorr[gq + 8];
#pragma unroll
            for (int n = 0; n < LA_TC_MAX_NT; ++n) {
                const int cb = warp * cw + n * 8;
                if (n * 8 >= cw || cb >= rk) break;
                o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    uint32_t b[2];
                    b[0] = to_tf32(sk[(size_t)(ks * 8 + tq) * DS + cb + gq]);
                    b[1] = to_tf32(sk[(size_t)(ks * 8 + tq + 4) * DS + cb + gq]);
                    mma_tf32_1688(o[n], a[ks], b);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPW; ++i)
        if (lane == 0) { sml[(warp * RPW + i) * 2] = m[i]; sml[(warp * RPW + i) * 2 + 1] = l[i]; }
    __syncthreads();
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        const int r = gq + hrow * 8;
        const int qi = r / HG, h = h0 + r % HG;
        if (qi >= nt || h >= p.H) continue;
        float* dst = p.part + (((size_t)(t0 + qi) * p.H + h) * p.nsplit + blockIdx.z) * (rk + 2);
#pragma unroll
        for (int n = 0; n < LA_TC_MAX_NT; ++n) {
            const int cb = warp * cw + n * 8;
            if (n * 8 >= cw || cb >= rk) break;
            const int d = cb + tq * 2;
            if (d < rk) dst[d] = o[n][hrow * 2];
            if (d + 1 < rk) dst[d + 1] = o[n][hrow * 2 + 1];
        }
        if (warp == 0 && tq == 0) { dst[rk] = sml[r * 2]; dst[rk + 1] = sml[r * 2 + 1]; }
    }
}

struct LatentMergeParams {
    const float* part;
    float* out;                                    // [T, H * rk]
    int H, rk, nsplit;
    MetaView meta;
};

__global__ void __launch_bounds__(128) latent_merge_kernel(const LatentMergeParams p) {
    const int t = blockIdx.x, h = blockIdx.y;
    if (t >= p.meta.T()) return;
    const float* src = p.part + ((size_t)t * p.H + h) * p.nsplit * (p.rk + 2);
    float M = -CUDART_INF_F;
    for (int z = 0; z < p.nsplit; ++z) M = fmaxf(M, src[(size_t)z * (p.rk + 2) + p.rk]);
    float Lsum = 0.f;
    for (int z = 0; z < p.nsplit; ++z) {
        const float mz = src[(size_t)z * (p.rk + 2) + p.rk];
        if (mz > -CUDART_INF_F) Lsum += src[(size_t)z * (p.rk + 2) + p.rk + 1] * expf(mz - M);
    }
    const float inv = 1.f / Lsum;
    for (int d = threadIdx.x; d < p.rk; d += blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < p.nsplit; ++z) {
            const float mz = src[(size_t)z * (p.rk + 2) + p.rk];
            if (mz > -CUDART_INF_F) acc += src[(size_t)z * (p.rk + 2) + d] * expf(mz - M);
        }
        p.out[(size_t)t * p.H * p.rk + (size_t)h * p.rk + d] = acc * inv;
    }
}

}  // namespace b200
