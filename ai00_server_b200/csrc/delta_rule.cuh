// Gated delta rule with a per-key-channel decay, and the short causal convolutions in front of it.
//
// Per value head, with the [dk, dv] f32 state S, unit-length key k and query q (q also times dk^-1/2), a decay vector g in
// (0, 1)^dk acting on the rows of S, and a write strength beta in (0, 1):
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees this token's write)
//     g = exp(-exp(A_h) * softplus(z)),  z = low-rank projection + bias,  beta = sigmoid(b)
// The read-out is divided by its root mean square over dv, times a weight vector shared by the heads, times sigmoid of a
// low-rank gate.  Several value heads may share one key / query head (value head h uses head h / (H / G)).
//
//   short_conv_kernel     y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1) + j, c]): per-channel causal convolution over time, the
//                         last column is the current token's; inputs before the step come from the sequence's tail rows
//                         (the last taps - 1 inputs, zeros at the start of a sequence)
//   conv_commit_kernel    the step's last taps - 1 inputs become the sequence's new tail rows (own launch: every token of the
//                         step has read the old tail by then)
//   delta_rule_reg_kernel the state column of thread j in registers (dk <= 128, dv <= 256): the form that runs for usual head sizes
//   delta_rule_kernel     one CTA per (value head, sequence of the step): the state sits in shared memory for the sequence's
//                         tokens of this step, column j belongs to thread j (two passes over the column per token: decay +
//                         S^T k, then update + read-out; no cross-thread traffic besides the unit norms and the output norm)
// Decays, logarithms, softplus, gates, unit norms, state and read-out are f32.
#pragma once
#include <cuda_runtime.h>
#include "common.cuh"

namespace b200 {

struct ShortConvParams {
    const float* x; int ldx;                      // [T, >= C] inputs (projection output rows)
    float* y; int ldy;                            // [T, C] silu(conv), or conv
    const float* w;                               // [C][taps]
    float* tail;                                  // [S][taps - 1][C] of this layer; row taps - 2 is the most recent input
    int C, taps;
    MetaView meta;
    int silu = 1;                                 // 0: the plain convolution
};

__global__ void __launch_bounds__(256) short_conv_kernel(const ShortConvParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int slot = p.meta.tok_slot()[t];
    // index of the token inside its sequence's run of this step: walk the prev links (runs are contiguous: t - first)
    int first = t;
    {
        const int* prev = p.meta.tok_prev();
        // tok_prev[t] = t - 1 inside a run, -1 at its first token; only taps - 1 steps back matter
        for (int d = 0; d < p.taps - 1 && prev[first] >= 0; ++d) first = prev[first];
    }
    const int back = t - first;                   // rows of this step available behind t (capped at taps - 1)
    const float* tl = p.tail + (size_t)slot * (p.taps - 1) * p.C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < p.taps; ++j) {
            const int d = p.taps - 1 - j;         // steps back
            const float xv = d <= back ? p.x[(size_t)(t - d) * p.ldx + c] : tl[(size_t)(p.taps - 1 + back - d) * p.C + c];
            acc = fmaf(p.w[(size_t)c * p.taps + j], xv, acc);
        }
        p.y[(size_t)t * p.ldy + c] = p.silu ? acc / (1.f + expf(-acc)) : acc;
    }
}

__global__ void __launch_bounds__(256) conv_commit_kernel(const ShortConvParams p) {
    const int i = blockIdx.x;
    if (i >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[i], t0 = p.meta.slot_start()[i], nt = p.meta.slot_count()[i];
    const int keep = p.taps - 1;
    float* tl = p.tail + (size_t)slot * keep * p.C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += gridDim.y * blockDim.x) {
        // new row r holds the input nt - keep + r of this step, or, for a short step, the old row r + nt (read before any
        // later row is written: r ascends and r + nt > r)
        for (int r = 0; r < keep; ++r) {
            const int idx = nt - keep + r;
            tl[(size_t)r * p.C + c] = idx >= 0 ? p.x[(size_t)(t0 + idx) * p.ldx + c] : tl[(size_t)(r + nt) * p.C + c];
        }
    }
}

struct DeltaRuleParams {
    const float* q; const float* k; const float* v; int ld;      // conv outputs: q, k [T, G * dk], v [T, H * dv], row stride ld
    const float* z; int ldz;                      // decay pre-activation [T, H * dk] (bias added)
    const float* b; int ldb;                      // write-strength logits [T, H]
    const float* gate; int ldgate;                // output-gate logits [T, H * dv]
    const float* a_log;                           // [H]
    const float* norm_w;                          // [dv]
    float* state;                                 // [S][H][dk][dv] of this layer
    float* out; int ldo;                          // [T, H * dv]
    int H, G, dk, dv;
    float q_scale, unit_eps, eps;
    MetaView meta;
};

__host__ __device__ inline size_t delta_rule_smem_bytes(int dk, int dv) { return ((size_t)dk * dv + 3 * (size_t)dk + 64) * sizeof(float); }

__global__ void delta_rule_kernel(const DeltaRuleParams p) {
    const int h = blockIdx.x, si = blockIdx.y;
    if (si >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[si], t0 = p.meta.slot_start()[si], nt = p.meta.slot_count()[si];
    const int dk = p.dk, dv = p.dv, j = threadIdx.x, hk = h / (p.H / p.G);
    const int nw = (blockDim.x + 31) >> 5;
    extern __shared__ __align__(16) float dr_smem[];
    float* S = dr_smem;                           // [dk][dv]
    float* sq = S + (size_t)dk * dv;              // [dk]
    float* sk = sq + dk;
    float* sg = sk + dk;
    float* red = sg + dk;                         // [2][32]
    float* gS = p.state + ((size_t)slot * p.H + h) * dk * dv;
    const int nst = dk * dv;
    const bool vec = (nst % 4) == 0;
    if (vec) {
#pragma unroll 8
        for (int e = j; e < nst / 4; e += blockDim.x) reinterpret_cast<float4*>(S)[e] = __ldg(reinterpret_cast<const float4*>(gS) + e);
    } else {
        for (int e = j; e < nst; e += blockDim.x) S[e] = gS[e];
    }
    const float rate = expf(p.a_log[h]);
    for (int t = t0; t < t0 + nt; ++t) {
        __syncthreads();
        float qq = 0.f, kk = 0.f;
        for (int i = j; i < dk; i += blockDim.x) {
            const float qv = p.q[(size_t)t * p.ld + (size_t)hk * dk + i], kv = p.k[(size_t)t * p.ld + (size_t)hk * dk + i];
            sq[i] = qv; sk[i] = kv;
            qq = fmaf(qv, qv, qq); kk = fmaf(kv, kv, kk);
            const float zz = p.z[(size_t)t * p.ldz + (size_t)h * dk + i];
            const float sp = fmaxf(zz, 0.f) + log1pf(expf(-fabsf(zz)));      // softplus
            sg[i] = expf(-rate * sp);
        }
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) { qq += __shfl_xor_sync(0xffffffffu, qq, of); kk += __shfl_xor_sync(0xffffffffu, kk, of); }
        if ((j & 31) == 0) { red[j >> 5] = qq; red[32 + (j >> 5)] = kk; }
        __syncthreads();
        qq = 0.f; kk = 0.f;
        for (int w = 0; w < nw; ++w) { qq += red[w]; kk += red[32 + w]; }
        const float qn = p.q_scale / sqrtf(qq + p.unit_eps), kn = 1.f / sqrtf(kk + p.unit_eps);
        const float bl = p.b[(size_t)t * p.ldb + h];
        const float beta = 1.f / (1.f + expf(-bl));
        float o = 0.f;
        if (j < dv) {
            const float vj = p.v[(size_t)t * p.ld + (size_t)h * dv + j];
            float sk_dot = 0.f;
            for (int i = 0; i < dk; ++i) {
                const float s = sg[i] * S[(size_t)i * dv + j];
                S[(size_t)i * dv + j] = s;
                sk_dot = fmaf(s, sk[i] * kn, sk_dot);
            }
            const float u = beta * (vj - sk_dot);
            for (int i = 0; i < dk; ++i) {
                const float s = fmaf(sk[i] * kn, u, S[(size_t)i * dv + j]);
                S[(size_t)i * dv + j] = s;
                o = fmaf(s, sq[i] * qn, o);
            }
        }
        float ss = j < dv ? o * o : 0.f;
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
        __syncthreads();                           // red has been read by every thread
        if ((j & 31) == 0) red[j >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < nw; ++w) ss += red[w];
        if (j < dv) {
            const float gl = p.gate[(size_t)t * p.ldgate + (size_t)h * dv + j];
            p.out[(size_t)t * p.ldo + (size_t)h * dv + j] = o / sqrtf(ss / (float)dv + p.eps) * p.norm_w[j] * (1.f / (1.f + expf(-gl)));
        }
    }
    __syncthreads();
    if (vec) {
#pragma unroll 8
        for (int e = j; e < nst / 4; e += blockDim.x) reinterpret_cast<float4*>(gS)[e] = reinterpret_cast<const float4*>(S)[e];
    } else {
        for (int e = j; e < nst; e += blockDim.x) gS[e] = S[e];
    }
}

// The same recurrence with the state column in REGISTERS (dk <= DKC <= 128, dv <= 256): thread j keeps S[0..dk)[j] for the whole
// step, so the two passes over the column are straight-line FMAs on registers fed by broadcast reads of q, k and g from shared
// memory (the shared-memory form above pays a load-after-store round trip per element).  Four partial sums shorten the
// dependency chains of the two dot products.
constexpr int DR_REG_MAX_DK = 128, DR_REG_MAX_DV = 256;

template <int DKC>
__global__ void __launch_bounds__(DR_REG_MAX_DV) delta_rule_reg_kernel(const DeltaRuleParams p) {
    const int h = blockIdx.x, si = blockIdx.y;
    if (si >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[si], t0 = p.meta.slot_start()[si], nt = p.meta.slot_count()[si];
    const int dk = p.dk, dv = p.dv, j = threadIdx.x, hk = h / (p.H / p.G);
    const int nw = (blockDim.x + 31) >> 5;
    __shared__ __align__(16) float sq[DKC], sk[DKC], sg[DKC];
    __shared__ float red[64];
    float* gS = p.state + ((size_t)slot * p.H + h) * dk * dv;
    float s[DKC];
#pragma unroll
    for (int i = 0; i < DKC; ++i) s[i] = (i < dk && j < dv) ? gS[(size_t)i * dv + j] : 0.f;
    const float rate = expf(p.a_log[h]);
    for (int t = t0; t < t0 + nt; ++t) {
        __syncthreads();
        float qq = 0.f, kk = 0.f;
        for (int i = j; i < DKC; i += blockDim.x) {
            float qv = 0.f, kv = 0.f, gv = 1.f;
            if (i < dk) {
                qv = p.q[(size_t)t * p.ld + (size_t)hk * dk + i]; kv = p.k[(size_t)t * p.ld + (size_t)hk * dk + i];
                const float zz = p.z[(size_t)t * p.ldz + (size_t)h * dk + i];
                gv = expf(-rate * (fmaxf(zz, 0.f) + log1pf(expf(-fabsf(zz)))));
            }
            sq[i] = qv; sk[i] = kv; sg[i] = gv;
            qq = fmaf(qv, qv, qq); kk = fmaf(kv, kv, kk);
        }
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) { qq += __shfl_xor_sync(0xffffffffu, qq, of); kk += __shfl_xor_sync(0xffffffffu, kk, of); }
        if ((j & 31) == 0) { red[j >> 5] = qq; red[32 + (j >> 5)] = kk; }
        __syncthreads();
        qq = 0.f; kk = 0.f;
        for (int w = 0; w < nw; ++w) { qq += red[w]; kk += red[32 + w]; }
        const float qn = p.q_scale / sqrtf(qq + p.unit_eps), kn = 1.f / sqrtf(kk + p.unit_eps);
        const float beta = 1.f / (1.f + expf(-p.b[(size_t)t * p.ldb + h]));
        float o = 0.f;
        if (j < dv) {
            const float vj = p.v[(size_t)t * p.ld + (size_t)h * dv + j];
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int i = 0; i < DKC; i += 4) {
                s[i] *= sg[i]; s[i + 1] *= sg[i + 1]; s[i + 2] *= sg[i + 2]; s[i + 3] *= sg[i + 3];
                d0 = fmaf(s[i], sk[i], d0); d1 = fmaf(s[i + 1], sk[i + 1], d1);
                d2 = fmaf(s[i + 2], sk[i + 2], d2); d3 = fmaf(s[i + 3], sk[i + 3], d3);
            }
            const float u = beta * (vj - ((d0 + d1) + (d2 + d3)) * kn) * kn;       // u * kn: the write is k_unit u^T
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int i = 0; i < DKC; i += 4) {
                s[i] = fmaf(sk[i], u, s[i]); s[i + 1] = fmaf(sk[i + 1], u, s[i + 1]);
                s[i + 2] = fmaf(sk[i + 2], u, s[i + 2]); s[i + 3] = fmaf(sk[i + 3], u, s[i + 3]);
                o0 = fmaf(s[i], sq[i], o0); o1 = fmaf(s[i + 1], sq[i + 1], o1);
                o2 = fmaf(s[i + 2], sq[i + 2], o2); o3 = fmaf(s[i + 3], sq[i + 3], o3);
            }
            o = ((o0 + o1) + (o2 + o3)) * qn;
        }
        float ss = j < dv ? o * o : 0.f;
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
        __syncthreads();                           // red has been read by every thread
        if ((j & 31) == 0) red[j >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < nw; ++w) ss += red[w];
        if (j < dv) {
            const float gl = p.gate[(size_t)t * p.ldgate + (size_t)h * dv + j];
            p.out[(size_t)t * p.ldo + (size_t)h * dv + j] = o / sqrtf(ss / (float)dv + p.eps) * p.norm_w[j] * (1.f / (1.f + expf(-gl)));
        }
    }
    if (j < dv) {
#pragma unroll
        for (int i = 0; i < DKC; ++i)
            if (i < dk) gS[(size_t)i * dv + j] = s[i];
    }
}

}  // namespace b200
