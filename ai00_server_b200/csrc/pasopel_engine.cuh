// Engine methods of the Pasopel family (see pasopel.cuh): weight upload, sequence memory of every layer run, and the launch
// sequence of the stack.  The step function, step metadata, cache pages, slot / snapshot interface and CUDA graphs are the ones
// of kemirax_engine.cuh.  Included by engine.cu after it.
#pragma once

using namespace b200;

typedef void (*SinkAttnKernel)(const SinkAttnParams);
static inline SinkAttnKernel ps_attn_kernel(int rb) {
    return rb >= 4 ? sink_attn_kernel<4> : (rb == 2 ? sink_attn_kernel<2> : sink_attn_kernel<1>);
}

// the attention launch sees every mixer as (H query heads, G key heads, key size, value size, value = leading part of the key?)
struct PsAttnShape { int H, G, dk, dv; bool valias; };
static inline PsAttnShape ps_attn_shape(const KxLayerCfg& c) {
    if (c.mixer == KX_LATENT) return {c.heads, 1, c.kv_rank + c.rot_dim, c.kv_rank, true};        // absorbed form: one shared row
    return {c.heads, c.kv_heads, c.dim, c.vdim, false};
}

// query heads per CTA: whole key heads, or a part of one key head's query heads; about `want`
static inline int ps_heads_per_cta(int H, int G, int want) {
    const int rep = H / G;
    want = std::max(1, std::min(want, H));
    if (G == 1) return want;
    if (rep >= want) {
        int d = want;
        while (rep % d) --d;
        return d;
    }
    return rep * (want / rep);
}

// the register form is built for key rows of one 512-byte piece per head.  (With three and five pieces, which the kernel's
// template allows, a decode step of a 576-float latent row took 120 us where the tile form takes 84: every piece's loads wait
// for the registers of the piece before it.)
static inline SinkAttnKernel ps_attn_reg_kernel(int rb) {
    return rb >= 4 ? sink_attn_reg_kernel<4, 1> : (rb == 2 ? sink_attn_reg_kernel<2, 1> : sink_attn_reg_kernel<1, 1>);
}

// how one attention launch of a layer runs: which kernel, its block size and shared memory, and the tile parameters
struct PsAttnPlan { SinkAttnKernel kern; int threads; size_t smem; int gt, nbuf, qb, ks, hb; };

static PsAttnPlan ps_attn_plan(const KxLayer& l, int qb_prompt, bool decode) {
    const PsAttnShape a = ps_attn_shape(l.c);
    const int rep = a.H / a.G, HB = decode ? l.sa_hb_decode : l.sa_hb;
    const int nhc = std::min(rep, HB), ncv = HB / nhc;
    PsAttnPlan p;
    p.hb = HB;
    if (l.sa_reg) {
        const int qb = decode ? 1 : qb_prompt, rows = qb * nhc;              // rows of one key head in a full chunk
        const int rb = rows >= 4 ? 4 : (rows >= 2 ? 2 : 1);
        const int items = ncv * cdiv(rows, rb);
        int ks = 1;                                // few items (decode): the 8 warps share each item's key tiles
        while (ks < 8 && items * ks * 2 <= SAR_THREADS / 32) ks *= 2;
        p.kern = ps_attn_reg_kernel(rb); p.threads = SAR_THREADS; p.smem = sink_attn_reg_smem(qb, HB, rep, a.dv, rb, ks);
        p.gt = 1; p.nbuf = 1; p.qb = qb; p.ks = ks;
        return p;
    }
    const int qb = decode ? 1 : l.sa_qb, rows = qb * nhc;
    const int gt = decode ? l.sa_gt_decode : l.sa_gt, nbuf = decode ? l.sa_nbuf_decode : l.sa_nbuf;
    // rows per warp: every key float a lane reads from the tile feeds one product per row, and the tile loop is bound by
    // shared-memory reads, so as many rows as still leave 4 warps an item (8 in decode-shaped
    int rb = SA_RB;
    while (rb > 1 && std::min(gt, ncv) * cdiv(rows, rb) < (decode ? 8 : 4)) rb >>= 1;    // steps, whose CTAs have an SM to themselves)
    p.kern = ps_attn_kernel(rb);
    p.threads = std::min(gt, ncv) * cdiv(rows, rb) >= 16 ? SA_THREADS : 256;
    p.smem = sink_attn_smem(qb, HB, a.dk, a.dv, gt, nbuf, a.valias);
    p.gt = gt; p.nbuf = nbuf; p.qb = qb; p.ks = 1;
    return p;
}

void b200rwkv_engine::ps_load(const StFile& st, KxSizes& z) {
    SeqModel& m = *kx;
    const int W = m.W, nr = (int)m.cfg.layers.size();
    auto plus_one = [](std::vector<float> v) { for (float& f : v) f += 1.f; return v; };     // norm weights are stored as offsets from one
    m.embed = kx_up16(kx_host_bf16(st, "embed", m.V, W));
    m.head = m.embed;                              // the embedding table is the output matrix
    m.final_w = kx_up32(plus_one(kx_host_f32(st, "final.norm", W)));
    int passes = 0, ntens = 0;
    for (const KxLayerCfg& c : m.cfg.layers) { passes = std::max(passes, c.opens_pass + 1); ntens = std::max(ntens, c.tensors_of + 1); }
    if (passes > 0) m.pass_vec = kx_up32(kx_host_f32(st, "loop.step", (int64_t)passes * W));
    // ---- tensors, once per layer of the file ----
    std::vector<KxLayer> own(ntens);
    std::vector<char> loaded(ntens, 0);
    for (const KxLayerCfg& c : m.cfg.layers) {
        const int i = c.tensors_of;
        if (loaded[i]) continue;
        loaded[i] = 1;
        KxLayer& l = own[i];
        l.c = c;
        const std::string p = "l" + std::to_string(i) + ".";
        const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim;
        REQUIRE(H_ >= 1 && dk >= 1 && dv >= 1, B200RWKV_ERR_INVALID, "config: bad mixer sizes");
        l.norm1_w = kx_up32(plus_one(kx_host_f32(st, p + "norm1", W)));
        l.sink = kx_up32(kx_host_f32(st, p + "mix.sink", H_));
        l.o = kx_up16(kx_host_bf16(st, p + "mix.o", W, (int64_t)H_ * dv));
        if (st.find(p + "mix.o.b")) l.o_b = kx_up32(kx_host_f32(st, p + "mix.o.b", W));
        if (c.mixer == KX_SINK) {
            REQUIRE(l.o_b, B200RWKV_ERR_INVALID, "missing tensor: " + p + "mix.o.b");
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)H_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)G_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.g", (int64_t)H_ * dv, W));
            l.conv_C = H_ * dk + G_ * dk;
            l.proj_n = l.conv_C + H_ * dv;
            l.proj = kx_up16(w);
            auto b = kx_host_f32(st, p + "mix.q.b", (int64_t)H_ * dk);
            auto bk = kx_host_f32(st, p + "mix.k.b", (int64_t)G_ * dk);
            b.insert(b.end(), bk.begin(), bk.end());
            b.resize((size_t)l.proj_n, 0.f);       // the gate has no bias
            l.proj_b = kx_up32(b);
            auto cw = kx_host_f32(st, p + "mix.q.conv", (int64_t)H_ * dk * c.taps);
            auto ck = kx_host_f32(st, p + "mix.k.conv", (int64_t)G_ * dk * c.taps);
            cw.insert(cw.end(), ck.begin(), ck.end());
            l.conv_w = kx_up32(cw);
        } else {
            const int dr = c.rot_dim, rk = c.kv_rank, D = rk + dr;
            auto w = kx_host_bf16(st, p + "mix.dq", c.q_rank, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.dkv", D, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.g", (int64_t)H_ * dv, W));
            l.proj_n = c.q_rank + D + H_ * dv;
            l.proj = kx_up16(w);
            l.dq_norm = kx_up32(kx_host_f32(st, p + "mix.dq.norm", c.q_rank));
            l.dkv_norm = kx_up32(kx_host_f32(st, p + "mix.dkv.norm", rk));
            l.uq = kx_up16(kx_host_bf16(st, p + "mix.uq", (int64_t)H_ * (dk + dr), c.q_rank));
            {   // W_uk [H * dk, rk] -> per head transposed [rk, dk]: the query's share of the score against the latent is a linear
                auto uk = kx_host_bf16(st, p + "mix.uk", (int64_t)H_ * dk, rk);
                std::vector<uint16_t> t(uk.size());
                for (int hh = 0; hh < H_; ++hh)
                    for (int d = 0; d < dk; ++d)
                        for (int r = 0; r < rk; ++r) t[((size_t)hh * rk + r) * dk + d] = uk[((size_t)hh * dk + d) * rk + r];
                l.ukT = kx_up16(t);
            }
            l.uv = kx_up16(kx_host_bf16(st, p + "mix.uv", (int64_t)H_ * dv, rk));
            std::vector<double> fr(std::max(c.rot.dims / 2, 1), 0.0);
            for (int f = 0; f < c.rot.dims / 2; ++f) fr[f] = std::pow(c.rot.base, -2.0 * f / c.rot.dims);
            l.freq_d = (double*)dalloc(fr.size() * 8, false);
            CK(cudaMemcpy(l.freq_d, fr.data(), fr.size() * 8, cudaMemcpyHostToDevice));
        }
        if (c.has_mlp) {
            l.norm2_w = kx_up32(plus_one(kx_host_f32(st, p + "norm2", W)));
            if (c.mlp_dense) {                     // one unit without a gate: kept where the other families keep their always-on unit
                l.sh_gu = kx_up16(kx_host_bf16(st, p + "mlp.up", c.ff, W));
                l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.down", W, c.ff));
            } else {
                const int E = c.experts, ff = c.ff;
                REQUIRE(E >= 1 && E <= 2048 && c.top >= 1 && c.top <= MOE_MAX_TOP && c.top <= E, B200RWKV_ERR_UNSUPPORTED,
                        "config: router sizes out of range (1 <= top <= 8, top <= experts <= 2048)");
                l.router = kx_up16(kx_host_bf16(st, p + "mlp.router", E, W));
                l.corr = kx_up32(kx_host_f32(st, p + "mlp.router.b", E));
                std::vector<uint16_t> gu, dw;
                for (int e = 0; e < E; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    kx_cat(gu, kx_interleave(kx_host_bf16(st, q + "gate", ff, W), kx_host_bf16(st, q + "up", ff, W), ff, W));
                    kx_cat(dw, kx_host_bf16(st, q + "down", W, ff));
                }
                l.gu = kx_up16(gu); l.down = kx_up16(dw);
                if (c.has_shared) {
                    l.sh_gu = kx_up16(kx_interleave(kx_host_bf16(st, p + "mlp.shared.gate", c.sff, W), kx_host_bf16(st, p + "mlp.shared.up", c.sff, W),
                                                    c.sff, W));
                    l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.shared.down", W, c.sff));
                }
            }
        }
    }
    // ---- the layer runs: the tensors of their layer, sequence memory of their own ----
    m.layers.resize(nr);
    const int qb = 4;                              // tokens per chunk of a prompt step; a layer whose rows do not fit takes a part of a chunk per CTA
    for (int r = 0; r < nr; ++r) {
        KxLayer& l = m.layers[r];
        l = own[m.cfg.layers[r].tensors_of];
        l.c = m.cfg.layers[r];
        const KxLayerCfg& c = l.c;
        const PsAttnShape a = ps_attn_shape(c);
        if (c.mixer == KX_SINK) {
            l.cache_D = a.G * (a.dk + a.dv);
            if (c.pool > 0) {
                l.prow = cdiv(m.page, c.pool);
                l.pcache = (float*)dalloc((size_t)m.npages * l.prow * l.cache_D * 4);
            }
            const size_t tail = (size_t)(c.taps - 1) * l.conv_C;
            l.conv_tail = (float*)dalloc(std::max<size_t>((size_t)S * tail, 1) * 4);
            l.fixed.push_back({l.conv_tail, tail});
            z.n_cv = std::max(z.n_cv, (size_t)l.conv_C); z.n_q = std::max(z.n_q, (size_t)a.H * a.dk);
        } else {
            l.cache_D = c.kv_rank + c.rot_dim;
            z.n_cq = std::max(z.n_cq, (size_t)c.q_rank); z.n_q = std::max(z.n_q, (size_t)a.H * (c.dim + c.rot_dim));
            z.n_qa = std::max(z.n_qa, (size_t)a.H * a.dk); z.n_olat = std::max(z.n_olat, (size_t)a.H * a.dv);
        }
        l.cache = (float*)dalloc((size_t)m.npages * m.page * l.cache_D * 4);
        z.n_pr = std::max(z.n_pr, (size_t)l.proj_n); z.n_vout = std::max(z.n_vout, (size_t)c.heads * c.vdim);
        if (c.has_mlp) {
            if (c.mlp_dense) z.n_ys = std::max(z.n_ys, (size_t)c.ff);
            else {
                z.n_yc = std::max(z.n_yc, (size_t)c.ff); z.n_rl = std::max(z.n_rl, (size_t)c.experts);
                z.max_top = std::max(z.max_top, c.top); z.max_E = std::max(z.max_E, c.experts);
                if (c.has_shared) z.n_ys = std::max(z.n_ys, (size_t)c.sff);
            }
        }
        // launch shape of the attention kernel: about 16 query heads per CTA, fewer (and then shorter chunks) where the rows of a
        // chunk would not fit into shared memory beside one tile
        // the register form takes key / value sizes that are multiples of four up to 128; longer rows (a latent) and odd sizes
        // go through shared-memory tiles
        l.sa_reg = a.dk % 4 == 0 && a.dv % 4 == 0 && l.cache_D % 4 == 0 && a.dk <= 128 && a.dv <= 128;
        l.sa_hb = ps_heads_per_cta(a.H, a.G, 16);
        l.sa_qb = qb;
        // tile form: rows (tokens x heads) per CTA such that two CTAs fit an SM beside one tile each (one loads while the other
        // multiplies); where that would leave fewer than four rows, one CTA per SM
        const int hb0 = l.sa_hb;
        for (size_t target : {(size_t)112 * 1024, (size_t)160 * 1024}) {
            if (l.sa_reg) break;
            l.sa_qb = qb; l.sa_hb = hb0;
            while (sink_attn_smem(l.sa_qb, l.sa_hb, a.dk, a.dv, 1, 1, a.valias) > target) {
                if (l.sa_qb > 1) l.sa_qb /= 2;
                else if (l.sa_hb > 1 && ps_heads_per_cta(a.H, a.G, l.sa_hb / 2) < l.sa_hb) l.sa_hb = ps_heads_per_cta(a.H, a.G, l.sa_hb / 2);
                else break;
            }
            if (sink_attn_smem(l.sa_qb, l.sa_hb, a.dk, a.dv, 1, 1, a.valias) <= target && l.sa_qb * l.sa_hb >= 4) break;
        }
        REQUIRE(l.sa_reg || sink_attn_smem(l.sa_qb, l.sa_hb, a.dk, a.dv, 1, 1, a.valias) <= 160 * 1024, B200RWKV_ERR_UNSUPPORTED,
                "attention heads too large for shared memory");
    }
    m.qb_prompt = qb;
    m.sa_ygroups = m.sa_ygroups_decode = 1 << 30;
    for (KxLayer& l : m.layers) {                  // as many key heads per tile load, and two tile buffers, where they fit
        const PsAttnShape a = ps_attn_shape(l.c);
        // decode-shaped steps have one row per head: the register form then takes one key head per CTA, so that a chunk's tiles
        // are spread over more warps
        l.sa_hb_decode = l.sa_reg ? ps_heads_per_cta(a.H, a.G, std::max(1, a.H / a.G)) : l.sa_hb;
        m.sa_ygroups = std::min(m.sa_ygroups, cdiv(a.H, l.sa_hb));
        m.sa_ygroups_decode = std::min(m.sa_ygroups_decode, cdiv(a.H, l.sa_hb_decode));
        for (int dec = 0; dec < 2; ++dec) {
            const int q = dec ? 1 : l.sa_qb;
            const int hb = dec ? l.sa_hb_decode : l.sa_hb, ncv = std::max(1, hb / std::max(1, a.H / a.G));
            int nbuf = 2, gt = ncv;
            if (sink_attn_smem(q, hb, a.dk, a.dv, 1, 2, a.valias) > (size_t)(dec ? 200 : 112) * 1024) nbuf = 1;
            while (gt > 1 && sink_attn_smem(q, hb, a.dk, a.dv, gt, nbuf, a.valias) > (dec ? 160 : 112) * 1024) gt = (gt + 1) / 2;
            (dec ? l.sa_gt_decode : l.sa_gt) = gt;
            (dec ? l.sa_nbuf_decode : l.sa_nbuf) = nbuf;
        }
    }
    for (int rb = 1; rb <= SA_RB; rb *= 2) {
        CK(cudaFuncSetAttribute(ps_attn_kernel(rb), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        CK(cudaFuncSetAttribute(ps_attn_reg_kernel(rb), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    // the largest cluster the attention launch may ask for: what the device can co-schedule at this layer's shared memory
    m.max_split = 8;
    m.wa_ctas_prompt = m.wa_ctas_decode = 8;
    for (const KxLayer& l : m.layers) {
        const PsAttnPlan pp = ps_attn_plan(l, qb, false), pd = ps_attn_plan(l, qb, true);
        REQUIRE(pp.smem <= 200 * 1024 && pd.smem <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "attention heads too large for shared memory");
        int cl = 8, cl_ok = 0;
        for (; cl > 1; cl >>= 1) {
            bool ok = true;
            for (const PsAttnPlan* a : {&pp, &pd}) {
                int lg = 0;
                while ((1 << lg) < cl) ++lg;
                cudaLaunchConfig_t cfg;
                memset(&cfg, 0, sizeof(cfg));
                cfg.gridDim = dim3(cl); cfg.blockDim = dim3(a->threads);
                cfg.dynamicSmemBytes = a->smem;
                cudaLaunchAttribute at;
                at.id = cudaLaunchAttributeClusterDimension;
                at.val.clusterDim.x = (unsigned)cl; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
                cfg.attrs = &at; cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, a->kern, &cfg) != cudaSuccess || n <= 0) { ok = false; n = 0; }
                cudaGetLastError();
                int& cap = (a == &pd ? m.cl_cap_decode : m.cl_cap_prompt)[lg];      // clusters of this size the GPU holds at once
                cap = std::min(cap, n);
            }
            if (ok && cl_ok == 0) cl_ok = cl;
        }
        m.max_split = std::min(m.max_split, std::max(cl_ok, 1));
        int np = 1, nd = 1;
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&np, pp.kern, pp.threads, pp.smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nd, pd.kern, pd.threads, pd.smem));
        m.wa_ctas_prompt = std::max(1, std::min(m.wa_ctas_prompt, np));
        m.wa_ctas_decode = std::max(1, std::min(m.wa_ctas_decode, nd));
    }
    REQUIRE((size_t)W * 4 <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "width too large for the norm kernel");
    CK(cudaFuncSetAttribute(pre_norm_kernel<NORM_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    CK(cudaFuncSetAttribute(pre_norm_kernel<PRE_NORM_THREADS_FEW_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
}

// block means of a sequence's first n tokens, rebuilt from its cache rows (after a state import)
void b200rwkv_engine::ps_repool(int slot, int n) {
    SeqModel& m = *kx;
    for (KxLayer& l : m.layers) {
        if (!l.pcache || n / l.c.pool == 0) continue;
        PoolWriteParams pw{l.cache, l.pcache, m.d_table, m.npages, m.page, l.cache_D, l.c.pool, l.prow, slot, n / l.c.pool, MetaView{d_meta, maxT, S}, m.sm};
        pool_rebuild_kernel<<<n / l.c.pool, 128, 0, stream>>>(pw);
        CK(cudaGetLastError());
    }
}

// the whole stack and the last norm: every sublayer begins with one pre_norm launch (the routed experts that just finished are
// combined into the residual there, a pass of the looped layers adds its vectors, the normed row is written)
void b200rwkv_engine::ps_enqueue_layers(cudaStream_t s, int rows, int nslot_grid, bool decode, int nsplit, Profiler* prof) {
    SeqModel& m = *kx;
    const int W = m.W;
    MetaView mv{d_meta, maxT, S};
    const int* cntT = d_meta;
    auto lin = [&](const float* X, int ldx, const __nv_bfloat16* Wt, float* Y, int ldy, int N_, int K_, int epi = LE_STORE, const float* bias = nullptr) {
        LinParams p;
        memset(&p, 0, sizeof(p));
        p.X = X; p.ldx = ldx; p.W = Wt; p.Y = Y; p.ldy = ldy; p.N = N_; p.K = K_; p.cnt = cntT; p.epi = epi; p.bias = bias;
        return p;
    };
    struct Pending { const float* rows = nullptr; int top = 0; const float* shared = nullptr; };
    Pending pend;
    auto boundary = [&](float* snap, const __nv_bfloat16* table, const float* vec, const float* weight, float* h, int compact, float* hidden) {
        PreNormParams pn{m.x, pend.rows, m.row_of, m.wgt, pend.top, pend.shared, snap, table, vec, weight, m.cfg.eps, h, compact, hidden, W, mv};
        if (rows <= 32) launch_k(pre_norm_kernel<PRE_NORM_THREADS_FEW_ROWS>, dim3(rows), dim3(PRE_NORM_THREADS_FEW_ROWS), (size_t)W * 4, pn, KC_LN, s, prof);
        else launch_k(pre_norm_kernel<NORM_THREADS>, dim3(rows), dim3(NORM_THREADS), (size_t)W * 4, pn, KC_LN, s, prof);
        pend = Pending();
    };
    const int chunks_grid = decode ? rows : cdiv(rows, m.qb_prompt) + nslot_grid;
    for (size_t li = 0; li < m.layers.size(); ++li) {
        KxLayer& l = m.layers[li];
        const KxLayerCfg& c = l.c;
        const int H_ = c.heads, dv = c.vdim, PN = l.proj_n;
        const PsAttnShape a = ps_attn_shape(c);
        const PsAttnPlan plan = ps_attn_plan(l, m.qb_prompt, decode);
        boundary(nullptr, c.opens_pass > 0 ? m.embed : nullptr, c.opens_pass >= 0 ? m.pass_vec + (size_t)c.opens_pass * W : nullptr, l.norm1_w, m.h, 0,
                 nullptr);
        kx_lin(s, prof, lin(m.h, W, l.proj, m.pr, PN, PN, W, LE_STORE, l.proj_b), rows, 1);
        SinkAttnParams sp;
        memset(&sp, 0, sizeof(sp));
        sp.cache = l.cache; sp.table = m.d_table; sp.stride = m.npages; sp.page = m.page; sp.D = l.cache_D;
        sp.sink = l.sink; sp.H = a.H; sp.G = a.G; sp.dk = a.dk; sp.dv = a.dv; sp.HB = plan.hb; sp.win = c.window;
        sp.qb = plan.qb; sp.gt = plan.gt; sp.cl = nsplit; sp.nbuf = plan.nbuf; sp.valias = a.valias ? 1 : 0; sp.ks = plan.ks;
        sp.nsub = decode ? 1 : m.qb_prompt / plan.qb;
        sp.meta = mv; sp.sm = m.sm;
        const dim3 attn_grid(chunks_grid * sp.nsub * nsplit, cdiv(a.H, plan.hb));
        if (c.mixer == KX_SINK) {
            const int G_ = c.kv_heads, dk = c.dim, C_ = l.conv_C;
            ShortConvParams cp{m.pr, PN, m.cv, C_, l.conv_w, l.conv_tail, C_, c.taps, mv, 0};
            launch_k(short_conv_kernel, dim3(rows, cdiv(C_, 256)), dim3(256), 0, cp, KC_OTHER, s, prof);
            if (c.taps > 1) launch_k(conv_commit_kernel, dim3(nslot_grid, cdiv(C_, 256)), dim3(256), 0, cp, KC_OTHER, s, prof);
            // unit-RMS queries (times the score scale) to the step buffer, unit-RMS keys and the keys as they are (the values) to the cache
            BiasAttnPrepParams ap{m.cv, m.cv + H_ * dk, m.cv + H_ * dk, C_, m.q, H_ * dk, l.cache, m.d_table, m.npages, m.page,
                                  m.vfirst, 0, BA_V_PLAIN, 0.f, H_, G_, dk, dv, c.scale, m.cfg.eps, mv, m.sm};
            launch_k(bias_attn_prep_kernel, dim3(rows), dim3(128), 0, ap, KC_OTHER, s, prof);
            if (c.pool > 0) {
                PoolWriteParams pw{l.cache, l.pcache, m.d_table, m.npages, m.page, l.cache_D, c.pool, l.prow, 0, 0, mv, m.sm};
                launch_k(pool_write_kernel, dim3(rows, cdiv(l.cache_D, 128)), dim3(128), 0, pw, KC_OTHER, s, prof);
            }
            sp.q = m.q; sp.ldq = H_ * dk; sp.pcache = l.pcache; sp.koff = 0; sp.voff = G_ * dk; sp.out = m.vout; sp.ldo = H_ * dv;
            sp.gate = m.pr + C_; sp.ldg = PN; sp.scale = 1.f; sp.pool = c.pool; sp.prow = l.prow;
            launch_cluster = nsplit;
            launch_k(plan.kern, attn_grid, dim3(plan.threads), plan.smem, sp, KC_WKV, s, prof);
        } else {
            const int dn = c.dim, dr = c.rot_dim, rk = c.kv_rank, D = rk + dr, QW = H_ * (dn + dr);
            RmsRowsParams rr{m.pr, PN, m.cq, c.q_rank, l.dq_norm, c.q_rank, 1, m.cfg.eps, cntT};
            launch_k(rms_rows_kernel, dim3(rows, 1), dim3(128), 0, rr, KC_LN, s, prof);
            kx_lin(s, prof, lin(m.cq, c.q_rank, l.uq, m.q, QW, QW, c.q_rank), rows, 1);
            RopeParams rp{m.q, QW, dn + dr, dn, m.qa, H_ * D, D, rk, H_, c.rot.dims, dr, nullptr, 1.f, mv, m.sm, l.freq_d};
            launch_k(rope_rows_kernel, dim3(rows), dim3(128), 0, rp, KC_OTHER, s, prof);
            {
                LinParams p = lin(m.q, QW, l.ukT, m.qa, H_ * D, rk, dn);
                p.x_gstride = dn + dr; p.w_gstride = (long long)rk * dn; p.y_gstride = D;
                kx_lin(s, prof, p, rows, H_);
            }
            KvWriteParams kw{m.pr + c.q_rank, PN, l.cache, m.d_table, m.npages, m.page, l.dkv_norm, rk, dr, c.rot.dims, nullptr, 1.f, m.cfg.eps, mv, m.sm,
                             l.freq_d};
            launch_k(kv_write_kernel, dim3(rows), dim3(128), 0, kw, KC_OTHER, s, prof);
            sp.q = m.qa; sp.ldq = H_ * D; sp.out = m.olat; sp.ldo = H_ * rk; sp.scale = c.scale;
            launch_cluster = nsplit;
            launch_k(plan.kern, attn_grid, dim3(plan.threads), plan.smem, sp, KC_WKV, s, prof);
            {   // values of every head from its weighted latent, through the output gate
                LinParams p = lin(m.olat, H_ * rk, l.uv, m.vout, H_ * dv, dv, rk, LE_MUL_SIGMOID);
                p.x_gstride = rk; p.w_gstride = (long long)dv * rk; p.y_gstride = dv;
                p.gate = m.pr + c.q_rank + D; p.ldg = PN; p.gate_gstride = dv;
                kx_lin(s, prof, p, rows, H_);
            }
        }
        kx_lin(s, prof, lin(m.vout, H_ * dv, l.o, m.x, W, W, H_ * dv, LE_ADD, l.o_b), rows, 1);
        if (c.has_mlp) {
            boundary(nullptr, nullptr, nullptr, l.norm2_w, m.h, 0, nullptr);
            if (c.mlp_dense) {
                kx_lin(s, prof, lin(m.h, W, l.sh_gu, m.ys, c.ff, c.ff, W, LE_RELU_SQ), rows, 1);
                kx_lin(s, prof, lin(m.ys, c.ff, l.sh_down, m.x, W, W, c.ff, LE_ADD), rows, 1);
            } else {
                const int E = c.experts, ff = c.ff;
                MoeRouteParams rp{m.h, W, l.router, W, l.corr, E, c.top, m.sel, m.wgt, mv, MOE_TOP_LOGITS};
                launch_k(moe_route_kernel, dim3(rows), dim3(MOE_ROUTE_THREADS), moe_route_smem(W, E), rp, KC_OTHER, s, prof);
                MoeGroupParams gp{m.sel, c.top, E, m.cnt, m.off, m.list, m.row_of, mv};
                launch_k(moe_group_kernel, dim3(1), dim3(256), ((size_t)E * 2 + (size_t)maxT * c.top) * 4, gp, KC_OTHER, s, prof);
                LinParams p1 = lin(m.h, W, l.gu, m.yc, ff, 2 * ff, W, LE_GLU_SILU);
                p1.w_gstride = (long long)2 * ff * W; p1.cnt = m.cnt; p1.cnt_gstride = 1; p1.off = m.off; p1.xlist = m.list;
                kx_lin(s, prof, p1, rows, E);
                LinParams p2 = lin(m.yc, ff, l.down, m.dn, W, W, ff);
                p2.w_gstride = (long long)W * ff; p2.cnt = m.cnt; p2.cnt_gstride = 1; p2.off = m.off;
                kx_lin(s, prof, p2, rows, E);
                if (c.has_shared) {
                    kx_lin(s, prof, lin(m.h, W, l.sh_gu, m.ys, c.sff, 2 * c.sff, W, LE_GLU_SILU), rows, 1);
                    kx_lin(s, prof, lin(m.ys, c.sff, l.sh_down, m.ds, W, W, c.sff), rows, 1);
                }
                pend.rows = m.dn; pend.top = c.top; pend.shared = c.has_shared ? m.ds : nullptr;
            }
        }
        if (m.dbg_layers && !use_graph) {          // bring-up aid: the residual as this run leaves it
            float* dst = m.dbg_layers + li * (size_t)maxT * W;
            if (pend.rows) boundary(dst, nullptr, nullptr, nullptr, nullptr, 0, nullptr);
            else CK(cudaMemcpyAsync(dst, m.x, (size_t)maxT * W * 4, cudaMemcpyDeviceToDevice, s));
        }
    }
    boundary(nullptr, nullptr, nullptr, m.final_w, m.hn, 1, d_hidden);
}
