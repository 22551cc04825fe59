// Engine methods of the Zufulix family (see zufulix.cuh): weight upload and the launch sequence of the layer stack.  The step
// function, step metadata, cache pages, slot / snapshot interface and CUDA graphs are the ones of kemirax_engine.cuh.  Included
// by engine.cu after it.
#pragma once

using namespace b200;

// rows of one key / value head a warp of the attention kernel takes together: as many (of 4, 2, 1) as still leave a work item
// for each of 8 warps
static inline int zf_rows_per_warp(int gt, int G_, int rep_rows) {
    int rb = BA_RB;
    while (rb > 1 && std::min(gt, G_) * cdiv(rep_rows, rb) < 8) rb >>= 1;
    return rb;
}
typedef void (*BiasAttnKernel)(const BiasAttnParams);
static inline BiasAttnKernel zf_attn_kernel(int rb) {
    return rb >= 4 ? bias_attn_kernel<4> : (rb == 2 ? bias_attn_kernel<2> : bias_attn_kernel<1>);
}
static inline BiasAttnKernel zf_attn_reg_kernel(int rb) {
    return rb >= 4 ? bias_attn_reg_kernel<4> : (rb == 2 ? bias_attn_reg_kernel<2> : bias_attn_reg_kernel<1>);
}

// the stream kernel unrolled for up to 4, 8 or 16 streams, with large blocks for steps of few tokens
typedef void (*HcStepKernel)(const HcStepParams);
static inline HcStepKernel zf_hc_kernel(bool few, int ns) {
    if (few) return ns <= 4 ? hc_step_kernel<HC_THREADS_FEW_ROWS, 4> : (ns <= 8 ? hc_step_kernel<HC_THREADS_FEW_ROWS, 8> : hc_step_kernel<HC_THREADS_FEW_ROWS, HC_MAX_STREAMS>);
    return ns <= 4 ? hc_step_kernel<NORM_THREADS, 4> : (ns <= 8 ? hc_step_kernel<NORM_THREADS, 8> : hc_step_kernel<NORM_THREADS, HC_MAX_STREAMS>);
}

// how one attention launch of a layer runs: which kernel, its block size and shared memory, and the tile / split parameters
struct ZfAttnPlan { BiasAttnKernel kern; int threads; size_t smem; int gt, ks; };

static ZfAttnPlan zf_attn_plan(const KxLayer& l, int qb_prompt, bool decode) {
    const int H_ = l.c.heads, G_ = l.c.kv_heads, dk = l.c.dim, dv = l.c.vdim, qb = decode ? 1 : qb_prompt;
    const int rows = qb * (H_ / G_);               // rows of one key / value head in a full chunk
    ZfAttnPlan a;
    if (l.attn_reg) {
        const int rb = rows >= 4 ? 4 : (rows >= 2 ? 2 : 1);
        const int items = G_ * cdiv(rows, rb);
        int ks = 1;                                // few items (decode): the 8 warps share each item's key tiles
        while (ks < 8 && items * ks * 2 <= BAR_THREADS / 32) ks *= 2;
        a.kern = zf_attn_reg_kernel(rb); a.threads = BAR_THREADS; a.smem = bias_attn_reg_smem(qb, H_, G_, dv, rb, ks); a.gt = 1; a.ks = ks;
        return a;
    }
    const int gt = decode ? l.gt_decode : l.wa_gt;
    const int rb = zf_rows_per_warp(gt, G_, rows);
    // 16 warps where every warp finds a work item (some rows of one key / value head), 8 otherwise
    a.kern = zf_attn_kernel(rb); a.threads = std::min(gt, G_) * cdiv(rows, rb) >= 16 ? BA_THREADS : 256;
    a.smem = bias_attn_smem(qb, H_, dk, dv, gt); a.gt = gt; a.ks = 1;
    return a;
}

void b200rwkv_engine::zf_load(const StFile& st, KxSizes& z) {
    SeqModel& m = *kx;
    const int W = m.W, nl = (int)m.cfg.layers.size();
    const bool hc = m.cfg.streams > 0;
    const int NS = hc ? m.cfg.streams : 1;
    m.streams = NS;
    z.n_streams = (size_t)NS;
    m.embed = kx_up16(kx_host_bf16(st, "embed", m.V, W));
    m.head = m.embed;                              // the embedding table is the output matrix
    m.final_w = kx_up32(kx_host_f32(st, "final.norm", W));
    m.final_b = kx_up32(kx_host_f32(st, "final.norm.b", W));
    float* ones = kx_up32(std::vector<float>((size_t)NS * NS, 1.f));      // one stream: a = b = M = 1 is the plain residual
    m.layers.resize(nl);
    int first_vmix = -1;
    int qb = 4;
    for (int i = 0; i < nl; ++i) {
        KxLayer& l = m.layers[i];
        l.c = m.cfg.layers[i];
        const KxLayerCfg& c = l.c;
        const std::string p = "l" + std::to_string(i) + ".";
        const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim;
        REQUIRE(H_ >= 1 && dk >= 1 && dv >= 1, B200RWKV_ERR_INVALID, "config: bad mixer sizes");
        l.norm1_w = kx_up32(kx_host_f32(st, p + "norm1", W));
        l.norm1_b = kx_up32(kx_host_f32(st, p + "norm1.b", W));
        for (int q = 0; q < (c.has_mlp ? 2 : 1); ++q) {
            const std::string hp = p + "hc" + std::to_string(q + 1) + ".";
            l.hc_in[q] = hc ? kx_up32(kx_host_f32(st, hp + "in", NS)) : ones;
            l.hc_out[q] = hc ? kx_up32(kx_host_f32(st, hp + "out", NS)) : ones;
            l.hc_mix[q] = hc ? kx_up32(kx_host_f32(st, hp + "mix", (int64_t)NS * NS)) : ones;
        }
        {
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)H_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)G_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.v", (int64_t)G_ * dv, W));
            l.proj_n = H_ * dk + G_ * dk + G_ * dv;
            l.proj = kx_up16(w);
            auto b = kx_host_f32(st, p + "mix.q.b", (int64_t)H_ * dk);
            auto bk = kx_host_f32(st, p + "mix.k.b", (int64_t)G_ * dk);
            auto bv = kx_host_f32(st, p + "mix.v.b", (int64_t)G_ * dv);
            b.insert(b.end(), bk.begin(), bk.end());
            b.insert(b.end(), bv.begin(), bv.end());
            l.proj_b = kx_up32(b);
        }
        l.o = kx_up16(kx_host_bf16(st, p + "mix.o", W, (int64_t)H_ * dv));
        {
            const StTensor* rt = st.find(p + "mix.rel");
            REQUIRE(rt && rt->shape.size() == 2 && (int)rt->shape[1] == H_, B200RWKV_ERR_INVALID, "tensor " + p + "mix.rel has an unexpected shape");
            const int B_ = (int)rt->shape[0];
            l.rel_bias = kx_up32(zf_bias_table(kx_host_f32(st, p + "mix.rel", (int64_t)B_ * H_), B_, H_, c.bias_max, l.rel_n));
        }
        l.vmode = BA_V_PLAIN;
        if (c.v_mix) {
            if (first_vmix < 0) { first_vmix = i; l.vmode = BA_V_FIRST; }
            else {
                const KxLayerCfg& f = m.cfg.layers[first_vmix];
                REQUIRE(f.kv_heads == G_ && f.vdim == dv, B200RWKV_ERR_INVALID, "config: layers that blend values must agree in kv_heads and vdim");
                l.vmode = BA_V_BLEND;
                l.lam = kx_host_f32(st, p + "mix.vmix", 1)[0];
            }
            z.n_vf = std::max(z.n_vf, (size_t)G_ * dv);
        }
        if (c.has_mlp) {
            l.norm2_w = kx_up32(kx_host_f32(st, p + "norm2", W));
            l.norm2_b = kx_up32(kx_host_f32(st, p + "norm2.b", W));
            if (c.mlp_dense) {                     // one unit without a gate: kept where the other families keep their always-on unit
                l.sh_gu = kx_up16(kx_host_bf16(st, p + "mlp.up", c.ff, W));
                l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.down", W, c.ff));
                z.n_ys = std::max(z.n_ys, (size_t)c.ff);
            } else {
                const int E = c.experts, ff = c.ff;
                REQUIRE(E >= 1 && E <= 2048 && c.top >= 1 && c.top <= MOE_MAX_TOP && c.top <= E, B200RWKV_ERR_UNSUPPORTED,
                        "config: router sizes out of range (1 <= top <= 8, top <= experts <= 2048)");
                l.router = kx_up16(kx_host_bf16(st, p + "mlp.router", E, W));
                std::vector<uint16_t> up, dw;
                for (int e = 0; e < E; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    kx_cat(up, kx_host_bf16(st, q + "up", ff, W));
                    kx_cat(dw, kx_host_bf16(st, q + "down", W, ff));
                }
                l.gu = kx_up16(up); l.down = kx_up16(dw);
                z.n_yc = std::max(z.n_yc, (size_t)ff); z.n_rl = std::max(z.n_rl, (size_t)E);
                z.max_top = std::max(z.max_top, c.top); z.max_E = std::max(z.max_E, E);
            }
        }
        l.cache_D = G_ * (dk + dv);
        l.cache = (float*)dalloc((size_t)m.npages * m.page * l.cache_D * 4);
        l.attn_reg = dk % 4 == 0 && dv % 4 == 0 && dk <= 128 && dv <= 128;       // the register form of the attention kernel
        if (l.attn_reg) {
            while (qb > 1 && bias_attn_reg_smem(qb, H_, G_, dv, 4, 1) > 160 * 1024) qb /= 2;
        } else {
            while (qb > 1 && bias_attn_smem(qb, H_, dk, dv, 1) > 112 * 1024) qb /= 2;   // two CTAs per SM where the heads allow it
            REQUIRE(bias_attn_smem(1, H_, dk, dv, 1) <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "attention heads too large for shared memory");
        }
        z.n_pr = std::max(z.n_pr, (size_t)l.proj_n); z.n_q = std::max(z.n_q, (size_t)H_ * dk); z.n_vout = std::max(z.n_vout, (size_t)H_ * dv);
    }
    m.qb_prompt = qb;
    for (KxLayer& l : m.layers) {                  // as many key / value heads per tile load as fit beside the chunk's rows
        l.wa_gt = l.c.kv_heads;
        while (l.wa_gt > 1 && bias_attn_smem(qb, l.c.heads, l.c.dim, l.c.vdim, l.wa_gt) > 112 * 1024) l.wa_gt = (l.wa_gt + 1) / 2;
        // decode-shaped steps have few rows and few CTAs: one CTA per SM may take more heads per load
        l.gt_decode = l.c.kv_heads;
        while (l.gt_decode > 1 && bias_attn_smem(1, l.c.heads, l.c.dim, l.c.vdim, l.gt_decode) > 160 * 1024) l.gt_decode = (l.gt_decode + 1) / 2;
    }
    for (int rb = 1; rb <= BA_RB; rb *= 2) {
        CK(cudaFuncSetAttribute(zf_attn_kernel(rb), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        CK(cudaFuncSetAttribute(zf_attn_reg_kernel(rb), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    // the largest cluster the attention launch may ask for: what the device can co-schedule at this layer's shared memory
    m.max_split = 8;
    m.wa_ctas_prompt = m.wa_ctas_decode = 8;
    for (const KxLayer& l : m.layers) {
        const ZfAttnPlan pp = zf_attn_plan(l, qb, false), pd = zf_attn_plan(l, qb, true);
        REQUIRE(pp.smem <= 200 * 1024 && pd.smem <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "too many attention heads for shared memory");
        int cl = 8, cl_ok = 0;
        for (; cl > 1; cl >>= 1) {
            bool ok = true;
            for (const ZfAttnPlan* a : {&pp, &pd}) {
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
    REQUIRE((size_t)W * 4 <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "width too large for the stream kernel");
    for (int few = 0; few < 2; ++few)
        for (int ns : {4, 8, HC_MAX_STREAMS}) CK(cudaFuncSetAttribute(zf_hc_kernel(few != 0, ns), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
}

// the whole stack and the last norm: every sublayer boundary is one hc_step launch (write the finished sublayer's output into the
// streams, read + norm for the next one)
void b200rwkv_engine::zf_enqueue_layers(cudaStream_t s, int rows, int nslot_grid, bool decode, int nsplit, Profiler* prof) {
    SeqModel& m = *kx;
    const int W = m.W, NS = m.streams;
    MetaView mv{d_meta, maxT, S};
    const int* cntT = d_meta;
    auto lin = [&](const float* X, int ldx, const __nv_bfloat16* Wt, float* Y, int ldy, int N_, int K_, int epi = LE_STORE, const float* bias = nullptr) {
        LinParams p;
        memset(&p, 0, sizeof(p));
        p.X = X; p.ldx = ldx; p.W = Wt; p.Y = Y; p.ldy = ldy; p.N = N_; p.K = K_; p.cnt = cntT; p.epi = epi; p.bias = bias;
        return p;
    };
    struct Pending { const float* mix = nullptr; const float* out = nullptr; const float* y = nullptr; const float* rows = nullptr; int top = 0; };
    Pending pend;
    auto boundary = [&](int read, const float* rd_in, const float* ln_w, const float* ln_b, float* h, int compact, float* hidden) {
        HcStepParams hp{m.x, NS, W, pend.mix, pend.out, pend.y, pend.rows, m.row_of, m.wgt, pend.top, read, rd_in, ln_w, ln_b, m.cfg.eps,
                        h, compact, hidden, mv};
        const bool few = rows <= 32;
        launch_k(zf_hc_kernel(few, NS), dim3(rows), dim3(few ? HC_THREADS_FEW_ROWS : NORM_THREADS), (size_t)W * 4, hp, KC_LN, s, prof);
        pend = Pending();
    };
    for (size_t li = 0; li < m.layers.size(); ++li) {
        KxLayer& l = m.layers[li];
        const KxLayerCfg& c = l.c;
        const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim, PN = l.proj_n;
        boundary(HC_READ_MIX, l.hc_in[0], l.norm1_w, l.norm1_b, m.h, 0, nullptr);
        kx_lin(s, prof, lin(m.h, W, l.proj, m.pr, PN, PN, W, LE_STORE, l.proj_b), rows, 1);
        BiasAttnPrepParams ap{m.pr, m.pr + H_ * dk, m.pr + H_ * dk + G_ * dk, PN, m.q, H_ * dk, l.cache, m.d_table, m.npages, m.page,
                              m.vfirst, G_ * dv, l.vmode, l.lam, H_, G_, dk, dv, c.scale, m.cfg.eps, mv, m.sm};
        launch_k(bias_attn_prep_kernel, dim3(rows), dim3(128), 0, ap, KC_OTHER, s, prof);
        const int qb = decode ? 1 : m.qb_prompt;
        const ZfAttnPlan ap_ = zf_attn_plan(l, m.qb_prompt, decode);
        BiasAttnParams wp{m.q, H_ * dk, l.cache, m.d_table, m.npages, m.page, m.vout, H_ * dv, l.rel_bias, l.rel_n, H_, G_, dk, dv, qb, ap_.gt,
                          nsplit, ap_.ks, mv, m.sm};
        launch_cluster = nsplit;
        launch_k(ap_.kern, dim3((decode ? rows : cdiv(rows, qb) + nslot_grid) * nsplit), dim3(ap_.threads), ap_.smem, wp, KC_WKV, s, prof);
        kx_lin(s, prof, lin(m.vout, H_ * dv, l.o, m.y, W, W, H_ * dv), rows, 1);
        pend.mix = l.hc_mix[0]; pend.out = l.hc_out[0]; pend.y = m.y;
        if (c.has_mlp) {
            boundary(HC_READ_MIX, l.hc_in[1], l.norm2_w, l.norm2_b, m.h, 0, nullptr);
            if (c.mlp_dense) {
                kx_lin(s, prof, lin(m.h, W, l.sh_gu, m.ys, c.ff, c.ff, W, LE_GELU_ERF), rows, 1);
                kx_lin(s, prof, lin(m.ys, c.ff, l.sh_down, m.y, W, W, c.ff), rows, 1);
                pend.mix = l.hc_mix[1]; pend.out = l.hc_out[1]; pend.y = m.y;
            } else {
                const int E = c.experts, ff = c.ff;
                MoeRouteParams rp{m.h, W, l.router, W, nullptr, E, c.top, m.sel, m.wgt, mv, MOE_SIGMOID_GROUPS, c.groups, c.groups_keep};
                launch_k(moe_route_kernel, dim3(rows), dim3(MOE_ROUTE_THREADS), moe_route_smem(W, E), rp, KC_OTHER, s, prof);
                MoeGroupParams gp{m.sel, c.top, E, m.cnt, m.off, m.list, m.row_of, mv};
                launch_k(moe_group_kernel, dim3(1), dim3(256), ((size_t)E * 2 + (size_t)maxT * c.top) * 4, gp, KC_OTHER, s, prof);
                LinParams p1 = lin(m.h, W, l.gu, m.yc, ff, ff, W, LE_RELU_SQ);
                p1.w_gstride = (long long)ff * W; p1.cnt = m.cnt; p1.cnt_gstride = 1; p1.off = m.off; p1.xlist = m.list;
                kx_lin(s, prof, p1, rows, E);
                LinParams p2 = lin(m.yc, ff, l.down, m.dn, W, W, ff);
                p2.w_gstride = (long long)W * ff; p2.cnt = m.cnt; p2.cnt_gstride = 1; p2.off = m.off;
                kx_lin(s, prof, p2, rows, E);
                pend.mix = l.hc_mix[1]; pend.out = l.hc_out[1]; pend.rows = m.dn; pend.top = c.top;
            }
        }
        if (m.dbg_layers && !use_graph) {          // bring-up aid: the layer's output lands in the streams now, their sum is kept
            boundary(HC_READ_NONE, nullptr, nullptr, nullptr, nullptr, 0, nullptr);
            HcSumParams sp{m.x, m.dbg_layers + li * (size_t)maxT * W, NS, W, mv};
            launch_k(hc_sum_kernel, dim3(rows), dim3(NORM_THREADS), 0, sp, KC_LN, s, prof);
        }
    }
    boundary(HC_READ_SUM, nullptr, m.final_w, m.final_b, m.hn, 1, d_hidden);
}
