// Engine methods of the Kemirax family (see kemirax.cuh): build, the per-step launch sequence, and the sequence memory
// behind the slot / snapshot interface.  Included by engine.cu after the engine struct.
#pragma once

namespace b200 {

static void kx_cat(std::vector<uint16_t>& a, const std::vector<uint16_t>& b) { a.insert(a.end(), b.begin(), b.end()); }
// (gate, up) -> rows interleaved so that outputs (2i, 2i+1) are one gated unit
static std::vector<uint16_t> kx_interleave(const std::vector<uint16_t>& gt, const std::vector<uint16_t>& upw, int ff, int K) {
    std::vector<uint16_t> o((size_t)2 * ff * K);
    for (int i = 0; i < ff; ++i) {
        memcpy(&o[(size_t)(2 * i) * K], &gt[(size_t)i * K], (size_t)K * 2);
        memcpy(&o[(size_t)(2 * i + 1) * K], &upw[(size_t)i * K], (size_t)K * 2);
    }
    return o;
}

static std::vector<uint16_t> kx_host_bf16(const StFile& st, const std::string& name, int64_t rows, int64_t cols) {
    const StTensor* t = st.find(name);
    REQUIRE(t, B200RWKV_ERR_INVALID, "missing tensor: " + name);
    REQUIRE(t->numel() == rows * cols, B200RWKV_ERR_INVALID, "tensor " + name + " has an unexpected shape");
    std::vector<uint16_t> v((size_t)(rows * cols));
    if (t->dtype == "BF16") {
        memcpy(v.data(), t->data, v.size() * 2);
    } else {
        for (size_t i = 0; i < v.size(); ++i) {
            const float f = st_elem_f32(*t, i);
            uint32_t u; memcpy(&u, &f, 4);
            u += 0x7FFFu + ((u >> 16) & 1u);
            v[i] = (uint16_t)(u >> 16);
        }
    }
    return v;
}

static std::vector<float> kx_host_f32(const StFile& st, const std::string& name, int64_t count) {
    const StTensor* t = st.find(name);
    REQUIRE(t, B200RWKV_ERR_INVALID, "missing tensor: " + name);
    REQUIRE(t->numel() == count, B200RWKV_ERR_INVALID, "tensor " + name + " has an unexpected shape");
    std::vector<float> v((size_t)count);
    for (size_t i = 0; i < v.size(); ++i) v[i] = st_elem_f32(*t, i);
    return v;
}

}  // namespace b200

using namespace b200;

__nv_bfloat16* b200rwkv_engine::kx_up16(const std::vector<uint16_t>& v) {
    __nv_bfloat16* d = (__nv_bfloat16*)dalloc(std::max<size_t>(v.size(), 1) * 2, false);
    if (!v.empty()) CK(cudaMemcpy(d, v.data(), v.size() * 2, cudaMemcpyHostToDevice));
    weight_bytes_total += v.size() * 2;
    return d;
}
float* b200rwkv_engine::kx_up32(const std::vector<float>& v) {
    float* d = (float*)dalloc(std::max<size_t>(v.size(), 1) * 4, false);
    if (!v.empty()) CK(cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    return d;
}

size_t SeqModel::flat_floats(int ctx_rows) const {
    size_t n = 4;                                          // [0] tokens held
    for (const KxLayer& l : layers) {
        for (const KxLayer::Block& b : l.fixed) n += b.per_slot;
        n += (size_t)ctx_rows * l.cache_D;
    }
    return n;
}

// tensors of a Kemirax model -> device, stacked / interleaved / transposed as the grouped launches want them
void b200rwkv_engine::kx_load(const StFile& st, KxSizes& z) {
    SeqModel& m = *kx;
    const int W = m.W, nl = (int)m.cfg.layers.size();
    m.embed = kx_up16(kx_host_bf16(st, "embed", m.V, W));
    m.head = kx_up16(kx_host_bf16(st, "head", m.V, W));
    m.final_gain = kx_host_f32(st, "final.norm", 1)[0];
    emb = nullptr;

    m.layers.resize(nl);
    for (int i = 0; i < nl; ++i) {
        KxLayer& l = m.layers[i];
        l.c = m.cfg.layers[i];
        const KxLayerCfg& c = l.c;
        const std::string p = "l" + std::to_string(i) + ".";
        l.gain = kx_host_f32(st, p + "norm1", 1)[0];
        l.mu = kx_up32(kx_host_f32(st, p + "shift", W));
        l.shift_state = (float*)dalloc((size_t)S * W * 4);
        l.fixed.push_back({l.shift_state, (size_t)W});
        {
            auto g = kx_host_bf16(st, p + "rg1", W, W);
            auto b = kx_host_f32(st, p + "rg1.b", W);
            if (c.has_mlp) {
                kx_cat(g, kx_host_bf16(st, p + "rg2", W, W));
                auto b2 = kx_host_f32(st, p + "rg2.b", W);
                b.insert(b.end(), b2.begin(), b2.end());
            }
            l.rg = kx_up16(g); l.rg_b = kx_up32(b);
        }
        REQUIRE(c.heads >= 1 && c.dim >= 1 && c.vdim >= 1, B200RWKV_ERR_INVALID, "config: bad mixer sizes");
        if (c.mixer == KX_LATENT) {
            const int H_ = c.heads, dn = c.dim, dr = c.rot_dim, dv = c.vdim, rk = c.kv_rank, D = rk + dr;
            REQUIRE(rk >= 1 && rk <= 32 * LA_MAX_RK_CHUNKS, B200RWKV_ERR_UNSUPPORTED, "kv_rank must be in 1..512");
            REQUIRE(c.rot.dims % 2 == 0 && c.rot.dims <= dr, B200RWKV_ERR_INVALID, "config: rot.dims must be even and <= rot_dim");
            REQUIRE((latent_attn_smem<1, 16>(D)) <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "kv_rank + rot_dim too large for the attention tile");
            l.dq = kx_up16(kx_host_bf16(st, p + "mix.dq", c.q_rank, W));
            l.dq_norm = kx_up32(kx_host_f32(st, p + "mix.dq.norm", c.q_rank));
            l.uq = kx_up16(kx_host_bf16(st, p + "mix.uq", (int64_t)H_ * (dn + dr), c.q_rank));
            {   // W_uk [H * dn, rk] -> per head transposed [rk, dn]: qa[h] = W_uk[h]^T q_plain[h] becomes a linear
                auto uk = kx_host_bf16(st, p + "mix.uk", (int64_t)H_ * dn, rk);
                std::vector<uint16_t> t(uk.size());
                for (int hh = 0; hh < H_; ++hh)
                    for (int d = 0; d < dn; ++d)
                        for (int r = 0; r < rk; ++r) t[((size_t)hh * rk + r) * dn + d] = uk[((size_t)hh * dn + d) * rk + r];
                l.ukT = kx_up16(t);
            }
            l.uv = kx_up16(kx_host_bf16(st, p + "mix.uv", (int64_t)H_ * dv, rk));
            l.o = kx_up16(kx_host_bf16(st, p + "mix.o", W, (int64_t)H_ * dv));
            std::vector<float> fr;
            kx_rot_table(c.rot, fr, l.mag);
            l.freq = kx_up32(fr);
            if (c.kv_from < 0) {
                l.dkv = kx_up16(kx_host_bf16(st, p + "mix.dkv", D, W));
                l.dkv_norm = kx_up32(kx_host_f32(st, p + "mix.dkv.norm", rk));
                l.cache = (float*)dalloc((size_t)m.npages * m.page * D * 4);
                l.cache_D = D;
            } else {
                REQUIRE(c.kv_from < i, B200RWKV_ERR_INVALID, "config: kv_from must name an earlier layer");
                const KxLayer& src = m.layers[c.kv_from];
                REQUIRE(src.c.mixer == KX_LATENT && src.c.kv_from < 0 && src.c.kv_rank == rk && src.c.rot_dim == dr, B200RWKV_ERR_INVALID,
                        "config: kv_from must name a latent-attention layer with its own cache of the same shape");
                l.cache = src.cache;
            }
            z.n_cq = std::max(z.n_cq, (size_t)c.q_rank); z.n_q = std::max(z.n_q, (size_t)H_ * (dn + dr)); z.n_qa = std::max(z.n_qa, (size_t)H_ * D);
            z.n_kv = std::max(z.n_kv, (size_t)D); z.n_part = std::max(z.n_part, (size_t)H_ * m.max_split * (rk + 2));
            z.n_olat = std::max(z.n_olat, (size_t)H_ * rk); z.n_vout = std::max(z.n_vout, (size_t)H_ * dv);
            m.max_D = std::max(m.max_D, D);
        } else {
            const int H_ = c.heads, dk = c.dim, dv = c.vdim;
            REQUIRE(dv <= 1024, B200RWKV_ERR_UNSUPPORTED, "gla vdim must be <= 1024");
            REQUIRE(gla_smem_bytes(dk, dv) <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "gla head state too large for shared memory");
            const StTensor* a1 = st.find(p + "mix.a1");
            REQUIRE(a1 && a1->shape.size() == 2, B200RWKV_ERR_INVALID, "missing tensor: " + p + "mix.a1");
            l.a_rank = (int)a1->shape[0];
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)H_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)H_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.v", (int64_t)H_ * dv, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.g", (int64_t)H_ * dv, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.a1", l.a_rank, W));
            l.proj_n = 2 * H_ * dk + 2 * H_ * dv + l.a_rank;
            l.proj = kx_up16(w);
            l.a2 = kx_up16(kx_host_bf16(st, p + "mix.a2", (int64_t)H_ * dk, l.a_rank));
            l.a2_b = kx_up32(kx_host_f32(st, p + "mix.a2.b", (int64_t)H_ * dk));
            l.norm_w = kx_up32(kx_host_f32(st, p + "mix.norm", dv));
            l.o = kx_up16(kx_host_bf16(st, p + "mix.o", W, (int64_t)H_ * dv));
            l.gla_state = (float*)dalloc((size_t)S * H_ * dk * dv * 4);
            l.fixed.push_back({l.gla_state, (size_t)H_ * dk * dv});
            z.n_pr = std::max(z.n_pr, (size_t)l.proj_n); z.n_z = std::max(z.n_z, (size_t)H_ * dk); z.n_vout = std::max(z.n_vout, (size_t)H_ * dv);
        }
        if (c.has_mlp) {
            const int E = c.experts, NE = E + c.identity, ff = c.ff;
            REQUIRE(c.top >= 1 && c.top <= MOE_MAX_TOP && c.top <= NE && E >= 0 && NE >= 1 && NE <= 2048, B200RWKV_ERR_UNSUPPORTED,
                    "config: router sizes out of range (top <= 8, outputs <= 2048)");
            l.router = kx_up16(kx_host_bf16(st, p + "mlp.router", NE, W));
            if (st.find(p + "mlp.correction")) l.corr = kx_up32(kx_host_f32(st, p + "mlp.correction", NE));
            if (E > 0) {
                std::vector<uint16_t> gu, dw;
                for (int e = 0; e < E; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    kx_cat(gu, kx_interleave(kx_host_bf16(st, q + "gate", ff, W), kx_host_bf16(st, q + "up", ff, W), ff, W));
                    kx_cat(dw, kx_host_bf16(st, q + "down", W, ff));
                }
                l.gu = kx_up16(gu); l.down = kx_up16(dw);
            }
            if (c.has_shared) {
                l.sh_gu = kx_up16(kx_interleave(kx_host_bf16(st, p + "mlp.shared.gate", c.sff, W), kx_host_bf16(st, p + "mlp.shared.up", c.sff, W), c.sff, W));
                l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.shared.down", W, c.sff));
                l.sg = kx_up16(kx_host_bf16(st, p + "mlp.shared.sg", 1, W));
                z.n_ys = std::max(z.n_ys, (size_t)c.sff);
            }
            z.n_rl = std::max(z.n_rl, (size_t)NE); z.n_yc = std::max(z.n_yc, (size_t)ff);
            z.max_top = std::max(z.max_top, c.top); z.max_E = std::max(z.max_E, std::max(E, 1));
        }
    }

}

void b200rwkv_engine::kx_build(const StFile& st, const char* cfg_json, size_t cfg_len) {
    kx.reset(new SeqModel());
    SeqModel& m = *kx;
    m.cfg = kx_parse_config(cfg_json, cfg_len);
    m.exact = precision == 1;
    m.W = m.cfg.width; m.V = m.cfg.vocab;
    const int W = m.W, nl = (int)m.cfg.layers.size();
    memset(&info, 0, sizeof(info));
    info.version = m.cfg.family == KX_FAMILY_PASOPEL ? B200RWKV_ARCH_PASOPEL
                   : m.cfg.family == KX_FAMILY_ZUFULIX ? B200RWKV_ARCH_ZUFULIX
                   : (m.cfg.family == KX_FAMILY_DEGAVIK ? B200RWKV_ARCH_DEGAVIK : B200RWKV_ARCH_KEMIRAX); info.num_layer = nl; info.num_emb = W; info.num_vocab = m.V;
    L = nl; C = W; V = m.V; Vl = V; Cl = C; H = Hl = 0; N = 0; F = Fl = 0;
    REQUIRE(world == 1, B200RWKV_ERR_UNSUPPORTED, "models that come with a config.json run on one GPU in this version");
    REQUIRE(quant_layers == 0 && loras.empty(), B200RWKV_ERR_UNSUPPORTED, "models that come with a config.json take no LoRA / quantised layers");
    use_pdl = false;                                       // these kernels carry no programmatic-dependency waits
    // steps of up to 512 tokens when the caller's token_chunk_size asks for them (prompts then stream the weights once per 512
    // tokens and fill the experts' row tiles); 128 otherwise, like the other families
    maxT = chunk > 256 ? 512 : (chunk > 128 ? 256 : 128);
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&sm_stream, cudaStreamNonBlocking));
    CK(cudaEventCreateWithFlags(&step_done, cudaEventDisableTiming));
    for (auto& ev : meta_ev) CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));

    // ---- step metadata: the common block, then positions / attention chunks / page-table updates ----
    const size_t mv_ints = MetaView::ints(maxT, S);
    meta_ints = mv_ints + SeqMeta::ints(maxT);
    d_meta = (int*)dalloc(meta_ints * 4);
    CK(cudaMallocHost(&h_meta, meta_ints * 4 * META_RING));
    memset(h_meta, 0, meta_ints * 4 * META_RING);
    m.sm = SeqMeta{d_meta + mv_ints, maxT};

    // ---- pages ----
    m.page = kv_page > 0 ? kv_page : 64;
    const long long want_tokens = kv_tokens > 0 ? kv_tokens : (long long)S * 4096;
    m.npages = (int)((want_tokens + m.page - 1) / m.page) + S;          // every sequence may hold one partly filled page
    m.state_ctx = (int)std::min<long long>((long long)m.npages * m.page, 8192);
    m.d_table = (int*)dalloc((size_t)S * m.npages * 4);
    m.pos.assign(S, 0);
    m.pages.assign(S, {});
    for (int i = m.npages - 1; i >= 0; --i) m.free_pages.push_back(i);

    KxSizes z;
    if (m.cfg.family == KX_FAMILY_PASOPEL) ps_load(st, z);
    else if (m.cfg.family == KX_FAMILY_ZUFULIX) zf_load(st, z);
    else if (m.cfg.family == KX_FAMILY_DEGAVIK) dg_load(st, z);
    else kx_load(st, z);
    emb = nullptr;

    // ---- activations (maxT rows each) ----
    const size_t T_ = (size_t)maxT;
    auto fa = [&](size_t n) { return (float*)dalloc(n * 4); };
    m.x = fa(T_ * W * z.n_streams); m.h = fa(T_ * W); m.hs = fa(T_ * W); m.G = fa(T_ * 2 * W); m.hn = fa(T_ * W);
    m.cq = fa(T_ * z.n_cq); m.q = fa(T_ * z.n_q); m.qa = fa(T_ * z.n_qa); m.kv = fa(T_ * z.n_kv); m.part = fa(T_ * z.n_part);
    m.olat = fa(T_ * z.n_olat); m.vout = fa(T_ * z.n_vout); m.pr = fa(T_ * z.n_pr); m.z = fa(T_ * z.n_z);
    m.rl = fa(T_ * z.n_rl); m.wgt = fa(T_ * z.max_top); m.yc = fa(T_ * z.max_top * z.n_yc); m.dn = fa(T_ * z.max_top * W);
    m.ys = fa(T_ * z.n_ys); m.ds = fa(T_ * W);
    m.y = fa(T_ * W); m.cv = fa(T_ * z.n_cv); m.gl = fa(T_ * z.n_gl); m.vfirst = fa(T_ * z.n_vf);
    m.lin_ws_floats = (size_t)4 << 20;                   // split-k partial sums of one projection launch
    m.lin_ws = fa(m.lin_ws_floats);
    m.sel = (int*)dalloc(T_ * z.max_top * 4); m.row_of = (int*)dalloc(T_ * z.max_top * 4); m.list = (int*)dalloc(T_ * z.max_top * 4);
    m.cnt = (int*)dalloc((size_t)z.max_E * 4); m.off = (int*)dalloc((size_t)z.max_E * 4);
    d_hidden = fa(T_ * W);
    d_logits = fa(T_ * V);
    d_api = fa(m.flat_floats(m.state_ctx));
    x_a = m.x;

    // ---- logits rows kept for sampling (sample.cuh) ----
    keep_valid.assign(S, 0);
    d_keep = (float*)dalloc((size_t)S * V * 4);
    {
        const int nseg = cdiv(V, TOPK_SEG);
        if (nseg <= TOPK_MAX_SEGS) {
            tk_cand_x = (float*)dalloc((size_t)S * nseg * TOPK_MAX * 4);
            tk_cand_id = (unsigned*)dalloc((size_t)S * nseg * TOPK_MAX * 4);
            tk_stats = (float2*)dalloc((size_t)S * nseg * 8);
            tk_out_id = (unsigned*)dalloc((size_t)S * TOPK_MAX * 4);
            tk_out_p = (float*)dalloc((size_t)S * TOPK_MAX * 4);
        }
    }
    comm_base = (uint8_t*)d_logits; off_logits = 0;       // the keep-rows gather reads the (single) logits shard from here
    peer_base[0] = comm_base;
    connected = true;

    if (m.max_D > 0) {
        const int smem = (int)latent_attn_smem<1, 16>(m.max_D);
        CK(cudaFuncSetAttribute(latent_attn_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CK(cudaFuncSetAttribute(latent_attn_kernel<1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        CK(cudaFuncSetAttribute(latent_attn_kernel<1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        const int smem_tc = (int)latent_attn_tc_smem(m.max_D);
        CK(cudaFuncSetAttribute(latent_attn_tc_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tc));
        CK(cudaFuncSetAttribute(latent_attn_tc_kernel<1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tc));
        CK(cudaFuncSetAttribute(latent_attn_tc_kernel<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tc));
    }
    CK(cudaFuncSetAttribute(gla_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    CK(cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    REQUIRE(moe_route_smem(W, 2048) <= 128 * 1024, B200RWKV_ERR_UNSUPPORTED, "width too large for the router kernel");
    CK(cudaFuncSetAttribute(lin_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LIN_TC_SMEM));
    CK(cudaDeviceSynchronize());
}

// one grouped linear launch; `rows` bounds the row count of any group (the step's bucket)
void b200rwkv_engine::kx_lin(cudaStream_t s, Profiler* prof, LinParams p, int rows, int groups, bool force_exact) {
    p.max_rows = rows;
    const bool exact = kx->exact || force_exact;
    if (!exact && rows <= 16) {
        launch_k(lin_mma16_kernel, dim3(cdiv(p.N, LIN_M16_BN), 1, groups), dim3(LIN_M16_WARPS * 32), 0, p, KC_GEMM, s, prof);
    } else if (rows <= LIN_SK_ROWS || (exact && rows <= 16)) {
        launch_k(lin_skinny_kernel, dim3(cdiv(p.N, 2 * LIN_SK_WARPS), 1, groups), dim3(LIN_SK_WARPS * 32), 0, p, KC_GEMM, s, prof);
    } else if (exact) {
        launch_k(lin_tile_kernel<true>, dim3(cdiv(p.N, LIN_BN), cdiv(rows, LIN_BM), groups), dim3(LIN_THREADS), 0, p, KC_GEMM, s, prof);
    } else {
        const int ctas = cdiv(p.N, LIN_BN) * cdiv(rows, LIN_BM), nslab = cdiv(p.K, LIN_TC_BK);
        int ks = 1;
        if (groups == 1 && !p.off && !p.xlist && p.cnt_gstride == 0)
            while (ks < 8 && ctas * ks * 2 <= 2 * num_sms && nslab / (ks * 2) >= 4 && (size_t)ks * 2 * rows * p.N <= kx->lin_ws_floats) ks *= 2;
        if (ks > 1) { p.ksplit = ks; p.ws = kx->lin_ws; }
        launch_k(lin_tile_kernel<false>, dim3(cdiv(p.N, LIN_BN) * ks, cdiv(rows, LIN_BM), groups), dim3(LIN_THREADS), LIN_TC_SMEM, p, KC_GEMM, s, prof);
        if (ks > 1) launch_k(lin_splitk_finish_kernel, dim3(cdiv(p.N, 512), rows), dim3(256), 0, p, KC_GEMM, s, prof);
    }
}

void b200rwkv_engine::kx_enqueue_step(cudaStream_t s, int rows, int rrows, bool decode, int nsplit, Profiler* prof) {
    launches_last_step = 0;
    SeqModel& m = *kx;
    const int W = m.W;
    MetaView mv{d_meta, maxT, S};
    const int* cntT = d_meta;            // T
    const int* cntR = d_meta + 2;        // R
    auto lin = [&](const float* X, int ldx, const __nv_bfloat16* Wt, float* Y, int ldy, int N_, int K_, int epi = LE_STORE,
                   const float* bias = nullptr, bool force_exact = false) {
        LinParams p;
        memset(&p, 0, sizeof(p));
        p.X = X; p.ldx = ldx; p.W = Wt; p.Y = Y; p.ldy = ldy; p.N = N_; p.K = K_; p.cnt = cntT; p.epi = epi; p.bias = bias;
        return p;
    };
    {
        PageUpdateParams pu{m.sm, m.d_table, m.npages};
        launch_k(page_update_kernel, dim3(1), dim3(128), 0, pu, KC_OTHER, s, prof);
        EmbedRowsParams ep{m.embed, m.x, W, mv, m.cfg.embed_scale, m.streams};
        launch_k(embed_rows_kernel, dim3(rows), dim3(NORM_THREADS), 0, ep, KC_LN, s, prof);
    }
    const int nslot_grid = std::min(S, rows);
    const bool own_stack = m.cfg.family == KX_FAMILY_ZUFULIX || m.cfg.family == KX_FAMILY_PASOPEL;    // these end with the last norm
    if (m.cfg.family == KX_FAMILY_ZUFULIX) zf_enqueue_layers(s, rows, nslot_grid, decode, nsplit, prof);
    if (m.cfg.family == KX_FAMILY_PASOPEL) ps_enqueue_layers(s, rows, nslot_grid, decode, nsplit, prof);
    for (size_t li = 0; li < m.layers.size() && !own_stack; ++li) {
        KxLayer& l = m.layers[li];
        const KxLayerCfg& c = l.c;
        if (m.cfg.family == KX_FAMILY_DEGAVIK) {
            dg_enqueue_layer(s, l, rows, nslot_grid, decode, nsplit, prof);
            if (m.dbg_layers && !use_graph)
                CK(cudaMemcpyAsync(m.dbg_layers + li * (size_t)maxT * W, m.x, (size_t)maxT * W * 4, cudaMemcpyDeviceToDevice, s));
            continue;
        }
        NormShiftParams ns{m.x, m.h, m.hs, l.mu, l.shift_state, l.gain, m.cfg.eps, W, mv};
        launch_k(norm_shift_kernel, dim3(rows), dim3(NORM_THREADS), 0, ns, KC_LN, s, prof);
        launch_k(shift_commit_kernel, dim3(nslot_grid), dim3(NORM_THREADS), 0, ns, KC_LN, s, prof);
        const int GW = c.has_mlp ? 2 * W : W;
        kx_lin(s, prof, lin(m.h, W, l.rg, m.G, GW, GW, W, LE_SIGMOID, l.rg_b), rows, 1);
        if (c.mixer == KX_LATENT) {
            const int H_ = c.heads, dn = c.dim, dr = c.rot_dim, dv = c.vdim, rk = c.kv_rank, D = rk + dr, QW = H_ * (dn + dr);
            kx_lin(s, prof, lin(m.hs, W, l.dq, m.cq, c.q_rank, c.q_rank, W), rows, 1);
            RmsRowsParams rr{m.cq, c.q_rank, m.cq, c.q_rank, l.dq_norm, c.q_rank, 1, m.cfg.eps, cntT};
            launch_k(rms_rows_kernel, dim3(rows, 1), dim3(128), 0, rr, KC_LN, s, prof);
            kx_lin(s, prof, lin(m.cq, c.q_rank, l.uq, m.q, QW, QW, c.q_rank), rows, 1);
            RopeParams rp{m.q, QW, dn + dr, dn, m.qa, H_ * D, D, rk, H_, c.rot.dims, dr, l.freq, l.mag, mv, m.sm};
            launch_k(rope_rows_kernel, dim3(rows), dim3(128), 0, rp, KC_OTHER, s, prof);
            {
                LinParams p = lin(m.q, QW, l.ukT, m.qa, H_ * D, rk, dn);
                p.x_gstride = dn + dr; p.w_gstride = (long long)rk * dn; p.y_gstride = D;
                kx_lin(s, prof, p, rows, H_);
            }
            if (c.kv_from < 0) {
                kx_lin(s, prof, lin(m.hs, W, l.dkv, m.kv, D, D, W), rows, 1);
                KvWriteParams kw{m.kv, D, l.cache, m.d_table, m.npages, m.page, l.dkv_norm, rk, dr, c.rot.dims, l.freq, l.mag, m.cfg.eps, mv, m.sm};
                launch_k(kv_write_kernel, dim3(rows), dim3(128), 0, kw, KC_OTHER, s, prof);
            }
            LatentAttnParams ap{m.qa, l.cache, m.d_table, m.npages, m.page, m.part, H_, rk, dr, nsplit, c.scale, mv, m.sm};
            if (!m.exact) {         // serving precision: both products on the tensor cores (TF32 operands, f32 accumulation and softmax)
                const size_t sm_b = latent_attn_tc_smem(D);
                if (!decode) launch_k(latent_attn_tc_kernel<4, 4>, dim3(cdiv(rows, 4) + nslot_grid, cdiv(H_, 4), nsplit), dim3(LA_THREADS), sm_b, ap, KC_WKV, s, prof);
                else if (H_ > 8) launch_k(latent_attn_tc_kernel<1, 16>, dim3(rows, cdiv(H_, 16), nsplit), dim3(LA_THREADS), sm_b, ap, KC_WKV, s, prof);
                else launch_k(latent_attn_tc_kernel<2, 8>, dim3(rows, cdiv(H_, 8), nsplit), dim3(LA_THREADS), sm_b, ap, KC_WKV, s, prof);
            } else if (!decode) {
                launch_k(latent_attn_kernel<4, 4>, dim3(cdiv(rows, 4) + nslot_grid, cdiv(H_, 4), nsplit), dim3(LA_THREADS), latent_attn_smem<4, 4>(D), ap,
                         KC_WKV, s, prof);
            } else if (H_ > 8) {
                launch_k(latent_attn_kernel<1, 16>, dim3(rows, cdiv(H_, 16), nsplit), dim3(LA_THREADS), latent_attn_smem<1, 16>(D), ap, KC_WKV, s, prof);
            } else {
                launch_k(latent_attn_kernel<1, 8>, dim3(rows, cdiv(H_, 8), nsplit), dim3(LA_THREADS), latent_attn_smem<1, 8>(D), ap, KC_WKV, s, prof);
            }
            LatentMergeParams mp{m.part, m.olat, H_, rk, nsplit, mv};
            launch_k(latent_merge_kernel, dim3(rows, H_), dim3(128), 0, mp, KC_WKV, s, prof);
            {
                LinParams p = lin(m.olat, H_ * rk, l.uv, m.vout, H_ * dv, dv, rk);
                p.x_gstride = rk; p.w_gstride = (long long)dv * rk; p.y_gstride = dv;
                kx_lin(s, prof, p, rows, H_);
            }
            LinParams po = lin(m.vout, H_ * dv, l.o, m.x, W, W, H_ * dv, LE_GATED_ADD);
            po.gate = m.G; po.ldg = GW;
            kx_lin(s, prof, po, rows, 1);
        } else {
            const int H_ = c.heads, dk = c.dim, dv = c.vdim;
            kx_lin(s, prof, lin(m.hs, W, l.proj, m.pr, l.proj_n, l.proj_n, W), rows, 1);
            kx_lin(s, prof, lin(m.pr + 2 * H_ * dk + 2 * H_ * dv, l.proj_n, l.a2, m.z, H_ * dk, H_ * dk, l.a_rank, LE_STORE, l.a2_b), rows, 1);
            GlaParams gp{m.pr, m.pr + H_ * dk, m.pr + 2 * H_ * dk, m.pr + 2 * H_ * dk + H_ * dv, l.proj_n, m.z, H_ * dk, l.gla_state, m.vout, H_ * dv,
                         l.norm_w, H_, dk, dv, 1.f / c.tau, 1.f / sqrtf((float)dk), m.cfg.eps, mv};
            launch_k(gla_kernel, dim3(H_, nslot_grid), dim3(rup(dv, 32)), gla_smem_bytes(dk, dv), gp, KC_WKV, s, prof);
            LinParams po = lin(m.vout, H_ * dv, l.o, m.x, W, W, H_ * dv, LE_GATED_ADD);
            po.gate = m.G; po.ldg = GW;
            kx_lin(s, prof, po, rows, 1);
        }
        if (c.has_mlp) {
            const int E = c.experts, NE = E + c.identity, ff = c.ff;
            MoeRouteParams rp{m.h, W, l.router, W, l.corr, NE, c.top, m.sel, m.wgt, mv};
            launch_k(moe_route_kernel, dim3(rows), dim3(MOE_ROUTE_THREADS), moe_route_smem(W, NE), rp, KC_OTHER, s, prof);
            MoeGroupParams gp{m.sel, c.top, E, m.cnt, m.off, m.list, m.row_of, mv};
            launch_k(moe_group_kernel, dim3(1), dim3(256), ((size_t)std::max(E, 1) * 2 + (size_t)maxT * c.top) * 4, gp, KC_OTHER, s, prof);
            if (E > 0) {
                LinParams p1 = lin(m.h, W, l.gu, m.yc, ff, 2 * ff, W, LE_GLU_CLAMP);
                p1.w_gstride = (long long)2 * ff * W; p1.cnt = m.cnt; p1.cnt_gstride = 1; p1.off = m.off; p1.xlist = m.list; p1.limit = c.limit;
                kx_lin(s, prof, p1, rows, E);
                LinParams p2 = lin(m.yc, ff, l.down, m.dn, W, W, ff);
                p2.w_gstride = (long long)W * ff; p2.cnt = m.cnt; p2.cnt_gstride = 1; p2.off = m.off;
                kx_lin(s, prof, p2, rows, E);
            }
            if (c.has_shared) {
                LinParams p1 = lin(m.h, W, l.sh_gu, m.ys, c.sff, 2 * c.sff, W, LE_GLU_CLAMP);
                p1.limit = c.slimit;
                kx_lin(s, prof, p1, rows, 1);
                kx_lin(s, prof, lin(m.ys, c.sff, l.sh_down, m.ds, W, W, c.sff), rows, 1);
            }
            MoeCombineParams cp{m.x, m.h, m.G + W, GW, m.dn, m.row_of, m.wgt, c.top, c.has_shared ? m.ds : nullptr, l.sg, W, mv};
            launch_k(moe_combine_kernel, dim3(rows), dim3(256), 0, cp, KC_OTHER, s, prof);
        }
        if (m.dbg_layers && !use_graph)
            CK(cudaMemcpyAsync(m.dbg_layers + li * (size_t)maxT * W, m.x, (size_t)maxT * W * 4, cudaMemcpyDeviceToDevice, s));
    }
    if (!own_stack) {
        FinalNormParams fn{m.x, m.hn, d_hidden, m.final_gain, m.cfg.eps, W, mv, m.final_w};
        launch_k(final_norm_kernel, dim3(rows), dim3(NORM_THREADS), 0, fn, KC_LN, s, prof);
    }
    if (rrows > 0) {
        LinParams ph = lin(m.hn, W, m.head, d_logits, V, V, W);
        if (m.cfg.logit_cap > 0.f) { ph.epi = LE_TANH_CAP; ph.limit = m.cfg.logit_cap; }
        ph.cnt = cntR;
        kx_lin(s, prof, ph, rrows, 1);
    }
}

static inline int kx_bucket(int n) {
    for (int b = 8; b < 512; b *= 2)
        if (n <= b) return b;
    return 512;
}

// positions, attention chunks and page-table updates of one step; hands out pages
void b200rwkv_engine::kx_fill_step(int* hm, const std::vector<int>& slots, const std::vector<int>& counts, bool* decode, int* nsplit) {
    SeqModel& m = *kx;
    int* base = hm + MetaView::ints(maxT, S);
    int* tok_pos = base + 8;
    int* ch_start = base + 8 + maxT;
    int* ch_count = base + 8 + 2 * maxT;
    int* upd = base + 8 + 3 * maxT;
    int T = 0, nch = 0, nupd = 0, ctx_max = 1;
    bool dec = true;
    for (int c : counts) dec = dec && c == 1;
    const int QB = dec ? 1 : m.qb_prompt;
    // hand out pages first: the step either fits or fails as a whole
    size_t need = 0;
    for (size_t i = 0; i < slots.size(); ++i) {
        const int have = (int)m.pages[slots[i]].size(), want = cdiv(m.pos[slots[i]] + counts[i], m.page);
        need += (size_t)std::max(0, want - have);
    }
    REQUIRE(need <= m.free_pages.size(), B200RWKV_ERR_STATE, "attention cache is full: live sequences hold more tokens than kv_tokens");
    for (size_t i = 0; i < slots.size(); ++i) {
        const int sl = slots[i];
        const int want = cdiv(m.pos[sl] + counts[i], m.page);
        while ((int)m.pages[sl].size() < want) {
            const int pg = m.free_pages.back();
            m.free_pages.pop_back();
            upd[3 * nupd] = sl; upd[3 * nupd + 1] = (int)m.pages[sl].size(); upd[3 * nupd + 2] = pg;
            ++nupd;
            m.pages[sl].push_back(pg);
        }
        for (int j = 0; j < counts[i]; j += QB) {
            ch_start[nch] = T + j;
            ch_count[nch] = std::min(QB, counts[i] - j);
            ++nch;
        }
        for (int j = 0; j < counts[i]; ++j) tok_pos[T++] = m.pos[sl] + j;
        m.pos[sl] += counts[i];
        ctx_max = std::max(ctx_max, m.pos[sl]);
    }
    base[0] = nupd; base[1] = nch;
    // long contexts at few chunks: split the keys so that the launch fills the GPU
    int hg_min = 1 << 30;
    for (const KxLayer& l : m.layers)
        if (l.c.mixer == KX_LATENT) hg_min = std::min(hg_min, cdiv(l.c.heads, dec ? (l.c.heads > 8 ? 16 : 8) : 4));
    int ns = 1;
    if (hg_min < (1 << 30)) {
        const int ctas = std::max(1, nch * hg_min), tiles = cdiv(ctx_max, LA_KT);
        while (ns < m.max_split && ctas * ns < 2 * num_sms && tiles / (ns * 2) >= 2) ns *= 2;
    }
    if (m.cfg.family != KX_FAMILY_KEMIRAX) {               // CTAs per attention chunk (a cluster): the keys a chunk can see, in tiles
        int seen = 0;
        for (const KxLayer& l : m.layers) {
            if (l.c.mixer == KX_WINDOW) seen = std::max(seen, std::min(ctx_max, l.c.window + l.c.keep_first + QB));
            if (l.c.mixer == KX_BIASED) seen = std::max(seen, ctx_max);
            if (m.cfg.family == KX_FAMILY_PASOPEL)         // the window, and one row per block of older tokens
                seen = std::max(seen, std::min(ctx_max, l.c.window + QB) + (l.c.pool > 0 ? ctx_max / l.c.pool : 0));
        }
        const int tiles = cdiv(seen, WA_KT);
        ns = 1;
        const int room = num_sms * (dec ? m.wa_ctas_decode : m.wa_ctas_prompt) / std::max(1, dec ? m.sa_ygroups_decode : m.sa_ygroups);   // CTAs the GPU holds at once
        const int* cap = dec ? m.cl_cap_decode : m.cl_cap_prompt;
        auto lg2 = [](int v) { int l = 0; while ((1 << l) < v) ++l; return l; };
        while (ns < m.max_split && std::max(1, nch) * ns * 2 <= room && std::max(1, nch) <= cap[lg2(ns * 2)] && tiles / (ns * 2) >= 1)
            ns *= 2;                                       // at most one wave of CTAs, and of clusters
    }
    *decode = dec; *nsplit = ns;
}

void b200rwkv_engine::kx_run_step(int T, int R, bool decode, int nsplit) {
    const int rows = kx_bucket(T), rrows = R > 0 ? kx_bucket(R) : 0;
    if (!use_graph) {
        kx_enqueue_step(stream, rows, rrows, decode, nsplit, nullptr);
        enqueue_keep(stream, rrows / 16 + (rrows % 16 ? 1 : 0));
        launch_total += launches_last_step;
        return;
    }
    int lg = 0;
    while ((1 << lg) < nsplit) ++lg;
    const int key = 1000000 + (((rows / 8) * 128 + rrows / 8) * 2 + (decode ? 1 : 0)) * 8 + lg;
    auto it = graphs.find(key);
    if (it == graphs.end()) {
        cudaGraph_t g = nullptr;
        CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        try {
            kx_enqueue_step(stream, rows, rrows, decode, nsplit, nullptr);
            enqueue_keep(stream, rrows / 16 + (rrows % 16 ? 1 : 0));
        } catch (...) {
            cudaStreamEndCapture(stream, &g);
            if (g) cudaGraphDestroy(g);
            throw;
        }
        CK(cudaStreamEndCapture(stream, &g));
        cudaGraphExec_t ge = nullptr;
        CK(cudaGraphInstantiate(&ge, g, 0));
        CK(cudaGraphDestroy(g));
        it = graphs.emplace(key, ge).first;
        graph_launches[key] = launches_last_step;
    }
    CK(cudaGraphLaunch(it->second, stream));
    launch_total += graph_launches[key];
}

// ---- sequence memory <-> flat record: [4 header floats][per layer: its fixed blocks (shift row, recurrent state, ...) | cache rows x D] ----
void b200rwkv_engine::kx_release(int slot) {
    SeqModel& m = *kx;
    for (int pg : m.pages[slot]) m.free_pages.push_back(pg);
    m.pages[slot].clear();
    m.pos[slot] = 0;
}

struct KxRowsParams { float* flat; float* cache; const int* table; int page, D, n; bool to_cache; };

__global__ void kx_cache_rows_kernel(const KxRowsParams p) {
    const int j = blockIdx.x;
    if (j >= p.n) return;
    float* c = p.cache + ((size_t)p.table[j / p.page] * p.page + j % p.page) * p.D;
    float* f = p.flat + (size_t)j * p.D;
    for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
        if (p.to_cache) c[d] = f[d];
        else f[d] = c[d];
    }
}

// export (import = false): slot -> record with `ctx_rows` cache rows per layer; import: record holding `n` tokens -> slot
void b200rwkv_engine::kx_xfer(int slot, float* rec, int ctx_rows, bool import, int n) {
    SeqModel& m = *kx;
    if (import) {
        kx_release(slot);
        REQUIRE(n >= 0 && n <= ctx_rows, B200RWKV_ERR_INVALID, "state record holds more tokens than it has rows");
        const int want = cdiv(n, m.page);
        REQUIRE((size_t)want <= m.free_pages.size(), B200RWKV_ERR_STATE, "attention cache is full");
        for (int i = 0; i < want; ++i) { m.pages[slot].push_back(m.free_pages.back()); m.free_pages.pop_back(); }
        if (want > 0) CK(cudaMemcpyAsync(m.d_table + (size_t)slot * m.npages, m.pages[slot].data(), (size_t)want * 4, cudaMemcpyHostToDevice, stream));
        CK(cudaStreamSynchronize(stream));                  // the pageable source above is read by now
        m.pos[slot] = n;
    } else {
        n = m.pos[slot];
        REQUIRE(n <= ctx_rows, B200RWKV_ERR_STATE, "sequence is longer than the state tensor's cache rows");
    }
    size_t o = 4;
    auto copy = [&](float* dev, size_t cnt) {
        if (import) CK(cudaMemcpyAsync(dev, rec + o, cnt * 4, cudaMemcpyDeviceToDevice, stream));
        else CK(cudaMemcpyAsync(rec + o, dev, cnt * 4, cudaMemcpyDeviceToDevice, stream));
        o += cnt;
    };
    for (KxLayer& l : m.layers) {
        for (const KxLayer::Block& b : l.fixed) copy(b.base + (size_t)slot * b.per_slot, b.per_slot);
        if (l.cache_D > 0) {
            if (n > 0) {
                KxRowsParams rp{rec + o, l.cache, m.d_table + (size_t)slot * m.npages, m.page, l.cache_D, n, import};
                kx_cache_rows_kernel<<<n, 128, 0, stream>>>(rp);
                CK(cudaGetLastError());
            }
            o += (size_t)ctx_rows * l.cache_D;
        }
    }
    if (import && m.cfg.family == KX_FAMILY_PASOPEL) ps_repool(slot, n);      // block means are derived from the cache rows
}

// host copy between two records of the same model whose cache blocks have different row counts
static void kx_relayout(const SeqModel& m, const float* src, int src_rows, float* dst, int dst_rows, int n) {
    size_t a = 4, b = 4;
    memset(dst, 0, 16);                                    // header: the caller writes the token count
    for (const KxLayer& l : m.layers) {
        for (const KxLayer::Block& blk : l.fixed) { memcpy(dst + b, src + a, blk.per_slot * 4); a += blk.per_slot; b += blk.per_slot; }
        if (l.cache_D > 0) {
            memcpy(dst + b, src + a, (size_t)n * l.cache_D * 4);
            a += (size_t)src_rows * l.cache_D; b += (size_t)dst_rows * l.cache_D;
        }
    }
}

// an empty sequence in `slot`: pages back to the pool, the fixed blocks (shift rows, recurrent states, convolution tails) zero
void b200rwkv_engine::kx_reset(int slot) {
    SeqModel& m = *kx;
    kx_release(slot);
    for (KxLayer& l : m.layers)
        for (const KxLayer::Block& b : l.fixed)
            if (b.per_slot) CK(cudaMemsetAsync(b.base + (size_t)slot * b.per_slot, 0, b.per_slot * 4, stream));
}
