// Kemirax model family: parallel blocks  x += G1(h) * Mixer(shift(h)) + G2(h) * FF(h),  h = scalar-gain RMS norm of x,
// mixers = latent attention over a paged cache (latent_attn.cuh) or gated linear attention (gla.cuh), feed-forward = routed
// mixture of clamped gated experts with identity experts and a gated shared expert (moe.cuh), projections = grouped linears
// (linear.cuh).  Every size and constant comes from config.json / the tensor shapes.  This file is the host side: config
// parsing, weight upload (stacking / interleaving / transposing the matrices the grouped launches want), the per-step launch
// sequence, and the sequence memory (shift rows, recurrent states, cache pages) behind the engine's slot / snapshot interface.
//
// Included by engine.cu after the engine struct; uses its allocation, launch, metadata and graph plumbing.
#pragma once

namespace b200 {

// ------------------------------------------------------------------------------------------------------------------
// minimal JSON value (config.json)
// ------------------------------------------------------------------------------------------------------------------
struct JVal {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    double num = 0;
    bool b = false;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const std::string& k) const {
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
    const JVal& at(const std::string& k) const {
        const JVal* v = get(k);
        REQUIRE(v, B200RWKV_ERR_INVALID, "config: missing key '" + k + "'");
        return *v;
    }
    double number(const std::string& k) const {
        const JVal& v = at(k);
        REQUIRE(v.kind == NUM, B200RWKV_ERR_INVALID, "config: '" + k + "' is not a number");
        return v.num;
    }
    int integer(const std::string& k) const {
        const double d = number(k);
        REQUIRE(d >= 0 && d <= 1e9 && d == std::floor(d), B200RWKV_ERR_INVALID, "config: '" + k + "' is not a size");
        return (int)d;
    }
    bool has(const std::string& k) const { const JVal* v = get(k); return v && v->kind != NUL; }
};

class JsonParser {
public:
    JsonParser(const char* s, size_t n) : s_(s), n_(n) {}
    JVal parse() { JVal v = value(0); ws(); REQUIRE(i_ == n_, B200RWKV_ERR_INVALID, "config: trailing characters"); return v; }
private:
    const char* s_; size_t n_, i_ = 0;
    void ws() { while (i_ < n_ && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_; }
    char peek() { return i_ < n_ ? s_[i_] : '\0'; }
    void expect(char c) { REQUIRE(peek() == c, B200RWKV_ERR_INVALID, std::string("config: expected '") + c + "'"); ++i_; }
    std::string string_() {
        expect('"');
        std::string o;
        while (i_ < n_ && s_[i_] != '"') {
            if (s_[i_] == '\\' && i_ + 1 < n_) { ++i_; if (s_[i_] == 'u') { i_ += 4; o.push_back('?'); } else o.push_back(s_[i_] == 'n' ? '\n' : s_[i_]); }
            else o.push_back(s_[i_]);
            ++i_;
        }
        expect('"');
        return o;
    }
    JVal value(int depth) {
        REQUIRE(depth < 32, B200RWKV_ERR_INVALID, "config: nested too deeply");
        ws();
        JVal v;
        const char c = peek();
        if (c == '{') {
            v.kind = JVal::OBJ; ++i_; ws();
            if (peek() == '}') { ++i_; return v; }
            for (;;) {
                ws(); std::string k = string_(); ws(); expect(':');
                v.obj.emplace_back(std::move(k), value(depth + 1));
                ws();
                if (peek() == ',') { ++i_; continue; }
                expect('}'); break;
            }
        } else if (c == '[') {
            v.kind = JVal::ARR; ++i_; ws();
            if (peek() == ']') { ++i_; return v; }
            for (;;) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (peek() == ',') { ++i_; continue; }
                expect(']'); break;
            }
        } else if (c == '"') { v.kind = JVal::STR; v.str = string_(); }
        else if (n_ - i_ >= 4 && !strncmp(s_ + i_, "null", 4)) { i_ += 4; }
        else if (n_ - i_ >= 4 && !strncmp(s_ + i_, "true", 4)) { i_ += 4; v.kind = JVal::BOOL; v.b = true; }
        else if (n_ - i_ >= 5 && !strncmp(s_ + i_, "false", 5)) { i_ += 5; v.kind = JVal::BOOL; }
        else {
            size_t j = i_;
            while (j < n_ && (isdigit((unsigned char)s_[j]) || s_[j] == '-' || s_[j] == '+' || s_[j] == '.' || s_[j] == 'e' || s_[j] == 'E')) ++j;
            REQUIRE(j > i_, B200RWKV_ERR_INVALID, "config: unexpected character");
            v.kind = JVal::NUM; v.num = strtod(std::string(s_ + i_, j - i_).c_str(), nullptr);
            i_ = j;
        }
        return v;
    }
};

// ------------------------------------------------------------------------------------------------------------------
// configuration
// ------------------------------------------------------------------------------------------------------------------
struct RotCfg { int dims = 0; double base = 10000.0; bool scaled = false; double factor = 1, original = 0, fast = 0, slow = 0; };

enum KxMixer { KX_LATENT = 0, KX_GLA = 1, KX_RETENTION = 2, KX_DELTA = 3, KX_WINDOW = 4, KX_BIASED = 5, KX_SINK = 6 };
enum KxFamily { KX_FAMILY_KEMIRAX = 0, KX_FAMILY_DEGAVIK = 1, KX_FAMILY_ZUFULIX = 2, KX_FAMILY_PASOPEL = 3 };

struct KxLayerCfg {
    int mixer = KX_LATENT;
    int heads = 0, dim = 0, vdim = 0;
    // Degavik mixers (degavik.cuh)
    int kv_heads = 0;                                            // delta rule, windowed attention
    int taps = 0;                                                // delta rule: short convolution length
    int window = 0, keep_first = 0;                              // windowed attention
    float softcap = 0.f;
    std::vector<double> decay;                                   // retention: one per head
    int weights_of = -1;                                         // the layer whose tensors this layer uses (-1: its own)
    bool mlp_dense = false;                                      // feed-forward is one dense unit, not routed experts
    // Zufulix (zufulix.cuh): attention with a bias per (distance bucket, head), blended values, grouped sigmoid router
    double bias_max = 0;                                         // distance from which every key shares the last bucket
    bool v_mix = false;                                          // values blended with the first such layer's
    int groups = 0, groups_keep = 0;                             // router: groups of neighbouring experts / groups kept (0: none)
    // Pasopel (pasopel.cuh): attention whose values are its keys, behind short convolutions, over a window extended by block
    // means, with a sink term; latent attention over a window with a sink term; a run of layers executed several times
    int pool = 0;                                                // tokens per block mean behind the window (0: none)
    int tensors_of = -1;                                         // index in the tensor names ("l<i>."); -1: the layer's own place
    int opens_pass = -1;                                         // >= 0: this run opens pass number `opens_pass` of the looped layers
    int rot_dim = 0, kv_rank = 0, q_rank = 0, kv_from = -1;     // latent attention
    float scale = 1.f;
    RotCfg rot;
    float tau = 1.f;                                             // gla
    bool has_mlp = false;
    int experts = 0, identity = 0, top = 0, ff = 0;
    float limit = 0.f;
    bool has_shared = false;
    int sff = 0;
    float slimit = 0.f;
};

struct KxConfig {
    int family = KX_FAMILY_KEMIRAX;
    int vocab = 0, width = 0;
    float eps = 1e-5f;
    int streams = 0;                                             // copies of the residual (0: the plain residual)
    float embed_scale = 1.f;                                     // factor on the embedding row
    float logit_cap = 0.f;                                       // logits <- cap * tanh(logits / cap) (0: none)
    bool has_loop = false;                                       // a run of layers is executed several times (`layers` lists every run)
    std::vector<KxLayerCfg> layers;
};

static KxConfig dg_parse_config(const JVal& root);
static KxConfig zf_parse_config(const JVal& root);
static KxConfig ps_parse_config(const JVal& root);

// model registry of the families that come with a config.json: `architecture` names the design
static KxConfig kx_parse_config(const char* json, size_t n) {
    JVal root = JsonParser(json, n).parse();
    REQUIRE(root.kind == JVal::OBJ, B200RWKV_ERR_INVALID, "config: not an object");
    REQUIRE(root.has("architecture") && root.at("architecture").kind == JVal::STR, B200RWKV_ERR_INVALID, "config: no architecture");
    const std::string arch = root.at("architecture").str;
    if (arch == "Degavik") return dg_parse_config(root);
    if (arch == "Zufulix") return zf_parse_config(root);
    if (arch == "Pasopel") return ps_parse_config(root);
    REQUIRE(arch == "Kemirax", B200RWKV_ERR_UNSUPPORTED, "config: unknown architecture '" + arch + "'");
    KxConfig c;
    c.vocab = root.integer("vocab");
    c.width = root.integer("width");
    c.eps = (float)root.at("norm").number("eps");
    const JVal& ls = root.at("layers");
    REQUIRE(ls.kind == JVal::ARR && !ls.arr.empty(), B200RWKV_ERR_INVALID, "config: layers");
    for (const JVal& l : ls.arr) {
        KxLayerCfg k;
        const std::string type = l.at("type").str;
        const JVal& m = l.at("mixer");
        k.heads = m.integer("heads"); k.dim = m.integer("dim"); k.vdim = m.integer("vdim");
        if (type == "latent_attention") {
            k.mixer = KX_LATENT;
            k.rot_dim = m.integer("rot_dim"); k.kv_rank = m.integer("kv_rank"); k.q_rank = m.integer("q_rank");
            k.scale = (float)m.number("scale");
            if (m.has("kv_from")) k.kv_from = m.integer("kv_from");
            const JVal& r = m.at("rot");
            k.rot.dims = r.integer("dims"); k.rot.base = r.number("base");
            if (r.has("scaling")) {
                const JVal& s = r.at("scaling");
                k.rot.scaled = true;
                k.rot.factor = s.number("factor"); k.rot.original = s.number("original");
                k.rot.fast = s.number("fast"); k.rot.slow = s.number("slow");
            }
        } else if (type == "gla") {
            k.mixer = KX_GLA;
            k.tau = (float)m.number("tau");
        } else {
            throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown layer type '" + type + "'");
        }
        if (l.has("mlp")) {
            const JVal& f = l.at("mlp");
            REQUIRE(f.at("kind").str == "moe", B200RWKV_ERR_UNSUPPORTED, "config: unknown mlp kind");
            k.has_mlp = true;
            const JVal& r = f.at("router");
            k.experts = r.integer("experts"); k.top = r.integer("top");
            k.identity = r.has("identity") ? r.integer("identity") : 0;
            k.ff = f.at("expert").integer("ff"); k.limit = (float)f.at("expert").number("limit");
            if (f.has("shared")) {
                k.has_shared = true;
                k.sff = f.at("shared").integer("ff"); k.slimit = (float)f.at("shared").number("limit");
            }
        }
        c.layers.push_back(k);
    }
    return c;
}

// rotary frequency table with the long-context rescaling folded in (double arithmetic on the host, f32 table on the device)
static void kx_rot_table(const RotCfg& r, std::vector<float>& freq, float& mag) {
    const int half = r.dims / 2;
    freq.resize(std::max(half, 1));
    mag = 1.f;
    int lo = 0, hi = 0;
    if (r.scaled) {
        auto turn_dim = [&](double turns) { return r.dims * std::log(r.original / (2.0 * M_PI * turns)) / (2.0 * std::log(r.base)); };
        lo = std::max((int)std::floor(turn_dim(r.fast)), 0);
        hi = std::min((int)std::ceil(turn_dim(r.slow)), r.dims - 1);
        mag = (float)(0.1 * std::log(r.factor) + 1.0);
    }
    for (int i = 0; i < half; ++i) {
        double f = std::pow(r.base, -2.0 * i / r.dims);
        if (r.scaled) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max((double)(hi - lo), 0.001)));
            f = f / r.factor * ramp + f * (1.0 - ramp);
        }
        freq[i] = (float)f;
    }
}

// ------------------------------------------------------------------------------------------------------------------
// device-side model
// ------------------------------------------------------------------------------------------------------------------
struct KxLayer {
    KxLayerCfg c;
    float gain = 1.f;
    float* mu = nullptr;
    float* shift_state = nullptr;                 // [S][W]
    __nv_bfloat16* rg = nullptr; float* rg_b = nullptr;          // [2W, W] rg1 over rg2, [2W]
    // latent attention
    __nv_bfloat16 *dq = nullptr, *uq = nullptr, *dkv = nullptr, *ukT = nullptr, *uv = nullptr, *o = nullptr;
    float *dq_norm = nullptr, *dkv_norm = nullptr, *freq = nullptr;
    float mag = 1.f;
    float* cache = nullptr;                       // [pages][page][rk + dr]; a borrowing layer points at the lender's pool
    // gla
    __nv_bfloat16 *proj = nullptr, *a2 = nullptr;               // proj = [q; k; v; g; a1] stacked
    float *a2_b = nullptr, *norm_w = nullptr, *gla_state = nullptr;
    int a_rank = 0, proj_n = 0;
    // feed-forward
    __nv_bfloat16 *router = nullptr, *gu = nullptr, *down = nullptr, *sh_gu = nullptr, *sh_down = nullptr, *sg = nullptr;
    float* corr = nullptr;
    // Degavik: norms on the sublayers' outputs, retention / delta-rule / windowed-attention mixers
    float *norm1_w = nullptr, *norm2_w = nullptr;
    float *decay = nullptr;                                      // retention [H]
    __nv_bfloat16 *g2 = nullptr;                                 // delta rule: output-gate up-projection (a2 = decay up-projection)
    float *a_log = nullptr, *conv_w = nullptr, *conv_tail = nullptr;   // delta rule: [H], [C][taps], [S][taps - 1][C]
    int g_rank = 0, conv_C = 0;
    float *qn_w = nullptr, *kn_w = nullptr, *talk = nullptr, *temp = nullptr;   // windowed attention
    double* freq_d = nullptr;                                    // rotary frequencies in double (retention, windowed attention)
    int wa_gt = 1;                                               // key / value heads per tile load of the attention kernel
    float* rec_state = nullptr;                                  // retention / delta rule: [S][H][dk][dv]
    int cache_D = 0;                                             // floats per cached token when the layer owns a pool
    // Zufulix: layer norms with bias, stream coefficients of the two sublayers, projection biases, distance-bias table
    float *norm1_b = nullptr, *norm2_b = nullptr;
    float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
    float *proj_b = nullptr, *rel_bias = nullptr;                // [proj_n], [rel_n + 1][H]
    int rel_n = 0, vmode = 0;
    int gt_decode = 1;                                           // key / value heads per tile load in decode-shaped steps
    bool attn_reg = false;                                       // head sizes fit the attention kernel's register form
    float lam = 0.f;
    // Pasopel: sink terms, output-gate offset in the projection row, block-mean rows, launch shape of the attention kernel
    float *sink = nullptr, *o_b = nullptr, *pcache = nullptr;
    int prow = 0;                                                // block-mean rows per page
    int sa_hb = 1, sa_gt = 1, sa_gt_decode = 1, sa_nbuf = 2, sa_nbuf_decode = 2;
    int sa_qb = 1;                                               // tokens per chunk of the tile form in prompt steps
    int sa_hb_decode = 1;                                        // query heads per CTA in decode-shaped steps
    bool sa_reg = false;                                         // head sizes fit the register form of the attention kernel
    // per-sequence memory of fixed size, in the order of the flat state record
    struct Block { float* base; size_t per_slot; };
    std::vector<Block> fixed;
};

// largest per-token widths of the activation buffers over the layers of a model (filled by the family's loader)
struct KxSizes {
    size_t n_cq = 1, n_q = 1, n_qa = 1, n_kv = 1, n_part = 1, n_olat = 1, n_vout = 1, n_pr = 1, n_z = 1, n_rl = 1, n_yc = 1, n_ys = 1,
           n_cv = 1, n_gl = 1, n_vf = 1, n_streams = 1;
    int max_top = 1, max_E = 1;
};

// the device-side model of every config.json family (which one: cfg.family) and the sequence memory of its slots
struct SeqModel {
    KxConfig cfg;
    std::vector<KxLayer> layers;
    bool exact = false;
    int W = 0, V = 0, page = 64, npages = 0, state_ctx = 0;
    float final_gain = 1.f;
    float* final_w = nullptr;                     // weight vector of the last norm (families that have one)
    float* final_b = nullptr;                     // its bias (layer-norm families)
    float* pass_vec = nullptr;                    // [passes][W] vector a looped run of layers adds when a pass begins
    int streams = 1;                              // copies of the residual a token row of x holds
    float* vfirst = nullptr;                      // [T, G * dv] values of the first blending attention layer, this step's tokens
    int qb_prompt = 4;                            // tokens per attention chunk of a prompt step
    int wa_ctas_prompt = 1, wa_ctas_decode = 1;   // windowed-attention CTAs one SM holds at once (prompt / decode shape)
    int cl_cap_prompt[4] = {1 << 30, 1 << 30, 1 << 30, 1 << 30};   // clusters of 1 / 2 / 4 / 8 attention CTAs the GPU holds at once, where a
    int cl_cap_decode[4] = {1 << 30, 1 << 30, 1 << 30, 1 << 30};   // family's loader has asked the device (a launch should stay within one wave)
    float *y = nullptr, *cv = nullptr, *gl = nullptr;   // sublayer output, convolution output, output-gate logits
    __nv_bfloat16 *embed = nullptr, *head = nullptr;
    // sequence memory
    int* d_table = nullptr;                       // [S][npages]
    std::vector<int> pos;                         // [S] tokens held
    std::vector<std::vector<int>> pages;          // [S] pages held, in order
    std::vector<int> free_pages;
    // activations
    float *x = nullptr, *h = nullptr, *hs = nullptr, *G = nullptr, *cq = nullptr, *q = nullptr, *qa = nullptr, *kv = nullptr, *part = nullptr,
          *olat = nullptr, *vout = nullptr, *pr = nullptr, *z = nullptr, *rl = nullptr, *wgt = nullptr, *yc = nullptr, *dn = nullptr, *ys = nullptr,
          *ds = nullptr, *hn = nullptr;
    int *sel = nullptr, *cnt = nullptr, *off = nullptr, *list = nullptr, *row_of = nullptr;
    float* lin_ws = nullptr; size_t lin_ws_floats = 0;
    float* dbg_layers = nullptr;                  // [L][maxT][W] residual after every layer (bring-up aid; nullptr: off)
    int max_split = 16;
    int sa_ygroups = 1, sa_ygroups_decode = 1;    // head groups (grid rows) of the smallest windowed-attention launch of the model (prompt / decode shape)
    SeqMeta sm{nullptr, 0};
    size_t flat_floats(int ctx_rows) const;
    int max_D = 0;
};

}  // namespace b200
