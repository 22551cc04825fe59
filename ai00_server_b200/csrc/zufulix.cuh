// Zufulix model family: pre-norm blocks (layer norm with weight and bias) around several copies of the residual,
//     u = sum_s a[s] x_s;   y = Sublayer(LN(u));   x_t <- sum_s M[s, t] x_s + b[t] y                           (hyper.cuh)
// or the plain x <- x + Sublayer(LN(x)) when the configuration names no streams.  Mixer = causal softmax attention with grouped
// key / value heads, biased projections, unit-RMS queries and keys, a learned bias per (distance bucket, head) and values
// blended with those of the first blending layer (bias_attn.cuh); feed-forward = W_down gelu(W_up h), or routed experts
// W_down relu(W_up h)^2 chosen by sigmoid scores inside the best groups of neighbouring experts (moe.cuh).  The embedding row is
// scaled on the way in and the embedding table itself is the output matrix.  Every size and constant that can differ between
// models comes from config.json / the tensor shapes.  The family shares the sequence-model engine of the other config.json
// families (kemirax.cuh: configuration structs, slot / page / snapshot plumbing); this file reads its configuration.
#pragma once

namespace b200 {

static KxConfig zf_parse_config(const JVal& root) {
    KxConfig c;
    c.family = KX_FAMILY_ZUFULIX;
    c.vocab = root.integer("vocab");
    c.width = root.integer("width");
    c.eps = (float)root.at("norm").number("eps");
    if (root.has("embedding") && root.at("embedding").has("scale")) c.embed_scale = (float)root.at("embedding").number("scale");
    if (root.has("streams")) {
        c.streams = root.integer("streams");
        REQUIRE(c.streams >= 1 && c.streams <= HC_MAX_STREAMS, B200RWKV_ERR_UNSUPPORTED, "config: streams must be in 1..16");
    }
    const JVal& ls = root.at("layers");
    REQUIRE(ls.kind == JVal::ARR && !ls.arr.empty(), B200RWKV_ERR_INVALID, "config: layers");
    for (const JVal& l : ls.arr) {
        KxLayerCfg k;
        REQUIRE(l.kind == JVal::OBJ && l.has("type") && l.at("type").kind == JVal::STR, B200RWKV_ERR_INVALID, "config: layer without a type");
        const std::string type = l.at("type").str;
        REQUIRE(type == "attention", B200RWKV_ERR_UNSUPPORTED, "config: unknown layer type '" + type + "'");
        const JVal& m = l.at("mixer");
        k.mixer = KX_BIASED;
        k.heads = m.integer("heads"); k.dim = m.integer("dim"); k.vdim = m.integer("vdim");
        k.kv_heads = m.has("kv_heads") ? m.integer("kv_heads") : k.heads;
        REQUIRE(k.heads >= 1 && k.kv_heads >= 1 && k.heads % k.kv_heads == 0, B200RWKV_ERR_INVALID, "config: heads must be a multiple of kv_heads");
        k.scale = (float)m.number("scale");
        k.bias_max = m.number("bias_max");
        const JVal* vm = m.get("v_mix");
        k.v_mix = vm && ((vm->kind == JVal::BOOL && vm->b) || (vm->kind == JVal::NUM && vm->num != 0));
        if (l.has("mlp")) {
            const JVal& f = l.at("mlp");
            const std::string kind = f.at("kind").str;
            k.has_mlp = true;
            if (kind == "dense") {
                k.mlp_dense = true;
                k.ff = f.integer("ff");
            } else if (kind == "moe") {
                const JVal& r = f.at("router");
                k.experts = r.integer("experts"); k.top = r.integer("top");
                k.ff = f.at("expert").integer("ff");
                if (r.has("groups")) {
                    k.groups = r.at("groups").integer("count"); k.groups_keep = r.at("groups").integer("keep");
                    REQUIRE(k.groups >= 1 && k.experts % k.groups == 0 && k.groups_keep >= 1 && k.groups_keep <= k.groups, B200RWKV_ERR_INVALID,
                            "config: groups.count must divide experts and groups.keep must be in 1..count");
                    REQUIRE((long long)k.groups_keep * (k.experts / k.groups) >= k.top, B200RWKV_ERR_INVALID,
                            "config: the kept groups hold fewer experts than top");
                }
            } else {
                throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown mlp kind '" + kind + "'");
            }
        }
        c.layers.push_back(k);
    }
    return c;
}

// bias of every distance 0 .. nb for every head, from the bucket table rel[B][H]: distance n < B/2 has bucket n, larger ones
// share buckets evenly spaced in log(n) up to `far`; n >= far takes the last bucket (so nb = ceil(far) closes the table).
// Double arithmetic on the host; the kernel indexes by min(distance, nb).
static std::vector<float> zf_bias_table(const std::vector<float>& rel, int B, int H_, double far, int& nb) {
    const int half = B / 2;
    REQUIRE(B >= 2 && far > (double)half && far <= 1e7, B200RWKV_ERR_INVALID, "config: bias_max must exceed half the bias table's rows");
    nb = (int)std::ceil(far);
    std::vector<float> t((size_t)(nb + 1) * H_);
    for (int n = 0; n <= nb; ++n) {
        int b = n;
        if (n >= half) {
            const double f = std::floor(std::log((double)n / half) / std::log(far / half) * (double)(B - half));
            b = (int)std::min<double>((double)(B - 1), (double)half + f);
        }
        for (int h = 0; h < H_; ++h) t[(size_t)n * H_ + h] = rel[(size_t)b * H_ + h];
    }
    return t;
}

}  // namespace b200
