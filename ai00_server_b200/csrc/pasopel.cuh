// Pasopel model family: pre-norm blocks  x += Mixer(N1(x));  x += FF(N2(x))  with RMS norms whose weights are stored as
// offsets from one.  A run of consecutive layers (`loop`: start, stop, times) is executed `times` times with the same tensors
// and sequence memory of its own per pass; a pass begins by adding a learned per-pass vector to the residual, every pass after
// the first also adds the token's embedding row again.
// Mixers: "attention" = grouped-head softmax attention whose values are its un-normalised keys, queries and keys behind short
// causal convolutions and divided by their root mean square, a sliding window extended by block means of older keys / values,
// a sink term per head in the softmax denominator, a sigmoid output gate, biased projections (sink_attn.cuh);
// "latent_attention" = low-rank queries, one shared key / value latent plus one shared rotated key part (neighbouring entries
// turn together), sliding window, sink, output gate (latent_attn.cuh prepares, sink_attn.cuh attends, in the absorbed form).
// Feed-forward: W_down relu(W_up h)^2, or routed silu-gated experts (largest logits, softmax over the chosen) plus an always-on
// expert (moe.cuh).  The embedding table is the output matrix; the logits are squashed by cap * tanh(z / cap).
// Every size and constant that can differ between models comes from config.json / the tensor shapes.  The family shares the
// sequence-model engine of the Kemirax family (kemirax.cuh: configuration structs, slot / page / snapshot plumbing); this file
// reads its configuration and unrolls the looped layers into the list of layer runs the engine executes.
#pragma once

namespace b200 {

static KxConfig ps_parse_config(const JVal& root) {
    KxConfig c;
    c.family = KX_FAMILY_PASOPEL;
    c.vocab = root.integer("vocab");
    c.width = root.integer("width");
    c.eps = (float)root.at("norm").number("eps");
    if (root.has("logit_softcap")) {
        c.logit_cap = (float)root.number("logit_softcap");
        REQUIRE(c.logit_cap > 0.f, B200RWKV_ERR_INVALID, "config: logit_softcap must be positive");
    }
    const JVal& ls = root.at("layers");
    REQUIRE(ls.kind == JVal::ARR && !ls.arr.empty(), B200RWKV_ERR_INVALID, "config: layers");
    std::vector<KxLayerCfg> own;
    for (const JVal& l : ls.arr) {
        KxLayerCfg k;
        REQUIRE(l.kind == JVal::OBJ && l.has("type") && l.at("type").kind == JVal::STR, B200RWKV_ERR_INVALID, "config: layer without a type");
        const std::string type = l.at("type").str;
        const JVal& m = l.at("mixer");
        k.heads = m.integer("heads"); k.dim = m.integer("dim");
        k.vdim = m.has("vdim") ? m.integer("vdim") : k.dim;
        k.scale = (float)m.number("scale");
        const JVal& mk = m.at("mask");
        k.window = mk.integer("size");
        REQUIRE(k.window >= 1, B200RWKV_ERR_INVALID, "config: mask.size must be >= 1");
        if (type == "attention") {
            k.mixer = KX_SINK;
            k.kv_heads = m.has("kv_heads") ? m.integer("kv_heads") : k.heads;
            k.taps = m.has("conv") ? m.integer("conv") : 1;
            k.pool = mk.has("pool") ? mk.integer("pool") : 0;
            REQUIRE(k.taps >= 1, B200RWKV_ERR_INVALID, "config: conv must be >= 1");
            REQUIRE(k.vdim == k.dim, B200RWKV_ERR_INVALID, "config: the values of this mixer are its keys, vdim must equal dim");
            REQUIRE(k.kv_heads >= 1 && k.heads % k.kv_heads == 0, B200RWKV_ERR_INVALID, "config: heads must be a multiple of kv_heads");
        } else if (type == "latent_attention") {
            k.mixer = KX_LATENT;
            k.kv_heads = 1;
            k.rot_dim = m.integer("rot_dim"); k.kv_rank = m.integer("kv_rank"); k.q_rank = m.integer("q_rank");
            const JVal& r = m.at("rot");
            k.rot.dims = r.integer("dims"); k.rot.base = r.number("base");
            REQUIRE(k.rot.dims % 2 == 0 && k.rot.dims <= k.rot_dim, B200RWKV_ERR_INVALID, "config: rot.dims must be even and <= rot_dim");
            REQUIRE(k.kv_rank >= 1 && k.q_rank >= 1, B200RWKV_ERR_INVALID, "config: ranks must be >= 1");
        } else {
            throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown layer type '" + type + "'");
        }
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
                if (f.has("shared")) { k.has_shared = true; k.sff = f.at("shared").integer("ff"); }
            } else {
                throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown mlp kind '" + kind + "'");
            }
        }
        own.push_back(k);
    }
    // the layer runs in execution order: layers before the loop, the looped layers once per pass, the rest
    const int nl = (int)own.size();
    int start = 0, stop = 0, times = 1;
    if (root.has("loop")) {
        const JVal& lp = root.at("loop");
        start = lp.integer("start"); stop = lp.integer("stop"); times = lp.integer("times");
        REQUIRE(start <= stop && stop <= nl && times >= 1, B200RWKV_ERR_INVALID, "config: loop must name layers start .. stop - 1 and times >= 1");
        REQUIRE((long long)(stop - start) * times + nl <= 4096, B200RWKV_ERR_UNSUPPORTED, "config: too many layer runs");
        c.has_loop = stop > start;
    }
    auto run = [&](int i, int opens) {
        KxLayerCfg k = own[i];
        k.tensors_of = i;
        k.opens_pass = opens;
        c.layers.push_back(k);
    };
    for (int i = 0; i < (c.has_loop ? start : nl); ++i) run(i, -1);
    if (c.has_loop) {
        for (int t = 0; t < times; ++t)
            for (int i = start; i < stop; ++i) run(i, i == start ? t : -1);
        for (int i = stop; i < nl; ++i) run(i, -1);
    }
    return c;
}

}  // namespace b200
