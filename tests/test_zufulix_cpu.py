"""CPU tests of the Zufulix pieces that need no GPU: the NumPy restatement against independent formulations of the same
mechanisms (a batched masked attention over materialised keys / values, the bucket law by its defining properties, hand-made
router cases, one stream = the plain residual), invariance of the restatement to how a sequence is cut, the synthetic-model
writer, and the host-only model detection of the C ABI."""
import json
import math

import numpy as np

from ai00_server_b200 import capi, synth
from oracle import zufulix_numpy as Z

L = synth.zufulix_layer


def model(layers, **kw):
    cfgb, st, w = synth.make_zufulix(layers, **kw)
    return json.loads(cfgb), st, w


def test_writer_round_trips():
    cfg, st, w = model([L(), L(mlp="moe"), L(mlp=None)], seed=2)
    back = Z.read_safetensors(bytes(st))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], w[k]), k
    assert w["l1.mix.vmix"].shape == () and "l2.hc2.in" not in w and "l2.norm2" not in w
    assert cfg["streams"] == 3 and w["l0.hc1.mix"].shape == (3, 3)


def test_distance_buckets():
    rows, far = 12, 40
    b = [Z.distance_bucket(n, rows, far) for n in range(200)]
    assert b[:6] == list(range(6))                              # one bucket per distance below rows / 2
    assert b[6] == 6 and all(x <= y for x, y in zip(b, b[1:]))  # monotone, continuous at the switch
    assert all(x == rows - 1 for x in b[40:]) and max(b) == rows - 1    # everything from `far` on shares the last bucket
    # log spacing: bucket 6 + k starts where n / 6 first reaches (far / 6)^(k / 6)
    for k in range(1, 6):
        first = b.index(6 + k)
        assert first == math.ceil(6 * (far / 6) ** (k / 6) - 1e-9)
    assert [Z.distance_bucket(n, 2, 3.0) for n in range(5)] == [0, 1, 1, 1, 1]


def test_attention_equals_a_batched_form():
    cfg, st, w = model([L(heads=6, kv_heads=2, dim=8, vdim=5, bias_max=9, mlp=None)], width=24, seed=1, rel_rows=6)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    rng = np.random.default_rng(3)
    hs = rng.standard_normal((21, 24))
    mem, got = {}, []
    for t, h in enumerate(hs):
        got.append(Z.attention(w, p, c, 1e-5, h, mem, t, {}))
    H, G, dk, dv, n = 6, 2, 8, 5, len(hs)
    q = (hs @ w[p + "q"].T + w[p + "q.b"]).reshape(n, H, dk)
    k = (hs @ w[p + "k"].T + w[p + "k.b"]).reshape(n, G, dk)
    v = (hs @ w[p + "v"].T + w[p + "v.b"]).reshape(n, G, dv)
    q = q / np.sqrt((q ** 2).mean(-1, keepdims=True) + 1e-5)
    k = k / np.sqrt((k ** 2).mean(-1, keepdims=True) + 1e-5)
    k, v = np.repeat(k, H // G, 1), np.repeat(v, H // G, 1)     # query head h reads key / value head h // (H / G)
    dist = np.arange(n)[:, None] - np.arange(n)[None, :]
    bucket = np.vectorize(lambda d: Z.distance_bucket(int(d), 6, 9) if d >= 0 else 0)(dist)
    s = np.einsum("ihd,jhd->hij", q, k) * c["scale"] + np.transpose(w[p + "rel"][bucket], (2, 0, 1))
    s = np.where(dist[None] >= 0, s, -np.inf)
    a = np.exp(s - s.max(-1, keepdims=True))
    a /= a.sum(-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", a, v).reshape(n, H * dv) @ w[p + "o"].T
    assert np.abs(o - np.stack(got)).max() < 1e-10


def test_values_blend_with_the_first_blending_layer_only():
    layers = [L(v_mix=False, mlp=None), L(mlp=None), L(v_mix=None, mlp=None), L(mlp=None)]
    cfg, st, w = model(layers, seed=4)
    toks = [3, 9, 27, 5, 1]
    mem = Z.new_memory(cfg)
    Z.run(cfg, w, toks, mem=mem)
    hs = {}

    def spy(name):
        orig = Z.MIXERS[name]

        def f(w_, p, c, eps, h, m, pos, shared):
            hs.setdefault(p, []).append(h.copy())
            return orig(w_, p, c, eps, h, m, pos, shared)
        return orig, f
    orig, f = spy("attention")
    Z.MIXERS["attention"] = f
    try:
        Z.run(cfg, w, toks)
    finally:
        Z.MIXERS["attention"] = orig
    plain = lambda i, t: (w["l%d.mix.v" % i] @ hs["l%d.mix." % i][t] + w["l%d.mix.v.b" % i]).reshape(4, 16)
    for t in range(len(toks)):
        assert np.allclose(mem["layers"][0]["v"][t], plain(0, t))                     # no blend asked for
        assert np.allclose(mem["layers"][1]["v"][t], plain(1, t))                     # the first blending layer keeps its own
        assert np.allclose(mem["layers"][2]["v"][t], plain(2, t))
        lam = float(w["l3.mix.vmix"])
        assert np.allclose(mem["layers"][3]["v"][t], (1 - lam) * plain(3, t) + lam * plain(1, t))


def test_router_groups_and_weights():
    s = np.array([0.9, 0.1, 0.1, 0.1,   0.5, 0.5, 0.1, 0.1,   0.45, 0.45, 0.45, 0.45,   0.2, 0.3, 0.1, 0.0])
    # group scores (two best): 1.0, 1.0, 0.9, 0.5 -> groups 0 and 1 stay (tie with the lower index first); 0.45s are out
    idx, wt = Z.route(s, 3, (4, 2))
    assert list(idx) == [0, 4, 5] and np.allclose(wt, np.array([0.9, 0.5, 0.5]) / 1.9)
    idx, wt = Z.route(s, 3, None)                              # without groups the 0.45s win places
    assert list(idx) == [0, 4, 5]
    idx, wt = Z.route(s, 4, None)
    assert list(idx) == [0, 4, 5, 8]
    idx, wt = Z.route(s, 2, (4, 1))
    assert list(idx) == [0, 1]                                 # only group 0: its second best is 0.1
    idx, wt = Z.route(s, 1, (16, 3))                           # groups of one expert: the score itself
    assert list(idx) == [0] and np.allclose(wt, [1.0])
    assert np.allclose(Z.route(np.zeros(4), 2, None)[1], 0.0)  # all-zero scores: the guard in the denominator


def test_one_stream_with_unit_coefficients_is_the_plain_residual():
    layers = [L(mlp="dense"), L(mlp="moe")]
    cfg, st, w = model(layers, seed=5, streams=None)
    cfg1, st1, w1 = model(layers, seed=5, streams=None)
    cfg1["streams"] = 1
    for i in range(2):
        for q in (1, 2):
            w1["l%d.hc%d.in" % (i, q)] = np.ones(1)
            w1["l%d.hc%d.out" % (i, q)] = np.ones(1)
            w1["l%d.hc%d.mix" % (i, q)] = np.ones((1, 1))
    toks = [1, 2, 3, 4, 5, 6]
    assert np.abs(Z.run(cfg, w, toks) - Z.run(cfg1, w1, toks)).max() < 1e-12


def test_streams_follow_the_written_update():
    cfg, st, w = model([L(mlp="dense")], seed=6, streams=2)
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][7] * cfg["embedding"]["scale"]
    xs = np.stack([x0, x0])
    a, b, M = w["l0.hc1.in"], w["l0.hc1.out"], w["l0.hc1.mix"]
    u = a[0] * xs[0] + a[1] * xs[1]
    h = (u - u.mean()) / np.sqrt(u.var() + eps) * w["l0.norm1"] + w["l0.norm1.b"]
    y = Z.attention(w, "l0.mix.", cfg["layers"][0]["mixer"], eps, h, {}, 0, {})
    new = np.stack([M[0, 0] * xs[0] + M[1, 0] * xs[1] + b[0] * y, M[0, 1] * xs[0] + M[1, 1] * xs[1] + b[1] * y])
    got = Z.sublayer(cfg, w, "l0.", 1, xs, lambda hh: Z.attention(w, "l0.mix.", cfg["layers"][0]["mixer"], eps, hh, {}, 0, {}))
    assert np.abs(got - new).max() < 1e-12


def test_sequence_memory_makes_the_cut_irrelevant():
    cfg, st, w = model([L(kv_heads=2, mlp="moe"), L(kv_heads=2, mlp="dense")], seed=8)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 96, 30)]
    whole = Z.run(cfg, w, toks)
    mem = Z.new_memory(cfg)
    parts = [Z.run(cfg, w, toks[a:b], mem=mem) for a, b in ((0, 7), (7, 8), (8, 30))]
    assert np.array_equal(np.concatenate(parts), whole)


def test_model_detection_and_info_without_a_gpu():
    cfg, st, w = model([L(), L(mlp="moe")], width=40, vocab=77)
    info = capi.info_from_st(st)
    assert info["version"] == capi.ARCH_ZUFULIX and info["num_layer"] == 2 and info["num_emb"] == 40 and info["num_vocab"] == 77
