"""CPU tests of the Pasopel pieces that need no GPU: the NumPy restatement against independent formulations of the same
mechanisms (batched masked attention over materialised keys / values with the block means appended as extra keys, the latent
attention with per-head keys / values rebuilt for the whole sequence, a direct convolution, hand-made router cases, the loop
written out by hand), invariance of the restatement to how a sequence is cut, the synthetic-model writer, and the host-only
model detection of the C ABI."""
import json

import numpy as np

from ai00_server_b200 import capi, synth
from oracle import pasopel_numpy as P

L = synth.pasopel_layer


def model(layers, **kw):
    cfgb, st, w = synth.make_pasopel(layers, **kw)
    return json.loads(cfgb), st, w


def test_writer_round_trips():
    cfg, st, w = model([L("attention"), L("latent_attention", mlp="moe"), L("attention", mlp=None, pool=0)], seed=2, loop=(1, 3, 2))
    back = P.read_safetensors(bytes(st))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], w[k]), k
    assert "l2.norm2" not in w and "l1.mix.o.b" not in w and "l0.mix.v" not in w and "head" not in w
    assert w["loop.step"].shape == (2, 64) and "pool" not in cfg["layers"][2]["mixer"]["mask"]


def test_visibility_sets():
    # window 5, blocks of 3: position 9 sees tokens 5..9 and the blocks that end at or before position 4: only block 0 (0..2)
    assert list(P.visible_tokens(9, 5)) == [5, 6, 7, 8, 9] and list(P.visible_blocks(9, 5, 3)) == [0]
    assert list(P.visible_blocks(10, 5, 3)) == [0, 1]           # block 1 = 3..5 ends at 5 = 10 - 5
    assert list(P.visible_blocks(7, 5, 3)) == [0] and list(P.visible_blocks(6, 5, 3)) == []
    assert list(P.visible_tokens(3, 5)) == [0, 1, 2, 3] and list(P.visible_blocks(3, 5, 3)) == []
    assert list(P.visible_blocks(50, 5, 0)) == []
    for i in range(40):                                         # no token is seen twice; tokens between block and window are unseen
        covered = [b * 3 + u for b in P.visible_blocks(i, 5, 3) for u in range(3)] + list(P.visible_tokens(i, 5))
        assert len(set(covered)) == len(covered) and max(covered) == i


def test_sink_softmax():
    s = np.array([0.3, -1.0, 2.0])
    w = P.sink_softmax(s, 0.5)
    e = np.exp(s)
    assert np.allclose(w, e / (e.sum() + np.exp(0.5))) and w.sum() < 1.0
    assert np.allclose(P.sink_softmax(s, -1e9), e / e.sum())
    assert P.sink_softmax(s, 80.0).sum() < 1e-30                # a dominant sink takes (nearly) all the weight, nothing overflows


def test_convolution_is_causal_and_starts_from_zeros():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((5, 4))
    u = rng.standard_normal((9, 5))
    hist, got = [], []
    for t in range(9):
        hist.append(u[t])
        hist = hist[-4:]
        got.append(P.short_conv(w, [np.zeros(5)] * (4 - len(hist)) + hist))
    want = np.zeros((9, 5))
    for t in range(9):
        for j in range(4):
            if t - 3 + j >= 0:
                want[t] += w[:, j] * u[t - 3 + j]
    assert np.abs(np.array(got) - want).max() < 1e-12


def test_rotation_turns_neighbouring_entries():
    x = np.arange(1.0, 9.0)
    y = P.rotate_pairs(x, 3, 4, 100.0)
    assert np.array_equal(y[4:], x[4:])
    for i in range(2):
        a = 3 * 100.0 ** (-2.0 * i / 4)
        z = complex(x[2 * i], x[2 * i + 1]) * complex(np.cos(a), np.sin(a))
        assert abs(y[2 * i] - z.real) < 1e-12 and abs(y[2 * i + 1] - z.imag) < 1e-12
    # relative positions: the score of two rotated vectors depends on the distance only
    q, k = np.array([0.3, -1.2, 0.8, 0.1]), np.array([1.1, 0.4, -0.6, 0.9])
    assert abs(P.rotate_pairs(q, 17, 4, 50.0) @ P.rotate_pairs(k, 11, 4, 50.0) - P.rotate_pairs(q, 106, 4, 50.0) @ P.rotate_pairs(k, 100, 4, 50.0)) < 1e-9


def test_attention_equals_a_batched_form():
    H, G, dk, win, pool, taps, n = 6, 2, 8, 7, 3, 3, 31
    cfg, st, w = model([L("attention", heads=H, kv_heads=G, dim=dk, window=win, pool=pool, conv=taps, mlp=None)], width=24, seed=1)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    hs = np.random.default_rng(3).standard_normal((n, 24))
    mem = P.new_layer_memory(cfg["layers"][0])
    got = np.array([P.attention(w, p, c, 1e-5, h, mem, t) for t, h in enumerate(hs)])
    conv = lambda u, cw: np.stack([sum(cw[:, j] * (u[t - taps + 1 + j] if t - taps + 1 + j >= 0 else 0.0) for j in range(taps)) for t in range(n)])
    q = conv(hs @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).reshape(n, H, dk)
    v = conv(hs @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).reshape(n, G, dk)
    q = q / np.sqrt((q ** 2).mean(-1, keepdims=True) + 1e-5)
    k = v / np.sqrt((v ** 2).mean(-1, keepdims=True) + 1e-5)
    nb = n // pool
    kb = k[: nb * pool].reshape(nb, pool, G, dk).mean(1)        # block means of the normalised keys and of the values
    vb = v[: nb * pool].reshape(nb, pool, G, dk).mean(1)
    K, V = np.concatenate([kb, k]), np.concatenate([vb, v])     # blocks first, then tokens: one softmax over both
    i = np.arange(n)[:, None]
    mask = np.concatenate([(np.arange(nb)[None, :] + 1) * pool - 1 <= i - win, (np.arange(n)[None, :] <= i) & (np.arange(n)[None, :] > i - win)], 1)
    out = np.zeros((n, H, dk))
    for h in range(H):
        s = np.where(mask, q[:, h] @ K[:, h // (H // G)].T * c["scale"], -np.inf)
        e = np.exp(s - s.max(1, keepdims=True))
        den = e.sum(1, keepdims=True) + np.exp(w[p + "sink"][h] - s.max(1, keepdims=True))
        out[:, h] = (e / den) @ V[:, h // (H // G)]
    want = (out.reshape(n, -1) * P.sigmoid(hs @ w[p + "g"].T)) @ w[p + "o"].T + w[p + "o.b"]
    assert np.abs(got - want).max() < 1e-10


def test_latent_attention_equals_a_batched_form():
    H, dn, dr, dv, rk, win, n = 3, 6, 4, 5, 10, 6, 20
    cfg, st, w = model([L("latent_attention", heads=H, dim=dn, rot_dim=dr, rot_dims=2, vdim=dv, kv_rank=rk, q_rank=7, window=win, base=50.0, mlp=None)],
                       width=24, seed=4)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    hs = np.random.default_rng(5).standard_normal((n, 24))
    mem = P.new_layer_memory(cfg["layers"][0])
    got = np.array([P.latent_attention(w, p, c, 1e-5, h, mem, t) for t, h in enumerate(hs)])
    rms = lambda x: x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-5)
    q = ((rms(hs @ w[p + "dq"].T) * w[p + "dq.norm"]) @ w[p + "uq"].T).reshape(n, H, dn + dr)
    kv = hs @ w[p + "dkv"].T
    lat = rms(kv[:, :rk]) * w[p + "dkv.norm"]
    turn = lambda x, pos: np.stack([P.rotate_pairs(x[t], pos[t], 2, 50.0) for t in range(len(x))])
    kr = turn(kv[:, rk:], np.arange(n))
    k = np.concatenate([(lat @ w[p + "uk"].T).reshape(n, H, dn), np.repeat(kr[:, None], H, 1)], -1)
    v = (lat @ w[p + "uv"].T).reshape(n, H, dv)
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    mask = (j <= i) & (j > i - win)
    out = np.zeros((n, H, dv))
    for h in range(H):
        qh = np.concatenate([q[:, h, :dn], turn(q[:, h, dn:], np.arange(n))], -1)
        s = np.where(mask, qh @ k[:, h].T * c["scale"], -np.inf)
        e = np.exp(s - s.max(1, keepdims=True))
        out[:, h] = (e / (e.sum(1, keepdims=True) + np.exp(w[p + "sink"][h] - s.max(1, keepdims=True)))) @ v[:, h]
    want = (out.reshape(n, -1) * P.sigmoid(hs @ w[p + "g"].T)) @ w[p + "o"].T
    assert np.abs(got - want).max() < 1e-10


def test_router_cases():
    f = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 3}}
    w = {"r.router": np.eye(4), "r.router.b": np.array([0.0, 0.0, 0.5, 0.0])}
    chosen, wt = P.route(w, "r.", f, np.array([1.0, 2.0, 1.6, -1.0]))
    assert chosen == [2, 1]                                     # the bias is part of the logit: 2.1 beats 2.0
    assert np.allclose(wt, np.exp([2.1, 2.0]) / np.exp([2.1, 2.0]).sum()) and abs(wt.sum() - 1.0) < 1e-12
    chosen, _ = P.route(w, "r.", f, np.array([1.0, 1.0, 0.5, 1.0]))
    assert chosen == [0, 1]                                     # ties go to the lower index
    f["router"]["top"] = 1
    chosen, wt = P.route(w, "r.", f, np.array([0.0, 3.0, 0.0, 0.0]))
    assert chosen == [1] and wt.tolist() == [1.0]               # a single winner has weight one


def test_feed_forward_forms():
    cfg, st, w = model([L("attention", mlp="dense", ff=5), L("attention", mlp="moe", experts=3, top=3, ff=4, shared_ff=6)], width=16, seed=3)
    h = np.random.default_rng(1).standard_normal(16)
    d = P.feed_forward(w, "l0.mlp.", cfg["layers"][0]["mlp"], h)
    assert np.allclose(d, w["l0.mlp.down"] @ np.maximum(w["l0.mlp.up"] @ h, 0) ** 2)
    z = w["l1.mlp.router"] @ h + w["l1.mlp.router.b"]
    g = np.exp(z - z.max()) / np.exp(z - z.max()).sum()         # all experts chosen: the plain softmax
    unit = lambda q: w[q + "down"] @ ((lambda a: a / (1 + np.exp(-a)))(w[q + "gate"] @ h) * (w[q + "up"] @ h))
    want = sum(g[e] * unit("l1.mlp.e%d." % e) for e in range(3)) + unit("l1.mlp.shared.")
    assert np.allclose(P.feed_forward(w, "l1.mlp.", cfg["layers"][1]["mlp"], h), want)


def test_layer_runs_and_the_loop_written_out():
    cfg, st, w = model([L("attention", mlp=None), L("latent_attention", mlp="dense"), L("attention", mlp="dense")], seed=6, loop=(1, 3, 2), softcap=None)
    assert P.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    cfg0 = dict(cfg)
    del cfg0["loop"]
    assert P.layer_runs(cfg0) == [(0, None), (1, None), (2, None)]
    assert P.layer_runs(dict(cfg, loop={"start": 0, "stop": 3, "times": 1})) == [(0, 0), (1, None), (2, None)]
    # one token by hand: every run has a memory of its own, pass t adds step[t], passes after the first add the embedding row again
    eps, x0 = cfg["norm"]["eps"], w["embed"][5]
    mems = [P.new_layer_memory(cfg["layers"][i]) for i in (0, 1, 2, 1, 2)]
    lay = lambda x, i, mem: (lambda y: y + (P.feed_forward(w, "l%d.mlp." % i, cfg["layers"][i]["mlp"], P.offset_norm(y, w["l%d.norm2" % i], eps))
                                            if cfg["layers"][i]["mlp"] else 0.0))(
        x + P.MIXERS[cfg["layers"][i]["type"]](w, "l%d.mix." % i, cfg["layers"][i]["mixer"], eps, P.offset_norm(x, w["l%d.norm1" % i], eps), mem, 0))
    x = lay(x0, 0, mems[0])
    x = lay(lay(x + w["loop.step"][0], 1, mems[1]), 2, mems[2])
    x = lay(lay(x + x0 + w["loop.step"][1], 1, mems[3]), 2, mems[4])
    want = w["embed"] @ P.offset_norm(x, w["final.norm"], eps)
    assert np.abs(P.run(cfg, w, [5])[0] - want).max() < 1e-10
    capped = P.run(dict(cfg, logit_softcap=3.0), w, [5])[0]
    assert np.allclose(capped, 3.0 * np.tanh(want / 3.0)) and np.abs(capped).max() < 3.0


def test_offset_norm():
    x = np.array([3.0, -4.0])
    assert np.allclose(P.offset_norm(x, np.array([0.0, 0.5]), 0.0), x / np.sqrt(12.5) * np.array([1.0, 1.5]))


def test_sequence_memory_makes_the_cut_irrelevant():
    cfg, st, w = model([L("attention", kv_heads=2, mlp="moe"), L("latent_attention", mlp="dense")], seed=8, loop=(0, 2, 2))
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 96, 30)]
    whole = P.run(cfg, w, toks)
    mem = P.new_memory(cfg)
    parts = [P.run(cfg, w, toks[a:b], mem=mem) for a, b in ((0, 7), (7, 8), (8, 30))]
    assert np.array_equal(np.concatenate(parts), whole)


def test_model_detection_and_info_without_a_gpu():
    cfg, st, w = model([L("attention"), L("latent_attention", mlp="moe")], width=40, vocab=77)
    info = capi.info_from_st(st)
    assert info["version"] == capi.ARCH_PASOPEL and info["num_layer"] == 2 and info["num_emb"] == 40 and info["num_vocab"] == 77
