"""GPU tests of the Zufulix family: the CUDA engine (through runtime.Model, i.e. the C ABI's infer / state / sampling entry
points and its own step packing) against the plain NumPy restatement in oracle/zufulix_numpy.py, on small random models made
here.  precision 1 (every product in f32) is held to a tight bound, precision 0 (bf16 tensor-core products) to the
restatement's own bf16 operand-rounding error.
"""
import json

import numpy as np
import pytest

from ai00_server_b200 import capi, runtime, synth
from oracle import zufulix_numpy as Z

pytestmark = pytest.mark.gpu

TIGHT = 2e-4        # f32 engine vs float64 oracle, relative to the logits' spread
L = synth.zufulix_layer


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())


def err(got, want):
    return float(row_errs(got, want).max())


class Bundle:
    def __init__(self, layers, precision=1, slots=3, kv_tokens=2048, kv_page=16, seed=0, chunk=128, tweak=None, **kw):
        self.cfg_bytes, self.st, self.w = synth.make_zufulix(layers, seed=seed, **kw)
        self.cfg = json.loads(self.cfg_bytes)
        if tweak:                                   # planted weights: edit the rounded arrays, write them again
            tweak(self.cfg, self.w)
            self.st = synth.pack_st_bf16({k: np.asarray(v, np.float32) for k, v in self.w.items()})
            self.w = {k: v.astype(np.float64) for k, v in Z.read_safetensors(bytes(self.st)).items()}
        self.m = runtime.Model(self.st, max_batch=slots, token_chunk_size=chunk, precision=precision, config=self.cfg_bytes,
                               kv_tokens=kv_tokens, kv_page=kv_page)
        self.vocab = self.cfg["vocab"]

    def tokens(self, n, seed=0):
        return [int(t) for t in np.random.default_rng(seed).integers(0, self.vocab, n)]

    def oracle(self, toks, layers=False):
        return Z.run(self.cfg, self.w, toks, layers=layers)

    def feed(self, slot, toks, opt=capi.OPTION_FULL):
        return self.m.infer_raw([slot], [len(toks)], list(toks), [opt])[0].copy()

    def close(self):
        self.m.close()


def bf16_floor(b, toks, want):
    """How far the restatement itself moves when every projection's activation operand is rounded to bfloat16: the yardstick
    for precision 0, whose tensor-core steps round exactly those operands."""
    Z.ROUND_OPERANDS = True
    try:
        return row_errs(b.oracle(toks), want)
    finally:
        Z.ROUND_OPERANDS = False


def assert_serving(got, want, floor):
    """Typical rows sit at the rounding floor; a rare row may sit far above it where operand rounding flips a close router
    decision (the restatement's own rounded run has such rows too), so rows are counted, not maximised."""
    e = row_errs(got, want)
    assert np.median(e) <= 2.0 * np.median(floor)
    assert (e > 3.0 * floor.max()).sum() <= max(1, 0.02 * len(e))


STACK = [L(kv_heads=2, mlp="dense"), L(kv_heads=2, vdim=16, mlp="moe"), L(heads=2, kv_heads=1, dim=8, vdim=32, bias_max=25, v_mix=False, mlp=None),
         L(kv_heads=2, v_mix=False, mlp="moe", experts=6, top=3, groups=None), L(kv_heads=2, mlp="moe", experts=6, groups=(3, 1))]


@pytest.fixture(scope="module")
def stack():
    b = Bundle(STACK)
    yield b
    b.close()


@pytest.fixture(scope="module")
def stack_ref(stack):
    toks = stack.tokens(150, 5)
    return toks, stack.oracle(toks)


# ---- each mechanism alone: one- or two-layer models, residual stream (sum of the streams) after every layer and logits ----
@pytest.mark.parametrize("layers,kw", [
    ([L(mlp=None)], {}),
    ([L(kv_heads=1, mlp=None)], {"rel_rows": 7}),
    ([L(mlp=None)], {"streams": None, "embed_scale": None}),
    ([L(mlp="dense")], {"streams": 1}),
    ([L(mlp="dense")], {"streams": 8}),
    ([L(mlp="moe", top=3)], {"streams": 16}),
    ([L(mlp="moe")], {}),
    ([L(mlp="moe", experts=6, top=6, groups=None)], {}),
    ([L(mlp="moe", experts=4, top=1, groups=(4, 2))], {}),
    ([L(kv_heads=2, v_mix=False, mlp=None), L(kv_heads=2, mlp=None), L(kv_heads=2, mlp="dense"), L(kv_heads=2, v_mix=None, mlp=None),
      L(kv_heads=2, heads=8, dim=8, mlp=None)], {}),
], ids=["attention", "attention-one-kv-head-odd-table", "plain-residual-unscaled-embedding", "one-stream", "eight-streams", "sixteen-streams", "experts-in-groups",
        "experts-all-chosen-no-groups", "groups-of-one-expert", "value-blend-first-layer-not-layer-0"])
def test_single_mechanisms(layers, kw):
    b = Bundle(layers, seed=3, **kw)
    try:
        toks = b.tokens(37, 1)
        b.m.debug_read("layers_on", 1)
        got = b.feed(0, toks)
        want, lay = b.oracle(toks, layers=True)
        buf = np.empty(len(layers) * 128 * b.cfg["width"], np.float32)
        capi.check(capi.lib().b200rwkv_debug_read(b.m._h, b"layers", capi.ptr(buf), buf.size), b.m._h)
        buf = buf.reshape(len(layers), 128, -1)[:, :len(toks)]
        for i in range(len(layers)):
            assert np.abs(buf[i] - lay[i]).max() <= 1e-4 * max(1.0, np.abs(lay[i]).max()), i
        assert err(got, want) <= TIGHT
    finally:
        b.close()


def test_whole_prompt_and_first_tokens(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    assert err(stack.feed(0, toks), want) <= TIGHT
    for n in (1, 2, 3):                                        # sequences of one to three tokens
        stack.m.state.reset(1)
        assert err(stack.feed(1, toks[:n]), want[:n]) <= TIGHT


def test_prefill_against_token_by_token(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    rows = np.concatenate([stack.feed(0, [t], capi.OPTION_LAST) for t in toks])
    assert err(rows, want) <= TIGHT


@pytest.mark.parametrize("cuts", [[2, 2, 3, 64, 5, 2, 31, 17, 16, 8], [15, 1, 1, 16, 17, 2, 98], [128, 22], [7] * 21 + [3], [1, 2] * 50])
def test_portions(stack, stack_ref, cuts):
    toks, want = stack_ref
    assert sum(cuts) == len(toks)
    stack.m.state.reset(0)
    out, at = [], 0
    for c in cuts:
        out.append(stack.feed(0, toks[at:at + c]))
        at += c
    assert err(np.concatenate(out), want) <= TIGHT


def test_unequal_batch_against_each_alone(stack):
    reqs = [stack.tokens(n, 10 + n) for n in (41, 1, 19)]
    want = [stack.oracle(r) for r in reqs]
    for s in range(3):
        stack.m.state.reset(s)
    rows = stack.m.infer_raw([0, 1, 2], [len(r) for r in reqs], [t for r in reqs for t in r], [capi.OPTION_FULL] * 3)
    for r, w in zip(rows, want):
        assert err(r, w) <= TIGHT
    nxt = [3, 4, 5]                                            # decode all three together: the rows do not depend on the company
    together = stack.m.infer_raw([0, 1, 2], [1, 1, 1], nxt, [capi.OPTION_LAST] * 3)
    for s in range(3):
        assert err(together[s], stack.oracle(reqs[s] + [nxt[s]])[-1:]) <= TIGHT
    # a prompt portion of one sequence beside single tokens of two others
    more = [stack.tokens(9, 77), [6], [7]]
    mixed = stack.m.infer_raw([1, 0, 2], [9, 1, 1], more[0] + more[1] + more[2], [capi.OPTION_FULL, capi.OPTION_LAST, capi.OPTION_LAST])
    assert err(mixed[0], stack.oracle(reqs[1] + [nxt[1]] + more[0])[-9:]) <= TIGHT
    assert err(mixed[1], stack.oracle(reqs[0] + [nxt[0]] + more[1])[-1:]) <= TIGHT
    assert err(mixed[2], stack.oracle(reqs[2] + [nxt[2]] + more[2])[-1:]) <= TIGHT


def test_pages_and_slots_reused():
    b = Bundle(STACK[:3], slots=2, kv_tokens=64, kv_page=8, seed=4)
    try:
        a, c = b.tokens(60, 1), b.tokens(50, 2)
        wa, wc = b.oracle(a), b.oracle(c)
        assert err(b.feed(0, a), wa) <= TIGHT
        with pytest.raises(capi.B200Error):                    # the pool is for 64 tokens (+ one partly filled page per slot)
            b.feed(1, c)
        b.m.state.reset(1)
        b.m.state.reset(0)                                     # pages go back ...
        assert err(b.feed(1, c), wc) <= TIGHT                  # ... and are used again by another slot, in another order
        b.m.state.reset(1)
        assert err(b.feed(0, c[:9]), wc[:9]) <= TIGHT
        assert err(b.feed(1, a[:33]), wa[:33]) <= TIGHT        # two live sequences share the pool
        assert err(b.feed(0, c[9:40]), wc[9:40]) <= TIGHT
    finally:
        b.close()


def sharp_buckets(cfg, w):
    """Bias tables whose neighbouring rows differ by many units: nearly all of a row's weight sits on the keys of ONE distance
    bucket, so a key counted into the bucket next door (or a distance clamped one off) changes the row completely."""
    rng = np.random.default_rng(0)
    for k in w:
        if k.endswith("mix.rel"):
            rows, H = w[k].shape
            w[k] = np.stack([rng.permutation(rows) for _ in range(H)], 1) * 6.0


@pytest.mark.parametrize("rows,far", [(8, 20), (8, 16), (9, 33), (2, 3), (16, 17), (6, 70)])
def test_bucket_edges_far_distances_and_page_borders(rows, far):
    layers = [L(heads=2, kv_heads=1, bias_max=far, mlp=None), L(heads=4, kv_heads=4, bias_max=far, v_mix=False, mlp="dense")]
    b = Bundle(layers, kv_page=16, seed=6, rel_rows=rows, tweak=sharp_buckets)
    try:
        toks = b.tokens(120, 3)
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT             # in a prompt
        b.m.state.reset(1)
        out = [b.feed(1, toks[:13])]
        for i in range(13, 90):                                # decoded alone while the first keys cross every bucket's edge, `far`
            out.append(b.feed(1, [toks[i]], capi.OPTION_LAST))  # itself, and the page borders at 16, 32, 48, 64, 80
        out.append(b.feed(1, toks[90:93]))
        out.append(b.feed(1, toks[93:]))                       # portions that start and end inside pages and buckets
        assert err(np.concatenate(out), want) <= TIGHT
    finally:
        b.close()


def test_the_bias_edges_matter():
    # the inputs do what the test above needs: distances counted one off, or clamped one early, give other rows altogether
    layers = [L(heads=2, kv_heads=1, bias_max=20, mlp=None)]
    cfgb, st, w = synth.make_zufulix(layers, seed=6, rel_rows=8)
    cfg = json.loads(cfgb)
    sharp_buckets(cfg, w)
    toks = [int(t) for t in np.random.default_rng(3).integers(0, 96, 40)]
    a = Z.run(cfg, w, toks)
    orig = Z.distance_bucket
    try:
        Z.distance_bucket = lambda n, rows, far: orig(n + 1, rows, far)
        off = Z.run(cfg, w, toks)
        Z.distance_bucket = lambda n, rows, far: orig(min(n, 12), rows, far)
        early = Z.run(cfg, w, toks)
    finally:
        Z.distance_bucket = orig
    assert err(a[1:], off[1:]) > 1000 * TIGHT
    assert err(a[:13], early[:13]) == 0.0 and err(a[14:], early[14:]) > 1000 * TIGHT


def plant_far_key(cfg, w):
    """Every query of layer 0 points along the key of token 1, which stands at position 1 only: that key outscores every other
    by a wide margin at every later position, near or hundreds of tokens away."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][1] * cfg["embedding"]["scale"]
    u = w["l0.hc1.in"].sum() * x0
    h = Z.layer_norm(u, w["l0.norm1"], w["l0.norm1.b"], eps)
    k = w["l0.mix.k"] @ h + w["l0.mix.k.b"]
    w["l0.mix.q.b"] = 50.0 * k / np.linalg.norm(k)
    w["l0.mix.rel"] = np.zeros_like(w["l0.mix.rel"])


def test_a_far_key_carries_the_row():
    b = Bundle([L(heads=1, kv_heads=1, dim=16, scale=2.0, mlp=None)], seed=11, vocab=8, tweak=plant_far_key)
    try:
        toks = [0, 1] + [int(t) for t in np.random.default_rng(1).integers(2, 8, 400)]
        c, p = b.cfg["layers"][0]["mixer"], "l0.mix."
        eps = b.cfg["norm"]["eps"]
        hs = [Z.layer_norm(b.w["l0.hc1.in"].sum() * b.w["embed"][t] * b.cfg["embedding"]["scale"], b.w["l0.norm1"], b.w["l0.norm1.b"], eps)
              for t in toks]
        K = np.stack([Z.unit_rms(b.w[p + "k"] @ h + b.w[p + "k.b"], eps) for h in hs])
        wins = 0
        for t in range(10, 402):
            q = Z.unit_rms(b.w[p + "q"] @ hs[t] + b.w[p + "q.b"], eps)
            s = K[: t + 1] @ q * c["scale"]
            e = np.exp(s - s.max())
            wins += int(e[1] / e.sum() > 0.9)
        assert wins > 380                                      # the inputs do what the test needs: the rows hang on key 1
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT
        b.m.state.reset(1)
        b.feed(1, toks[:250], capi.OPTION_NONE)
        rows = np.concatenate([b.feed(1, [t], capi.OPTION_LAST) for t in toks[250:]])
        assert err(rows, want[250:]) <= TIGHT
    finally:
        b.close()


def test_long_decoding(stack):
    toks = stack.tokens(200, 9)
    want = stack.oracle(toks)
    stack.m.state.reset(0)
    out = [stack.feed(0, toks[:60])] + [stack.feed(0, [t], capi.OPTION_LAST) for t in toks[60:]]
    assert err(np.concatenate(out), want) <= TIGHT


ODD = [L(heads=3, kv_heads=3, dim=10, vdim=20, bias_max=7.5, v_mix=False, mlp="moe", experts=3, top=3, ff=10, groups=(1, 1)),
       L(heads=6, kv_heads=2, dim=6, vdim=12, bias_max=300, v_mix=False, mlp="moe", experts=1, top=1, ff=7, groups=None),
       L(heads=1, kv_heads=1, dim=8, vdim=5, mlp=None),
       L(heads=5, kv_heads=1, dim=40, vdim=5, mlp="dense", ff=9),
       L(heads=6, kv_heads=3, dim=6, vdim=10, v_mix=False, mlp="moe", experts=9, top=4, ff=5, groups=(3, 2)),
       L(heads=1, kv_heads=1, dim=34, vdim=5, bias_max=11, mlp="dense", ff=3)]


@pytest.mark.parametrize("precision", [1, 0])
def test_other_sizes(precision):
    b = Bundle(ODD, precision=precision, width=50, vocab=61, seed=7, streams=5, rel_rows=9)
    try:
        toks = b.tokens(90, 4)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:70]), b.feed(0, toks[70:72])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[72:]])
        if precision == 1:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


WIDE = [L(heads=8, kv_heads=2, dim=64, vdim=64, bias_max=128, mlp="moe", experts=8, top=2, ff=64),
        L(heads=4, kv_heads=4, dim=128, vdim=64, bias_max=64, v_mix=None, mlp="dense", ff=320),
        L(heads=8, kv_heads=2, dim=64, vdim=64, bias_max=1000, mlp="dense", ff=320)]


@pytest.mark.parametrize("precision", [1, 0])
def test_wider_layers(precision):
    b = Bundle(WIDE, precision=precision, width=256, vocab=300, seed=5, streams=2, rel_rows=32)
    try:
        toks = b.tokens(140, 6)
        want = b.oracle(toks)
        got = np.concatenate([b.feed(0, toks[:100])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[100:120]] + [b.feed(0, toks[120:])])
        if precision == 1:
            assert err(got, want) <= TIGHT
        else:
            assert_serving(got, want, bf16_floor(b, toks, want))
    finally:
        b.close()


# head sizes and head ratios around the attention kernel's two forms (registers: multiples of four up to 128; tiles in shared
# memory: everything else), with 1 to 8 query heads per key / value head, in prompts of several chunks and in decoding
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(1, 1, 4, 4), (2, 2, 128, 128), (3, 1, 12, 100), (5, 1, 64, 8), (8, 1, 32, 32), (12, 4, 20, 24),
                                                     (6, 3, 136, 16), (2, 1, 16, 132), (7, 7, 9, 6), (4, 2, 30, 34), (32, 32, 8, 8), (40, 20, 4, 64),
                                                     (16, 16, 64, 64)])
def test_head_shapes(heads, kv_heads, dim, vdim):
    layers = [L(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, bias_max=50, mlp=None),
              L(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, bias_max=13, mlp="dense")]
    b = Bundle(layers, seed=heads + dim, width=40, vocab=50, rel_rows=10, kv_page=8)
    try:
        toks = b.tokens(100, 2)
        want = b.oracle(toks)
        assert err(b.feed(0, toks), want) <= TIGHT
        out = [b.feed(1, toks[:41])] + [b.feed(1, [t], capi.OPTION_LAST) for t in toks[41:80]] + [b.feed(1, toks[80:83]), b.feed(1, toks[83:])]
        assert err(np.concatenate(out), want) <= TIGHT
    finally:
        b.close()


def random_model(seed):
    """A configuration drawn at random: every size, count and constant of the family varies, layers differ from one another."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    blend_shape = (pick(1, 2, 3), pick(4, 8, 10, 24))          # (kv_heads, vdim) shared by the layers that blend values
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        blend = bool(rng.integers(2))
        kv, vdim = blend_shape if blend else (pick(1, 2, 4), pick(4, 6, 16, 20, 36))
        mlp = pick("dense", "moe", None)
        experts, groups = pick((4, (2, 1)), (6, (3, 2)), (8, (8, 3)), (5, None), (9, (3, 3)), (2, (1, 1)))
        per_kept = experts if not groups else experts // groups[0] * groups[1]
        layers.append(L(heads=kv * pick(1, 2, 3, 4), kv_heads=kv, dim=pick(4, 8, 12, 18, 32, 40), vdim=vdim, scale=float(rng.uniform(0.1, 0.6)),
                        bias_max=float(pick(21, 37.5, 64, 150, 1000)), v_mix=pick(True, None) if blend else pick(False, None), mlp=mlp,
                        ff=pick(8, 24, 33), experts=experts, top=int(rng.integers(1, min(per_kept, 4) + 1)), groups=groups))
    kw = dict(width=pick(24, 40, 56, 100), vocab=pick(31, 64, 150), streams=pick(None, 1, 2, 4, 6), embed_scale=pick(None, 0.25, 1.5),
              rel_rows=pick(2, 5, 8, 13, 20, 32), eps=pick(1e-5, 1e-6, 1e-3))
    return layers, kw


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(seed):
    layers, kw = random_model(seed)
    b = Bundle(layers, seed=seed, kv_page=int(np.random.default_rng(seed).choice([4, 8, 16, 64])), **kw)
    try:
        toks = b.tokens(150, seed)
        want = b.oracle(toks)
        assert err(b.feed(0, toks), want) <= TIGHT                                        # a prompt of two steps
        out = [b.feed(1, toks[:57]), b.feed(1, toks[57:59])] + [b.feed(1, [t], capi.OPTION_LAST) for t in toks[59:110]] + [b.feed(1, toks[110:])]
        assert err(np.concatenate(out), want) <= TIGHT                                    # portions, then decoding, then a portion
    finally:
        b.close()


def test_serving_precision(stack_ref):
    toks, want = stack_ref
    b = Bundle(STACK, precision=0)
    try:
        floor = bf16_floor(b, toks, want)
        assert_serving(b.feed(0, toks), want, floor)
        b.m.state.reset(0)
        out = [b.feed(0, toks[:50])] + [b.feed(0, [t], capi.OPTION_LAST) for t in toks[50:90]] + [b.feed(0, toks[90:])]
        assert_serving(np.concatenate(out), want, floor)
    finally:
        b.close()


def test_steps_of_up_to_512_tokens_and_long_contexts(stack_ref):
    toks, want = stack_ref
    b = Bundle(STACK, chunk=512)
    try:
        long = toks + b.tokens(550, 8)                         # several key tiles per cluster rank, three steps
        ref = b.oracle(long)
        assert err(b.feed(0, long), ref) <= TIGHT
        b.m.state.reset(0)
        b.feed(0, long[:690], capi.OPTION_NONE)
        rows = np.concatenate([b.feed(0, [t], capi.OPTION_LAST) for t in long[690:]])     # decoding with the keys split over a cluster
        assert err(rows, ref[690:]) <= TIGHT
    finally:
        b.close()


def test_greedy_generation_through_the_runtime(stack):
    # the framework's own entry point: Runtime.infer (its token budget and slot batching) + the GPU sampling front half
    prompt = stack.tokens(21, 12)
    mem = Z.new_memory(stack.cfg)
    row = Z.run(stack.cfg, stack.w, prompt, mem=mem)[-1]
    want = []
    for _ in range(12):
        want.append(int(row.argmax()))
        row = Z.run(stack.cfg, stack.w, [want[-1]], mem=mem)[-1]
    stack.m.state.reset(0)
    inp = runtime.RnnInput([runtime.RnnInputBatch(list(prompt), runtime.RnnOption.Last)], token_chunk_size=8)
    got = []
    while len(got) < 12:
        inp, out = stack.m.runtime.infer(inp)
        if out[0].is_empty():
            continue
        ids, probs = stack.m.sample_topk([0], top_k=4)
        assert int(ids[0, 0]) == int(out[0].data[0].argmax())
        got.append(int(ids[0, 0]))
        inp = runtime.RnnInput([runtime.RnnInputBatch([got[-1]], runtime.RnnOption.Last)], token_chunk_size=8)
    assert got == want


def test_state_snapshots_and_host_round_trip(stack, stack_ref):
    toks, want = stack_ref
    m = stack.m
    m.state.reset(0)
    stack.feed(0, toks[:50], capi.OPTION_LAST)
    snap = m.state.read(0)
    host = m.state.back(0)
    assert int(host.reshape(-1)[0]) == 50
    a = stack.feed(0, toks[50:90])
    m.state.write(snap, 1)                                     # device snapshot into another slot
    b_ = stack.feed(1, toks[50:90])
    m.state.load(host, 2)                                      # host tensor into a third
    c = stack.feed(2, toks[50:90])
    assert err(a, want[50:90]) <= TIGHT
    assert np.array_equal(a, b_) and np.array_equal(a, c)
    snap.free()
