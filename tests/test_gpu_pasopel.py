"""GPU tests of the Pasopel family: the CUDA engine (through runtime.Model, i.e. the C ABI's infer / state / sampling entry
points and its own step packing) against the plain NumPy restatement in oracle/pasopel_numpy.py, on small random models made
here.  precision 1 (every product in f32) is held to a tight bound, precision 0 (bf16 tensor-core products) to the
restatement's own bf16 operand-rounding error.
"""
import json

import numpy as np
import pytest

from ai00_server_b200 import capi, runtime, synth
from oracle import pasopel_numpy as P

pytestmark = pytest.mark.gpu

TIGHT = 2e-4        # f32 engine vs float64 oracle, relative to the logits' spread
L = synth.pasopel_layer
A, M = "attention", "latent_attention"


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())


def err(got, want):
    return float(row_errs(got, want).max())


class Bundle:
    def __init__(self, layers, precision=1, slots=3, kv_tokens=2048, kv_page=16, seed=0, chunk=128, tweak=None, **kw):
        self.cfg_bytes, self.st, self.w = synth.make_pasopel(layers, seed=seed, **kw)
        self.cfg = json.loads(self.cfg_bytes)
        if tweak:                                   # planted weights: edit the rounded arrays, write them again
            tweak(self.cfg, self.w)
            self.cfg_bytes = json.dumps(self.cfg).encode()
            self.st = synth.pack_st_bf16({k: np.asarray(v, np.float32) for k, v in self.w.items()})
            self.w = {k: v.astype(np.float64) for k, v in P.read_safetensors(bytes(self.st)).items()}
        self.m = runtime.Model(self.st, max_batch=slots, token_chunk_size=chunk, precision=precision, config=self.cfg_bytes,
                               kv_tokens=kv_tokens, kv_page=kv_page)
        self.vocab = self.cfg["vocab"]
        self.runs = len(P.layer_runs(self.cfg))

    def tokens(self, n, seed=0):
        return [int(t) for t in np.random.default_rng(seed).integers(0, self.vocab, n)]

    def oracle(self, toks, layers=False):
        return P.run(self.cfg, self.w, toks, layers=layers)

    def feed(self, slot, toks, opt=capi.OPTION_FULL):
        return self.m.infer_raw([slot], [len(toks)], list(toks), [opt])[0].copy()

    def close(self):
        self.m.close()


def bf16_floor(b, toks, want):
    """How far the restatement itself moves when every projection's activation operand is rounded to bfloat16: the yardstick
    for precision 0, whose tensor-core steps round exactly those operands."""
    P.ROUND_OPERANDS = True
    try:
        return row_errs(b.oracle(toks), want)
    finally:
        P.ROUND_OPERANDS = False


def assert_serving(got, want, floor):
    """Typical rows sit at the rounding floor; a rare row may sit far above it where operand rounding flips a close router
    decision (the restatement's own rounded run has such rows too), so rows are counted, not maximised."""
    e = row_errs(got, want)
    assert np.median(e) <= 2.0 * np.median(floor)
    assert (e > 3.0 * floor.max()).sum() <= max(1, 0.02 * len(e))


# windows, blocks and pages that share no edge; the loop covers the middle of the stack
STACK = [L(A, kv_heads=2, window=11, pool=3, mlp="dense"),
         L(M, window=9, mlp="moe"),
         L(A, heads=6, kv_heads=1, dim=8, window=20, pool=5, conv=2, mlp="moe", experts=6, top=3),
         L(M, heads=2, dim=8, vdim=24, rot_dim=12, rot_dims=6, kv_rank=16, q_rank=9, window=33, mlp=None),
         L(A, kv_heads=4, window=7, pool=0, conv=4, mlp="moe", experts=5, top=1, shared_ff=0)]
STACK_KW = dict(loop=(1, 4, 3))


@pytest.fixture(scope="module")
def stack():
    b = Bundle(STACK, **STACK_KW)
    yield b
    b.close()


@pytest.fixture(scope="module")
def stack_ref(stack):
    toks = stack.tokens(150, 5)
    return toks, stack.oracle(toks)


# ---- each mechanism alone: small models, residual stream after every layer run and logits ----
@pytest.mark.parametrize("layers,kw", [
    ([L(A, mlp=None)], {"loop": None, "softcap": None}),
    ([L(A, kv_heads=1, pool=0, mlp=None)], {"loop": None}),
    ([L(A, kv_heads=2, conv=1, window=5, pool=2, mlp=None)], {"loop": None}),
    ([L(A, window=1, pool=1, mlp=None)], {"loop": None}),
    ([L(A, window=6, pool=9, mlp=None)], {"loop": None}),
    ([L(A, window=4, pool=20, mlp=None)], {"loop": None, "kv_page": 8}),
    ([L(M, mlp=None)], {"loop": None, "softcap": None}),
    ([L(M, rot_dims=0, vdim=8, window=3, mlp=None)], {"loop": None}),
    ([L(M, rot_dim=6, rot_dims=2, q_rank=5, kv_rank=33, mlp=None)], {"loop": None}),
    ([L(A, mlp="dense")], {"loop": None}),
    ([L(M, mlp="moe")], {"loop": None}),
    ([L(A, mlp="moe", experts=6, top=6, shared_ff=0)], {"loop": None}),
    ([L(M, mlp="moe", experts=1, top=1)], {"loop": None}),
    ([L(A, mlp=None), L(M, mlp=None)], {"loop": (0, 2, 3)}),
    ([L(A, mlp="dense"), L(M, mlp="moe"), L(A, mlp="moe")], {"loop": (1, 2, 2)}),
    ([L(A, mlp="moe"), L(M, mlp="moe")], {"loop": (1, 2, 1)}),
    ([L(M, mlp="dense"), L(A, mlp="moe")], {"loop": (0, 1, 4), "softcap": 2.0}),
], ids=["attention", "attention-no-blocks", "attention-one-tap", "window-of-one-blocks-of-one", "blocks-longer-than-window", "blocks-longer-than-a-page",
        "latent", "latent-no-rotation", "latent-partial-rotation", "dense", "experts", "experts-all-chosen-no-shared", "one-expert",
        "loop-whole-stack", "loop-in-the-middle", "loop-once-at-the-end", "loop-first-layer-tight-cap"])
def test_single_mechanisms(layers, kw):
    kw = dict(kw)
    page = kw.pop("kv_page", 16)
    b = Bundle(layers, seed=3, kv_page=page, **kw)
    try:
        toks = b.tokens(61, 1)
        b.m.debug_read("layers_on", 1)
        got = b.feed(0, toks)
        want, lay = b.oracle(toks, layers=True)
        buf = np.empty(b.runs * 128 * b.cfg["width"], np.float32)
        capi.check(capi.lib().b200rwkv_debug_read(b.m._h, b"layers", capi.ptr(buf), buf.size), b.m._h)
        buf = buf.reshape(b.runs, 128, -1)[:, :len(toks)]
        assert lay.shape[0] == b.runs
        for i in range(b.runs):
            assert np.abs(buf[i] - lay[i]).max() <= 1e-4 * max(1.0, np.abs(lay[i]).max()), i
        assert err(got, want) <= TIGHT
    finally:
        b.close()


def test_whole_prompt_and_first_tokens(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    assert err(stack.feed(0, toks), want) <= TIGHT
    for n in (1, 2, 3, 4):                                     # sequences shorter than any convolution, window or block
        stack.m.state.reset(1)
        assert err(stack.feed(1, toks[:n]), want[:n]) <= TIGHT


def test_prefill_against_token_by_token(stack, stack_ref):
    toks, want = stack_ref
    stack.m.state.reset(0)
    rows = np.concatenate([stack.feed(0, [t], capi.OPTION_LAST) for t in toks])
    assert err(rows, want) <= TIGHT


@pytest.mark.parametrize("cuts", [[2, 2, 3, 64, 5, 2, 31, 17, 16, 8], [15, 1, 1, 16, 17, 2, 98], [128, 22], [7] * 21 + [3], [1, 2] * 50, [2] * 75])
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
    b = Bundle(STACK[:3], slots=2, kv_tokens=64, kv_page=8, seed=4, loop=(0, 2, 2))
    try:
        a, c = b.tokens(60, 1), b.tokens(50, 2)
        wa, wc = b.oracle(a), b.oracle(c)
        assert err(b.feed(0, a), wa) <= TIGHT
        with pytest.raises(capi.B200Error):                    # the pool is for 64 tokens (+ one partly filled page per slot)
            b.feed(1, c)
        b.m.state.reset(1)
        b.m.state.reset(0)                                     # pages go back ...
        assert err(b.feed(1, c), wc) <= TIGHT                  # ... and are used again by another slot, in another order:
        b.m.state.reset(1)                                     # stale rows, block means and convolution tails must not show
        assert err(b.feed(0, c[:9]), wc[:9]) <= TIGHT
        assert err(b.feed(1, a[:33]), wa[:33]) <= TIGHT        # two live sequences share the pool
        assert err(b.feed(0, c[9:40]), wc[9:40]) <= TIGHT
    finally:
        b.close()


# ---- edges: peaked softmaxes, so that one key seen too much or too little changes the row ----
def sharpen(cfg, w):
    """Scores many units apart: nearly all of a row's weight sits on its best key (or block), wherever that is."""
    for l in cfg["layers"]:
        l["mixer"]["scale"] *= 12.0
    for k in w:
        if k.endswith("mix.sink"):
            w[k] = w[k] * 0.0 + 3.0                             # a sink that counts: about as large as a good score
        if k.endswith("mix.k.b"):
            w[k] = w[k] * 12.0                                  # keys share a direction: a block's mean is as long as a key and wins as often


EDGE_MODELS = [
    ([L(A, heads=2, kv_heads=1, window=8, pool=4, mlp=None), L(M, heads=2, window=8, mlp="dense")], 16),
    ([L(A, heads=4, kv_heads=4, window=13, pool=3, conv=2, mlp=None), L(M, heads=3, window=17, rot_dims=4, mlp=None)], 16),
    ([L(A, heads=2, kv_heads=2, window=16, pool=16, mlp=None), L(M, heads=2, window=16, mlp=None)], 16),
    ([L(A, heads=3, kv_heads=1, window=5, pool=7, conv=1, mlp=None), L(M, heads=1, window=1, mlp=None)], 8),
    ([L(A, heads=2, kv_heads=1, window=33, pool=2, mlp=None), L(M, heads=2, window=40, mlp=None)], 32),
]


@pytest.mark.parametrize("which", range(len(EDGE_MODELS)))
def test_window_block_and_page_edges(which):
    layers, page = EDGE_MODELS[which]
    b = Bundle(layers, kv_page=page, seed=6, loop=(0, 2, 2), tweak=sharpen)
    try:
        toks = b.tokens(130, 3)
        want = b.oracle(toks)
        b.m.state.reset(0)
        assert err(b.feed(0, toks), want) <= TIGHT             # in a prompt (chunks of four tokens cross every edge)
        b.m.state.reset(1)
        out = [b.feed(1, toks[:5])]
        for i in range(5, 100):                                # decoded alone while the first tokens leave every window, blocks close
            out.append(b.feed(1, [toks[i]], capi.OPTION_LAST))  # and become visible, and the sequence crosses page borders
        out.append(b.feed(1, toks[100:103]))
        out.append(b.feed(1, toks[103:105]))
        out.append(b.feed(1, toks[105:]))                      # portions that start and end inside windows, blocks and pages
        assert err(np.concatenate(out), want) <= TIGHT
    finally:
        b.close()


def test_the_edges_matter():
    # the inputs do what the test above needs: a window, a block or a sink that is one off gives other rows altogether
    layers, _ = EDGE_MODELS[0]
    cfgb, st, w = synth.make_pasopel(layers, seed=6, loop=(0, 2, 2))
    cfg = json.loads(cfgb)
    sharpen(cfg, w)
    toks = [int(t) for t in np.random.default_rng(3).integers(0, 96, 60)]
    a = P.run(cfg, w, toks)
    vt, vb, ss = P.visible_tokens, P.visible_blocks, P.sink_softmax
    try:
        P.visible_tokens = lambda i, win: vt(i, win + 1)
        wide = P.run(cfg, w, toks)
        P.visible_tokens = lambda i, win: vt(i, win - 1)
        narrow = P.run(cfg, w, toks)
        P.visible_tokens = vt
        P.visible_blocks = lambda i, win, pool: vb(i + 1, win, pool)
        early = P.run(cfg, w, toks)
        P.visible_blocks = lambda i, win, pool: vb(i - 1, win, pool)
        late = P.run(cfg, w, toks)
        P.visible_blocks = vb
        P.sink_softmax = lambda s, sink: ss(s, -1e30)
        nosink = P.run(cfg, w, toks)
    finally:
        P.visible_tokens, P.visible_blocks, P.sink_softmax = vt, vb, ss
    for other in (wide, narrow, early, late):
        assert err(a[:7], other[:7]) < 1e-9                     # nothing has left a window of 8 yet
    for other in (wide, narrow, nosink):
        assert err(a[12:], other[12:]) > 1000 * TIGHT
    for other in (early, late):                                 # a block's mean is a milder key than a token, still far from rounding
        assert err(a[12:], other[12:]) > 100 * TIGHT


def plant_far_key(cfg, w):
    """Every query of layer 0 points along the key of token 1, which stands at position 1 only.  Once it has left the window
    it is seen through its block's mean alone, which still outscores every other key, near or hundreds of tokens away."""
    eps = cfg["norm"]["eps"]
    h = P.offset_norm(w["embed"][1], w["l0.norm1"], eps)
    k = (w["l0.mix.k"] @ h + w["l0.mix.k.b"]) * w["l0.mix.k.conv"][:, 0]
    w["l0.mix.q.b"] = 50.0 * k / np.linalg.norm(k) / w["l0.mix.q.conv"][:, 0]
    w["l0.mix.sink"] = w["l0.mix.sink"] * 0.0


def test_a_far_key_carries_the_row():
    b = Bundle([L(A, heads=1, kv_heads=1, dim=16, conv=1, window=6, pool=2, scale=3.0, mlp=None)], seed=11, vocab=8, loop=None, tweak=plant_far_key)
    try:
        toks = [0, 1] + [int(t) for t in np.random.default_rng(1).integers(2, 8, 400)]
        want = b.oracle(toks)
        vb = P.visible_blocks
        try:                                                   # the inputs do what the test needs: without block 0 the rows change
            P.visible_blocks = lambda i, win, pool: [x for x in vb(i, win, pool) if x != 0]
            blind = b.oracle(toks)
        finally:
            P.visible_blocks = vb
        assert (row_errs(blind[10:], want[10:]) > 1000 * TIGHT).mean() > 0.95
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


ODD = [L(A, heads=3, kv_heads=3, dim=10, window=7, pool=3, conv=5, mlp="moe", experts=3, top=3, ff=10, shared_ff=7),
       L(M, heads=5, dim=6, vdim=9, rot_dim=10, rot_dims=4, kv_rank=13, q_rank=21, window=50, mlp="moe", experts=1, top=1, ff=7, shared_ff=0),
       L(A, heads=1, kv_heads=1, dim=34, window=2, pool=0, conv=1, mlp=None),
       L(M, heads=1, dim=5, vdim=3, rot_dim=2, kv_rank=7, q_rank=3, window=12, mlp="dense", ff=9),
       L(A, heads=6, kv_heads=2, dim=6, window=300, pool=4, conv=2, mlp="moe", experts=9, top=4, ff=5),
       L(A, heads=5, kv_heads=1, dim=9, window=3, pool=1, mlp="dense", ff=3)]


@pytest.mark.parametrize("precision", [1, 0])
def test_other_sizes(precision):
    b = Bundle(ODD, precision=precision, width=50, vocab=61, seed=7, loop=(2, 5, 2), softcap=7.5, eps=1e-6)
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


WIDE = [L(A, heads=8, kv_heads=2, dim=64, window=48, pool=8, mlp="moe", experts=8, top=2, ff=64, shared_ff=96),
        L(M, heads=16, dim=32, vdim=32, rot_dim=16, kv_rank=128, q_rank=96, window=64, mlp="dense", ff=320),
        L(A, heads=4, kv_heads=4, dim=128, window=100, pool=16, mlp="dense", ff=320),
        L(M, heads=4, dim=64, vdim=128, rot_dim=32, kv_rank=256, q_rank=64, window=30, mlp="moe", experts=4, top=2, ff=128)]


@pytest.mark.parametrize("precision", [1, 0])
def test_wider_layers(precision):
    b = Bundle(WIDE, precision=precision, width=256, vocab=300, seed=5, loop=(0, 2, 2))
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


# head counts, head ratios and head sizes around the attention kernel's launch shapes (heads per CTA, key heads per tile load,
# vector and scalar tile loads), in prompts of several chunks and in decoding
@pytest.mark.parametrize("kind,heads,kv_heads,dim,extra", [
    (A, 1, 1, 4, {}), (A, 2, 2, 128, {}), (A, 3, 1, 12, {}), (A, 12, 4, 20, {}), (A, 7, 7, 9, {}), (A, 32, 32, 8, {}), (A, 40, 20, 4, {}),
    (A, 24, 1, 16, {}), (A, 34, 2, 6, {}), (A, 16, 16, 64, {}),
    (M, 1, 1, 4, dict(rot_dim=2, kv_rank=5, vdim=3)), (M, 20, 1, 16, dict(rot_dim=8, kv_rank=64, vdim=16)),
    (M, 17, 1, 8, dict(rot_dim=4, kv_rank=30, vdim=10)), (M, 4, 1, 64, dict(rot_dim=64, kv_rank=512, vdim=64)),
    (M, 2, 1, 7, dict(rot_dim=6, kv_rank=11, vdim=5))])
def test_head_shapes(kind, heads, kv_heads, dim, extra):
    kw = dict(heads=heads, dim=dim, **extra)
    if kind == A:
        kw["kv_heads"] = kv_heads
    layers = [L(kind, window=21, pool=4, mlp=None, **kw), L(kind, window=9, pool=3, mlp="dense", **kw)]
    b = Bundle(layers, seed=heads + dim, width=40, vocab=50, kv_page=8, loop=(1, 2, 2))
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
    rng = np.random.default_rng(2000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        mlp = pick("dense", "moe", None)
        experts = pick(2, 4, 5, 9)
        ff = dict(mlp=mlp, ff=pick(8, 24, 33), experts=experts, top=int(rng.integers(1, min(experts, 4) + 1)), shared_ff=pick(0, 8, 20))
        if rng.integers(2):
            kv = pick(1, 2, 4)
            layers.append(L(A, heads=kv * pick(1, 2, 3, 4), kv_heads=kv, dim=pick(4, 8, 12, 18, 32, 40), window=pick(1, 5, 16, 31, 64, 200),
                            pool=pick(0, 1, 2, 4, 5, 8, 16), conv=pick(1, 2, 3, 4), scale=float(rng.uniform(0.1, 0.6)), **ff))
        else:
            dr = pick(2, 4, 8, 12)
            layers.append(L(M, heads=pick(1, 2, 3, 8), dim=pick(4, 8, 12, 20), vdim=pick(4, 6, 16, 20), rot_dim=dr, rot_dims=pick(0, 2, dr),
                            kv_rank=pick(6, 16, 33, 64), q_rank=pick(4, 16, 30), window=pick(1, 6, 16, 37, 128), base=pick(100.0, 10000.0, 5e5),
                            scale=float(rng.uniform(0.1, 0.6)), **ff))
    n = len(layers)
    start = int(rng.integers(0, n))
    loop = pick(None, (start, int(rng.integers(start + 1, n + 1)), pick(1, 2, 3)))
    kw = dict(width=pick(24, 40, 56, 100), vocab=pick(31, 64, 150), loop=loop, softcap=pick(None, 5.0, 30.0), eps=pick(1e-5, 1e-6, 1e-3))
    return layers, kw


@pytest.mark.parametrize("seed", range(10))
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
    b = Bundle(STACK, precision=0, **STACK_KW)
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
    b = Bundle(STACK, chunk=512, **STACK_KW)
    try:
        long = toks + b.tokens(550, 8)                         # hundreds of block rows: several key tiles per cluster rank, three steps
        ref = b.oracle(long)
        assert err(b.feed(0, long), ref) <= TIGHT
        b.m.state.reset(0)
        b.feed(0, long[:660], capi.OPTION_NONE)
        rows = np.concatenate([b.feed(0, [t], capi.OPTION_LAST) for t in long[660:]])     # decoding with the keys split over a cluster
        assert err(rows, ref[660:]) <= TIGHT
    finally:
        b.close()


def test_greedy_generation_through_the_runtime(stack):
    # the framework's own entry point: Runtime.infer (its token budget and slot batching) + the GPU sampling front half
    prompt = stack.tokens(21, 12)
    mem = P.new_memory(stack.cfg)
    row = P.run(stack.cfg, stack.w, prompt, mem=mem)[-1]
    want = []
    for _ in range(12):
        want.append(int(row.argmax()))
        row = P.run(stack.cfg, stack.w, [want[-1]], mem=mem)[-1]
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
    m.state.write(snap, 1)                                     # device snapshot into another slot: its block means are rebuilt
    b_ = stack.feed(1, toks[50:90])
    m.state.load(host, 2)                                      # host tensor into a third
    c = stack.feed(2, toks[50:90])
    assert err(a, want[50:90]) <= TIGHT
    assert np.array_equal(a, b_) and np.array_equal(a, c)
    snap.free()
