"""Plain NumPy restatement of the Zufulix decoder: one function per mechanism, token by token, written for clarity.  It
shares no code with the CUDA engine and is test infrastructure only.

Notation: W[out, in] applied as W @ x; `cfg` is the parsed config.json; weights are a dict name -> float64 array.
A model is a stack of pre-norm blocks over `streams` copies of the residual (hyper-connections):
    u = sum_s a[s] x_s;   y = Sublayer(LN(u));   x_t <- sum_s M[s, t] x_s + b[t] y        (all streams from the old ones)
with one (a, b, M) per sublayer; without `streams` in the config the block is the plain  x <- x + Sublayer(LN(x)).
LN is a layer norm with weight and bias.  The mixer is causal softmax attention with grouped key / value heads, biased
projections, unit-RMS queries and keys, a learned bias per (log-spaced distance bucket, head) and a blend of the values with
those of the first blending layer; the feed-forward is W_down gelu(W_up h) or routed experts W_down relu(W_up h)^2 chosen by
sigmoid scores inside the best groups of neighbouring experts.  The logits come from the (unscaled) embedding table.
"""
from __future__ import annotations

import math

import numpy as np

from .kemirax_numpy import bf16_round, read_safetensors  # noqa: F401  (file helpers only)

ROUND_OPERANDS = False      # True: the activation operand of every projection is rounded to bfloat16 first (noise-floor runs)


def lin(W, x):
    return W @ (bf16_round(x) if ROUND_OPERANDS else x)


def layer_norm(x, w, b, eps):
    d = x - x.mean()
    return d / np.sqrt(np.mean(d * d) + eps) * w + b


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_erf(z):
    return np.array([0.5 * v * (1.0 + math.erf(v / math.sqrt(2.0))) for v in np.ravel(z)]).reshape(np.shape(z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ----------------------------------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------------------------------
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for distance n >= 0: the first rows / 2 distances have a row each, the others share rows that are
    evenly spaced in log(distance) up to `far`; everything at or beyond `far` takes the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def attention(w, p, c, eps, h, mem, pos, shared):
    """mem: {'k': [list of [G, dk]], 'v': [list of [G, dv]]} of this layer; shared: per-token dict that carries the first
    blending layer's values to the later ones."""
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (lin(w[p + "q"], h) + w[p + "q.b"]).reshape(H, dk)
    k = (lin(w[p + "k"], h) + w[p + "k.b"]).reshape(G, dk)
    v = (lin(w[p + "v"], h) + w[p + "v.b"]).reshape(G, dv)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    if c.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v.copy()
        else:
            lam = float(w[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
    mem.setdefault("k", []).append(k)
    mem.setdefault("v", []).append(v)
    rel = w[p + "rel"]
    K, V = np.stack(mem["k"]), np.stack(mem["v"])      # [pos + 1, G, d]
    bucket = [distance_bucket(pos - j, rel.shape[0], c["bias_max"]) for j in range(pos + 1)]
    out = np.zeros((H, dv))
    for hh in range(H):
        g = hh // (H // G)
        s = K[:, g] @ q[hh] * c["scale"] + rel[bucket, hh]
        e = np.exp(s - s.max())
        out[hh] = (e / e.sum()) @ V[:, g]
    return lin(w[p + "o"], out.reshape(-1))


MIXERS = {"attention": attention}


# ----------------------------------------------------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------------------------------------------------
def route(s, top, groups=None):
    """Chosen experts (largest scores first; ties: lower index) and their weights.  With groups = (count, keep) only experts of
    the `keep` groups with the largest sum of their two best scores can be chosen."""
    E = len(s)
    allowed = np.ones(E, bool)
    if groups:
        count, keep = groups
        per = E // count
        gs = np.array([np.sort(s[g * per:(g + 1) * per])[::-1][:2].sum() for g in range(count)])
        best = np.argsort(-gs, kind="stable")[:keep]
        allowed[:] = False
        for g in best:
            allowed[g * per:(g + 1) * per] = True
    masked = np.where(allowed, s, -np.inf)
    idx = np.argsort(-masked, kind="stable")[:top]
    return idx, s[idx] / (s[idx].sum() + 1e-20)


def feed_forward(w, p, c, h):
    if c["kind"] == "dense":
        return lin(w[p + "down"], gelu_erf(lin(w[p + "up"], h)))
    r = c["router"]
    s = sigmoid(w[p + "router"] @ h)                    # the router reads the unrounded row
    g = r.get("groups")
    idx, wt = route(s, r["top"], (g["count"], g["keep"]) if g else None)
    y = 0.0
    for n, e in enumerate(idx):
        a = np.maximum(lin(w[p + "e%d.up" % e], h), 0.0) ** 2
        y = y + wt[n] * lin(w[p + "e%d.down" % e], a)
    return y


# ----------------------------------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------------------------------
def new_memory(cfg):
    return {"pos": 0, "layers": [dict() for _ in cfg["layers"]]}


def sublayer(cfg, w, p, q, xs, fn):
    """Sublayer q (1: mixer, 2: feed-forward) of the layer with prefix p on the streams xs [s, W] (or the single residual)."""
    eps = cfg["norm"]["eps"]
    nw, nb = w[p + "norm%d" % q], w[p + "norm%d.b" % q]
    if "streams" not in cfg:
        return xs + fn(layer_norm(xs[0], nw, nb, eps))[None, :]
    a, b, M = w[p + "hc%d.in" % q], w[p + "hc%d.out" % q], w[p + "hc%d.mix" % q]
    y = fn(layer_norm(a @ xs, nw, nb, eps))
    return M.T @ xs + np.outer(b, y)


def step(cfg, w, mem, token, residuals=None):
    """One token through the stack; returns the logits row and advances `mem`."""
    eps = cfg["norm"]["eps"]
    x0 = np.array(w["embed"][token], np.float64) * cfg.get("embedding", {}).get("scale", 1.0)
    xs = np.tile(x0, (cfg.get("streams", 1), 1))
    shared = {}
    for i, l in enumerate(cfg["layers"]):
        p = "l%d." % i
        xs = sublayer(cfg, w, p, 1, xs,
                      lambda h: MIXERS[l["type"]](w, p + "mix.", l["mixer"], eps, h, mem["layers"][i], mem["pos"], shared))
        if l.get("mlp"):
            xs = sublayer(cfg, w, p, 2, xs, lambda h: feed_forward(w, p + "mlp.", l["mlp"], h))
        if residuals is not None:
            residuals.append(xs.sum(0))
    mem["pos"] += 1
    return lin(w["embed"], layer_norm(xs.sum(0), w["final.norm"], w["final.norm.b"], eps))


def run(cfg, w, toks, layers=False, mem=None):
    """Logits rows [len(toks), vocab] (and, with layers, the residual after every layer [L, len(toks), width])."""
    mem = mem if mem is not None else new_memory(cfg)
    rows, res = [], []
    for t in toks:
        r = []
        rows.append(step(cfg, w, mem, int(t), r))
        res.append(np.stack(r))
    if layers:
        return np.stack(rows), np.stack(res, 1)
    return np.stack(rows)
