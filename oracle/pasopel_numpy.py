"""Plain NumPy restatement of the Pasopel decoder: one function per mechanism, token by token, written for clarity.  It
shares no code with the CUDA engine and is test infrastructure only.

Notation: W[out, in] applied as W @ x; `cfg` is the parsed config.json; weights are a dict name -> float64 array.
A model is a stack of pre-norm blocks  x <- x + Mixer(N1(x));  x <- x + FF(N2(x))  where N is an RMS norm whose stored weight
is an offset from one.  A run of consecutive layers (`loop`) is executed several times with the same tensors and a memory of
its own per pass; every pass begins by adding a learned per-pass vector to the residual, and every pass after the first also
adds the token's embedding row again.  Two mixers: grouped-head softmax attention whose values are the (un-normalised) keys,
behind short causal convolutions, over a sliding window extended by block means of the older keys; and latent attention (low
rank queries, one shared key/value latent plus one shared rotated key part) over a sliding window.  Both add a learned
per-head "sink" term to the softmax denominator and gate their output with a sigmoid of a projection of the mixer input.
Feed-forward: W_down relu(W_up h)^2, or routed silu-gated experts (largest logits win, softmax over the winners) plus an
always-on expert.  The logits come from the embedding table and are squashed by cap * tanh(z / cap).
"""
from __future__ import annotations

import numpy as np

from .kemirax_numpy import bf16_round, read_safetensors  # noqa: F401  (file helpers only)

ROUND_OPERANDS = False      # True: the activation operand of every projection is rounded to bfloat16 first (noise-floor runs)


def lin(W, x):
    return W @ (bf16_round(x) if ROUND_OPERANDS else x)


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def sink_softmax(scores, sink):
    """Weights of the keys when the denominator holds one more term exp(sink) that belongs to no key."""
    m = max(float(np.max(scores)), float(sink))
    e = np.exp(scores - m)
    return e / (e.sum() + np.exp(sink - m))


def short_conv(taps_w, history):
    """taps_w [C, taps]; history: the last `taps` inputs, oldest first (zeros before the start of the sequence)."""
    return sum(taps_w[:, j] * history[j] for j in range(taps_w.shape[1]))


def rotate_pairs(x, pos, dims, base):
    """Neighbouring entries (2i, 2i + 1) of the first `dims` entries turn by pos * base^(-2i / dims); the rest stay."""
    y = np.array(x, np.float64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, v = x[2 * i], x[2 * i + 1]
        y[2 * i] = u * np.cos(a) - v * np.sin(a)
        y[2 * i + 1] = v * np.cos(a) + u * np.sin(a)
    return y


def visible_tokens(i, window):
    return range(max(0, i - window + 1), i + 1)


def visible_blocks(i, window, pool):
    """Blocks of `pool` consecutive positions that lie wholly before the window of position i."""
    return range(max(0, i - window + 1) // pool) if pool else range(0)


# ----------------------------------------------------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------------------------------------------------
def attention(w, p, c, eps, h, mem, pos):
    """mem: {'hist_q': list, 'hist_k': list, 'k': [[G, dk] per token], 'v': [[G, dk] per token]}."""
    H, G, dk = c["heads"], c["kv_heads"], c["dim"]
    taps = c["conv"]
    win, pool = c["mask"]["size"], c["mask"].get("pool", 0)
    q_in = lin(w[p + "q"], h) + w[p + "q.b"]
    k_in = lin(w[p + "k"], h) + w[p + "k.b"]
    for name, val in (("hist_q", q_in), ("hist_k", k_in)):
        mem[name].append(val)
        del mem[name][:-taps]
    pad = lambda hist: [np.zeros_like(hist[-1])] * (taps - len(hist)) + hist
    q = short_conv(w[p + "q.conv"], pad(mem["hist_q"])).reshape(H, dk)
    k = short_conv(w[p + "k.conv"], pad(mem["hist_k"])).reshape(G, dk)
    mem["v"].append(k.copy())                      # the value is the key before it is normalised
    mem["k"].append(unit_rms(k, eps))
    q = unit_rms(q, eps)
    toks = list(visible_tokens(pos, win))
    blocks = list(visible_blocks(pos, win, pool))
    out = np.zeros((H, dk))
    for hd in range(H):
        g = hd // (H // G)
        keys = [np.mean([mem["k"][b * pool + u][g] for u in range(pool)], 0) for b in blocks] + [mem["k"][j][g] for j in toks]
        vals = [np.mean([mem["v"][b * pool + u][g] for u in range(pool)], 0) for b in blocks] + [mem["v"][j][g] for j in toks]
        s = np.array([q[hd] @ kk for kk in keys]) * c["scale"]
        out[hd] = sink_softmax(s, w[p + "sink"][hd]) @ np.array(vals)
    gate = sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], out.reshape(-1) * gate) + w[p + "o.b"]


def latent_attention(w, p, c, eps, h, mem, pos):
    """mem: {'c': [[kv_rank] per token], 'kr': [[rot_dim] per token]}; keys and values are rebuilt from the latent."""
    H, dn, dr, dv, rk = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    win = c["mask"]["size"]
    rot = c["rot"]
    cq = unit_rms(lin(w[p + "dq"], h), eps) * w[p + "dq.norm"]
    q = lin(w[p + "uq"], cq).reshape(H, dn + dr)
    kv = lin(w[p + "dkv"], h)
    mem["c"].append(unit_rms(kv[:rk], eps) * w[p + "dkv.norm"])
    mem["kr"].append(rotate_pairs(kv[rk:], pos, rot["dims"], rot["base"]))
    toks = list(visible_tokens(pos, win))
    out = np.zeros((H, dv))
    for hd in range(H):
        q_rot = rotate_pairs(q[hd, dn:], pos, rot["dims"], rot["base"])
        s = np.zeros(len(toks))
        vals = np.zeros((len(toks), dv))
        for n, j in enumerate(toks):
            k_plain = lin(w[p + "uk"][hd * dn:(hd + 1) * dn], mem["c"][j])
            vals[n] = lin(w[p + "uv"][hd * dv:(hd + 1) * dv], mem["c"][j])
            s[n] = (q[hd, :dn] @ k_plain + q_rot @ mem["kr"][j]) * c["scale"]
        out[hd] = sink_softmax(s, w[p + "sink"][hd]) @ vals
    gate = sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], out.reshape(-1) * gate)


MIXERS = {"attention": attention, "latent_attention": latent_attention}


def new_layer_memory(layer):
    if layer["type"] == "attention":
        return {"hist_q": [], "hist_k": [], "k": [], "v": []}
    return {"c": [], "kr": []}


# ----------------------------------------------------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------------------------------------------------
def gated_unit(w, p, h):
    return lin(w[p + "down"], silu(lin(w[p + "gate"], h)) * lin(w[p + "up"], h))


def route(w, p, f, h):
    """(chosen experts, their weights): the `top` largest logits win, ties to the lower index; softmax over the winners."""
    z = w[p + "router"] @ h + w[p + "router.b"]
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[: f["router"]["top"]]
    e = np.exp(z[order] - z[order].max())
    return order, e / e.sum()


def feed_forward(w, p, f, h):
    if f["kind"] == "dense":
        return lin(w[p + "down"], np.maximum(lin(w[p + "up"], h), 0.0) ** 2)
    chosen, weights = route(w, p, f, h)
    y = sum(g * gated_unit(w, p + "e%d." % e, h) for e, g in zip(chosen, weights))
    if f.get("shared"):
        y = y + gated_unit(w, p + "shared.", h)
    return y


# ----------------------------------------------------------------------------------------------------------------------
# model
# ----------------------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer index, pass number if the run opens a pass else None)] in execution order."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def new_memory(cfg):
    return {"pos": 0, "runs": [new_layer_memory(cfg["layers"][i]) for i, _ in layer_runs(cfg)]}


def step(cfg, w, mem, token, residuals=None):
    """One token through the stack; returns the logits row and advances `mem`."""
    eps = cfg["norm"]["eps"]
    x0 = np.array(w["embed"][token], np.float64)
    x = x0.copy()
    for r, (i, opens) in enumerate(layer_runs(cfg)):
        l = cfg["layers"][i]
        p = "l%d." % i
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"][opens]
        x = x + MIXERS[l["type"]](w, p + "mix.", l["mixer"], eps, offset_norm(x, w[p + "norm1"], eps), mem["runs"][r], mem["pos"])
        if l.get("mlp"):
            x = x + feed_forward(w, p + "mlp.", l["mlp"], offset_norm(x, w[p + "norm2"], eps))
        if residuals is not None:
            residuals.append(x.copy())
    mem["pos"] += 1
    z = lin(w["embed"], offset_norm(x, w["final.norm"], eps))
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z


def run(cfg, w, toks, layers=False, mem=None):
    """Logits rows [len(toks), vocab] (and, with layers, the residual after every layer run [runs, len(toks), width])."""
    mem = mem if mem is not None else new_memory(cfg)
    rows, res = [], []
    for t in toks:
        r = []
        rows.append(step(cfg, w, mem, int(t), r))
        res.append(np.stack(r))
    if layers:
        return np.stack(rows), np.stack(res, 1)
    return np.stack(rows)
