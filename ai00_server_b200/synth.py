"""Deterministic synthetic RWKV weights in the reference's on-disk `.st` layout.

No RWKV checkpoints exist offline, so tests and bench.py use
random-init weights of the named architectures.  The file image written here
follows /root/reference/assets/scripts/convert_safetensors.py:22-101 exactly:
safetensors container, metadata {"format": "pt"}, every tensor float16, lower-case
keys after the `time_maa->time_mix` / `time_faaaa->time_first` renames, LoRA
matrices already transposed to [out, in].

Values come from a counter-based hash (murmur3 finaliser over the element index,
keyed by FNV-1a of the tensor name and the seed), so any element of any tensor
can be regenerated independently and bit-identically by NumPy here and by the
OpenMP C helper (csrc/synth_fill.c) that fills the 15 GB 7B image in seconds.
This module is bench/test tooling: the engine itself only ever sees `.st` bytes.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


@dataclass
class Shape:
    version: int
    L: int
    C: int
    F: int
    V: int = 65536
    N: int = 64
    Dm: int = 32      # v6 time-mix LoRA rank
    Dd: int = 64      # v6 decay LoRA rank / v7 w rank
    Da: int = 64      # v7
    Dv: int = 32      # v7
    Dg: int = 128     # v7
    time_state: bool = False

    @property
    def H(self) -> int:
        return self.C // self.N


PRESETS = {
    # CI-sized
    "tiny6": Shape(6, 2, 256, 896, V=512, Dm=32, Dd=64),
    "tiny5": Shape(5, 2, 256, 896, V=512),
    "tiny7": Shape(7, 3, 256, 1024, V=512, Dd=32, Da=32, Dv=16, Dg=64),
    "small6": Shape(6, 4, 512, 1792, V=2048, Dm=32, Dd=64),
    "small5": Shape(5, 3, 512, 1792, V=2048),                                   # 8 heads: shards over 8 GPUs
    "small7": Shape(7, 3, 512, 2048, V=2048, Dd=32, Da=32, Dv=16, Dg=64),
    # BASELINE.json shapes (last row)
    "v6-1b6": Shape(6, 24, 2048, 7168, Dm=32, Dd=64),
    "v6-3b": Shape(6, 32, 2560, 8960, Dm=32, Dd=64),
    "v6-7b": Shape(6, 32, 4096, 14336, Dm=64, Dd=128),
    "v7-2b9": Shape(7, 32, 2560, 10240, Dd=96, Da=96, Dv=64, Dg=320),
}


def _sq(c):
    return float(np.sqrt(3.0) / np.sqrt(c))    # uniform(-a,a) with std 1/sqrt(c)


def tensor_spec(s: Shape) -> list[tuple[str, tuple[int, ...], float, float]]:
    """[(name, shape, lo, hi)] in file order."""
    C, F, V, H, N, L = s.C, s.F, s.V, s.H, s.N, s.L
    out: list[tuple[str, tuple[int, ...], float, float]] = []

    def add(name, shape, lo, hi):
        out.append((name, tuple(shape), float(lo), float(hi)))

    def ln(prefix):
        add(prefix + ".weight", (C,), 0.9, 1.1)
        add(prefix + ".bias", (C,), -0.05, 0.05)

    add("emb.weight", (V, C), -1.0, 1.0)
    for l in range(L):
        b = f"blocks.{l}."
        if l == 0:
            ln(b + "ln0")
        ln(b + "ln1")
        ln(b + "ln2")
        a = b + "att."
        if s.version == 6:
            for n in ("x", "w", "k", "v", "r", "g"):
                add(a + f"time_mix_{n}", (1, 1, C), 0.0, 1.0)
            add(a + "time_mix_w1", (5 * s.Dm, C), -0.5 * _sq(C), 0.5 * _sq(C))
            add(a + "time_mix_w2", (5, C, s.Dm), -0.2 * _sq(s.Dm), 0.2 * _sq(s.Dm))
            add(a + "time_decay", (1, 1, C), -6.0, -1.0)
            add(a + "time_decay_w1", (s.Dd, C), -0.5 * _sq(C), 0.5 * _sq(C))
            add(a + "time_decay_w2", (C, s.Dd), -0.5 * _sq(s.Dd), 0.5 * _sq(s.Dd))
            add(a + "time_first", (H, N), -0.5, 0.5)
        elif s.version == 5:
            for n in ("k", "v", "r", "g"):
                add(a + f"time_mix_{n}", (1, 1, C), 0.0, 1.0)
            add(a + "time_decay", (H, N), -6.0, -1.0)
            add(a + "time_first", (H, N), -0.5, 0.5)
        else:
            for n in ("r", "w", "k", "v", "a", "g"):
                add(a + f"x_{n}", (1, 1, C), 0.0, 1.0)
            add(a + "w0", (1, 1, C), -3.0, 1.0)
            add(a + "w1", (s.Dd, C), -0.5 * _sq(C), 0.5 * _sq(C))
            add(a + "w2", (C, s.Dd), -1.0 * _sq(s.Dd), 1.0 * _sq(s.Dd))
            add(a + "a0", (1, 1, C), -1.0, 1.0)
            add(a + "a1", (s.Da, C), -0.5 * _sq(C), 0.5 * _sq(C))
            add(a + "a2", (C, s.Da), -1.0 * _sq(s.Da), 1.0 * _sq(s.Da))
            add(a + "v0", (1, 1, C), -1.0, 1.0)
            add(a + "v1", (s.Dv, C), -0.5 * _sq(C), 0.5 * _sq(C))
            add(a + "v2", (C, s.Dv), -1.0 * _sq(s.Dv), 1.0 * _sq(s.Dv))
            add(a + "g1", (s.Dg, C), -1.0 * _sq(C), 1.0 * _sq(C))
            # gate LoRA / output gains sized so that the synthetic model is as well conditioned as the RWKV-6 presets: with
            # gain 2 / 0.5 here the random RWKV-7 stack is chaotic (two f32 implementations that differ only in summation
            # order are 3e-3 apart after one token at 32 layers, f16 vs f32 operands 0.3: profiles/r02_findings.md), which
            # says nothing about an engine; trained RWKV-7 checkpoints initialise both near zero.
            add(a + "g2", (C, s.Dg), -1.0 * _sq(s.Dg), 1.0 * _sq(s.Dg))
            add(a + "k_k", (1, 1, C), 0.5, 1.2)
            add(a + "k_a", (1, 1, C), 0.0, 1.0)
            add(a + "r_k", (H, N), -0.3, 0.3)
        for n in ("receptance", "key", "value"):
            add(a + n + ".weight", (C, C), -_sq(C), _sq(C))
        if s.version != 7:
            add(a + "gate.weight", (C, C), -_sq(C), _sq(C))
        og = 0.25 if s.version == 7 else 0.5
        add(a + "output.weight", (C, C), -og * _sq(C), og * _sq(C))
        add(a + "ln_x.weight", (C,), 0.8, 1.2)
        add(a + "ln_x.bias", (C,), -0.05, 0.05)
        if s.time_state:
            add(a + "time_state", (H, N, N), -0.5, 0.5)
        f = b + "ffn."
        if s.version == 7:
            add(f + "x_k", (1, 1, C), 0.0, 1.0)
        else:
            add(f + "time_mix_k", (1, 1, C), 0.0, 1.0)
            add(f + "time_mix_r", (1, 1, C), 0.0, 1.0)
            add(f + "receptance.weight", (C, C), -_sq(C), _sq(C))
        add(f + "key.weight", (F, C), -_sq(C), _sq(C))
        add(f + "value.weight", (C, F), -0.5 * _sq(F), 0.5 * _sq(F))
    ln("ln_out")
    add("head.weight", (V, C), -2.0 * _sq(C), 2.0 * _sq(C))
    return out


def name_seed(name: str, seed: int) -> int:
    h = 0x811C9DC5
    for ch in name.encode("utf-8"):
        h = ((h ^ ch) * 0x01000193) & 0xFFFFFFFF
    return (h ^ ((seed * 0x9E3779B1) & 0xFFFFFFFF)) & 0xFFFFFFFF


def fill_numpy(dst: np.ndarray, seed32: int, lo: float, hi: float) -> None:
    """dst: flat float16 array.  Reference implementation of the fill."""
    n = dst.size
    chunk = 1 << 22
    lo32, span = np.float32(lo), np.float32(np.float32(hi) - np.float32(lo))
    for off in range(0, n, chunk):
        m = min(chunk, n - off)
        h = np.arange(off, off + m, dtype=np.uint64).astype(np.uint32)
        h = h * np.uint32(0x9E3779B1) + np.uint32(seed32)
        h ^= h >> np.uint32(16)
        h *= np.uint32(0x85EBCA6B)
        h ^= h >> np.uint32(13)
        h *= np.uint32(0xC2B2AE35)
        h ^= h >> np.uint32(16)
        u = (h >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)
        dst[off:off + m] = (u * span + lo32).astype(np.float16)


_lib = None


def _fill_lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "_synthfill.so")
        if os.path.exists(path):
            lib = ctypes.CDLL(path)
            lib.synth_fill_f16.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32,
                                           ctypes.c_float, ctypes.c_float]
            lib.synth_fill_f16.restype = None
            _lib = lib
        else:
            _lib = False
    return _lib


def fill(dst: np.ndarray, seed32: int, lo: float, hi: float, force_numpy: bool = False) -> None:
    lib = None if force_numpy else _fill_lib()
    if lib:
        lib.synth_fill_f16(dst.ctypes.data, dst.size, seed32, lo, hi)
    else:
        fill_numpy(dst, seed32, lo, hi)


def make_st(shape: Shape | str, seed: int = 0, force_numpy: bool = False) -> np.ndarray:
    """Build the `.st` file image (uint8 array) for `shape`."""
    if isinstance(shape, str):
        shape = PRESETS[shape]
    spec = tensor_spec(shape)
    header = {"__metadata__": {"format": "pt"}}
    off = 0
    for name, shp, _, _ in spec:
        nbytes = int(np.prod(shp)) * 2
        header[name] = {"dtype": "F16", "shape": list(shp), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((-len(hjson)) % 8)
    base = 8 + len(hjson)
    buf = np.empty(base + off, dtype=np.uint8)
    buf[:8] = np.frombuffer(struct.pack("<Q", len(hjson)), dtype=np.uint8)
    buf[8:base] = np.frombuffer(hjson, dtype=np.uint8)
    for name, shp, lo, hi in spec:
        b, e = header[name]["data_offsets"]
        view = buf[base + b:base + e].view(np.float16)
        fill(view, name_seed(name, seed), lo, hi, force_numpy)
    return buf


def pack_st(tensors: dict[str, np.ndarray]) -> np.ndarray:
    """safetensors image of a dict of arrays (F16 / F32), metadata {"format": "pt"}."""
    header = {"__metadata__": {"format": "pt"}}
    off, blobs = 0, []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        dt = {np.dtype(np.float16): "F16", np.dtype(np.float32): "F32"}[a.dtype]
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((-len(hjson)) % 8)
    return np.frombuffer(struct.pack("<Q", len(hjson)) + hjson + b"".join(blobs), dtype=np.uint8).copy()


def make_lora_st(shape: Shape | str, rank: int = 8, seed: int = 1, targets=("att.key", "att.value", "att.output", "ffn.key", "ffn.value")) -> np.ndarray:
    """Synthetic LoRA file in the layout the reference's converter writes (assets/scripts/convert_safetensors.py:96-101):
    `<name>.lora.0` = lora_A transposed = [in, r], `<name>.lora.1` = lora_B = [out, r], float16, for every block and `head`."""
    if isinstance(shape, str):
        shape = PRESETS[shape]
    dims = {n: shp for n, shp, _, _ in tensor_spec(shape)}
    out = {}
    names = [f"blocks.{l}.{t}" for l in range(shape.L) for t in targets if f"blocks.{l}.{t}.weight" in dims] + ["head"]
    for base in names:
        o, i = dims[base + ".weight"]
        for idx, (rows, gain) in enumerate(((i, 1.0), (o, 1.0))):
            a = np.empty(rows * rank, np.float16)
            fill(a, name_seed(f"{base}.lora.{idx}", seed), -gain * _sq(rank) * 0.5, gain * _sq(rank) * 0.5, True)
            out[f"{base}.lora.{idx}"] = a.reshape(rows, rank)
    return pack_st(out)


def num_params(shape: Shape | str) -> int:
    if isinstance(shape, str):
        shape = PRESETS[shape]
    return sum(int(np.prod(shp)) for _, shp, _, _ in tensor_spec(shape))


def algorithmic_bytes_per_step(s: Shape | str, batch: int) -> int:
    """SURVEY.md §8(d) / BASELINE.md §3 figure: f16 weights streamed once per decode step,
    f32 state read + written once, embedding rows in, f32 logits out."""
    if isinstance(s, str):
        s = PRESETS[s]
    C, F, V, L, H, N = s.C, s.F, s.V, s.L, s.H, s.N
    if s.version == 7:
        p_layer = 4 * C * C + 2 * C * (s.Dd + s.Da + s.Dv + s.Dg) + 2 * C * F + 19 * C
    elif s.version == 6:
        p_layer = 5 * C * C + 2 * C * (5 * s.Dm + s.Dd) + 2 * C * F + C * C + 16 * C
    else:
        p_layer = 5 * C * C + 2 * C * F + C * C + 12 * C
    return 2 * (L * p_layer + V * C + 4 * C) + batch * (2 * L * (H * N * N + 2 * C) * 4 + 2 * C + 4 * V)


# ----------------------------------------------------------------------------------------------------------------------
# Kemirax family (config.json + bf16 safetensors): random weights for tests and bench.py
# ----------------------------------------------------------------------------------------------------------------------
def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (round to nearest even)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def pack_st_bf16(tensors: dict) -> np.ndarray:
    """safetensors image with every float tensor stored as BF16 (integer tensors as I32)."""
    head, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.asarray(a)
        if a.dtype.kind in "iu":
            raw, dt = np.ascontiguousarray(a, np.int32).tobytes(), "I32"
        else:
            raw, dt = to_bf16_bits(a).tobytes(), "BF16"
        head[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    return np.frombuffer(struct.pack("<Q", len(hj)) + hj + b"".join(blobs), np.uint8).copy()


def kemirax_layer(kind: str, *, heads=4, dim=16, vdim=16, rot_dim=8, kv_rank=24, q_rank=20, kv_from=None, scale=None, base=10000.0,
                  scaling=None, tau=8.0, experts=4, identity=1, top=2, ff=24, limit=2.0, shared_ff=32, shared_limit=1.5, mlp=True) -> dict:
    """One entry of config['layers'].  kind: 'latent_attention' | 'gla'."""
    if kind == "latent_attention":
        rot = {"base": base, "dims": rot_dim}
        if scaling:
            rot["scaling"] = dict(scaling)
        mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
                 "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
        if kv_from is not None:
            mixer["kv_from"] = int(kv_from)
    else:
        mixer = {"heads": heads, "dim": dim, "vdim": vdim, "tau": float(tau)}
    layer = {"type": kind, "mixer": mixer, "mlp": None}
    if mlp:
        layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": limit}}
        if shared_ff:
            layer["mlp"]["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return layer


def make_kemirax(layers: list, width: int = 64, vocab: int = 96, eps: float = 1e-5, seed: int = 0, gain: float = 1.0, a_rank: int = 8,
                 arrays: bool = True):
    """(config.json bytes, safetensors image, dict of float64 arrays holding the bf16-rounded values, or None when `arrays` is
    off) for a random model of the family."""
    rng = np.random.default_rng(seed)
    W = width
    t = {}

    def mat(n, k, g=1.0):
        return (rng.standard_normal((n, k)) * (g * gain / np.sqrt(k))).astype(np.float32)

    t["embed"] = rng.standard_normal((vocab, W)).astype(np.float32)
    for i, l in enumerate(layers):
        p, m = "l%d." % i, l["mixer"]
        t[p + "norm1"] = np.float32(rng.uniform(0.8, 1.2))
        t[p + "shift"] = rng.uniform(0.0, 1.0, W).astype(np.float32)
        for r in ("rg1", "rg2") if l.get("mlp") else ("rg1",):
            t[p + r] = mat(W, W)
            t[p + r + ".b"] = rng.uniform(-0.5, 1.0, W).astype(np.float32)
        H, dn, dv = m["heads"], m["dim"], m["vdim"]
        if l["type"] == "latent_attention":
            dr, rk, rq = m["rot_dim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"] = mat(rq, W)
            t[p + "mix.dq.norm"] = rng.uniform(0.5, 1.5, rq).astype(np.float32)
            t[p + "mix.uq"] = mat(H * (dn + dr), rq, 2.0)
            if "kv_from" not in m:
                t[p + "mix.dkv"] = mat(rk + dr, W, 2.0)
                t[p + "mix.dkv.norm"] = rng.uniform(0.5, 1.5, rk).astype(np.float32)
            t[p + "mix.uk"] = mat(H * dn, rk, 2.0)
            t[p + "mix.uv"] = mat(H * dv, rk)
            t[p + "mix.o"] = mat(W, H * dv)
        else:
            t[p + "mix.q"] = mat(H * dn, W)
            t[p + "mix.k"] = mat(H * dn, W)
            t[p + "mix.v"] = mat(H * dv, W)
            t[p + "mix.g"] = mat(H * dv, W)
            t[p + "mix.o"] = mat(W, H * dv)
            t[p + "mix.norm"] = rng.uniform(0.5, 1.5, dv).astype(np.float32)
            t[p + "mix.a1"] = mat(a_rank, W)
            t[p + "mix.a2"] = mat(H * dn, a_rank, 2.0)
            t[p + "mix.a2.b"] = rng.uniform(1.0, 4.0, H * dn).astype(np.float32)
        f = l.get("mlp")
        if f:
            E, I = f["router"]["experts"], f["router"].get("identity", 0)
            t[p + "mlp.router"] = mat(E + I, W, 2.0)
            t[p + "mlp.correction"] = rng.uniform(-0.05, 0.05, E + I).astype(np.float32)
            for e in range(E):
                q = p + "mlp.e%d." % e
                t[q + "gate"] = mat(f["expert"]["ff"], W, 2.0)
                t[q + "up"] = mat(f["expert"]["ff"], W, 2.0)
                t[q + "down"] = mat(W, f["expert"]["ff"])
            if f.get("shared"):
                t[p + "mlp.shared.gate"] = mat(f["shared"]["ff"], W, 2.0)
                t[p + "mlp.shared.up"] = mat(f["shared"]["ff"], W, 2.0)
                t[p + "mlp.shared.down"] = mat(W, f["shared"]["ff"])
                t[p + "mlp.shared.sg"] = mat(1, W)
    t["final.norm"] = np.float32(rng.uniform(0.8, 1.2))
    t["head"] = mat(vocab, W)
    cfg = {"architecture": "Kemirax", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": W}
    if not arrays:
        return json.dumps(cfg).encode(), pack_st_bf16(t), None
    bits = {k: to_bf16_bits(np.asarray(v, np.float32).reshape(np.shape(v))) for k, v in t.items()}
    rounded = {k: (b.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(t[k])).astype(np.float64) for k, b in bits.items()}
    return json.dumps(cfg).encode(), pack_st_bf16(t), rounded


# ----------------------------------------------------------------------------------------------------------------------
# Degavik family (config.json + bf16 safetensors): random weights for tests and bench.py
# ----------------------------------------------------------------------------------------------------------------------
def degavik_layer(kind: str, *, heads=4, kv_heads=None, dim=16, vdim=16, rot_dims=None, base=10000.0, decay=None, conv=3, window=8,
                  keep_first=2, scale=None, softcap=20.0, mlp="dense", ff=48, experts=4, top=2, shared_ff=32, weights_of=None) -> dict:
    """One entry of config['layers'].  kind: 'retention' | 'channel_delta' | 'attention'; mlp: 'dense' | 'moe' | None."""
    if kind == "retention":
        mixer = {"heads": heads, "dim": dim, "vdim": vdim, "rot": {"base": float(base), "dims": int(dim if rot_dims is None else rot_dims)},
                 "decay": [float(d) for d in (decay if decay is not None else 1.0 - 2.0 ** (-2.0 - np.arange(heads) * 6.0 / max(heads, 1)))]}
    elif kind == "channel_delta":
        mixer = {"heads": heads, "kv_heads": int(kv_heads or heads), "dim": dim, "vdim": vdim, "conv": int(conv)}
    elif kind == "attention":
        mixer = {"heads": heads, "kv_heads": int(kv_heads or heads), "dim": dim, "vdim": vdim,
                 "rot": {"base": float(base), "dims": int(dim if rot_dims is None else rot_dims)},
                 "scale": float(scale if scale is not None else dim ** -0.5), "softcap": float(softcap),
                 "mask": {"size": int(window), "keep_first": int(keep_first)}}
    else:
        raise ValueError(kind)
    layer = {"type": kind, "mixer": mixer, "mlp": None}
    if mlp == "dense":
        layer["mlp"] = {"kind": "dense", "ff": int(ff)}
    elif mlp == "moe":
        layer["mlp"] = {"kind": "moe", "router": {"experts": int(experts), "top": int(top)}, "expert": {"ff": int(ff)}}
        if shared_ff:
            layer["mlp"]["shared"] = {"ff": int(shared_ff)}
    if weights_of is not None:
        layer["weights_of"] = int(weights_of)
    return layer


def make_degavik(layers: list, width: int = 64, vocab: int = 96, eps: float = 1e-5, seed: int = 0, low_rank: int = 8, arrays: bool = True):
    """(config.json bytes, safetensors image, dict of float64 arrays holding the bf16-rounded values, or None when `arrays` is
    off) for a random model of the family.  Layers with `weights_of` get no tensors."""
    rng = np.random.default_rng(seed)
    W = width
    t = {}

    def mat(n, k, g=1.0):
        return (rng.standard_normal((n, k)) * (g / np.sqrt(k))).astype(np.float32)

    def unit(p, ff):
        t[p + "gate"] = mat(ff, W, 2.0)
        t[p + "up"] = mat(ff, W, 2.0)
        t[p + "down"] = mat(W, ff)

    t["embed"] = rng.standard_normal((vocab, W)).astype(np.float32)
    for i, l in enumerate(layers):
        if l.get("weights_of") is not None:
            continue
        p, m = "l%d." % i, l["mixer"]
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        G = m.get("kv_heads", H)
        t[p + "norm1"] = rng.uniform(0.5, 1.5, W).astype(np.float32)
        if l["type"] == "retention":
            for n, rows in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv)):
                t[p + "mix." + n] = mat(rows, W, 2.0 if n in "qk" else 1.0)
        elif l["type"] == "channel_delta":
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[p + "mix." + n] = mat(rows, W, 2.0)
                t[p + "mix." + n + ".conv"] = (rng.standard_normal((rows, m["conv"])) * 0.6).astype(np.float32)
            t[p + "mix.b"] = mat(H, W, 2.0)
            t[p + "mix.A_log"] = rng.uniform(-4.0, 0.0, H).astype(np.float32)
            t[p + "mix.norm"] = rng.uniform(0.5, 1.5, dv).astype(np.float32)
            t[p + "mix.a1"] = mat(low_rank, W)
            t[p + "mix.a2"] = mat(H * dk, low_rank, 2.0)
            t[p + "mix.dt_bias"] = rng.uniform(-4.0, 1.0, H * dk).astype(np.float32)
            t[p + "mix.g1"] = mat(low_rank, W)
            t[p + "mix.g2"] = mat(H * dv, low_rank, 2.0)
        else:
            t[p + "mix.q"] = mat(H * dk, W, 2.0)
            t[p + "mix.k"] = mat(G * dk, W, 2.0)
            t[p + "mix.v"] = mat(G * dv, W)
            t[p + "mix.q.norm"] = rng.uniform(0.5, 1.5, dk).astype(np.float32)
            t[p + "mix.k.norm"] = rng.uniform(0.5, 1.5, dk).astype(np.float32)
            t[p + "mix.talk"] = (np.eye(H) + 0.3 * rng.standard_normal((H, H))).astype(np.float32)
            t[p + "mix.temp"] = rng.uniform(0.5, 1.5, H).astype(np.float32)
        t[p + "mix.o"] = mat(W, H * dv)
        f = l.get("mlp")
        if f:
            t[p + "norm2"] = rng.uniform(0.5, 1.5, W).astype(np.float32)
            if f["kind"] == "dense":
                unit(p + "mlp.", f["ff"])
            else:
                E = f["router"]["experts"]
                t[p + "mlp.router"] = mat(E, W, 2.0)
                t[p + "mlp.router.b"] = rng.uniform(-0.5, 0.5, E).astype(np.float32)
                for e in range(E):
                    unit(p + "mlp.e%d." % e, f["expert"]["ff"])
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
    t["final.norm"] = rng.uniform(0.5, 1.5, W).astype(np.float32)
    t["head"] = mat(vocab, W)
    cfg = {"architecture": "Degavik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": W}
    if not arrays:
        return json.dumps(cfg).encode(), pack_st_bf16(t), None
    bits = {k: to_bf16_bits(np.asarray(v, np.float32).reshape(np.shape(v))) for k, v in t.items()}
    rounded = {k: (b.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(t[k])).astype(np.float64) for k, b in bits.items()}
    return json.dumps(cfg).encode(), pack_st_bf16(t), rounded


# ----------------------------------------------------------------------------------------------------------------------
# Zufulix family (config.json + bf16 safetensors): random weights for tests and bench.py
# ----------------------------------------------------------------------------------------------------------------------
def zufulix_layer(*, heads=4, kv_heads=None, dim=16, vdim=16, scale=None, bias_max=40, v_mix=True, mlp="dense", ff=48, experts=8, top=2,
                  groups=(4, 2)) -> dict:
    """One entry of config['layers'] (attention mixer).  mlp: 'dense' | 'moe' | None; groups: (count, keep) or None."""
    mixer = {"heads": heads, "kv_heads": int(kv_heads or heads), "dim": dim, "vdim": vdim,
             "scale": float(scale if scale is not None else dim ** -0.5), "bias_max": bias_max}
    if v_mix is not None:
        mixer["v_mix"] = bool(v_mix)
    layer = {"type": "attention", "mixer": mixer, "mlp": None}
    if mlp == "dense":
        layer["mlp"] = {"kind": "dense", "ff": int(ff)}
    elif mlp == "moe":
        router = {"experts": int(experts), "top": int(top)}
        if groups:
            router["groups"] = {"count": int(groups[0]), "keep": int(groups[1])}
        layer["mlp"] = {"kind": "moe", "router": router, "expert": {"ff": int(ff)}}
    return layer


def make_zufulix(layers: list, width: int = 64, vocab: int = 96, eps: float = 1e-5, seed: int = 0, streams: int | None = 3,
                 embed_scale: float | None = 0.7, rel_rows: int = 12, arrays: bool = True, rel_gain: float = 1.0):
    """(config.json bytes, safetensors image, dict of float64 arrays holding the bf16-rounded values, or None when `arrays` is
    off) for a random model of the family.  streams None: the plain residual (no stream tensors)."""
    rng = np.random.default_rng(seed)
    W = width
    t = {}

    def mat(n, k, g=1.0):
        return (rng.standard_normal((n, k)) * (g / np.sqrt(k))).astype(np.float32)

    def norm(name):
        t[name] = rng.uniform(0.5, 1.5, W).astype(np.float32)
        t[name + ".b"] = (0.2 * rng.standard_normal(W)).astype(np.float32)

    t["embed"] = rng.standard_normal((vocab, W)).astype(np.float32)
    for i, l in enumerate(layers):
        p, m = "l%d." % i, l["mixer"]
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        G = m.get("kv_heads", H)
        norm(p + "norm1")
        for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
            t[p + "mix." + n] = mat(rows, W, 2.0 if n in "qk" else 1.0)
            t[p + "mix." + n + ".b"] = (0.3 * rng.standard_normal(rows)).astype(np.float32)
        t[p + "mix.rel"] = (rel_gain * rng.standard_normal((rel_rows, H))).astype(np.float32)
        t[p + "mix.vmix"] = np.float32(rng.uniform(0.2, 0.8))
        t[p + "mix.o"] = mat(W, H * dv)
        f = l.get("mlp")
        subs = [1]
        if f:
            subs.append(2)
            norm(p + "norm2")
            if f["kind"] == "dense":
                t[p + "mlp.up"] = mat(f["ff"], W, 2.0)
                t[p + "mlp.down"] = mat(W, f["ff"])
            else:
                E = f["router"]["experts"]
                t[p + "mlp.router"] = mat(E, W, 3.0)
                for e in range(E):
                    t[p + "mlp.e%d.up" % e] = mat(f["expert"]["ff"], W, 2.0)
                    t[p + "mlp.e%d.down" % e] = mat(W, f["expert"]["ff"])
        if streams is not None:
            for q in subs:
                hp = p + "hc%d." % q
                t[hp + "in"] = (np.full(streams, 1.0 / streams) + 0.2 * rng.standard_normal(streams)).astype(np.float32)
                t[hp + "out"] = rng.uniform(0.5, 1.2, streams).astype(np.float32)
                t[hp + "mix"] = (np.eye(streams) + 0.15 * rng.standard_normal((streams, streams))).astype(np.float32)
    norm("final.norm")
    cfg = {"architecture": "Zufulix", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": W}
    if streams is not None:
        cfg["streams"] = int(streams)
    if embed_scale is not None:
        cfg["embedding"] = {"scale": float(embed_scale)}
    if not arrays:
        return json.dumps(cfg).encode(), pack_st_bf16(t), None
    bits = {k: to_bf16_bits(np.asarray(v, np.float32).reshape(np.shape(v))) for k, v in t.items()}
    rounded = {k: (b.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(t[k])).astype(np.float64) for k, b in bits.items()}
    return json.dumps(cfg).encode(), pack_st_bf16(t), rounded


# ----------------------------------------------------------------------------------------------------------------------
# Pasopel family (config.json + bf16 safetensors): random weights for tests and bench.py
# ----------------------------------------------------------------------------------------------------------------------
def pasopel_layer(kind: str, *, heads=4, kv_heads=None, dim=16, vdim=None, conv=3, window=8, pool=4, rot_dim=8, rot_dims=None, kv_rank=24,
                  q_rank=20, base=10000.0, scale=None, mlp="dense", ff=48, experts=8, top=2, shared_ff=24) -> dict:
    """One entry of config['layers'].  kind: 'attention' | 'latent_attention'; mlp: 'dense' | 'moe' | None; pool 0: no block means."""
    if kind == "attention":
        mixer = {"heads": heads, "kv_heads": int(kv_heads or heads), "dim": dim, "vdim": dim, "conv": int(conv),
                 "scale": float(scale if scale is not None else dim ** -0.5), "mask": {"size": int(window)}}
        if pool:
            mixer["mask"]["pool"] = int(pool)
    elif kind == "latent_attention":
        mixer = {"heads": heads, "dim": dim, "rot_dim": int(rot_dim), "vdim": int(vdim or dim), "kv_rank": int(kv_rank), "q_rank": int(q_rank),
                 "rot": {"base": float(base), "dims": int(rot_dim if rot_dims is None else rot_dims)},
                 "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5), "mask": {"size": int(window)}}
    else:
        raise ValueError(kind)
    layer = {"type": kind, "mixer": mixer, "mlp": None}
    if mlp == "dense":
        layer["mlp"] = {"kind": "dense", "ff": int(ff)}
    elif mlp == "moe":
        layer["mlp"] = {"kind": "moe", "router": {"experts": int(experts), "top": int(top)}, "expert": {"ff": int(ff)}}
        if shared_ff:
            layer["mlp"]["shared"] = {"ff": int(shared_ff)}
    return layer


def make_pasopel(layers: list, width: int = 64, vocab: int = 96, eps: float = 1e-5, seed: int = 0, loop: tuple | None = (0, 1, 2),
                 softcap: float | None = 12.0, arrays: bool = True, sink_gain: float = 1.0):
    """(config.json bytes, safetensors image, dict of float64 arrays holding the bf16-rounded values, or None when `arrays` is
    off) for a random model of the family.  loop: (start, stop, times) or None."""
    rng = np.random.default_rng(seed)
    W = width
    t = {}

    def mat(n, k, g=1.0):
        return (rng.standard_normal((n, k)) * (g / np.sqrt(k))).astype(np.float32)

    def norm(name, n=W):
        t[name] = (0.3 * rng.standard_normal(n)).astype(np.float32)

    def unit(p, ff):
        t[p + "gate"] = mat(ff, W, 2.0)
        t[p + "up"] = mat(ff, W, 2.0)
        t[p + "down"] = mat(W, ff)

    t["embed"] = rng.standard_normal((vocab, W)).astype(np.float32)
    if loop is not None:
        t["loop.step"] = (0.5 * rng.standard_normal((loop[2], W))).astype(np.float32)
    for i, l in enumerate(layers):
        p, m = "l%d." % i, l["mixer"]
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        norm(p + "norm1")
        if l["type"] == "attention":
            G = m.get("kv_heads", H)
            for n, rows in (("q", H * dk), ("k", G * dk)):
                t[p + "mix." + n] = mat(rows, W, 2.0)
                t[p + "mix." + n + ".b"] = (0.3 * rng.standard_normal(rows)).astype(np.float32)
                t[p + "mix." + n + ".conv"] = (rng.standard_normal((rows, m["conv"])) * 0.6).astype(np.float32)
            t[p + "mix.o.b"] = (0.1 * rng.standard_normal(W)).astype(np.float32)
        else:
            dr, rk, rq = m["rot_dim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"] = mat(rq, W)
            t[p + "mix.dq.norm"] = rng.uniform(0.5, 1.5, rq).astype(np.float32)
            t[p + "mix.uq"] = mat(H * (dk + dr), rq, 2.0)
            t[p + "mix.dkv"] = mat(rk + dr, W, 2.0)
            t[p + "mix.dkv.norm"] = rng.uniform(0.5, 1.5, rk).astype(np.float32)
            t[p + "mix.uk"] = mat(H * dk, rk, 2.0)
            t[p + "mix.uv"] = mat(H * dv, rk)
        t[p + "mix.sink"] = (sink_gain * rng.standard_normal(H)).astype(np.float32)
        t[p + "mix.g"] = mat(H * dv, W, 2.0)
        t[p + "mix.o"] = mat(W, H * dv)
        f = l.get("mlp")
        if f:
            norm(p + "norm2")
            if f["kind"] == "dense":
                t[p + "mlp.up"] = mat(f["ff"], W, 2.0)
                t[p + "mlp.down"] = mat(W, f["ff"])
            else:
                E = f["router"]["experts"]
                t[p + "mlp.router"] = mat(E, W, 3.0)
                t[p + "mlp.router.b"] = rng.uniform(-0.5, 0.5, E).astype(np.float32)
                for e in range(E):
                    unit(p + "mlp.e%d." % e, f["expert"]["ff"])
                if f.get("shared"):
                    unit(p + "mlp.shared.", f["shared"]["ff"])
    norm("final.norm")
    cfg = {"architecture": "Pasopel", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": W}
    if loop is not None:
        cfg["loop"] = {"start": int(loop[0]), "stop": int(loop[1]), "times": int(loop[2])}
    if softcap is not None:
        cfg["logit_softcap"] = float(softcap)
    if not arrays:
        return json.dumps(cfg).encode(), pack_st_bf16(t), None
    bits = {k: to_bf16_bits(np.asarray(v, np.float32).reshape(np.shape(v))) for k, v in t.items()}
    rounded = {k: (b.astype(np.uint32) << 16).view(np.float32).reshape(np.shape(t[k])).astype(np.float64) for k, b in bits.items()}
    return json.dumps(cfg).encode(), pack_st_bf16(t), rounded
