"""Vedadra in plain NumPy, one function per mechanism, whole sequences, no cache.  Slow and
simple on purpose: it shares no code with the package and is what the kernels are compared
with.  Everything runs in the dtype of the tensors it is given (float64 in the tests).

Notation: x is the residual stream [T, d]; W are [out, in] and applied as W @ x; i is a
query's position and j a key's, both counted from 0."""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# ----------------------------------------------------------- small functions --

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """Division of the last axis by its root mean square, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def grouped_norm(x, w, groups, eps):
    """The row cut into ``groups`` equal runs, each divided by its own root mean square; then the weight."""
    T, d = x.shape
    return unit_rms(x.reshape(T, groups, d // groups), eps).reshape(T, d) * w


def softmax_rows(s, visible):
    """Softmax over the visible keys of every row; s and visible [..., T, T]."""
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.where(visible, np.exp(s), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def window_mask(T, size, keep_first=0):
    """visible[i, j]: j <= i, and j within the last ``size`` positions up to i or among the first ``keep_first``."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def head_slopes(H):
    return 2.0 ** (-8.0 * (np.arange(H) + 1.0) / H)


# -------------------------------------------------------------------- mixers --

def biased_attention(h, t, p, mx, eps):
    """The mixer of kind ``attention``: the values are the projected keys before their norm, scores carry a
    factor per head, lose slope_h (i - j), are then mixed across heads by a matrix, and the concatenated heads
    pass an output gate computed from the same input."""
    T = h.shape[0]
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, D)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, D)
    v = k.copy()
    q = unit_rms(q, eps) * t[p + "q.norm"]
    k = unit_rms(k, eps) * t[p + "k.norm"]
    kv_of = np.arange(H) // (H // G)
    s = np.einsum("ihd,jhd->hij", q, k[:, kv_of]) * mx["scale"]
    s = s * t[p + "temp"][:, None, None]
    dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(h.dtype)
    s = s - head_slopes(H)[:, None, None] * dist
    s = np.einsum("hg,gij->hij", t[p + "talk"], s)
    w = softmax_rows(s, window_mask(T, mx["mask"]["size"]))
    o = np.einsum("hij,jhd->ihd", w, v[:, kv_of]).reshape(T, H * D)
    o = o * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T + t[p + "o.b"]


def differential_lambda(t, p, diff):
    return float(np.exp(np.sum(t[p + "lq1"] * t[p + "lk1"])) - np.exp(np.sum(t[p + "lq2"] * t[p + "lk2"])) + diff)


def differential_attention(h, t, p, mx, eps):
    """The mixer of kind ``attention_2``: every head has two score maps over the same values; the second map's
    output is taken off the first's with the layer's factor, the difference divided by its root mean square and
    scaled.  The window also keeps the sequence's first tokens."""
    T = h.shape[0]
    H, G, D, Dv, diff = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["diff"]
    q = (h @ t[p + "q"].T).reshape(T, H, 2, D)
    k = (h @ t[p + "k"].T).reshape(T, G, 2, D)
    v = (h @ t[p + "v"].T).reshape(T, G, Dv)
    q = unit_rms(q, eps) * t[p + "q.norm"]
    k = unit_rms(k, eps) * t[p + "k.norm"]
    kv_of = np.arange(H) // (H // G)
    s = np.einsum("ihmd,jhmd->hmij", q, k[:, kv_of]) * mx["scale"]
    w = softmax_rows(s, window_mask(T, mx["mask"]["size"], mx["mask"].get("keep_first", 0)))
    a = np.einsum("hmij,jhd->imhd", w, v[:, kv_of])
    o = a[:, 0] - differential_lambda(t, p, diff) * a[:, 1]
    o = unit_rms(o, eps) * (1.0 - diff)
    return o.reshape(T, H * Dv) @ t[p + "o"].T


MIXERS = {"attention": biased_attention, "attention_2": differential_attention}


# -------------------------------------------------------------- feed-forward --

def gated_ff(h, t, p):
    return (gelu_tanh(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


# --------------------------------------------------------------------- model --

def run_order(cfg):
    """[(layer, adds the embedding first)]: the layers of ``loop`` run ``times`` times in a row."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, n = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(a)]
    for rep in range(n):
        out += [(i, rep > 0 and i == a) for i in range(a, b)]
    return out + [(i, False) for i in range(b, L)]


def forward(cfg, t, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the
    residual stream after every layer run."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x0 = t["embed"][np.asarray(tokens)]
    x = x0.copy()
    for i, again in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if again:
            x = x + x0
        y = MIXERS[layer["type"]](grouped_norm(x, t[p + "norm1"], groups, eps), t, p + "mix.", layer["mixer"], eps)
        x = x + grouped_norm(y, t[p + "norm1b"], groups, eps)
        if layer.get("mlp") is not None:
            y = gated_ff(grouped_norm(x, t[p + "norm2"], groups, eps), t, p + "mlp.")
            x = x + grouped_norm(y, t[p + "norm2b"], groups, eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return grouped_norm(x, t["final.norm"], groups, eps) @ t["head"].T


# ------------------------------------------------- tensors, files, configs --

def tensor_shapes(cfg):
    d, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],), "head": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        out[p + "norm1"] = out[p + "norm1b"] = (d,)
        if layer["type"] == "attention":
            out.update({p + "mix.q": (H * D, d), p + "mix.q.b": (H * D,), p + "mix.k": (G * D, d), p + "mix.k.b": (G * D,),
                        p + "mix.q.norm": (D,), p + "mix.k.norm": (D,), p + "mix.talk": (H, H), p + "mix.temp": (H,),
                        p + "mix.g": (H * Dv, d), p + "mix.o": (d, H * Dv), p + "mix.o.b": (d,)})
        else:
            out.update({p + "mix.q": (H * 2 * D, d), p + "mix.k": (G * 2 * D, d), p + "mix.v": (G * Dv, d),
                        p + "mix.q.norm": (D,), p + "mix.k.norm": (D,), p + "mix.lq1": (D,), p + "mix.lk1": (D,),
                        p + "mix.lq2": (D,), p + "mix.lk2": (D,), p + "mix.o": (d, H * Dv)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out[p + "norm2"] = out[p + "norm2b"] = (d,)
            out.update({p + "mlp.gate": (ff, d), p + "mlp.up": (ff, d), p + "mlp.down": (d, ff)})
    return out


def round_bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


def random_tensors(cfg, seed, gain=1.0):
    """Every tensor as float32 values that bfloat16 holds exactly."""
    rs = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        g = rs.standard_normal(shape).astype(np.float32)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            w = 0.5 * g
        elif last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            w = 1.0 + 0.1 * g
        elif name.endswith(".q.norm") or name.endswith(".k.norm"):
            w = 1.0 + 0.1 * g
        elif last == "temp":
            w = 1.0 + 0.2 * g
        elif last == "talk":
            w = np.eye(shape[0], dtype=np.float32) + 0.2 * g
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            w = 0.15 * g
        elif last == "b":
            w = 0.3 * g
        else:
            w = gain * g / np.sqrt(shape[-1])
        out[name] = round_bf16(w.astype(np.float32))
    return out


def write_safetensors(path, tensors):
    """Floats as BF16 (the values are exact in it)."""
    header, chunks, off = {}, [], 0
    for name, arr in tensors.items():
        raw = (np.ascontiguousarray(arr, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        chunks.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


def write_folder(folder, cfg, tensors):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def greedy_generate(cfg, t, prompt, n):
    """n tokens, each the arg max of the last position's logits (the whole sequence is run again every time)."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(cfg, t, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
