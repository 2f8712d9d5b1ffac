"""Tesozen in plain NumPy, one function per mechanism, whole sequences, no cache.  Slow and
simple on purpose: it shares no code with the package and is what the kernels are compared
with.  Everything runs in the dtype of the tensors it is given (float64 in the tests).

Notation: x is the residual stream [T, d]; W are [out, in] and applied as W @ x; i is a
query's position and j a key's, both counted from 0; t counts time steps of a recurrence."""

from __future__ import annotations

import numpy as np

from plain_vedadra import round_bf16, write_folder, write_safetensors  # noqa: F401  (file helpers only)


# ----------------------------------------------------------- small functions --

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def unit_rms(x, eps):
    """Division of the last axis by its root mean square, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.where(visible, np.exp(s), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def causal_mask(T):
    return np.arange(T)[None, :] <= np.arange(T)[:, None]


def chunk_mask(T, size):
    """visible[i, j]: j <= i and both in the same run of ``size`` positions counted from 0."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


# -------------------------------------------------------------------- mixers --

def differential_lambda(t, p, diff):
    return float(np.exp(np.sum(t[p + "lq1"] * t[p + "lk1"])) - np.exp(np.sum(t[p + "lq2"] * t[p + "lk2"])) + diff)


def chunked_differential_attention(h, t, p, mx, eps):
    """Two score maps per head over the same values, keys visible inside the query's chunk only; the second
    map's output is taken off the first's, the difference divided by its root mean square and scaled; one gate
    number per head from the same input."""
    T = h.shape[0]
    H, G, D, Dv, diff = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["diff"]
    q = (h @ t[p + "q"].T).reshape(T, H, 2, D)
    k = (h @ t[p + "k"].T).reshape(T, G, 2, D)
    v = (h @ t[p + "v"].T).reshape(T, G, Dv)
    q = unit_rms(q, eps) * t[p + "q.norm"]
    k = unit_rms(k, eps) * t[p + "k.norm"]
    kv_of = np.arange(H) // (H // G)
    s = np.einsum("ihmd,jhmd->hmij", q, k[:, kv_of]) * mx["scale"]
    mask = chunk_mask(T, mx["mask"]["size"]) if mx.get("mask") else causal_mask(T)
    w = softmax_rows(s, mask)
    a = np.einsum("hmij,jhd->imhd", w, v[:, kv_of])
    o = a[:, 0] - differential_lambda(t, p, diff) * a[:, 1]
    o = unit_rms(o, eps) * (1.0 - diff)
    o = o * sigmoid(h @ t[p + "g"].T)[:, :, None]
    return o.reshape(T, H * Dv) @ t[p + "o"].T


def mlstm_gates(h, t, p, cap):
    """Log input gate and log forget gate per (token, head), both behind a soft cap."""
    i = cap * np.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    f = log_sigmoid(cap * np.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f):
    """The matrix memory walked token by token from an empty state.  q, k [T, H, D], v [T, H, Dv], gates [T, H].
    The stabilizer m starts at 0."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = np.zeros((H, D, Dv), dtype=q.dtype)
    n = np.zeros((H, D), dtype=q.dtype)
    m = np.zeros((H,), dtype=q.dtype)
    out = np.zeros((T, H, Dv), dtype=q.dtype)
    for s in range(T):
        m_new = np.maximum(f[s] + m, i[s])
        keep, write = np.exp(f[s] + m - m_new), np.exp(i[s] - m_new)
        S = keep[:, None, None] * S + write[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[s]
        m = m_new
        num = np.einsum("hdv,hd->hv", S, q[s])
        den = np.maximum(np.abs(np.einsum("hd,hd->h", n, q[s])), np.exp(-m)) + 1e-6
        out[s] = num / den[:, None]
    return out


def mlstm(h, t, p, mx, eps):
    T = h.shape[0]
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    q = (h @ t[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ t[p + "k"].T).reshape(T, H, D)
    v = (h @ t[p + "v"].T).reshape(T, H, Dv)
    i, f = mlstm_gates(h, t, p, mx["gate_cap"])
    o = unit_rms(mlstm_recurrence(q, k, v, i, f), eps).reshape(T, H * Dv)
    o = o * t[p + "norm"] * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def plain_latent_attention(h, t, p, mx, eps):
    """Keys and values are up-projections of one normed latent per token; no positions; causal; a gate per
    output number."""
    T = h.shape[0]
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    q = (h @ t[p + "q"].T).reshape(T, H, D)
    c = unit_rms(h @ t[p + "dkv"].T, eps) * t[p + "dkv.norm"]
    k = (c @ t[p + "uk"].T).reshape(T, H, D)
    v = (c @ t[p + "uv"].T).reshape(T, H, Dv)
    s = np.einsum("ihd,jhd->hij", q, k) * mx["scale"]
    w = softmax_rows(s, causal_mask(T))
    o = np.einsum("hij,jhd->ihd", w, v).reshape(T, H * Dv)
    o = o * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


MIXERS = {"attention": chunked_differential_attention, "mlstm": mlstm, "latent_attention": plain_latent_attention}


# -------------------------------------------------------------- feed-forward --

def dense_ff(h, t, p):
    return (np.maximum(h @ t[p + "up"].T, 0.0) ** 2) @ t[p + "down"].T


def silu_expert(h, t, p):
    g = h @ t[p + "gate"].T
    return (g * sigmoid(g) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def route(z, correction, top, count, keep, scale, margin=None):
    """One token's routing from its logits z [E]: (chosen experts, their weights).  ``margin``: a list that
    receives how far the choice was from turning out otherwise (the smaller of the gap between the last kept
    group and the next one, and between the last chosen expert and the next allowed one)."""
    E = z.shape[0]
    s = sigmoid(z)
    ranking = s + correction
    per = E // count
    group_score = np.array([np.sort(ranking[g * per:(g + 1) * per])[-2:].sum() for g in range(count)])
    order = sorted(range(count), key=lambda g: (-group_score[g], g))
    allowed = np.full(E, -np.inf)
    for g in order[:keep]:
        allowed[g * per:(g + 1) * per] = ranking[g * per:(g + 1) * per]
    ranked = sorted(range(E), key=lambda e: (-allowed[e], e))
    chosen = ranked[:top]
    if margin is not None:
        gaps = [group_score[order[keep - 1]] - group_score[order[keep]]] if keep < count else []
        if top < E and np.isfinite(allowed[ranked[top]]):
            gaps.append(allowed[ranked[top - 1]] - allowed[ranked[top]])
        margin.append(min(gaps) if gaps else np.inf)
    w = s[chosen] / (s[chosen].sum() + 1e-20) * scale
    return chosen, w


def moe_ff(h, t, p, mlp, margins=None):
    """``margins``: a list that receives one array [T] of this layer's routing margins (see ``route``)."""
    r = mlp["router"]
    mine = [] if margins is not None else None
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ t[p + "router"].T
    out = np.zeros_like(h)
    for n in range(h.shape[0]):
        chosen, w = route(z[n], t[p + "correction"], r["top"], groups["count"], groups["keep"], r["scale"], mine)
        for e, we in zip(chosen, w):
            out[n] += we * silu_expert(h[n:n + 1], t, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + silu_expert(h, t, p + "shared.")
    if margins is not None:
        margins.append(np.asarray(mine))
    return out


def feed_forward(h, t, p, mlp, margins=None):
    return dense_ff(h, t, p) if mlp["kind"] == "dense" else moe_ff(h, t, p, mlp, margins)


# --------------------------------------------------------------------- model --

def forward(cfg, t, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the
    residual stream after every layer; ``margins``: see ``moe_ff``."""
    eps = cfg["norm"]["eps"]

    def ln(x, name):
        return layer_norm(x, t[name], t[name + ".b"], eps)

    x = t["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](ln(x, p + "norm1"), t, p + "mix.", layer["mixer"], eps)
        x = x + ln(y, p + "norm1b")
        if layer.get("mlp") is not None:
            y = feed_forward(ln(x, p + "norm2"), t, p + "mlp.", layer["mlp"], margins)
            x = x + ln(y, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.copy())
    return ln(x, "final.norm") @ t["embed"].T


# ------------------------------------------------- tensors, files, configs --

def tensor_shapes(cfg):
    d = cfg["width"]
    out = {"embed": (cfg["vocab"], d), "final.norm": (d,), "final.norm.b": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") is not None else [])
        for n in names:
            out[p + n] = out[p + n + ".b"] = (d,)
        m = p + "mix."
        if layer["type"] == "attention":
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            out.update({m + "q": (H * 2 * D, d), m + "k": (G * 2 * D, d), m + "v": (G * Dv, d), m + "q.norm": (D,),
                        m + "k.norm": (D,), m + "lq1": (D,), m + "lk1": (D,), m + "lq2": (D,), m + "lk2": (D,),
                        m + "g": (H, d), m + "o": (d, H * Dv)})
        elif layer["type"] == "mlstm":
            H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
            out.update({m + "q": (H * D, d), m + "k": (H * D, d), m + "v": (H * Dv, d), m + "g": (H * Dv, d),
                        m + "o": (d, H * Dv), m + "norm": (H * Dv,), m + "i": (H, d), m + "i.b": (H,),
                        m + "f": (H, d), m + "f.b": (H,)})
        else:
            H, D, Dv, R = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"]
            out.update({m + "q": (H * D, d), m + "dkv": (R, d), m + "dkv.norm": (R,), m + "uk": (H * D, R),
                        m + "uv": (H * Dv, R), m + "g": (H * Dv, d), m + "o": (d, H * Dv)})
        mlp = layer.get("mlp")
        f = p + "mlp."
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({f + "up": (mlp["ff"], d), f + "down": (d, mlp["ff"])})
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            out.update({f"{f}e{e}.gate": (ff, d), f"{f}e{e}.up": (ff, d), f"{f}e{e}.down": (d, ff)})
        out.update({f + "router": (mlp["router"]["experts"], d), f + "correction": (mlp["router"]["experts"],)})
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            out.update({f + "shared.gate": (sf, d), f + "shared.up": (sf, d), f + "shared.down": (d, sf)})
    return out


def random_tensors(cfg, seed, gain=1.0):
    """Every tensor as float32 values that bfloat16 holds exactly."""
    rs = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        g = rs.standard_normal(shape).astype(np.float32)
        last = name.rsplit(".", 1)[-1]
        stem = name[:-2] if last == "b" else name
        if name == "embed":
            w = 0.5 * g
        elif last == "b" and (stem.rsplit(".", 1)[-1] in ("norm1", "norm2", "norm1b", "norm2b") or stem == "final.norm"):
            w = 0.1 * g
        elif last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm" or last == "norm":
            w = 1.0 + 0.1 * g
        elif name.endswith(".i.b"):
            w = 0.5 * g
        elif name.endswith(".f.b"):
            w = 2.0 + 1.0 * g
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            w = 0.15 * g
        elif last == "correction":
            w = 0.2 * g
        elif last == "router":
            w = 2.0 * g / np.sqrt(shape[-1])
        else:
            w = gain * g / np.sqrt(shape[-1])
        out[name] = round_bf16(w.astype(np.float32))
    return out


def greedy_generate(cfg, t, prompt, n):
    """n tokens, each the arg max of the last position's logits (the whole sequence is run again every time)."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(cfg, t, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
