"""Two softmax attentions over the paged cache that share one set of kernels (``csrc/attention_grouped.cu``):
per-head RMS norm of queries and keys with one weight for all heads, keys and values grouped separately, a
window, no rotation.

``talking_attention``: q = W_q h + b_q, k = W_k h + b_k; the values are the projected keys as they are before
their norm.  The score of head g is (q_g . k) scale temp_g - slope_g (i - j) with slope_g = 2^(-c (g + 1) / H);
the heads' scores are then mixed, s'_h = sum_g talk[h, g] s_g, before the softmax over the window.  The mix is
linear in the scores, so it is applied to the queries instead (``ops.head_norm_prepare``), once per token and
not once per query and key: the attention kernel sees H query heads, one key of G * dim numbers per token and
G value heads.  The concatenated heads are multiplied by sigmoid(W_g h) before the output projection (with bias).

``differential_attention``: every head has two score maps (its query and its key/value head's key are
[map 1, map 2]) over the same values v = W_v h; with a1 and a2 the maps' outputs,
o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, then o / rms(o) * (1 - diff) per head.
The window also keeps the sequence's first ``keep_first`` tokens; with ``chunk`` a query sees only the keys of
its own run of that many positions (runs counted from position 0 of the sequence).  ``head_gate``: head h's
output is multiplied by sigmoid(W_g h)_h, one number per head, before the output projection.  The kernel sees
2 H query heads, 2 G key heads and G value heads.

Norms, scores, weights, the mix and lambda are 32-bit in both dtypes."""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import KVNeed, Mixer, TensorDecl, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


def _fuse(pieces, width: int, biases=None):
    """Matrices one under the other (rows padded to a multiple of 8) and their biases (zeros where none)."""
    rows = sum(p.shape[0] for p in pieces)
    fused = torch.zeros((_padded(rows), width), dtype=pieces[0].dtype, device=pieces[0].device)
    bias = torch.zeros((fused.shape[0],), dtype=torch.float32, device=fused.device) if biases is not None else None
    at, views = 0, []
    for i, p in enumerate(pieces):
        fused[at:at + p.shape[0]] = p
        if biases is not None and biases[i] is not None:
            bias[at:at + p.shape[0]] = biases[i]
        views.append(fused[at:at + p.shape[0]])
        at += p.shape[0]
    return fused, bias, views


def _check_heads(heads: int, kv_heads: int, dim: int, vdim: int) -> None:
    if heads % kv_heads:
        raise ValueError(f"{heads} heads cannot share {kv_heads} key/value heads")
    if not (1 <= dim and 1 <= vdim <= 256):
        raise ValueError(f"head sizes {dim} / {vdim}: the attention kernels take values of 1 to 256 numbers")


class TalkingAttention(Mixer):
    KIND = "talking_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, scale: float, eps: float,
                 window: int | None = None, slope_exponent: float = 8.0, dtype=torch.float32, device="cuda"):
        _check_heads(heads, kv_heads, dim, dim)
        if kv_heads * dim > 1024:
            raise ValueError(f"{kv_heads} key heads of {dim}: a token's keys side by side may have at most 1024 numbers")
        self.width, self.heads, self.kv_heads, self.dim = width, heads, kv_heads, dim
        self.scale, self.eps, self.window, self.slope_exponent, self.dtype = float(scale), float(eps), window, float(slope_exponent), dtype
        self.in_weight = self.in_bias = self.mix = self.slopes = None

    def tensors(self):
        d, hd, gd = self.width, self.heads * self.dim, self.kv_heads * self.dim
        return {"q_weight": TensorDecl((hd, d), "matrix"), "q_bias": TensorDecl((hd,), "vector"),
                "k_weight": TensorDecl((gd, d), "matrix"), "k_bias": TensorDecl((gd,), "vector"),
                "q_norm": TensorDecl((self.dim,), "vector"), "k_norm": TensorDecl((self.dim,), "vector"),
                "talk": TensorDecl((self.heads, self.heads), "vector"), "temp": TensorDecl((self.heads,), "vector"),
                "gate_weight": TensorDecl((hd, d), "matrix"),
                "out_weight": TensorDecl((d, hd), "matrix"), "out_bias": TensorDecl((d,), "vector")}

    def bind(self, tensors):
        """q | k | gate become one product.  The mix of the scores with each head's factors folded in
        (talk[h, g] temp[g] scale) and the mixed slopes are made once, from 64-bit products."""
        super().bind(tensors)
        self.in_weight, self.in_bias, (self.q_weight, self.k_weight, self.gate_weight) = _fuse(
            [self.q_weight, self.k_weight, self.gate_weight], self.width, [self.q_bias, self.k_bias, None])
        talk = self.talk.double()
        H = self.heads
        slopes = torch.tensor([2.0 ** (-self.slope_exponent * (h + 1) / H) for h in range(H)], dtype=torch.float64, device=talk.device)
        self.mix = (talk * (self.temp.double() * self.scale)[None, :]).float().contiguous()
        self.slopes = (talk @ slopes).float().contiguous()

    def cache_need(self):
        return KVNeed(kv_heads=self.kv_heads, head_dim=self.dim, window=self.window, value_heads=self.kv_heads, value_dim=self.dim)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        kpages, vpages = ctx.cache.kv_layer(cache.group, cache.layer)
        table = ctx.tables[cache.group]
        H, G, D = self.heads, self.kv_heads, self.dim
        proj = ops.linear(h, self.in_weight, self.in_bias, out_dtype=torch.float32)
        q = ops.head_norm_prepare(proj, kpages, vpages, self.q_norm, self.k_norm, ctx, table, H, G, D, 1, H * D, self.eps,
                                  cache.writes, self.dtype, mix=self.mix)
        o = ops.grouped_attention(q, kpages, vpages, table, ctx, heads=H, key_heads=1, key_dim=G * D, scale=1.0,
                                  slopes=self.slopes, window=self.window, gate=proj[:, (H + G) * D:(2 * H + G) * D])
        return ops.linear(o, self.out_weight, self.out_bias, residual=residual, out_dtype=torch.float32, out=residual)


class DifferentialAttention(Mixer):
    KIND = "differential_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, diff: float, eps: float,
                 window: int | None = None, keep_first: int = 0, chunk: int | None = None, head_gate: bool = False,
                 dtype=torch.float32, device="cuda"):
        _check_heads(heads, kv_heads, dim, vdim)
        if chunk is not None and chunk < 1:
            raise ValueError(f"a chunk of {chunk} positions")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.diff, self.eps, self.window, self.keep_first, self.dtype = float(scale), float(diff), float(eps), window, int(keep_first), dtype
        self.chunk, self.head_gate = chunk, bool(head_gate)
        self.in_weight = None
        self.lam = 0.0

    def tensors(self):
        d, D = self.width, self.dim
        out = {"q_weight": TensorDecl((self.heads * 2 * D, d), "matrix"), "k_weight": TensorDecl((self.kv_heads * 2 * D, d), "matrix"),
               "v_weight": TensorDecl((self.kv_heads * self.vdim, d), "matrix"),
               "q_norm": TensorDecl((D,), "vector"), "k_norm": TensorDecl((D,), "vector"),
               "out_weight": TensorDecl((d, self.heads * self.vdim), "matrix")}
        if self.head_gate:
            out["gate_weight"] = TensorDecl((self.heads, d), "matrix")
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = TensorDecl((D,), "vector")
        return out

    def bind(self, tensors):
        super().bind(tensors)
        if self.head_gate:
            self.in_weight, _, (self.q_weight, self.k_weight, self.v_weight, self.gate_weight) = _fuse(
                [self.q_weight, self.k_weight, self.v_weight, self.gate_weight], self.width)
        else:
            self.in_weight, _, (self.q_weight, self.k_weight, self.v_weight) = _fuse([self.q_weight, self.k_weight, self.v_weight], self.width)
        one = float((self.lq1.double() * self.lk1.double()).sum())
        two = float((self.lq2.double() * self.lk2.double()).sum())
        self.lam = math.exp(one) - math.exp(two) + self.diff

    def cache_need(self):
        return KVNeed(kv_heads=2 * self.kv_heads, head_dim=self.dim, window=self.window, value_heads=self.kv_heads,
                      value_dim=self.vdim, keep_first=self.keep_first if self.window is not None else 0, chunk=self.chunk)

    def forward(self, h, residual, ctx, cache):
        kpages, vpages = ctx.cache.kv_layer(cache.group, cache.layer)
        table = ctx.tables[cache.group]
        H, G, D = self.heads, self.kv_heads, self.dim
        proj = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)
        q = ops.head_norm_prepare(proj, kpages, vpages, self.q_norm, self.k_norm, ctx, table, H, G, D, 2, (H + G) * 2 * D,
                                  self.eps, cache.writes, self.dtype)
        gate = proj[:, (H + G) * 2 * D + G * self.vdim:] if self.head_gate else None
        o = ops.grouped_attention(q, kpages, vpages, table, ctx, heads=2 * H, key_heads=2 * G, key_dim=D, scale=self.scale,
                                  window=self.window, keep_first=self.keep_first, maps=2, lam=self.lam,
                                  post_scale=1.0 - self.diff, eps=self.eps, chunk=self.chunk, gate=gate)
        return ops.linear(o, self.out_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


register_part(TalkingAttention.KIND, TalkingAttention)
register_part(DifferentialAttention.KIND, DifferentialAttention)
