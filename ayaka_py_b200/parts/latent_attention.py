"""Latent attention: causal attention whose keys and values are up-projections of
one small latent per token.

Per token the input is projected down to ``kv_rank + rot_dim`` numbers: the first
``kv_rank``, RMS-normed, are the latent c; the last ``rot_dim`` are a key part that
is rotated by the position and shared by all heads.  A head's query is laid out as
[``dim`` unrotated | ``rot_dim`` rotated]; its unrotated key is U_k c, its value
U_v c, the score (q_n . k_n + q_r . k_r) * scale, softmax over the positions up to
the query's.  Each head's output is multiplied by sigmoid of a gate that is a
projection of the same input, and the heads are projected out.

``rot_dim`` 0 (``rot`` None): there is no rotated part and positions do not enter the scores.
``gate`` "element": the gate has one number per output number of every head (the concatenated
heads times sigmoid(W_g h) element by element) instead of one per head.

Only c and the rotated key part are cached (the cache manager's pages: "keys" hold
the rotated part, "values" the latent, one head each).  The kernels never expand
keys or values: with q' = U_k^T q_n the score is q' . c + q_r . k_r, and
sum_j p_j U_v c_j = U_v sum_j p_j c_j, so attention runs over the cached pairs and
U_v is applied once per row (``csrc/latent.cu``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import KVNeed, Mixer, PartSpec, TensorDecl, make_part, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttention(Mixer):
    KIND = "latent_attention"

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 eps: float, rot: dict | None, gate: str = "head", dtype=torch.float32, device="cuda"):
        if (rot is None) != (rot_dim == 0):
            raise ValueError(f"a rotated part of {rot_dim} and rotation constants {rot!r} do not go together")
        if rot is not None and (rot_dim < 2 or rot["dims"] > rot_dim):
            raise ValueError(f"{rot['dims']} rotated dimensions do not fit a rotated part of {rot_dim}")
        if gate not in ("head", "element"):
            raise ValueError(f"unknown gate {gate!r}; known: head, element")
        self.width, self.heads, self.dim, self.rot_dim, self.vdim, self.rank = width, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.dtype = float(scale), float(eps), dtype
        self.gate_width = heads if gate == "head" else heads * vdim
        self.rotary = None if rot is None else make_part(
            PartSpec("rotary", {"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling")}), dtype, device)
        self.no_freq = None
        self.q_width = heads * (dim + rot_dim)
        self.down_width = kv_rank + rot_dim
        self.in_weight = None

    def tensors(self):
        H = self.heads
        return {"q_weight": TensorDecl((self.q_width, self.width), "matrix"),
                "down_weight": TensorDecl((self.down_width, self.width), "matrix"),
                "down_norm": TensorDecl((self.rank,), "vector"),
                "uk_weight": TensorDecl((H * self.dim, self.rank), "matrix"),
                "uv_weight": TensorDecl((H * self.vdim, self.rank), "matrix"),
                "gate_weight": TensorDecl((self.gate_width, self.width), "matrix"),
                "out_weight": TensorDecl((self.width, H * self.vdim), "matrix")}

    def bind(self, tensors):
        """The three projections of the input become one product (q | down | gate, rows padded to a
        multiple of 8); the up-projections are laid out per head for the per-head products."""
        super().bind(tensors)
        H, total = self.heads, self.q_width + self.down_width + self.gate_width
        fused = torch.zeros((_padded(total), self.width), dtype=self.q_weight.dtype, device=self.q_weight.device)
        fused[:self.q_width] = self.q_weight
        fused[self.q_width:self.q_width + self.down_width] = self.down_weight
        fused[self.q_width + self.down_width:total] = self.gate_weight
        self.in_weight = fused
        self.q_weight = fused[:self.q_width]
        self.down_weight = fused[self.q_width:self.q_width + self.down_width]
        self.gate_weight = fused[self.q_width + self.down_width:total]
        self.uk_heads = self.uk_weight.view(H, self.dim, self.rank).transpose(1, 2).contiguous()      # [H, rank, dim]
        self.uv_heads = self.uv_weight.view(H, self.vdim, self.rank)                                   # [H, vdim, rank]

    def cache_need(self):
        return KVNeed(kv_heads=1, head_dim=self.rot_dim, window=None, value_heads=1, value_dim=self.rank)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        rope_pages, latent_pages = ctx.cache.kv_layer(cache.group, cache.layer)
        table = ctx.tables[cache.group]
        T, H = h.shape[0], self.heads
        proj = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)
        if self.rotary is None:
            if self.no_freq is None:
                self.no_freq = torch.zeros((1,), dtype=torch.float32, device=h.device)
            freq, gain, rot_dims = self.no_freq, 1.0, 0
        else:
            freq, gain, rot_dims = self.rotary.freq, self.rotary.gain, self.rotary.dims
        query = ops.latent_prepare(proj, latent_pages, rope_pages, self.down_norm, freq, gain, rot_dims, ctx, table, H,
                                   self.dim, self.rot_dim, self.rank, self.eps, cache.writes)
        q_plain = proj[:, :self.q_width].view(T, H, self.dim + self.rot_dim)[:, :, :self.dim]
        ops.head_matmul(q_plain, self.uk_heads, query[:, :, :self.rank])
        mixed = ops.latent_attention(query, latent_pages, rope_pages, table, ctx, self.scale)
        gate = proj[:, self.q_width + self.down_width:self.q_width + self.down_width + self.gate_width]
        o = torch.empty((T, H, self.vdim), dtype=self.dtype, device=h.device)
        ops.head_matmul(mixed, self.uv_heads, o, gate=gate)
        return ops.linear(o.view(T, H * self.vdim), self.out_weight, None, residual=residual,
                          out_dtype=torch.float32, out=residual)


register_part(LatentAttention.KIND, LatentAttention)
