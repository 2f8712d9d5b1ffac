"""Dense feed-forward: up projection, activation, down projection, residual
(``models/gpt2.py:400-403``, ``:437-438``).  Bias, activation (in 32-bit) and
the residual sum are fused into the two matrix products' epilogues."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_part


class MLP(FeedForward):
    KIND = "mlp"

    def __init__(self, width: int, inner: int, activation: str, bias: bool = True,
                 dtype=torch.float32, device="cuda"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.width, self.inner, self.activation, self.has_bias = width, inner, activation, bias
        self.dtype = dtype
        self.up_weight = self.up_bias = self.down_weight = self.down_bias = None

    def tensors(self):
        out = {"up_weight": TensorDecl((self.inner, self.width), "matrix"),
               "down_weight": TensorDecl((self.width, self.inner), "matrix")}
        if self.has_bias:
            out["up_bias"] = TensorDecl((self.inner,), "vector")
            out["down_bias"] = TensorDecl((self.width,), "vector")
        return out

    def forward(self, h, residual, ctx):
        u = ops.linear(h, self.up_weight, self.up_bias, activation=self.activation, out_dtype=self.dtype)
        return ops.linear(u, self.down_weight, self.down_bias, residual=residual,
                          out_dtype=torch.float32, out=residual)

    def lower(self, builder, h, residual):
        u = builder.linear(h, self.up_weight, self.up_bias, activation=self.activation, out_dtype=self.dtype)
        out = builder.linear(u, self.down_weight, self.down_bias, residual=residual, out_dtype=torch.float32, out=residual)
        builder.release(u)
        return out


class PolyNormMLP(FeedForward):
    """down(act(up h)) without biases, act = PolyNorm: a N(z) + b N(z^2) + c N(z^3) + e with powers
    taken element by element and N the division of a token's vector by its root mean square
    (eps inside the root); the four numbers are a tensor of the part.  The up projection is
    stored in 32-bit, the norms are 32-bit, the activation is stored in the compute dtype."""

    KIND = "polynorm_mlp"

    def __init__(self, width: int, inner: int, eps: float, dtype=torch.float32, device="cuda"):
        self.width, self.inner, self.eps, self.dtype = width, inner, float(eps), dtype
        self.up_weight = self.down_weight = self.coeff = None

    def tensors(self):
        return {"up_weight": TensorDecl((self.inner, self.width), "matrix"),
                "down_weight": TensorDecl((self.width, self.inner), "matrix"),
                "coeff": TensorDecl((4,), "vector")}

    def forward(self, h, residual, ctx):
        """residual + ff(h); with ``residual`` None the sublayer's output alone, float32."""
        z = ops.linear(h, self.up_weight, None, out_dtype=torch.float32)
        u = ops.polynorm(z, self.coeff, self.eps, self.dtype)
        return ops.linear(u, self.down_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


class GatedMLP(FeedForward):
    """down(act(gate h) * (up h)) without biases.  gate | up is one product, stored in 32-bit; the
    activation and the product of the halves are 32-bit, their result is stored in the compute dtype."""

    KIND = "gated_mlp"

    def __init__(self, width: int, inner: int, activation: str, dtype=torch.float32, device="cuda"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.width, self.inner, self.activation, self.dtype = width, inner, activation, dtype
        self.gate_weight = self.up_weight = self.down_weight = self.in_weight = None

    def tensors(self):
        return {"gate_weight": TensorDecl((self.inner, self.width), "matrix"),
                "up_weight": TensorDecl((self.inner, self.width), "matrix"),
                "down_weight": TensorDecl((self.width, self.inner), "matrix")}

    def bind(self, tensors):
        super().bind(tensors)
        self.in_weight = torch.cat([self.gate_weight, self.up_weight], dim=0).contiguous()
        self.gate_weight, self.up_weight = self.in_weight[:self.inner], self.in_weight[self.inner:]

    def forward(self, h, residual, ctx):
        """residual + ff(h); with ``residual`` None the sublayer's output alone, float32."""
        z = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)
        u = ops.gated_act(z, self.inner, self.activation, self.dtype)
        return ops.linear(u, self.down_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


register_part(MLP.KIND, MLP)
register_part(GatedMLP.KIND, GatedMLP)
register_part(PolyNormMLP.KIND, PolyNormMLP)
