"""LayerNorm and RMS norm: statistics and affine in 32-bit (``layers/norm.py:198-205``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorDecl, register_part


class LayerNorm(Norm):
    KIND = "layernorm"

    def __init__(self, width: int, eps: float, bias: bool = True, dtype=torch.float32, device="cuda"):
        self.width, self.eps, self.has_bias = width, float(eps), bias
        self.dtype = dtype
        self.weight = None
        self.bias = None

    def tensors(self):
        out = {"weight": TensorDecl((self.width,), "vector")}
        if self.has_bias:
            out["bias"] = TensorDecl((self.width,), "vector")
        return out

    def forward(self, x, ctx, rows=None):
        return ops.layernorm(x, self.weight, self.bias, self.eps, self.dtype, rows=rows)

    def lower(self, builder, x, wanted=False):
        return builder.layernorm(x, self.weight, self.bias, self.eps, self.width, self.dtype, wanted=wanted)

    def add_normed(self, x, y):
        """x += norm(y), in place; x and y float32 [T, width]: a norm that closes a sublayer."""
        ops.layernorm_residual(x, y, self.weight, self.bias, self.eps)
        return x

    def add_normed_then(self, x, y, following: "LayerNorm"):
        """x += norm(y) in place, and ``following``'s norm of the updated x from the same kernel; returns the
        latter in the compute dtype."""
        if not isinstance(following, LayerNorm):
            self.add_normed(x, y)
            return following.forward(x, None)
        return ops.layernorm_residual(x, y, self.weight, self.bias, self.eps,
                                      (following.weight, following.bias, following.eps), following.dtype)


class RMSNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * weight, eps inside the root, all in 32-bit.  ``out_scale`` is a
    constant factor on the result: a norm that closes a sublayer carries the residual multiplier
    there, and ``add_normed`` adds its scaled output to the residual stream in one kernel.
    ``offset``: the checkpoint stores weight - offset (a weight kept around zero has offset 1); the
    sum is made once, in 32-bit, when the tensor is bound.  ``groups`` > 1: the row is cut into that
    many equal consecutive runs and each is divided by its own root mean square; the weight spans
    the whole row."""

    KIND = "rmsnorm"

    def __init__(self, width: int, eps: float, out_scale: float = 1.0, offset: float = 0.0, groups: int = 1,
                 dtype=torch.float32, device="cuda"):
        if groups < 1 or width % groups:
            raise ValueError(f"a row of {width} is not {groups} equal groups")
        self.width, self.eps, self.out_scale, self.offset = width, float(eps), float(out_scale), float(offset)
        self.groups = int(groups)
        self.dtype = dtype
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.width,), "vector")}

    def bind(self, tensors):
        super().bind(tensors)
        if self.offset != 0.0:
            self.weight = self.weight + self.offset          # a tensor of the part's own: the stored one may be shared

    def forward(self, x, ctx, rows=None):
        if self.out_scale != 1.0:
            raise ValueError("an RMS norm with an output factor only adds to the residual stream (add_normed)")
        return ops.rmsnorm(x, self.weight, self.eps, self.dtype, rows=rows, groups=self.groups)

    def add_normed(self, x, y):
        """x += out_scale * norm(y), in place; x and y float32 [T, width]."""
        return ops.rmsnorm_residual(x, y, self.weight, self.eps, self.out_scale, groups=self.groups)


    def add_normed_then(self, x, y, following: "RMSNorm"):
        """x += out_scale * norm(y) in place, and ``following``'s norm of the updated x (one kernel when both
        norms cut the row alike); returns the latter in the compute dtype."""
        if following.groups != self.groups or following.out_scale != 1.0:
            self.add_normed(x, y)
            return following.forward(x, None)
        return ops.rmsnorm_residual_norm(x, y, self.weight, self.eps, self.out_scale, following.weight, following.eps,
                                         following.dtype, groups=self.groups)


register_part(LayerNorm.KIND, LayerNorm)
register_part(RMSNorm.KIND, RMSNorm)
