"""mLSTM: a matrix memory per head with exponential gates (the matrix cell of xLSTM).

Per head, q = W_q h / sqrt(dim) and k = W_k h of ``dim`` numbers, v = W_v h of ``vdim`` numbers, a log input
gate i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap)).
With a running maximum m that starts at 0,

    m_t = max(f_t + m_(t-1), i_t)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,    n_t the same with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).

Each head's o is divided by its root mean square; the concatenated heads are multiplied by a weight per
channel and by sigmoid(W_g h), then projected out.  S, n and m (float32) start at zero and live in the
request's state slot; gates, exponentials, state, sums and the norm are 32-bit in both dtypes
(``csrc/mlstm.cu``).  The six projections of the input are one product whose rows are stored in 32-bit."""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class MLSTM(Mixer):
    KIND = "mlstm"

    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 dtype=torch.float32, device="cuda"):
        if vdim < 1 or dim < 1 or (vdim > 256 and dim > 700):
            raise ValueError(f"heads of {dim} x {vdim}: values wider than 256 need keys of at most 700 numbers")
        if gate_cap <= 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.cap, self.eps, self.dtype = float(gate_cap), float(eps), dtype
        self.in_weight = self.in_bias = None

    def tensors(self):
        d, H, hd, hv = self.width, self.heads, self.heads * self.dim, self.heads * self.vdim
        return {"q_weight": TensorDecl((hd, d), "matrix"), "k_weight": TensorDecl((hd, d), "matrix"),
                "v_weight": TensorDecl((hv, d), "matrix"),
                "i_weight": TensorDecl((H, d), "matrix"), "i_bias": TensorDecl((H,), "vector"),
                "f_weight": TensorDecl((H, d), "matrix"), "f_bias": TensorDecl((H,), "vector"),
                "gate_weight": TensorDecl((hv, d), "matrix"), "norm_weight": TensorDecl((hv,), "vector"),
                "out_weight": TensorDecl((d, hv), "matrix")}

    def bind(self, tensors):
        """q | k | v | i | f | gate become one product (rows padded to a multiple of 8); the gates' biases are its bias."""
        super().bind(tensors)
        pieces = [self.q_weight, self.k_weight, self.v_weight, self.i_weight, self.f_weight, self.gate_weight]
        rows = sum(p.shape[0] for p in pieces)
        fused = torch.zeros((_padded(rows), self.width), dtype=self.q_weight.dtype, device=self.q_weight.device)
        bias = torch.zeros((fused.shape[0],), dtype=torch.float32, device=fused.device)
        at, views = 0, []
        for p in pieces:
            fused[at:at + p.shape[0]] = p
            views.append(fused[at:at + p.shape[0]])
            at += p.shape[0]
        H, gates_at = self.heads, 2 * self.heads * self.dim + self.heads * self.vdim
        bias[gates_at:gates_at + H] = self.i_bias
        bias[gates_at + H:gates_at + 2 * H] = self.f_bias
        self.in_weight, self.in_bias = fused, bias
        self.q_weight, self.k_weight, self.v_weight, self.i_weight, self.f_weight, self.gate_weight = views

    def cache_need(self):
        return StateNeed((self.heads, ops.mlstm_head_floats(self.dim, self.vdim)), torch.float32)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        state = ctx.cache.state_layer(cache.group, cache.layer)
        proj = ops.linear(h, self.in_weight, self.in_bias, out_dtype=torch.float32)
        o = ops.mlstm(proj, state, self.norm_weight, ctx, self.heads, self.dim, self.vdim, self.cap, self.eps, self.dtype)
        return ops.linear(o, self.out_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


register_part(MLSTM.KIND, MLSTM)
