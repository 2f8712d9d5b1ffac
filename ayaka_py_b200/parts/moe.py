"""Mixture of experts with a gated shared expert.

Router: z = W_r h in 32-bit; the ``top`` experts with the largest z are chosen and weighted by
the softmax over the chosen z only.  An expert (no biases): g = min(W_gate h, limit),
u = clamp(W_up h, -limit, limit), y = W_down (g sigmoid(1.702 g) (u + 1)).  The output is the
weighted sum of the chosen experts' y plus the shared expert's (same form, sizes and limit of
its own), which runs for every token and is multiplied by sigmoid(w_mix . h), one number per
token.

Variants, all by parameters: ``router="sigmoid_groups"`` chooses by s + correction with s = sigmoid(z)
and a correction per expert (a tensor of the part) among the experts of the ``keep`` best of ``groups``
equal runs of consecutive experts (a run's score: the sum of its two largest ranking scores; the others cannot be
chosen at all), and weights the chosen experts by s over their sum, times ``route_scale``.  ``slope`` and
``plus`` set the activation g sigmoid(slope g) (u + plus); a limit of None clamps nothing (slope 1, plus 0,
no limit: silu(gate) * up).  ``shared_gated`` False: the shared expert is added as it is;
``shared_inner`` 0: there is none.

The experts' matrices are kept stacked ([experts, 2 inner, width] with gate over up, and
[experts, width, inner]); a step sorts its (token, choice) pairs by expert on the device and runs
two grouped products over the sorted rows, so nothing about the routing comes back to the host
(``csrc/moe.cu``): on tcgen05 for bfloat16 steps of many pairs (every expert's rows padded to whole
128-row tiles), pair by pair as matrix-vector products for a handful of pairs, on mma.sync or the
FP32 pipes otherwise.  The shared expert's gate, up and mixing row are one dense product."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class MoE(FeedForward):
    KIND = "moe"
    GATE_SLOPE = 1.702

    def __init__(self, width: int, experts: int, top: int, inner: int, limit: float | None, shared_inner: int,
                 shared_limit: float | None, router: str = "softmax", groups: int = 1, keep: int = 1,
                 route_scale: float = 1.0, slope: float = GATE_SLOPE, plus: float = 1.0, shared_gated: bool = True,
                 dtype=torch.float32, device="cuda"):
        if not 1 <= top <= min(experts, 16):
            raise ValueError(f"top {top} of {experts} experts: the routing kernel picks 1 to 16")
        if router not in ("softmax", "sigmoid_groups"):
            raise ValueError(f"unknown router {router!r}; known: softmax, sigmoid_groups")
        if router == "sigmoid_groups" and not (1 <= keep <= groups <= 32 and experts % groups == 0 and keep * (experts // groups) >= top):
            raise ValueError(f"{experts} experts in {groups} groups (at most 32) of which {keep} are kept cannot give {top} choices")
        self.width, self.experts, self.top, self.inner = width, experts, top, inner
        self.limit = float("inf") if limit is None else float(limit)
        self.shared_inner, self.dtype = shared_inner, dtype
        self.shared_limit = float("inf") if shared_limit is None else float(shared_limit)
        self.router, self.groups, self.keep, self.route_scale = router, int(groups), int(keep), float(route_scale)
        self.slope, self.plus, self.shared_gated = float(slope), float(plus), bool(shared_gated) and shared_inner > 0
        self.correction = None
        # many pairs in bfloat16, rows in whole 16-byte pieces: the experts' products run on tcgen05
        self.tensor_cores = dtype == torch.bfloat16 and width % 8 == 0 and inner % 8 == 0

    def tensors(self):
        d, ff, sf = self.width, self.inner, self.shared_inner
        out = {"router_weight": TensorDecl((self.experts, d), "matrix")}
        if self.router == "sigmoid_groups":
            out["correction"] = TensorDecl((self.experts,), "vector")
        if sf:
            out.update({"shared_gate": TensorDecl((sf, d), "matrix"), "shared_up": TensorDecl((sf, d), "matrix"),
                        "shared_down": TensorDecl((d, sf), "matrix")})
        if self.shared_gated:
            out["shared_mix"] = TensorDecl((1, d), "matrix")
        for e in range(self.experts):
            out[f"gate_{e}"] = TensorDecl((ff, d), "matrix")
            out[f"up_{e}"] = TensorDecl((ff, d), "matrix")
            out[f"down_{e}"] = TensorDecl((d, ff), "matrix")
        return out

    def bind(self, tensors):
        E, d, ff, sf = self.experts, self.width, self.inner, self.shared_inner
        first = tensors["gate_0"]
        self.in_weight = torch.empty((E, 2 * ff, d), dtype=first.dtype, device=first.device)
        self.down_weight = torch.empty((E, d, ff), dtype=first.dtype, device=first.device)
        for e in range(E):
            self.in_weight[e, :ff], self.in_weight[e, ff:] = tensors[f"gate_{e}"], tensors[f"up_{e}"]
            self.down_weight[e] = tensors[f"down_{e}"]
        rows = _padded(max(E, 8))
        self.router_weight = torch.zeros((rows, d), dtype=first.dtype, device=first.device)
        self.router_weight[:E] = tensors["router_weight"]
        if "correction" in tensors:
            self.correction = tensors["correction"]
        if sf:
            self.shared_in = torch.zeros((_padded(2 * sf + (1 if self.shared_gated else 0)), d), dtype=first.dtype, device=first.device)
            self.shared_in[:sf], self.shared_in[sf:2 * sf] = tensors["shared_gate"], tensors["shared_up"]
            if self.shared_gated:
                self.shared_in[2 * sf] = tensors["shared_mix"][0]
            self.shared_down = tensors["shared_down"]
        for e in range(E):                         # per-expert views, as the loader's bookkeeping expects attributes
            setattr(self, f"gate_{e}", self.in_weight[e, :ff])
            setattr(self, f"up_{e}", self.in_weight[e, ff:])
            setattr(self, f"down_{e}", self.down_weight[e])
        if sf:
            self.shared_gate, self.shared_up = self.shared_in[:sf], self.shared_in[sf:2 * sf]
        if self.shared_gated:
            self.shared_mix = self.shared_in[2 * sf:2 * sf + 1]

    def forward(self, h, residual, ctx):
        """ff(h) (+ residual), float32 [T, width].  h: rows in the compute dtype."""
        T, d, K = h.shape[0], self.width, self.top
        logits = ops.linear(h, self.router_weight, None, out_dtype=torch.float32)
        scored = None
        if self.router == "sigmoid_groups":
            scored = {"correction": self.correction, "groups": self.groups, "keep": self.keep, "factor": self.route_scale}
        route = ops.moe_route(logits, self.experts, K, scored)
        rows = None
        glu = (self.limit, self.slope, self.plus)
        if self.tensor_cores and T * K >= ops.MOE_TENSOR_PAIRS:
            picked, rows = ops.moe_experts_tc(h, self.in_weight, self.down_weight, route, *glu)
        elif self.tensor_cores and ops.moe_gemv_takes(h, self.in_weight):
            # a handful of pairs (a step of single tokens): every pair streams its expert's matrices on its own
            hidden = ops.moe_gemv(h, self.in_weight, route, glu=glu)
            picked = ops.moe_gemv(hidden, self.down_weight, route, glu=None)                               # [T * K, d]
        else:
            hidden = ops.moe_gemm(h, self.in_weight, route, glu=glu, out_dtype=self.dtype)
            picked = ops.moe_gemm(hidden, self.down_weight, route, glu=None, out_dtype=torch.float32)      # [T * K, d]
        if self.shared_inner:
            sp = ops.linear(h, self.shared_in, None, out_dtype=torch.float32)
            sh = ops.glu_limited(sp, self.shared_inner, self.shared_limit, self.slope, self.dtype, self.plus)
            shared = ops.linear(sh, self.shared_down, None, out_dtype=torch.float32)
        else:
            shared = torch.zeros((T, d), dtype=torch.float32, device=h.device)
        out = ops.moe_combine(picked, route, shared, sp[:, 2 * self.shared_inner] if self.shared_gated else None, rows)
        if residual is not None:
            residual.add_(out)
            return residual
        return out


register_part(MoE.KIND, MoE)
