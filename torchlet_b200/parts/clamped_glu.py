"""Clamped gated feed-forward: with g = min(W_gate x, limit) and u = clamp(W_up x, -limit, limit),
y = g * sigmoid(alpha * g) * (u + 1), output W_down y; no biases, activation in float32.

Parameters: ``hidden_size``, ``intermediate_size``, ``limit``, ``alpha`` (default 1.702), and the
tensors' names below the prefix: ``gate_name``, ``up_name``, ``down_name``.
"""
from __future__ import annotations

from .. import ops
from ..config.spec import PartSpec
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .linear import Linear

import torch


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.limit = float(p["limit"])
        self.alpha = float(p.get("alpha", 1.702))
        self.gate_up_proj: Linear | None = None
        self.gate_up_interleaved = None  # bfloat16 fused path: gate/up rows interleaved by 16
        self.down_proj: Linear | None = None

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str):
        p = spec.params
        return (prefix + p.get("gate_name", "gate_proj.weight"), prefix + p.get("up_name", "up_proj.weight"),
                prefix + p.get("down_name", "down_proj.weight"))

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        gate, up, down = cls._names(spec, prefix)
        return [TensorSpec(gate, (inter, hidden)), TensorSpec(up, (inter, hidden)), TensorSpec(down, (hidden, inter))]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        from . import swiglu_bf16

        gate, up, down = self._names(self.spec, prefix)
        if dtype == torch.bfloat16 and swiglu_bf16.usable(self.hidden_size, self.intermediate_size):
            # bfloat16: ONE tcgen05 product over the 16-interleaved gate and up rows, the activation in its epilogue
            self.gate_up_interleaved = swiglu_bf16.interleave(
                tensors[gate].to(device=device, dtype=dtype), tensors[up].to(device=device, dtype=dtype))
        else:
            self.gate_up_proj = Linear(torch.cat([tensors[gate], tensors[up]], dim=0), None, device, dtype)
        self.down_proj = Linear(tensors[down], None, device, dtype)

    def forward(self, ctx, x, acc) -> None:
        tokens = x.shape[0]
        if self.gate_up_interleaved is not None and ops.gemm_tc_supported(x, self.gate_up_interleaved):
            act = ctx.buffer("clamped_glu.act", (tokens, self.intermediate_size), ctx.dtype)
            ops.gemm_tc_glu(x, self.gate_up_interleaved, act, self.limit, self.alpha)
            if not self.down_proj.accumulate_later(ctx, act, acc):
                self.down_proj.forward(act, acc, accumulate=True)
            return
        gate_up = ctx.buffer("clamped_glu.gate_up", (tokens, 2 * self.intermediate_size), ctx.dtype)
        self.gate_up_proj.forward(x, gate_up)
        act = ctx.buffer("clamped_glu.act", (tokens, self.intermediate_size), ctx.dtype)
        ops.clamped_glu(gate_up, act, self.limit, self.alpha)
        if not self.down_proj.accumulate_later(ctx, act, acc):
            self.down_proj.forward(act, acc, accumulate=True)
