"""Per-layer token input: every layer adds something looked up by the token id itself.

"gated_token_embedding": with e = table[token] (``dim`` wide: this layer's columns
``[offset, offset + dim)`` of a table all layers share), g = gelu_tanh(W_gate x) * e and
y = W_proj g, the stream gets  x += m * y / sqrt(mean(y^2) + eps) * w_norm.  W_gate reads the
stream itself (not a normed copy); the norm and the sum are float32.

Parameters: ``hidden_size``, ``dim``, ``eps``, ``vocab_size``, ``table_name`` (full tensor name
of the shared table), ``table_width``, ``offset``.  Tensors below the prefix: ``gate`` [dim,
hidden], ``proj`` [hidden, dim], ``norm`` [hidden].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import TOKEN_INPUTS, TensorSpec, TokenInput
from .linear import Linear


@TOKEN_INPUTS.register("gated_token_embedding")
class GatedTokenEmbedding(TokenInput):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size, self.dim = int(p["hidden_size"]), int(p["dim"])
        self.eps = float(p["eps"])
        self.offset = int(p.get("offset", 0))
        self.table = None
        self.gate: Linear | None = None
        self.proj: Linear | None = None
        self.norm_weight = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, dim = int(p["hidden_size"]), int(p["dim"])
        return [
            TensorSpec(p["table_name"], (int(p["vocab_size"]), int(p.get("table_width", dim)))),
            TensorSpec(prefix + "gate", (dim, hidden)),
            TensorSpec(prefix + "proj", (hidden, dim)),
            TensorSpec(prefix + "norm", (hidden,), init="ones"),
        ]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        table = tensors[self.spec.params["table_name"]]
        # this layer's columns only, as a table of its own: a row is then one contiguous read
        self.table = table[:, self.offset:self.offset + self.dim].to(device=device, dtype=dtype).contiguous()
        self.gate = Linear(tensors[prefix + "gate"], None, device, dtype)
        self.proj = Linear(tensors[prefix + "proj"], None, device, dtype)
        self.norm_weight = tensors[prefix + "norm"].to(device=device, dtype=torch.float32).contiguous()

    def wants_cast(self, ctx, acc):
        """A buffer for the stream in the compute type (the gate product's input), which the
        caller's residual kernel fills in passing; None when the stream itself is the input."""
        if ctx.dtype == torch.float32:
            return None
        return ctx.buffer("token_input.x", tuple(acc.shape), ctx.dtype)

    def forward(self, ctx, acc, m: float = 1.0, cast=None) -> None:
        tokens = acc.shape[0]
        if ctx.dtype == torch.float32:
            x = acc
        elif cast is not None:
            x = cast
        else:
            x = ctx.buffer("token_input.x", tuple(acc.shape), ctx.dtype)
            x.copy_(acc)
        gate = ctx.buffer("token_input.gate", (tokens, self.dim), torch.float32)
        self.gate.forward(x, gate)
        g = ctx.buffer("token_input.g", (tokens, self.dim), ctx.dtype)
        ops.gated_token_embed(gate, self.table, ctx.tokens, g)
        y = ctx.buffer("token_input.y", (tokens, self.hidden_size), torch.float32)
        self.proj.forward(g, y)
        ops.rms_scaled_add(acc, y, self.norm_weight, m, self.eps)
