"""Gated linear attention: a recurrent mixer with one D x V float32 state matrix per head and request
(key channel x value channel), kept in the request's slot between steps.

With q = W_q x * D^(-1/2), k = W_k x (heads x D), v = W_v x (heads x V) and a decay per key channel
a = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau), per head:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

Each head's o is divided by its root mean square and multiplied by a weight over V that all heads
share; the heads, concatenated, are multiplied by silu(W_g x) and go through W_o into the stream.
The five input products run as ONE product with float32 output; decay, state and recurrence are
float32 in both engines (csrc/gla.cu).

Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_dim``, ``decay_rank``, ``tau``, ``eps``.
Tensors below the prefix: q, k [H D, hidden]; v, g [H V, hidden]; a1 [rank, hidden]; a2 [H D, rank];
a2.b [H D]; norm [V]; o [hidden, H V].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, Mixer, StateSpec, TensorSpec
from .linear import Linear


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe = True  # nothing is planned on the host: requests and slots are read on the device

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p["v_dim"])
        self.rank = int(p["decay_rank"])
        self.tau = float(p["tau"])
        self.eps = float(p["eps"])
        if self.head_dim > 256 or self.v_dim > 256:
            raise ValueError(f"head sizes {self.head_dim} x {self.v_dim} are not supported by the scan kernel (up to 256)")
        self.k_size = self.num_heads * self.head_dim
        self.v_size = self.num_heads * self.v_dim
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.a2 = self.a2_bias = self.norm_weight = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.v_dim), "float32")

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, rank = int(p["hidden_size"]), int(p["decay_rank"])
        k_size, v_size = int(p["num_heads"]) * int(p["head_dim"]), int(p["num_heads"]) * int(p["v_dim"])
        return [TensorSpec(prefix + "q", (k_size, hidden)), TensorSpec(prefix + "k", (k_size, hidden)),
                TensorSpec(prefix + "v", (v_size, hidden)), TensorSpec(prefix + "g", (v_size, hidden)),
                TensorSpec(prefix + "o", (hidden, v_size)), TensorSpec(prefix + "norm", (int(p["v_dim"]),), init="ones"),
                TensorSpec(prefix + "a1", (rank, hidden)), TensorSpec(prefix + "a2", (k_size, rank)),
                TensorSpec(prefix + "a2.b", (k_size,))]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        fused = torch.cat([tensors[prefix + name] for name in ("q", "k", "v", "g", "a1")], dim=0)
        self.in_proj = Linear(fused, None, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], None, device, dtype)
        f32 = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32).contiguous()
        self.a2_bias, self.norm_weight = f32("a2.b"), f32("norm")
        self.a2 = f32("a2").t().contiguous()  # [rank, H D]: the threads of a block read consecutive entries

    def forward(self, ctx, x, acc, cache) -> None:
        tokens, H, D, V = x.shape[0], self.num_heads, self.head_dim, self.v_dim
        proj = ctx.buffer("gla.proj", (tokens, 2 * self.k_size + 2 * self.v_size + self.rank), torch.float32)
        self.in_proj.forward(x, proj)
        decay = ctx.buffer("gla.decay", (tokens, self.k_size), torch.float32)
        ops.gla_decay(proj, 2 * self.k_size + 2 * self.v_size, self.a2, self.a2_bias, decay, self.rank, self.tau)
        o = ctx.buffer("gla.o", (tokens, self.v_size), torch.float32)
        ops.gla_scan(proj, decay, ctx.req_indptr, ctx.slots, cache.state, o, ctx.num_requests, H, D, V, D ** -0.5)
        out = ctx.buffer("gla.out", (tokens, self.v_size), ctx.dtype)
        ops.gla_finish(o, proj, 2 * self.k_size + self.v_size, self.norm_weight, out, H, V, self.eps)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
