"""Generalized delta rule: a recurrent mixer with one D x D float32 state matrix per head and
request (key channel x value channel), kept in the request's slot between steps.

With r, k, v = W_r x, W_k x, W_v x (heads x D each), the unit key u = k / sqrt(sum(k^2) + 1e-6),
the decay w = exp(-exp(-1/2) sigmoid(W_w2 tanh(W_w1 x) + w0)) and the removal rate
a = sigmoid(W_a x + b_a), per head and key channel:

    S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T        o_t = S_t^T r_t

Each head's o is divided by its root mean square, multiplied by a weight over all heads and by
sigmoid(W_g x), and goes through W_o into the stream.  The six input products run as ONE product
with float32 output; gates, state and recurrence are float32 in both engines (csrc/delta_rule.cu).

Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``decay_rank``, ``eps``.  Tensors below
the prefix: r, k, v, g, a [H D, hidden]; a.b, w0, norm [H D]; w1 [rank, hidden]; w2 [H D, rank];
o [hidden, H D].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, Mixer, StateSpec, TensorSpec
from .linear import Linear


@MIXERS.register("general_delta")
class GeneralDeltaMixer(Mixer):
    graph_safe = True  # nothing is planned on the host: requests and slots are read on the device

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.head_dim = int(p["head_dim"])
        self.rank = int(p["decay_rank"])
        self.eps = float(p["eps"])
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not supported by the delta-rule kernels (up to 256)")
        self.size = self.num_heads * self.head_dim
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.w2 = self.w0 = self.a_bias = self.norm_weight = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.head_dim), "float32")

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, size, rank = int(p["hidden_size"]), int(p["num_heads"]) * int(p["head_dim"]), int(p["decay_rank"])
        out = [TensorSpec(prefix + name, (size, hidden)) for name in ("r", "k", "v", "g", "a")]
        out += [TensorSpec(prefix + "a.b", (size,)), TensorSpec(prefix + "w1", (rank, hidden)),
                TensorSpec(prefix + "w2", (size, rank)), TensorSpec(prefix + "w0", (size,)),
                TensorSpec(prefix + "norm", (size,), init="ones"), TensorSpec(prefix + "o", (hidden, size))]
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        fused = torch.cat([tensors[prefix + name] for name in ("r", "k", "v", "g", "a", "w1")], dim=0)
        self.in_proj = Linear(fused, None, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], None, device, dtype)
        f32 = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32).contiguous()
        self.w0, self.a_bias, self.norm_weight = f32("w0"), f32("a.b"), f32("norm")
        self.w2 = f32("w2").t().contiguous()  # [rank, H D]: the threads of a block read consecutive entries

    def forward(self, ctx, x, acc, cache) -> None:
        tokens, H, D = x.shape[0], self.num_heads, self.head_dim
        proj = ctx.buffer("delta.proj", (tokens, 5 * self.size + self.rank), torch.float32)
        self.in_proj.forward(x, proj)
        gates = ctx.buffer("delta.gates", (tokens, H * 3 * D), torch.float32)
        ops.delta_prepare(proj, self.w2, self.w0, self.a_bias, gates, H, D, self.rank)
        o = ctx.buffer("delta.o", (tokens, self.size), torch.float32)
        ops.delta_scan(proj, gates, ctx.req_indptr, ctx.slots, cache.state, o, ctx.num_requests, H, D)
        out = ctx.buffer("delta.out", (tokens, self.size), ctx.dtype)
        ops.delta_finish(o, proj, self.norm_weight, out, H, D, self.eps)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
