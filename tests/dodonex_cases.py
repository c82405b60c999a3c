"""Small Dodonex configurations of the tests, their random weights, and an engine around them.
No two agree in any size, and none has a size that is a convenient multiple: head sizes that are
no multiple of 32, a rotation over fewer entries than the rotated part has, one group and
several, a multiplier of 1 and another, a layer without a feed-forward, a model without the
per-layer token input, one head, a cache read by two later layers."""
from __future__ import annotations

import functools

import torch

import plain_dodonex

# Largest allowed |engine - plain| of a position's logits as a fraction of that position's largest |logit|.
# float32: summation order only (the recurrence is deep).  bfloat16: activations are rounded to 8 bits of
# mantissa between kernels; the faults these tests look for (a lost state, a wrong key, a wrong position) cost
# tens of percent and are caught at the float32 tolerance besides.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, dims=None, kv_from=None, scale=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "rot": {"base": base, "dims": rot_dim if dims is None else dims},
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def layer(kind, mixer, ff=None, limit=2.0):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


CASES = {
    # delta first, a shared cache read by two layers, rotation over part of the rotated entries
    "P": {"architecture": "Dodonex", "vocab": 97, "width": 96, "embedding": {"scale": 5.0},
          "norm": {"eps": 1e-5, "groups": 3}, "residual_mult": 0.6, "logit_scale": 1.5, "token_side": {"dim": 8},
          "layers": [
              layer("general_delta", {"heads": 2, "dim": 24, "decay_rank": 6}, ff=72, limit=0.8),
              layer("latent_attention", latent(3, 16, 8, 24, 40, 24, base=5000.0, dims=4), ff=40, limit=1.0),
              layer("latent_attention", latent(3, 16, 8, 24, 40, 24, base=5000.0, dims=4, kv_from=1)),
              layer("general_delta", {"heads": 3, "dim": 40, "decay_rank": 10}, ff=72, limit=0.8),
              layer("latent_attention", latent(2, 8, 8, 8, 40, 16, base=5000.0, dims=4, kv_from=1), ff=24),
          ]},
    # no token input, one group, multiplier 1, one head, sizes that are no multiples of 8
    "Q": {"architecture": "Dodonex", "vocab": 61, "width": 64, "embedding": {"scale": 1.0},
          "norm": {"eps": 1e-6, "groups": 1}, "residual_mult": 1.0, "logit_scale": 1.0,
          "layers": [
              layer("latent_attention", latent(1, 12, 6, 10, 22, 12, base=300.0), ff=36, limit=3.0),
              layer("general_delta", {"heads": 1, "dim": 20, "decay_rank": 3}),
              layer("latent_attention", latent(5, 12, 2, 4, 18, 20, base=300.0, scale=0.4), ff=36, limit=3.0),
          ]},
    # nothing is a multiple of 4: every kernel's plain form (odd rows in the cache, an odd width)
    "S": {"architecture": "Dodonex", "vocab": 33, "width": 50, "embedding": {"scale": 2.0},
          "norm": {"eps": 1e-5, "groups": 5}, "residual_mult": 0.9, "logit_scale": 3.0, "token_side": {"dim": 3},
          "layers": [
              layer("general_delta", {"heads": 2, "dim": 10, "decay_rank": 3}, ff=21, limit=1.0),
              layer("latent_attention", latent(2, 5, 6, 3, 13, 7, base=50.0), ff=21, limit=1.0),
          ]},
    # sizes the tensor-core kernels take: multiples of 16 throughout, 64-wide delta heads
    "R": {"architecture": "Dodonex", "vocab": 211, "width": 128, "embedding": {"scale": 3.0},
          "norm": {"eps": 1e-5, "groups": 2}, "residual_mult": 0.8, "logit_scale": 0.5, "token_side": {"dim": 16},
          "layers": [
              layer("latent_attention", latent(4, 32, 16, 32, 64, 48), ff=192, limit=1.2),
              layer("general_delta", {"heads": 2, "dim": 64, "decay_rank": 16}, ff=192, limit=1.2),
              layer("latent_attention", latent(4, 32, 16, 32, 64, 48, kv_from=0), ff=192, limit=1.2),
          ]},
}


def config_for(name: str):
    from torchlet_b200.config import DodonexConfig

    return DodonexConfig.from_dict(CASES[name])


@functools.lru_cache(maxsize=None)
def weights_for(name: str, seed: int = 0):
    """bfloat16-rounded random weights as float32 tensors by name (so that both engines and the
    plain implementation hold the same numbers)."""
    from torchlet_b200.weights import random_tensors

    tensors = random_tensors(config_for(name), seed=100 + seed, std=0.1, norm_std=0.1, dtype="bfloat16")
    return {k: v.float() for k, v in tensors.items()}


def make_ids(name: str, length: int, seed: int):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CASES[name]["vocab"], (length,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int):
    ids = make_ids(name, length, seed)
    return ids, plain_dodonex.forward(CASES[name], weights_for(name), ids).float()


def make_model(name: str, dtype: str, weights=None):
    from torchlet_b200.engine.loading import build_model

    w = weights if weights is not None else weights_for(name)
    return build_model(config_for(name), {k: v.to(torch.bfloat16) for k, v in w.items()}, dtype)


def make_runner(name: str, dtype: str, num_pages: int = 64, slots: int = 4, page_size: int = 16, budget: int = 512,
                max_seq_len: int = 512, cuda_graph: bool = False, weights=None):
    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine import ModelRunner

    engine = EngineConfig(dtype=dtype, max_decode_slots=slots, kv_block_size=page_size, max_num_blocks=num_pages,
                          max_seq_len=max_seq_len, max_num_batched_tokens=budget, cuda_graph=cuda_graph)
    return ModelRunner(make_model(name, dtype, weights), engine)


def replay(runner, rid, ids, cuts, finish=True):
    """Feed ``ids`` of one request in portions of the given sizes, asking for every position's
    logits; returns [len(ids), vocab] on the CPU."""
    from torchlet_b200.engine import StepEntry

    assert sum(cuts) == len(ids)
    runner.admit(rid)
    out, start = [], 0
    for size in cuts:
        logits = runner.step([StepEntry(rid, ids[start:start + size], list(range(size)))])
        out.append(logits.cpu().clone())
        start += size
    if finish:
        runner.finish(rid)
        runner.cache.check()
    return torch.cat(out)


def assert_close(got, want, dtype: str, what: str = ""):
    assert got.shape == want.shape, f"{what}: shapes {tuple(got.shape)} and {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    got, want = got.reshape(-1, got.shape[-1]).double(), want.reshape(-1, want.shape[-1]).double()
    err = (got - want).abs().amax(dim=1)
    scale = want.abs().amax(dim=1)
    ratio = err / scale
    worst = int(ratio.argmax())
    assert ratio[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst}: max |diff| {err[worst]:.3e} > {TOLERANCE[dtype]:.1e} * {scale[worst]:.3f}")
