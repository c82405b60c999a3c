"""Small Numuzen configurations of the tests, their random weights, and an engine around them.  No
two agree in any size: head sizes that are no multiple of 32, key and value sizes that differ, one
head and several, one KV head and as many as query heads, a window of one token, of less than a page
and of several pages, a rotation over all entries and over a few, with and without frequency scaling,
with and without a score cap, one expert of one, all experts of three, two of five, a layer without a
feed-forward, either mixer first."""
from __future__ import annotations

import functools

import torch

import plain_numuzen

# Largest allowed |engine - plain| of a position's logits as a fraction of that position's largest |logit|.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def attn(heads, kv_heads, dim, scale, window=None, softcap=None, rot_dims=None, base=10000.0, scaling=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window:
        mixer["mask"] = {"size": window}
    if softcap:
        mixer["softcap"] = softcap
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    return mixer


def layer(kind, mixer, experts=None, top=None, ff=None, limit=1.5):
    mlp = None if experts is None else {"kind": "moe", "expert": {"ff": ff, "limit": limit},
                                        "router": {"experts": experts, "top": top}}
    return {"type": kind, "mixer": mixer, "mlp": mlp}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}

CASES = {
    # attention first; a window shorter than a page; rotation over a few entries with frequency scaling
    "P": {"architecture": "Numuzen", "vocab": 101, "width": 96, "norm": {"eps": 1e-5},
          "layers": [
              layer("attention", attn(4, 2, 24, 0.3, window=13, softcap=5.0, rot_dims=8, base=500.0, scaling=YARN),
                    experts=5, top=2, ff=40, limit=1.0),
              layer("gla", gla(3, 12, 20, 4.0, 6), experts=5, top=2, ff=40, limit=1.0),
              layer("attention", attn(4, 2, 24, 0.3, window=37, softcap=5.0, rot_dims=8, base=500.0, scaling=YARN)),
              layer("gla", gla(2, 24, 8, 9.0, 5), experts=2, top=1, ff=56, limit=3.0),
          ]},
    # one head, one expert of one, all experts of three, a window of ONE token, no cap, full rotation, no scaling,
    # a head size that is no multiple of 8, no window
    "Q": {"architecture": "Numuzen", "vocab": 67, "width": 64, "norm": {"eps": 1e-6},
          "layers": [
              layer("gla", gla(1, 40, 8, 1.0, 3), experts=1, top=1, ff=24, limit=0.7),
              layer("attention", attn(2, 2, 16, 0.25, window=1, rot_dims=16, base=100.0), experts=3, top=3, ff=24),
              layer("attention", attn(3, 1, 20, 0.2, rot_dims=6, base=100.0), experts=3, top=3, ff=24),
              layer("gla", gla(5, 8, 16, 32.0, 7)),
          ]},
    # sizes the tensor-core kernels take: heads of 64 and 128, windows of several pages
    "R": {"architecture": "Numuzen", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
          "layers": [
              layer("gla", gla(2, 64, 64, 12.0, 16), experts=4, top=2, ff=64, limit=1.5),
              layer("attention", attn(4, 1, 64, 0.125, window=150, softcap=20.0, rot_dims=32, base=50000.0, scaling=YARN),
                    experts=4, top=2, ff=64, limit=1.5),
              layer("attention", attn(6, 2, 128, 0.09, window=70, softcap=25.0, rot_dims=64, base=50000.0),
                    experts=4, top=1, ff=128, limit=2.5),
              layer("gla", gla(1, 128, 32, 8.0, 8), experts=4, top=2, ff=64, limit=1.5),
          ]},
}


def _all_experts(case: dict) -> dict:
    import copy

    case = copy.deepcopy(case)
    for entry in case["layers"]:
        if entry["mlp"] is not None:
            entry["mlp"]["router"]["top"] = entry["mlp"]["router"]["experts"]
    return case


# "Pa", "Qa", "Ra": the same models with EVERY expert chosen.  Random routers have close calls: where two
# experts' scores lie within bfloat16 rounding of one another the bfloat16 engine may choose the other one,
# and that position, and through states and keys all behind it, then differs by a whole expert's output.
# So the bfloat16 engine is compared on these (same tensors, no discrete choice), the float32 engine on
# the true routing at every position, and the choice itself is tested on given inputs in
# test_numuzen_parts_gpu.py.
CASES.update({name + "a": _all_experts(case) for name, case in list(CASES.items())})


def variant(name: str, dtype: str) -> str:
    return name if dtype == "float32" else name + "a"


def config_for(name: str):
    from torchlet_b200.config import NumuzenConfig

    return NumuzenConfig.from_dict(CASES[name])


@functools.lru_cache(maxsize=None)
def weights_for(name: str, seed: int = 0):
    """bfloat16-rounded random weights as float32 tensors by name (so that both engines and the
    plain implementation hold the same numbers).  Routers are drawn wider, so that the experts'
    scores lie apart, and the decay's bias is raised, so that states last some hundred tokens."""
    from torchlet_b200.weights import random_tensors

    tensors = random_tensors(config_for(name), seed=300 + seed, std=0.1, norm_std=0.1, dtype="bfloat16")
    out = {}
    for k, v in tensors.items():
        v = v.float()
        if k.endswith(".router"):
            v = (v * 4).to(torch.bfloat16).float()
        if k.endswith("a2.b"):
            v = (v + 2.0).to(torch.bfloat16).float()
        out[k] = v
    return out


def make_ids(name: str, length: int, seed: int):
    g = torch.Generator().manual_seed(2000 + seed)
    return torch.randint(0, CASES[name]["vocab"], (length,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int):
    ids = make_ids(name, length, seed)
    return ids, plain_numuzen.forward(CASES[name], weights_for(name), ids).float()


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
    if dtype == "bfloat16":
        # A norm stands behind every sub-layer, so a sub-layer's output counts by its direction alone.  At the
        # first positions the recurrent state has rank one or two and a head's output is its first value vector
        # times the scalar k . q: where that scalar is within bfloat16 rounding of zero, its sign, and with it the
        # whole normed output, is a coin's toss.  Random weights have such positions; the float32 engine is held
        # to its tolerance at EVERY position of the same tests, the bfloat16 engine at nine in ten, and
        # nowhere may it be off by more than half of the largest logit.
        over = int((ratio > TOLERANCE[dtype]).sum())
        assert over <= max(1, ratio.numel() // 10) and ratio[worst] <= 0.5, (
            f"{what}: {over} of {ratio.numel()} rows over {TOLERANCE[dtype]:.1e}; worst row {worst}: {ratio[worst]:.3e}")
        return
    assert ratio[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst}: max |diff| {err[worst]:.3e} > {TOLERANCE[dtype]:.1e} * {scale[worst]:.3f}")
