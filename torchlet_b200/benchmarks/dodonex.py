"""Prefill and decode throughput of the Dodonex design at layer sizes that resemble a real model's,
beside a Qwen2 model of equal size (same width, layers, feed-forward width, heads and vocabulary).

    python -m torchlet_b200.benchmarks.dodonex [--size 2b|1b] [--layers N] [--prefill 2048] [--batch 8]
                                               [--context 2048] [--steps 32] [--kernels]

Random bfloat16 weights made on the GPU.  Prefill: one request's whole prompt in one step (CUDA
events around the step, best of three).  Decode: ``batch`` requests with ``context`` cached tokens,
replayed from the captured decode step.  ``--kernels`` also times the step with each kernel class
of the new design replaced by nothing: the difference is that class's cost in place.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..config import DodonexConfig, EngineConfig, Qwen2Config
from ..engine import ModelRunner, StepEntry
from ..sampling import SampleSpec
from .common import fill_context


def _latent(heads, dim, rot, vdim, kv_rank, q_rank, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "rot": {"base": 10000.0, "dims": rot}, "scale": (dim + rot) ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def dodonex_config(size: str, layers: int) -> dict:
    """Layers in the pattern latent, delta, latent (reading the first one's cache), delta, ..."""
    if size == "2b":
        width, ff, vocab, side = 2048, 8192, 32768, 256
        latent = dict(heads=16, dim=128, rot=64, vdim=128, kv_rank=512, q_rank=1536)
        delta = {"heads": 32, "dim": 64, "decay_rank": 64}
    else:
        width, ff, vocab, side = 1024, 4096, 32768, 128
        latent = dict(heads=8, dim=64, rot=32, vdim=64, kv_rank=256, q_rank=512)
        delta = {"heads": 16, "dim": 64, "decay_rank": 32}
    out = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
        if i % 2:
            out.append({"type": "general_delta", "mixer": dict(delta), "mlp": mlp})
        else:
            out.append({"type": "latent_attention", "mixer": _latent(**latent, kv_from=0 if i % 4 == 2 else None),
                        "mlp": mlp})
    return {"architecture": "Dodonex", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6, "groups": 4}, "residual_mult": 0.5, "logit_scale": 1.0, "token_side": {"dim": side},
            "layers": out}


def qwen2_config(size: str, layers: int) -> dict:
    width, ff, heads = (2048, 8192, 16) if size == "2b" else (1024, 4096, 8)
    return {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 32768, "hidden_size": width, "intermediate_size": ff,
            "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": heads // 4,
            "head_dim": width // heads, "max_position_embeddings": 32768, "rope_theta": 1000000.0,
            "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": True}


def build(config, seed: int):
    from ..engine.loading import build_model
    from ..weights import random_tensors

    tensors = random_tensors(config, seed, std=0.02, norm_std=0.0, dtype="bfloat16", device="cuda:0")
    model = build_model(config, tensors, "bfloat16")
    del tensors
    torch.cuda.empty_cache()
    return model


def time_prefill(model, tokens: int, repeats: int = 3) -> float:
    """Milliseconds of one whole prompt of ``tokens`` tokens (best of ``repeats`` after a warm-up)."""
    page = 16
    config = EngineConfig(dtype="bfloat16", max_decode_slots=1, kv_block_size=page, max_seq_len=tokens,
                          max_num_blocks=-(-tokens // page) + 2, max_num_batched_tokens=tokens, cuda_graph=False)
    runner = ModelRunner(model, config)
    ids = torch.randint(0, model.spec.vocab_size, (tokens,)).tolist()
    best = float("inf")
    for k in range(repeats + 1):
        runner.admit("p")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step([StepEntry("p", ids, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.finish("p")
        if k:
            best = min(best, begin.elapsed_time(end))
    del runner
    torch.cuda.empty_cache()
    return best


def time_decode(model, batch: int, context: int, steps: int, warmup: int = 4) -> float:
    """Microseconds of one decode step of ``batch`` requests near ``context`` cached tokens."""
    page = 16
    config = EngineConfig(dtype="bfloat16", max_decode_slots=batch, kv_block_size=page, max_seq_len=context,
                          max_num_blocks=batch * (-(-context // page)) + 1, max_num_batched_tokens=2048)
    runner = ModelRunner(model, config)
    ids = [f"d{i}" for i in range(batch)]
    fill_context(runner, ids, context - steps - warmup, seed=17)
    tokens = torch.randint(0, model.spec.vocab_size, (steps + warmup, batch)).tolist()

    def step(k):
        runner.run([StepEntry(rid, [tokens[k][i]], sample=SampleSpec(0.0, i, k)) for i, rid in enumerate(ids)])

    for k in range(warmup):
        step(k)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for k in range(warmup, warmup + steps):
        step(k)
    end.record()
    torch.cuda.synchronize()
    assert runner.graph_steps >= steps
    for rid in ids:
        runner.finish(rid)
    del runner
    torch.cuda.empty_cache()
    return begin.elapsed_time(end) / steps * 1e3


KERNEL_CLASSES = {
    "latent attention": ("latent_attention_mma", "latent_attention"),
    "latent prepare/absorb/expand": ("latent_prepare", "latent_absorb_q", "latent_expand_o"),
    "delta rule": ("delta_prepare", "delta_scan", "delta_finish"),
    "clamped glu": ("clamped_glu",),
    "token input (elementwise)": ("gated_token_embed", "rms_scaled_add"),
    "residual (zero, scaled add)": ("fill_zero", "scaled_add"),
}


def run(size: str = "2b", layers: int = 8, prefill: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32,
        kernels: bool = False) -> dict:
    record = {"workload": "dodonex", "size": size, "layers": layers, "prefill_tokens": prefill, "batch": batch,
              "context": context}
    for name, config in (("dodonex", DodonexConfig.from_dict(dodonex_config(size, layers))),
                         ("qwen2_equal_size", Qwen2Config.from_dict(qwen2_config(size, layers)))):
        model = build(config, seed=9)
        ms = time_prefill(model, prefill)
        us = time_decode(model, batch, context, steps)
        record[name] = {"prefill_ms": round(ms, 3), "prefill_tok_s": round(prefill / ms * 1e3, 1),
                        "decode_us": round(us, 1), "decode_tok_s": round(batch / us * 1e6, 1)}
        if kernels and name == "dodonex":
            costs = {}
            for label, names in KERNEL_CLASSES.items():
                saved = {n: getattr(ops, n) for n in names}
                for n in names:
                    setattr(ops, n, lambda *a, **k: None)
                try:
                    costs[label] = {"prefill_ms": round(ms - time_prefill(model, prefill), 3),
                                    "decode_us": round(us - time_decode(model, batch, context, steps), 1)}
                finally:
                    for n, fn in saved.items():
                        setattr(ops, n, fn)
            record["dodonex"]["in_place_costs"] = costs
        del model
        torch.cuda.empty_cache()
    record["value"] = record["dodonex"]["decode_tok_s"]
    record["unit"] = "tok/s"
    record["metric"] = f"decode tokens per second, batch {batch}, context {context}"
    return record


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--size", choices=["2b", "1b"], default="2b")
    parser.add_argument("--layers", type=int, default=8)
    parser.add_argument("--prefill", type=int, default=2048)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--kernels", action="store_true")
    args = parser.parse_args(argv)
    print(json.dumps(run(args.size, args.layers, args.prefill, args.batch, args.context, args.steps, args.kernels)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
