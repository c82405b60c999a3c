"""Prefill and decode throughput of the Numuzen design at layer sizes that resemble a real model's,
beside the two existing models of equal size: Dodonex (the other design with a recurrent mixer and a
clamped gated feed-forward) and Qwen2 (same width, layers, heads and vocabulary; its dense feed-forward
is as wide as the experts a token of Numuzen goes through).

    python -m torchlet_b200.benchmarks.numuzen [--size 2b|1b] [--layers N] [--prefill 2048] [--batch 8]
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
from ..config import DodonexConfig, NumuzenConfig, Qwen2Config
from .dodonex import build, dodonex_config, qwen2_config, time_decode, time_prefill


def numuzen_config(size: str, layers: int, experts: int = 8, top: int = 2, window: int = 1024) -> dict:
    """Layers in the pattern gla, attention, gla, attention, ...; every layer with ``experts`` experts of
    which a token uses ``top``, each 1 / top of the dense models' feed-forward width."""
    if size == "2b":
        width, ff, vocab = 2048, 8192, 32768
        gla = {"heads": 16, "dim": 64, "vdim": 128, "tau": 12.0, "decay_rank": 32}
        attention = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128}
    else:
        width, ff, vocab = 1024, 4096, 32768
        gla = {"heads": 8, "dim": 64, "vdim": 128, "tau": 12.0, "decay_rank": 16}
        attention = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 64}
    attention.update(scale=attention["dim"] ** -0.5, softcap=50.0, mask={"size": window},
                     rot={"base": 1000000.0, "dims": attention["dim"] // 2,
                          "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}})
    mlp = {"kind": "moe", "expert": {"ff": ff // top, "limit": 7.0}, "router": {"experts": experts, "top": top}}
    out = [{"type": "attention" if i % 2 else "gla", "mixer": dict(attention if i % 2 else gla), "mlp": mlp}
           for i in range(layers)]
    return {"architecture": "Numuzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


KERNEL_CLASSES = {
    "gla (decay, scan, finish)": ("gla_decay", "gla_scan", "gla_finish"),
    "attention (norm, rotation, cache write)": ("normed_qk_store",),
    "attention (scores and values)": ("attention_mma", "attention_generic"),
    "routing (route, plan, scatter, combine)": ("moe_route", "moe_plan", "moe_scatter", "moe_combine"),
    "expert products": ("gemm_tc_grouped", "moe_gemm_simt"),
    "side stream (zero, norm behind the sub-layer)": ("fill_zero", "rms_scaled_add"),
}


def run(size: str = "2b", layers: int = 8, prefill: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32,
        kernels: bool = False, experts: int = 8, top: int = 2, window: int = 1024) -> dict:
    record = {"workload": "numuzen", "size": size, "layers": layers, "prefill_tokens": prefill, "batch": batch,
              "context": context, "experts": experts, "top": top, "window": window}
    models = (("numuzen", NumuzenConfig.from_dict(numuzen_config(size, layers, experts, top, window))),
              ("dodonex_equal_size", DodonexConfig.from_dict(dodonex_config(size, layers))),
              ("qwen2_equal_size", Qwen2Config.from_dict(qwen2_config(size, layers))))
    for name, config in models:
        model = build(config, seed=9)
        ms = time_prefill(model, prefill)
        us = time_decode(model, batch, context, steps)
        record[name] = {"prefill_ms": round(ms, 3), "prefill_tok_s": round(prefill / ms * 1e3, 1),
                        "decode_us": round(us, 1), "decode_tok_s": round(batch / us * 1e6, 1)}
        if kernels and name == "numuzen":
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
            record["numuzen"]["in_place_costs"] = costs
        del model
        torch.cuda.empty_cache()
    record["value"] = record["numuzen"]["decode_tok_s"]
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
    parser.add_argument("--experts", type=int, default=8)
    parser.add_argument("--top", type=int, default=2)
    parser.add_argument("--window", type=int, default=1024)
    parser.add_argument("--kernels", action="store_true")
    args = parser.parse_args(argv)
    print(json.dumps(run(args.size, args.layers, args.prefill, args.batch, args.context, args.steps, args.kernels,
                         args.experts, args.top, args.window)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
