"""Typed configuration of the Numuzen design: a decoder-only model whose layers are listed one by
one in ``config.json``; a layer is a gated-linear-attention layer or a windowed softmax-attention
layer, each followed by an optional mixture-of-experts feed-forward.

    {"architecture": "Numuzen", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}} | null},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": ...}, ...]}

Every layer is a sandwich block: a norm before AND after each sub-layer, x += norm_b(f(norm_a(x))),
with RMS norms whose weights are stored around zero (applied as 1 + w): ``l<i>.norm1``,
``l<i>.norm1b`` around the mixer ``l<i>.mix.*``; ``l<i>.norm2``, ``l<i>.norm2b`` around the
feed-forward ``l<i>.mlp.*``.  The LM head is the embedding table, behind ``final.norm``.
The rank of a gla layer's decay projection is not in ``config.json``: it is the first dimension of
``l<i>.mix.a1`` (``with_tensor_shapes``), or the mixer's ``decay_rank``.
"""
from __future__ import annotations

import copy
import dataclasses
from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry

MIXER_TYPES = ("gla", "attention")
DEFAULT_MAX_POSITIONS = 1 << 17  # the design has no position limit of its own; the engine wants a bound
EXPERT_SLOPE = 1.702  # the expert's activation is g * sigmoid(1.702 g) * (u + 1)


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


@register_architecture("Numuzen")
@dataclass(frozen=True)
class NumuzenConfig:
    vocab: int
    width: int
    layers: tuple  # of dicts as in config.json: type, mixer, mlp
    norm_eps: float = 1e-6
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    architecture = "Numuzen"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.layers:
            raise ValueError("'layers' is empty")
        for i, layer in enumerate(self.layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            if not isinstance(mixer, dict):
                raise ValueError(f"layer {i}: 'mixer' must be an object")
            needed = ("heads", "dim", "vdim", "tau") if kind == "gla" else ("heads", "kv_heads", "dim", "vdim", "scale")
            missing = [key for key in needed if key not in mixer]
            if missing:
                raise ValueError(f"layer {i} ({kind}): the mixer lacks {', '.join(missing)}")
            for key in ("heads", "dim", "vdim"):
                _positive_int(mixer[key], f"layer {i}: mixer.{key}")
            if kind == "gla":
                if not float(mixer["tau"]) > 0:
                    raise ValueError(f"layer {i}: tau must be positive")
            else:
                _positive_int(mixer["kv_heads"], f"layer {i}: mixer.kv_heads")
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ValueError(f"layer {i}: heads {mixer['heads']} is no multiple of kv_heads {mixer['kv_heads']}")
                if mixer["vdim"] != mixer["dim"]:
                    raise ValueError(f"layer {i}: the values are the keys, so vdim {mixer['vdim']} must equal dim {mixer['dim']}")
                rot = mixer.get("rot")
                if rot is not None:
                    for key in ("base", "dims"):
                        if key not in rot:
                            raise ValueError(f"layer {i}: rot lacks {key!r}")
                    if rot["dims"] % 2 or not 0 < rot["dims"] <= mixer["dim"]:
                        raise ValueError(f"layer {i}: rot.dims {rot['dims']} must be even and at most dim {mixer['dim']}")
                    scaling = rot.get("scaling")
                    if scaling is not None:
                        lacking = [key for key in ("factor", "original", "fast", "slow") if key not in scaling]
                        if lacking:
                            raise ValueError(f"layer {i}: rot.scaling lacks {', '.join(lacking)}")
                mask = mixer.get("mask")
                if mask is not None and mask.get("size") is not None:
                    _positive_int(mask["size"], f"layer {i}: mask.size")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
                expert, router = mlp.get("expert") or {}, mlp.get("router") or {}
                lacking = [f"expert.{key}" for key in ("ff", "limit") if key not in expert]
                lacking += [f"router.{key}" for key in ("experts", "top") if key not in router]
                if lacking:
                    raise ValueError(f"layer {i}: the mlp lacks {', '.join(lacking)}")
                _positive_int(expert["ff"], f"layer {i}: expert.ff")
                _positive_int(router["experts"], f"layer {i}: router.experts")
                _positive_int(router["top"], f"layer {i}: router.top")
                if router["top"] > router["experts"]:
                    raise ValueError(f"layer {i}: router.top {router['top']} exceeds router.experts {router['experts']}")

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, raw: dict) -> "NumuzenConfig":
        missing = [key for key in ("vocab", "width", "layers") if key not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        values = dict(
            vocab=raw["vocab"], width=raw["width"], layers=tuple(copy.deepcopy(list(raw["layers"]))),
            norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)), eos_token_id=raw.get("eos_token_id"))
        if raw.get("max_position_embeddings") is not None:
            values["max_position_embeddings"] = int(raw["max_position_embeddings"])
        return cls(**values)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    def with_tensor_shapes(self, shapes: dict) -> "NumuzenConfig":
        """The sizes that only the checkpoint gives: a gla layer's decay rank is the number of rows
        of its ``a1``.  ``shapes``: tensor name -> shape."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            name = f"l{i}.mix.a1"
            if layer["type"] == "gla" and name in shapes and len(shapes[name]) == 2:
                layer["mixer"]["decay_rank"] = int(shapes[name][0])
        return dataclasses.replace(self, layers=tuple(layers))

    # ------------------------------------------------------------ structure
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("rms_norm", {"size": W, "eps": self.norm_eps, "weight_name": "", "weight_offset": 1.0})
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            mixer = layer["mixer"]
            if layer["type"] == "gla":
                if mixer.get("decay_rank") is None:
                    raise ValueError(f"layer {i}: the decay rank is unknown; it is the first dimension of l{i}.mix.a1 "
                                     "(with_tensor_shapes) or the mixer's 'decay_rank'")
                part = PartSpec("gated_linear_attention", {
                    "hidden_size": W, "num_heads": int(mixer["heads"]), "head_dim": int(mixer["dim"]),
                    "v_dim": int(mixer["vdim"]), "decay_rank": int(mixer["decay_rank"]), "tau": float(mixer["tau"]),
                    "eps": self.norm_eps})
            else:
                rot, mask = mixer.get("rot"), mixer.get("mask") or {}
                positions = None
                if rot is not None:
                    positions = PartSpec("rotary_partial", {
                        "head_dim": int(mixer["dim"]), "dims": int(rot["dims"]), "base": float(rot["base"]),
                        "scaling": copy.deepcopy(rot.get("scaling"))})
                part = PartSpec("gated_attention", {
                    "hidden_size": W, "num_heads": int(mixer["heads"]), "num_kv_heads": int(mixer["kv_heads"]),
                    "head_dim": int(mixer["dim"]), "scale": float(mixer["scale"]),
                    "softcap": float(mixer["softcap"]) if mixer.get("softcap") else None,
                    "window": int(mask["size"]) if mask.get("size") else None,
                    "sink": True, "values_from_keys": True, "qk_norm": "whole", "gate": "sigmoid",
                    "eps": self.norm_eps, "positions": positions})
            mlp = layer.get("mlp")
            feed_forward = None
            if mlp is not None:
                feed_forward = PartSpec("routed_clamped_glu", {
                    "hidden_size": W, "intermediate_size": int(mlp["expert"]["ff"]), "limit": float(mlp["expert"]["limit"]),
                    "alpha": EXPERT_SLOPE, "num_experts": int(mlp["router"]["experts"]), "top_k": int(mlp["router"]["top"]),
                    "score": "sigmoid", "renormalize": False, "weight_on": "input"})
            norms = [NormSlot("mixer_norm", norm, "norm1"), NormSlot("mixer_post_norm", norm, "norm1b")]
            if feed_forward is not None:
                norms += [NormSlot("feed_forward_norm", norm, "norm2"), NormSlot("feed_forward_post_norm", norm, "norm2b")]
            layers.append(LayerSpec(
                prefix=f"l{i}.", block="sandwich", mixer=part, feed_forward=feed_forward, norms=tuple(norms),
                mixer_prefix="mix.", feed_forward_prefix="mlp."))
            schedule.append(ScheduleEntry(layer=i))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            max_position_embeddings=self.max_position_embeddings, embedding_name="embed",
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
            lm_head_name="lm_head", tie_word_embeddings=True)
        spec.validate()
        return spec
