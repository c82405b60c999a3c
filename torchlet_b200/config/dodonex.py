"""Typed configuration of the Dodonex design: a decoder-only model whose layers are listed one
by one in ``config.json``, each with one of two mixers and an optional feed-forward.

    {"architecture": "Dodonex", "vocab": V, "width": W, "embedding": {"scale": s},
     "norm": {"eps": e, "groups": G}, "residual_mult": m, "logit_scale": c,
     "token_side": {"dim": d} or absent,
     "layers": [{"type": "latent_attention" | "general_delta", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F, "limit": L} | null}, ...]}

Every layer is a parallel block (one grouped RMS norm ``l<i>.norm1``; mixer ``l<i>.mix.*`` and
feed-forward ``l<i>.mlp.*`` side by side; residual multiplier m) followed, when ``token_side`` is
given, by a gated per-layer token embedding (``l<i>.side.*``, columns ``[i d, (i + 1) d)`` of the
shared table ``side.embed``).  The LM head is the embedding table itself (unscaled), the logits
are multiplied by ``logit_scale``.  A latent-attention layer with ``kv_from: j`` reads layer j's
cache rows.  The rank of a delta-rule layer's decay projection is not in ``config.json``: it is
the first dimension of ``l<i>.mix.w1`` (``with_tensor_shapes``), or the mixer's ``decay_rank``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry

MIXER_TYPES = ("latent_attention", "general_delta")
DEFAULT_MAX_POSITIONS = 1 << 17  # the design has no position limit of its own; the engine wants a bound


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


@register_architecture("Dodonex")
@dataclass(frozen=True)
class DodonexConfig:
    vocab: int
    width: int
    layers: tuple  # of dicts as in config.json: type, mixer, mlp
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
    norm_groups: int = 1
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    token_side_dim: Optional[int] = None
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    architecture = "Dodonex"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.norm_groups, "norm.groups")
        if self.width % self.norm_groups:
            raise ValueError(f"width {self.width} is not divisible by norm.groups {self.norm_groups}")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.token_side_dim is not None:
            _positive_int(self.token_side_dim, "token_side.dim")
        if not self.layers:
            raise ValueError("'layers' is empty")
        for i, layer in enumerate(self.layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            if not isinstance(mixer, dict):
                raise ValueError(f"layer {i}: 'mixer' must be an object")
            needed = ("dim", "heads") if kind == "general_delta" else \
                ("dim", "heads", "kv_rank", "q_rank", "rot_dim", "vdim", "scale", "rot")
            missing = [key for key in needed if key not in mixer]
            if missing:
                raise ValueError(f"layer {i} ({kind}): the mixer lacks {', '.join(missing)}")
            if kind == "latent_attention":
                source = mixer.get("kv_from")
                if source is not None:
                    if not isinstance(source, int) or not 0 <= source < i:
                        raise ValueError(f"layer {i}: kv_from must name an earlier layer, got {source!r}")
                    theirs = self.layers[source]
                    if theirs.get("type") != "latent_attention" or theirs["mixer"].get("kv_from") is not None:
                        raise ValueError(f"layer {i}: kv_from {source} is not a latent-attention layer with a cache of its own")
                    for key in ("kv_rank", "rot_dim", "rot"):
                        if theirs["mixer"].get(key) != mixer.get(key):
                            raise ValueError(f"layer {i}: {key} differs from layer {source}, whose cache it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
                for key in ("ff", "limit"):
                    if key not in mlp:
                        raise ValueError(f"layer {i}: the mlp lacks {key!r}")

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, raw: dict) -> "DodonexConfig":
        missing = [key for key in ("vocab", "width", "layers") if key not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        norm = raw.get("norm") or {}
        side = raw.get("token_side") or None
        values = dict(
            vocab=raw["vocab"], width=raw["width"], layers=tuple(copy.deepcopy(list(raw["layers"]))),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            norm_eps=float(norm.get("eps", 1e-6)), norm_groups=int(norm.get("groups", 1)),
            residual_mult=float(raw.get("residual_mult", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
            token_side_dim=side["dim"] if side else None,
            eos_token_id=raw.get("eos_token_id"),
        )
        if raw.get("max_position_embeddings") is not None:
            values["max_position_embeddings"] = int(raw["max_position_embeddings"])
        return cls(**values)

    def to_dict(self) -> dict:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
            "layers": copy.deepcopy(list(self.layers)),
        }
        if self.token_side_dim is not None:
            out["token_side"] = {"dim": self.token_side_dim}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    def with_tensor_shapes(self, shapes: dict) -> "DodonexConfig":
        """The sizes that only the checkpoint gives: a delta-rule layer's decay rank is the
        number of rows of its ``w1``.  ``shapes``: tensor name -> shape."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            name = f"l{i}.mix.w1"
            if layer["type"] == "general_delta" and name in shapes and len(shapes[name]) == 2:
                layer["mixer"]["decay_rank"] = int(shapes[name][0])
        import dataclasses

        return dataclasses.replace(self, layers=tuple(layers))

    # ------------------------------------------------------------ structure
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("rms_norm", {"size": W, "eps": self.norm_eps, "groups": self.norm_groups, "weight_name": ""})
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            mixer = layer["mixer"]
            if layer["type"] == "general_delta":
                if mixer.get("decay_rank") is None:
                    raise ValueError(f"layer {i}: the decay rank is unknown; it is the first dimension of l{i}.mix.w1 "
                                     "(with_tensor_shapes) or the mixer's 'decay_rank'")
                part = PartSpec("general_delta", {
                    "hidden_size": W, "num_heads": int(mixer["heads"]), "head_dim": int(mixer["dim"]),
                    "decay_rank": int(mixer["decay_rank"]), "eps": self.norm_eps})
                source = None
            else:
                rot = mixer["rot"]
                source = mixer.get("kv_from")
                part = PartSpec("latent_attention", {
                    "hidden_size": W, "num_heads": int(mixer["heads"]), "head_dim": int(mixer["dim"]),
                    "rot_dim": int(mixer["rot_dim"]), "v_dim": int(mixer["vdim"]), "q_rank": int(mixer["q_rank"]),
                    "kv_rank": int(mixer["kv_rank"]), "scale": float(mixer["scale"]),
                    "rot_base": float(rot["base"]), "rot_dims": int(rot.get("dims", mixer["rot_dim"])),
                    "eps": self.norm_eps, "own_kv": source is None})
            mlp = layer.get("mlp")
            feed_forward = None if mlp is None else PartSpec("clamped_glu", {
                "hidden_size": W, "intermediate_size": int(mlp["ff"]), "limit": float(mlp["limit"]), "alpha": 1.702,
                "gate_name": "gate", "up_name": "up", "down_name": "down"})
            side = None
            if self.token_side_dim is not None:
                side = PartSpec("gated_token_embedding", {
                    "hidden_size": W, "dim": self.token_side_dim, "eps": self.norm_eps, "vocab_size": self.vocab,
                    "table_name": "side.embed", "table_width": self.token_side_dim * len(self.layers),
                    "offset": i * self.token_side_dim})
            layers.append(LayerSpec(
                prefix=f"l{i}.", block="parallel_scaled", mixer=part, feed_forward=feed_forward,
                norms=(NormSlot("shared_norm", norm, "norm1"),), mixer_prefix="mix.", feed_forward_prefix="mlp.",
                block_params={"residual_mult": self.residual_mult}, token_input=side, token_input_prefix="side."))
            schedule.append(ScheduleEntry(layer=i, cache_from=source))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            max_position_embeddings=self.max_position_embeddings, embedding_name="embed",
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
            lm_head_name="lm_head", tie_word_embeddings=True,
            embedding_scale=self.embedding_scale, logit_scale=self.logit_scale)
        spec.validate()
        return spec
