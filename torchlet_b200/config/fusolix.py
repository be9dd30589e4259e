"""Typed configuration of the Fusolix design: a decoder-only model whose layers are listed one by one in
``config.json``.

    {"architecture": "Fusolix", "vocab": V, "width": W, "streams": n, "norm": {"eps": e},
     "embedding": {"scale": s}, "canon": {"taps": k},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "pool"}},
                           "right": {"heads", "dim", "vdim", "decay": [...], "rot": {"base", "dims"}},
                           "left_scale", "right_scale"},
                 "mlp": {"kind": "dense", "ff", "limit"}
                      | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}}}
                      | null}, ...]}

The model keeps ``streams`` copies of the residual stream (hyper-connections: ``l<i>.hc1.*`` for the mixer,
``l<i>.hc2.*`` for the feed-forward), norms with a layer norm (``l<i>.norm1``, ``l<i>.norm2`` with ``.b`` biases), and
puts a causal convolution over time of ``canon.taps`` taps in front of every sub-layer (``l<i>.canon1``,
``l<i>.canon2``).  The mixer ``l<i>.mix.*`` is two mixers side by side: ``left``, a softmax attention over a sliding
window and pooled blocks of older tokens, with biases and without positions; ``right``, a retention with rotated q
and k.  The feed-forward ``l<i>.mlp.*`` is a clamped gated unit or a mixture of plain gated experts with softmax
scores, group-limited choice and renormalized weights.  Output: ``head`` behind the layer norm ``final.norm``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry

DEFAULT_MAX_POSITIONS = 1 << 17  # the design has no position limit of its own; the engine wants a bound
DENSE_SLOPE = 1.702  # the dense unit's activation is g * sigmoid(1.702 g) * (u + 1)
RENORM_EPS = 1e-20  # added to the sum the chosen experts' scores are divided by


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


def _need(mapping, keys, what: str) -> None:
    if not isinstance(mapping, dict):
        raise ValueError(f"{what} must be an object")
    missing = [key for key in keys if key not in mapping]
    if missing:
        raise ValueError(f"{what} lacks {', '.join(missing)}")


@register_architecture("Fusolix")
@dataclass(frozen=True)
class FusolixConfig:
    vocab: int
    width: int
    layers: tuple  # of dicts as in config.json: type, mixer, mlp
    streams: int = 1
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    canon_taps: Optional[int] = None  # None: no convolution in front of the sub-layers
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    architecture = "Fusolix"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.streams, "streams")
        if self.streams > 8:
            raise ValueError("at most 8 streams are supported")
        if self.canon_taps is not None and not 1 <= self.canon_taps <= 8:
            raise ValueError(f"canon.taps {self.canon_taps} is not supported (1 to 8)")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.layers:
            raise ValueError("'layers' is empty")
        for i, layer in enumerate(self.layers):
            if layer.get("type") != "parallel":
                raise ValueError(f"layer {i}: unknown type {layer.get('type')!r} (known: parallel)")
            mixer = layer.get("mixer")
            _need(mixer, ("left", "right"), f"layer {i}: mixer")
            left, right = mixer["left"], mixer["right"]
            _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), f"layer {i}: mixer.left")
            _need(left["mask"], ("size", "pool"), f"layer {i}: mixer.left.mask")
            _need(right, ("heads", "dim", "vdim", "decay"), f"layer {i}: mixer.right")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(left[key], f"layer {i}: mixer.left.{key}")
            for key in ("heads", "dim", "vdim"):
                _positive_int(right[key], f"layer {i}: mixer.right.{key}")
            _positive_int(left["mask"]["size"], f"layer {i}: mask.size")
            _positive_int(left["mask"]["pool"], f"layer {i}: mask.pool")
            if left["heads"] % left["kv_heads"]:
                raise ValueError(f"layer {i}: heads {left['heads']} is no multiple of kv_heads {left['kv_heads']}")
            if len(right["decay"]) != right["heads"]:
                raise ValueError(f"layer {i}: {len(right['decay'])} decays for {right['heads']} heads")
            rot = right.get("rot")
            if rot is not None:
                _need(rot, ("base", "dims"), f"layer {i}: mixer.right.rot")
                if rot["dims"] % 2 or not 0 < rot["dims"] <= right["dim"]:
                    raise ValueError(f"layer {i}: rot.dims {rot['dims']} must be even and at most dim {right['dim']}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            kind = mlp.get("kind")
            if kind == "dense":
                _need(mlp, ("ff", "limit"), f"layer {i}: mlp")
                _positive_int(mlp["ff"], f"layer {i}: mlp.ff")
            elif kind == "moe":
                _need(mlp, ("expert", "router"), f"layer {i}: mlp")
                _need(mlp["expert"], ("ff",), f"layer {i}: mlp.expert")
                _need(mlp["router"], ("experts", "top"), f"layer {i}: mlp.router")
                experts = _positive_int(mlp["router"]["experts"], f"layer {i}: router.experts")
                top = _positive_int(mlp["router"]["top"], f"layer {i}: router.top")
                groups = mlp["router"].get("groups")
                count, keep = (1, 1) if groups is None else (groups.get("count", 1), groups.get("keep", groups.get("count", 1)))
                _positive_int(count, f"layer {i}: router.groups.count")
                _positive_int(keep, f"layer {i}: router.groups.keep")
                if experts % count or keep > count:
                    raise ValueError(f"layer {i}: {experts} experts cannot form {count} equal groups of which {keep} are kept")
                if top > keep * (experts // count):
                    raise ValueError(f"layer {i}: router.top {top} exceeds the experts of the {keep} kept groups")
            else:
                raise ValueError(f"layer {i}: unknown mlp kind {kind!r} (known: dense, moe)")

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, raw: dict) -> "FusolixConfig":
        missing = [key for key in ("vocab", "width", "layers") if key not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        canon = raw.get("canon") or {}
        values = dict(
            vocab=raw["vocab"], width=raw["width"], layers=tuple(copy.deepcopy(list(raw["layers"]))),
            streams=int(raw.get("streams", 1)), norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            canon_taps=int(canon["taps"]) if canon.get("taps") else None, eos_token_id=raw.get("eos_token_id"))
        if raw.get("max_position_embeddings") is not None:
            values["max_position_embeddings"] = int(raw["max_position_embeddings"])
        return cls(**values)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
               "layers": copy.deepcopy(list(self.layers))}
        if self.canon_taps is not None:
            out["canon"] = {"taps": self.canon_taps}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    # ------------------------------------------------------------ structure
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("layer_norm", {"size": W, "eps": self.norm_eps, "weight_name": "", "bias_name": ".b"})
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            rot = right.get("rot")
            positions = None
            if rot is not None:
                positions = PartSpec("rotary_partial", {"head_dim": int(right["dim"]), "dims": int(rot["dims"]),
                                                        "base": float(rot["base"]), "scaling": None})
            attention = PartSpec("pooled_window_attention", {
                "hidden_size": W, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
                "head_dim": int(left["dim"]), "v_dim": int(left["vdim"]), "scale": float(left["scale"]),
                "window": int(left["mask"]["size"]), "pool": int(left["mask"]["pool"]), "bias": True})
            retention = PartSpec("retention", {
                "hidden_size": W, "num_heads": int(right["heads"]), "head_dim": int(right["dim"]),
                "v_dim": int(right["vdim"]), "decay": tuple(float(a) for a in right["decay"]), "eps": self.norm_eps,
                "positions": positions})
            mixer = PartSpec("parallel_mixers", {"branches": (
                {"mixer": attention, "prefix": "left.", "scale": float(layer["mixer"].get("left_scale", 1.0))},
                {"mixer": retention, "prefix": "right.", "scale": float(layer["mixer"].get("right_scale", 1.0))})})
            mlp = layer.get("mlp")
            feed_forward = None
            if mlp is not None and mlp["kind"] == "dense":
                feed_forward = PartSpec("clamped_glu", {
                    "hidden_size": W, "intermediate_size": int(mlp["ff"]), "limit": float(mlp["limit"]),
                    "alpha": DENSE_SLOPE, "gate_name": "gate", "up_name": "up", "down_name": "down"})
            elif mlp is not None:
                groups = mlp["router"].get("groups") or {}
                count = int(groups.get("count", 1))
                feed_forward = PartSpec("routed_clamped_glu", {
                    "hidden_size": W, "intermediate_size": int(mlp["expert"]["ff"]), "limit": None,
                    "num_experts": int(mlp["router"]["experts"]), "top_k": int(mlp["router"]["top"]),
                    "score": "softmax", "renormalize": True, "renorm_eps": RENORM_EPS, "weight_on": "output",
                    "groups": count, "keep": int(groups.get("keep", count))})
            norms = [NormSlot("mixer_norm", norm, "norm1")]
            if feed_forward is not None:
                norms.append(NormSlot("feed_forward_norm", norm, "norm2"))
            layers.append(LayerSpec(
                prefix=f"l{i}.", block="hyper_connected", mixer=mixer, feed_forward=feed_forward, norms=tuple(norms),
                mixer_prefix="mix.", feed_forward_prefix="mlp.",
                block_params={"streams": self.streams, "taps": self.canon_taps, "connections": ("hc1.", "hc2."),
                              "convolutions": ("canon1", "canon2")}))
            schedule.append(ScheduleEntry(layer=i))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            max_position_embeddings=self.max_position_embeddings, embedding_name="embed",
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
            lm_head_name="head", tie_word_embeddings=False, embedding_scale=self.embedding_scale, streams=self.streams)
        spec.validate()
        return spec
