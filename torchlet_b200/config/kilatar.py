"""Typed configuration of the Kilatar design: a decoder-only model whose layers are listed one by one in
``config.json``, a stretch of which may run several times.

    {"architecture": "Kilatar", "vocab": V, "width": W, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "mamba2", "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                                    "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                           "right": {"heads", "dim", "vdim", "decay": [...]}}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}}, "mlp": ...}]}
    mlp: {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity", "scale"},
          "shared": {"ff"} or absent} | null

The embedding rows pass an RMS norm (``embed.norm``).  Every layer is a PARALLEL block: one RMS norm (``l<i>.norm1``)
whose output both the mixer ``l<i>.mix.*`` and the feed-forward ``l<i>.mlp.*`` read, x += mixer + feed-forward.  Layers
``loop.start .. loop.stop - 1`` run ``loop.times`` times in a row with the same weights and a cache or state of their
own each time; before every pass but the first the embedding output is added to the stream.  The mixers: a
state-space mixer ("mamba2"); a latent attention with direct queries, an interleaved rotation of the rotated part and a
sigmoid output gate; or ("parallel") a chunked attention with a partial interleaved rotation whose frequencies are
slowed down by wavelength BESIDE a linear attention with silu on q, k, v and a constant decay per head, each branch's
output RMS-normed over the width (``left.out``, ``right.out``) and the two averaged.  The feed-forward is a gated unit
with the tanh form of gelu and biases, or a mixture of silu-gated experts: softmax scores, the choice by
score + ``correction``, weights renormalized and scaled, identity experts behind the real ones, and a shared expert
with a sigmoid gate of one number a token.  Output: ``head`` behind the RMS norm ``final.norm``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry

DEFAULT_MAX_POSITIONS = 1 << 17  # the design has no position limit of its own; the engine wants a bound
RENORM_EPS = 1e-20  # added to the sum the chosen experts' scores are divided by
BRANCH_SCALE = 0.5  # the two branches of a parallel mixer are averaged


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


def _check_rot(rot, limit: int, what: str) -> None:
    _need(rot, ("base", "dims"), what)
    if not isinstance(rot["dims"], int) or rot["dims"] % 2 or not 0 < rot["dims"] <= limit:
        raise ValueError(f"{what}.dims {rot['dims']!r} must be even and at most {limit}")
    if rot.get("scaling") is not None:
        _need(rot["scaling"], ("factor", "low", "high", "original"), f"{what}.scaling")


MIXER_KEYS = {
    "mamba2": ("heads", "vdim", "state", "conv"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "parallel": ("left", "right"),
}


@register_architecture("Kilatar")
@dataclass(frozen=True)
class KilatarConfig:
    vocab: int
    width: int
    layers: tuple  # of dicts as in config.json: type, mixer, mlp
    norm_eps: float = 1e-6
    loop: Optional[tuple] = None  # (start, stop, times)
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    architecture = "Kilatar"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.layers:
            raise ValueError("'layers' is empty")
        if self.loop is not None:
            start, stop, times = self.loop
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(self.layers)):
                raise ValueError(f"loop: layers {start} .. {stop} - 1 do not lie within the {len(self.layers)} layers")
            _positive_int(times, "loop.times")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in MIXER_KEYS:
                raise ValueError(f"layer {i}: unknown type {kind!r} (known: {', '.join(sorted(MIXER_KEYS))})")
            mixer = layer.get("mixer")
            _need(mixer, MIXER_KEYS[kind], f"layer {i}: mixer")
            if kind == "mamba2":
                for key in ("heads", "vdim", "state", "conv"):
                    _positive_int(mixer[key], f"layer {i}: mixer.{key}")
                groups = _positive_int(mixer.get("groups", 1), f"layer {i}: mixer.groups")
                parts = _positive_int(mixer.get("norm_groups", 1), f"layer {i}: mixer.norm_groups")
                if mixer["heads"] % groups or (mixer["heads"] * mixer["vdim"]) % parts:
                    raise ValueError(f"layer {i}: {mixer['heads']} heads of {mixer['vdim']} do not split into {groups} "
                                     f"groups / {parts} norm groups")
            elif kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _positive_int(mixer[key], f"layer {i}: mixer.{key}")
                _check_rot(mixer["rot"], mixer["rot_dim"], f"layer {i}: mixer.rot")
                if mixer["rot"].get("scaling") is not None:
                    raise ValueError(f"layer {i}: frequency scaling is not part of the latent attention")
            else:
                left, right = mixer["left"], mixer["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), f"layer {i}: mixer.left")
                _need(left["mask"], ("size",), f"layer {i}: mixer.left.mask")
                _need(right, ("heads", "dim", "vdim", "decay"), f"layer {i}: mixer.right")
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(left[key], f"layer {i}: mixer.left.{key}")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right[key], f"layer {i}: mixer.right.{key}")
                _positive_int(left["mask"]["size"], f"layer {i}: mask.size")
                if left["heads"] % left["kv_heads"]:
                    raise ValueError(f"layer {i}: heads {left['heads']} is no multiple of kv_heads {left['kv_heads']}")
                if left.get("rot") is not None:
                    _check_rot(left["rot"], left["dim"], f"layer {i}: mixer.left.rot")
                if len(right["decay"]) != right["heads"]:
                    raise ValueError(f"layer {i}: {len(right['decay'])} decays for {right['heads']} heads")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
            elif mlp.get("kind") == "moe":
                _need(mlp, ("expert", "router"), f"layer {i}: mlp")
                _need(mlp["expert"], ("ff",), f"layer {i}: mlp.expert")
                _need(mlp["router"], ("experts", "top"), f"layer {i}: mlp.router")
                experts = _positive_int(mlp["router"]["experts"], f"layer {i}: router.experts")
                top = _positive_int(mlp["router"]["top"], f"layer {i}: router.top")
                identity = mlp["router"].get("identity", 0) or 0
                if not isinstance(identity, int) or identity < 0 or top > experts + identity:
                    raise ValueError(f"layer {i}: router.top {top} / identity {identity!r} do not fit {experts} experts")
                if mlp.get("shared") is not None:
                    _positive_int(mlp["shared"].get("ff"), f"layer {i}: mlp.shared.ff")
            else:
                raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r} (known: dense, moe)")

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, raw: dict) -> "KilatarConfig":
        missing = [key for key in ("vocab", "width", "layers") if key not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        loop = raw.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop"), "loop")
            loop = (loop["start"], loop["stop"], loop.get("times", 1))
        values = dict(vocab=raw["vocab"], width=raw["width"], layers=tuple(copy.deepcopy(list(raw["layers"]))),
                      norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)), loop=loop,
                      eos_token_id=raw.get("eos_token_id"))
        if raw.get("max_position_embeddings") is not None:
            values["max_position_embeddings"] = int(raw["max_position_embeddings"])
        return cls(**values)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    # ------------------------------------------------------------ structure
    def layer_runs(self) -> list:
        """The layers in the order they run: (layer, whether the embedding output is added before it)."""
        n = len(self.layers)
        if self.loop is None or self.loop[2] <= 1:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, False) for i in range(start)]
        for k in range(times):
            runs += [(i, k > 0 and i == start) for i in range(start, stop)]
        return runs + [(i, False) for i in range(stop, n)]

    def _mixer(self, kind: str, m: dict) -> PartSpec:
        W, eps = self.width, self.norm_eps
        if kind == "mamba2":
            return PartSpec("mamba2", {
                "hidden_size": W, "num_heads": int(m["heads"]), "v_dim": int(m["vdim"]), "state_size": int(m["state"]),
                "groups": int(m.get("groups", 1)), "conv_taps": int(m["conv"]), "norm_groups": int(m.get("norm_groups", 1)),
                "eps": eps})
        if kind == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                "v_dim": int(m["vdim"]), "q_rank": None, "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]),
                "rot_base": float(m["rot"]["base"]), "rot_dims": int(m["rot"]["dims"]), "eps": eps, "gate": "sigmoid",
                "pairing": "interleaved"})
        left, right = m["left"], m["right"]
        rot = left.get("rot")
        positions = None
        if rot is not None:
            scaling = dict(rot["scaling"]) if rot.get("scaling") else None
            positions = PartSpec("rotary_partial", {"head_dim": int(left["dim"]), "dims": int(rot["dims"]),
                                                    "base": float(rot["base"]), "scaling": scaling, "pairing": "interleaved"})
        attention = PartSpec("gated_attention", {
            "hidden_size": W, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
            "head_dim": int(left["dim"]), "v_dim": int(left["vdim"]), "scale": float(left["scale"]),
            "chunk": int(left["mask"]["size"]), "positions": positions, "eps": eps})
        linear = PartSpec("retention", {
            "hidden_size": W, "num_heads": int(right["heads"]), "head_dim": int(right["dim"]), "v_dim": int(right["vdim"]),
            "decay": tuple(float(a) for a in right["decay"]), "eps": eps, "positions": None, "k_scale": 1.0,
            "activation": "silu", "norm": "whole", "gate": "sigmoid"})
        out_norm = PartSpec("rms_norm", {"size": W, "eps": eps, "weight_name": ""})
        return PartSpec("parallel_mixers", {"branches": (
            {"mixer": attention, "prefix": "left.", "scale": BRANCH_SCALE, "norm": out_norm, "norm_prefix": "left.out"},
            {"mixer": linear, "prefix": "right.", "scale": BRANCH_SCALE, "norm": out_norm, "norm_prefix": "right.out"})})

    def _feed_forward(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        W = self.width
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": int(mlp["ff"]),
                                          "activation": "gelu_tanh", "bias": True})
        router = mlp["router"]
        shared = None
        if mlp.get("shared") is not None:
            shared = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": int(mlp["shared"]["ff"]),
                                            "activation": "silu", "bias": False, "token_gate": "sg"})
        return PartSpec("routed_clamped_glu", {
            "hidden_size": W, "intermediate_size": int(mlp["expert"]["ff"]), "limit": None,
            "num_experts": int(router["experts"]), "top_k": int(router["top"]), "score": "softmax",
            "renormalize": True, "renorm_eps": RENORM_EPS, "weight_on": "output", "correction": True,
            "weight_scale": float(router.get("scale", 1.0)), "identity": int(router.get("identity", 0) or 0),
            "shared": shared, "shared_prefix": "shared."})

    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("rms_norm", {"size": W, "eps": self.norm_eps, "weight_name": ""})
        layers = []
        for i, layer in enumerate(self.layers):
            layers.append(LayerSpec(
                prefix=f"l{i}.", block="parallel_scaled", mixer=self._mixer(layer["type"], layer["mixer"]),
                feed_forward=self._feed_forward(layer.get("mlp")), norms=(NormSlot("shared_norm", norm, "norm1"),),
                mixer_prefix="mix.", feed_forward_prefix="mlp.", block_params={"residual_mult": 1.0}))
        schedule = tuple(ScheduleEntry(layer=i, add_embedding=again) for i, again in self.layer_runs())
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W,
            max_position_embeddings=self.max_position_embeddings, embedding_name="embed",
            layers=tuple(layers), schedule=schedule, final_norm=norm, final_norm_prefix="final.norm",
            lm_head_name="head", tie_word_embeddings=False, embedding_norm=norm, embedding_norm_prefix="embed.norm")
        spec.validate()
        return spec
