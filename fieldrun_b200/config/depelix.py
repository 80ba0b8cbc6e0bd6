"""Configuration of the Depelix design, read from its own config.json keys.

The file names the design as ``"architecture": "Depelix"`` and lists the layers one by one:

    vocab, width                       sizes of the vocabulary and of the residual stream
    norm.eps                           eps of every norm of a layer and of the model
    embedding.bigram                   {buckets, mul_prev, mul_cur}: a second embedding row per token, chosen by a hash
                                       of the previous and the current token (absent: none)
    token_side.dim                     columns per layer of the per-layer token input (absent: none)
    layers[i].type                     "latent_attention" | "latent_attention_2"
    layers[i].mixer                    the mixer's sizes and constants (below)
    layers[i].mlp                      {"kind": "dense", "ff": n}, {"kind": "moe", "expert": {ff, limit},
                                       "router": {experts, top}}, or null for a layer without feed-forward

    mixer:  heads, dim (unrotated query/key entries per head), rot_dim (rotated ones), vdim, kv_rank, q_rank,
            rot {base, dims}, scale, mask {size} (``latent_attention`` only: the window), kv_from (optional: the
            index of the earlier layer whose latents and rotated key part this layer reads instead of making its own)

Everything that can differ between two models of the design is read here; what the design fixes per layer type
(the pairing of the rotation, window or not, the form of the output gate, the experts' activation) lives with the
plan in ``models/depelix.py``.  Inside a layer an unknown key is refused; at the top level it is a warning.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "Depelix"
LAYER_TYPES = ("latent_attention", "latent_attention_2")
WINDOWED_TYPES = ("latent_attention",)


@dataclass(frozen=True)
class DepelixMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    rot_base: float
    rot_dims: int
    scale: float
    window: Optional[int] = None
    kv_from: Optional[int] = None

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DepelixMlp:
    kind: str                            # "dense" | "moe"
    ff: int                              # width of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    def to_json(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class DepelixLayer:
    type: str
    mixer: DepelixMixer
    mlp: Optional[DepelixMlp]

    def to_json(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class DepelixBigram:
    buckets: int
    mul_prev: int
    mul_cur: int


def _only(raw: Mapping[str, Any], allowed: set[str], where: str) -> None:
    extra = sorted(set(raw) - allowed)
    if extra:
        raise ConfigError(f"{where}: keys this design does not have: {', '.join(extra)}")


def _mixer(raw: Mapping[str, Any], kind: str, where: str, index: int, before: list[DepelixLayer]) -> DepelixMixer:
    _only(raw, {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "rot", "scale", "mask", "kv_from"}, where)
    r = KeyReader(raw, where)
    dim = r.integer("dim", minimum=0)
    rot_dim = r.integer("rot_dim", minimum=0)
    if dim + rot_dim < 1:
        raise ConfigError(f"{where}: a head without query and key entries")
    rot_dims = r.integer("rot.dims", default=rot_dim, minimum=0)
    if rot_dims > rot_dim or rot_dims % 2:
        raise ConfigError(f"{where}: rot.dims {rot_dims} must be even and at most rot_dim {rot_dim}")
    if isinstance(raw.get("rot"), Mapping):
        _only(raw["rot"], {"base", "dims"}, where + ".rot")
    window = None
    if kind in WINDOWED_TYPES:
        if isinstance(raw.get("mask"), Mapping):
            _only(raw["mask"], {"size"}, where + ".mask")
        window = r.integer("mask.size", minimum=1)
    elif r.present("mask"):
        raise ConfigError(f"{where}: a mask on a layer of type {kind!r}, which sees every earlier key")
    mixer = DepelixMixer(
        heads=r.integer("heads", minimum=1), dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim", minimum=1),
        kv_rank=r.integer("kv_rank", minimum=1), q_rank=r.integer("q_rank", minimum=1),
        rot_base=r.real("rot.base", default=10000.0, positive=True), rot_dims=rot_dims,
        scale=r.real("scale", default=float(dim + rot_dim) ** -0.5, positive=True), window=window,
        kv_from=r.integer("kv_from", minimum=0) if r.present("kv_from") else None)
    if mixer.kv_from is not None:
        if mixer.kv_from >= index:
            raise ConfigError(f"{where}: kv_from {mixer.kv_from} must name an earlier layer")
        source = before[mixer.kv_from]
        if source.mixer.kv_from is not None:
            raise ConfigError(f"{where}: kv_from {mixer.kv_from} must name a layer with latents of its own")
        mine = (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims, kind in WINDOWED_TYPES)
        theirs = (source.mixer.kv_rank, source.mixer.rot_dim, source.mixer.rot_base, source.mixer.rot_dims,
                  source.type in WINDOWED_TYPES)
        if mine != theirs:
            raise ConfigError(f"{where}: layer {mixer.kv_from}'s latents (rank, rotated part, rotation: {theirs}) "
                              f"do not fit this layer's ({mine})")
    return mixer


def _mlp(raw: Any, where: str) -> Optional[DepelixMlp]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where} must be an object or null")
    kind = raw.get("kind")
    if kind == "dense":
        _only(raw, {"kind", "ff"}, where)
        return DepelixMlp("dense", KeyReader(raw, where).integer("ff", minimum=1))
    if kind == "moe":
        _only(raw, {"kind", "expert", "router"}, where)
        r = KeyReader(raw, where)
        for name, keys in (("expert", {"ff", "limit"}), ("router", {"experts", "top"})):
            if not isinstance(raw.get(name), Mapping):
                raise ConfigError(f"{where}.{name} must be an object")
            _only(raw[name], keys, f"{where}.{name}")
        experts = r.integer("router.experts", minimum=1)
        top = r.integer("router.top", minimum=1)
        if top > experts:
            raise ConfigError(f"{where}: the {top} best of {experts} experts")
        return DepelixMlp("moe", r.integer("expert.ff", minimum=1), experts, top, r.real("expert.limit", positive=True))
    raise ConfigError(f"{where}.kind is {kind!r}: this design has 'dense' and 'moe'")


@dataclass(frozen=True)
class DepelixConfig(ModelConfig):
    norm_eps: float = 1e-6
    bigram: Optional[DepelixBigram] = None
    side_dim: Optional[int] = None
    layers: tuple[DepelixLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "DepelixConfig":
        known = {"architecture", "architectures", "model_type", "vocab", "width", "embedding", "norm", "token_side",
                 "layers", "eos_token_id"}
        extra = sorted(set(raw) - known)
        if extra:
            print(f"{where}: warning: top-level keys this design does not have are ignored: {', '.join(extra)}", file=sys.stderr)
        for name, keys in (("embedding", {"bigram"}), ("norm", {"eps"}), ("token_side", {"dim"})):
            if isinstance(raw.get(name), Mapping):
                _only(raw[name], keys, f"{where}: {name}")
        r = KeyReader(raw, where)
        bigram = None
        if r.present("embedding.bigram"):
            _only(raw["embedding"]["bigram"], {"buckets", "mul_prev", "mul_cur"}, f"{where}: embedding.bigram")
            bigram = DepelixBigram(r.integer("embedding.bigram.buckets", minimum=1),
                                   r.integer("embedding.bigram.mul_prev", minimum=0),
                                   r.integer("embedding.bigram.mul_cur", minimum=0))
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError(f"{where}: key 'layers' must be a list of at least one layer")
        layers: list[DepelixLayer] = []
        for index, entry in enumerate(listed):
            at = f"{where}: layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{at} must be an object")
            _only(entry, {"type", "mixer", "mlp"}, at)
            kind = entry.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{at}.type is {kind!r}: this design has {' and '.join(repr(t) for t in LAYER_TYPES)}")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"{at}.mixer must be an object")
            layers.append(DepelixLayer(kind, _mixer(entry["mixer"], kind, at + ".mixer", index, layers),
                                       _mlp(entry.get("mlp"), at + ".mlp")))
        return cls(
            architecture=ARCHITECTURE,
            vocab_size=r.integer("vocab", minimum=1),
            hidden_size=r.integer("width", minimum=1),
            num_hidden_layers=len(layers),
            eos_token_id=tuple(t for t in r.integer_list("eos_token_id", default=()) if t >= 0),
            norm_eps=r.real("norm.eps", positive=True),
            bigram=bigram,
            side_dim=r.integer("token_side.dim", minimum=1) if r.present("token_side.dim") else None,
            layers=tuple(layers),
        )

    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_json() for layer in self.layers],
        }
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
