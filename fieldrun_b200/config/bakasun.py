"""Configuration of the Bakasun design, read from its own config.json keys.

The file names the design as ``"architecture": "Bakasun"`` and lists the layers one by one:

    vocab, width                       sizes of the vocabulary and of the residual stream
    norm.eps                           eps of every root-mean-square norm
    layers[i].type                     "attention" | "parallel"
    layers[i].mixer                    the mixer's sizes and constants (below)
    layers[i].mlp                      null | {"kind": "dense", "ff"} |
                                       {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}},
                                        "shared": {"ff"}}

    attention: heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims, scaling {factor}}, softcap
    parallel:  left   the same keys (an attention with biases on q, k, v and no norm of q and k)
               right  {heads, kv_heads, dim, vdim, conv}                 gated delta rule
               left_scale, right_scale                                    the two outputs' weights

Everything that can differ between two models of the design is read here: a key that is absent switches its mechanism
off (no ``mask``: every earlier key; no ``rot``: no rotation; no ``scaling``: angles as they are; no ``softcap``: scores
as they are; no ``groups``: every expert can be chosen; no ``shared``: no shared expert).  What the design fixes (the
activations, the sink of score zero, the 1e-20 of the experts' weights, which mixer has biases and which norms its
queries and keys) lives with the plan (``models/bakasun.py``).  A key the design does not have is a warning on stderr.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "Bakasun"


def _unknown(raw: Mapping[str, Any], allowed: set[str], where: str) -> None:
    extra = sorted(set(raw) - allowed)
    if extra:
        print(f"{where}: warning: keys this design does not have are ignored: {', '.join(extra)}", file=sys.stderr)


def _object(raw: Any, where: str) -> Mapping[str, Any]:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where} must be an object")
    return raw


@dataclass(frozen=True)
class BakasunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                 # None: every earlier key
    rot_dims: int                         # 0: no rotation
    rot_base: float
    rot_factor: float                     # every angle is divided by it
    softcap: Optional[float]

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_factor != 1.0:
                out["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class BakasunDeltaRule:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_json(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class BakasunParallel:
    left: BakasunAttention
    right: BakasunDeltaRule
    left_scale: float
    right_scale: float

    def to_json(self) -> dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class BakasunDense:
    ff: int

    def to_json(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class BakasunExperts:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0                    # 0: no shared expert
    # whether the file holds the choice correction and the shared expert's token gate; a folder's tensor names decide
    correction: bool = True
    shared_gate: bool = True

    def to_json(self) -> dict[str, Any]:
        router: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        out: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class BakasunLayer:
    type: str
    mixer: Any                            # BakasunAttention | BakasunParallel
    mlp: Any                              # None | BakasunDense | BakasunExperts

    def to_json(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


_ATTENTION_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot", "softcap"}


def _attention(raw: Mapping[str, Any], where: str) -> BakasunAttention:
    _unknown(raw, _ATTENTION_KEYS, where)
    r = KeyReader(raw, where)
    heads = r.integer("heads", minimum=1)
    kv_heads = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = r.integer("dim", minimum=1)
    window = None
    if raw.get("mask") is not None:
        _unknown(_object(raw["mask"], where + ".mask"), {"size"}, where + ".mask")
        window = r.integer("mask.size", minimum=1)
    rot_dims, rot_base, rot_factor = 0, 10000.0, 1.0
    if raw.get("rot") is not None:
        rot = _object(raw["rot"], where + ".rot")
        _unknown(rot, {"base", "dims", "scaling"}, where + ".rot")
        rot_dims = r.integer("rot.dims", default=dim, minimum=0)
        rot_base = r.real("rot.base", positive=True)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{where}.rot.dims is {rot_dims}: an even number up to dim = {dim}")
        if rot.get("scaling") is not None:
            _unknown(_object(rot["scaling"], where + ".rot.scaling"), {"factor"}, where + ".rot.scaling")
            rot_factor = r.real("rot.scaling.factor", default=1.0, positive=True)
    softcap = r.real("softcap", positive=True) if raw.get("softcap") is not None else None
    return BakasunAttention(heads, kv_heads, dim, r.integer("vdim", default=dim, minimum=1),
                            r.real("scale", default=float(dim) ** -0.5, positive=True), window, rot_dims, rot_base, rot_factor,
                            softcap)


def _parallel(raw: Mapping[str, Any], where: str) -> BakasunParallel:
    _unknown(raw, {"left", "right", "left_scale", "right_scale"}, where)
    left = _attention(_object(raw.get("left"), where + ".left"), where + ".left")
    right = _object(raw.get("right"), where + ".right")
    _unknown(right, {"heads", "kv_heads", "dim", "vdim", "conv"}, where + ".right")
    s = KeyReader(right, where + ".right")
    heads = s.integer("heads", minimum=1)
    kv_heads = s.integer("kv_heads", default=heads, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{where}.right: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = s.integer("dim", minimum=1)
    rule = BakasunDeltaRule(heads, kv_heads, dim, s.integer("vdim", default=dim, minimum=1), s.integer("conv", minimum=1))
    r = KeyReader(raw, where)
    return BakasunParallel(left, rule, r.real("left_scale", default=1.0), r.real("right_scale", default=1.0))


_MIXERS = {"attention": _attention, "parallel": _parallel}


def _mlp(raw: Any, where: str):
    if raw is None:
        return None
    m = _object(raw, where)
    kind = m.get("kind")
    k = KeyReader(m, where)
    if kind == "dense":
        _unknown(m, {"kind", "ff"}, where)
        return BakasunDense(k.integer("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{where}.kind is {kind!r}: this design has 'dense' and 'moe'")
    _unknown(m, {"kind", "expert", "router", "shared"}, where)
    experts, top = k.integer("router.experts", minimum=1), k.integer("router.top", minimum=1)
    if top > experts:
        raise ConfigError(f"{where}.router: top {top} of {experts} experts")
    groups, keep = 1, 1
    if _object(m.get("router"), where + ".router").get("groups") is not None:
        groups = k.integer("router.groups.count", minimum=1)
        keep = k.integer("router.groups.keep", default=groups, minimum=1)
        if keep > groups or experts % groups:
            raise ConfigError(f"{where}.router.groups: {experts} experts in {groups} equal groups of which {keep} stay")
        if keep * (experts // groups) < top:
            raise ConfigError(f"{where}.router: {keep} groups of {experts // groups} experts hold fewer than top = {top}")
    shared_ff = k.integer("shared.ff", minimum=1) if m.get("shared") is not None else 0
    return BakasunExperts(experts, top, k.integer("expert.ff", minimum=1), groups, keep, shared_ff)


@dataclass(frozen=True)
class BakasunConfig(ModelConfig):
    norm_eps: float = 1e-6
    layers: tuple[BakasunLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "BakasunConfig":
        _unknown(raw, {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "eos_token_id"}, where)
        r = KeyReader(raw, where)
        if isinstance(raw.get("norm"), Mapping):
            _unknown(raw["norm"], {"eps"}, f"{where}: norm")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError(f"{where}: key 'layers' must be a list of at least one layer")
        layers: list[BakasunLayer] = []
        for index, entry in enumerate(listed):
            at = f"{where}: layers[{index}]"
            entry = _object(entry, at)
            _unknown(entry, {"type", "mixer", "mlp"}, at)
            kind = entry.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{at}.type is {kind!r}: this design has {', '.join(sorted(_MIXERS))}")
            mixer = _MIXERS[kind](_object(entry.get("mixer"), at + ".mixer"), at + ".mixer")
            layers.append(BakasunLayer(kind, mixer, _mlp(entry.get("mlp"), at + ".mlp")))
        return cls(
            architecture=ARCHITECTURE,
            vocab_size=r.integer("vocab", minimum=1),
            hidden_size=r.integer("width", minimum=1),
            num_hidden_layers=len(layers),
            eos_token_id=tuple(t for t in r.integer_list("eos_token_id", default=()) if t >= 0),
            norm_eps=r.real("norm.eps", positive=True),
            layers=tuple(layers),
        )

    def with_tensor_names(self, shapes: Mapping[str, tuple[int, ...]]) -> "BakasunConfig":
        """The configuration completed from a folder's tensor names: a layer of experts has a choice correction and a
        token gate on its shared expert if the file holds their tensors."""
        layers = []
        for index, layer in enumerate(self.layers):
            if isinstance(layer.mlp, BakasunExperts):
                mlp = replace(layer.mlp, correction=f"l{index}.mlp.correction" in shapes,
                              shared_gate=f"l{index}.mlp.shared.sg" in shapes)
                layer = replace(layer, mlp=mlp)
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_json() for layer in self.layers],
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
