"""Typed configuration of the Famalorn decoder, read from its config.json.

config.json gives ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list whose entries name the
layer's mixer (``type``: ``delta``, ``mamba2`` or ``parallel``), the mixer's sizes (``mixer``) and the
feed-forward (``mlp``: ``{"kind": "dense", "ff": n}``, or null for a layer without one).  A
``parallel`` mixer holds an attention branch (``left``) and a Mamba-2 branch (``right``) with the
weights of their sum.  Every size and constant of a model is one of these numbers; the code holds
only what the design fixes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError

ARCHITECTURE = "Famalorn"


def _int(raw: dict, key: str, where: str, least: int = 1) -> int:
    value = raw.get(key)
    if value is None or isinstance(value, bool) or int(value) != value:
        raise ConfigError(f"config.json: {where} needs an integer {key!r}, got {value!r}")
    if int(value) < least:
        raise ConfigError(f"config.json: {where} has {key!r} = {value}, below {least}")
    return int(value)


def _float(raw: dict, key: str, where: str) -> float:
    value = raw.get(key)
    if value is None or isinstance(value, bool):
        raise ConfigError(f"config.json: {where} needs a number {key!r}, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class Mamba2Sizes:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @staticmethod
    def from_dict(raw: dict, where: str) -> "Mamba2Sizes":
        sizes = Mamba2Sizes(*(_int(raw, key, where) for key in ("heads", "vdim", "state", "groups", "norm_groups", "conv")))
        if sizes.heads % sizes.groups:
            raise ConfigError(f"config.json: {where}: {sizes.heads} heads are not a multiple of {sizes.groups} groups")
        if (sizes.heads * sizes.vdim) % sizes.norm_groups:
            raise ConfigError(f"config.json: {where}: the inner width is not a multiple of {sizes.norm_groups} norm groups")
        return sizes

    def to_dict(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups, "state": self.state,
                "vdim": self.vdim}


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @staticmethod
    def from_dict(raw: dict, where: str) -> "DeltaSizes":
        sizes = DeltaSizes(*(_int(raw, key, where) for key in ("heads", "kv_heads", "dim", "vdim", "conv")))
        if sizes.heads % sizes.kv_heads:
            raise ConfigError(f"config.json: {where}: {sizes.heads} heads are not a multiple of {sizes.kv_heads} query/key heads")
        return sizes

    def to_dict(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int           # 0: no rotation
    rot_base: float

    @staticmethod
    def from_dict(raw: dict, where: str) -> "AttentionSizes":
        rot = raw.get("rot") or {}
        dims = _int(rot, "dims", where + ".rot", 0) if rot else 0
        sizes = AttentionSizes(
            _int(raw, "heads", where), _int(raw, "kv_heads", where), _int(raw, "dim", where), _int(raw, "vdim", where),
            _float(raw, "scale", where), dims, _float(rot, "base", where + ".rot") if dims else 10000.0)
        if sizes.heads % sizes.kv_heads:
            raise ConfigError(f"config.json: {where}: {sizes.heads} query heads are not a multiple of {sizes.kv_heads} key/value heads")
        if sizes.rot_dims % 2 or sizes.rot_dims > sizes.dim:
            raise ConfigError(f"config.json: {where}: the rotated part must be even and at most {sizes.dim}, got {sizes.rot_dims}")
        return sizes

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        out.update({"scale": self.scale, "vdim": self.vdim})
        return out


@dataclass(frozen=True)
class ParallelSizes:
    left: AttentionSizes
    right: Mamba2Sizes
    left_scale: float
    right_scale: float

    @staticmethod
    def from_dict(raw: dict, where: str) -> "ParallelSizes":
        for key in ("left", "right"):
            if not isinstance(raw.get(key), dict):
                raise ConfigError(f"config.json: {where} needs the sizes of its {key!r} branch")
        return ParallelSizes(AttentionSizes.from_dict(raw["left"], where + ".left"), Mamba2Sizes.from_dict(raw["right"], where + ".right"),
                             _float(raw, "left_scale", where), _float(raw, "right_scale", where))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(), "right_scale": self.right_scale}


MIXER_SIZES = {"delta": DeltaSizes, "mamba2": Mamba2Sizes, "parallel": ParallelSizes}
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class FamalornLayer:
    type: str
    mixer: Any              # DeltaSizes, Mamba2Sizes or ParallelSizes
    ff: int | None          # width of the dense feed-forward; None: the layer has none

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense"}, "type": self.type}


@dataclass(frozen=True)
class FamalornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[FamalornLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "FamalornConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json is missing the 'norm' entry with its eps")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_SIZES:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known: {', '.join(sorted(MIXER_SIZES))}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs the sizes of its mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp must be null or of a kind among {MLP_KINDS}")
                ff = _int(mlp, "ff", where + ".mlp")
            layers.append(FamalornLayer(kind, MIXER_SIZES[kind].from_dict(entry["mixer"], where + ".mixer"), ff))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return FamalornConfig(_int(raw, "vocab", "the model"), _int(raw, "width", "the model"), _float(norm, "eps", "norm"),
                              tuple(layers), eos_ids)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
