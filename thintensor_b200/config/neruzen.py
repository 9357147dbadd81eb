"""Typed configuration of the Neruzen decoder, read from its config.json.

config.json gives ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``: the
hashed pair table that is added to the token embedding; absent: none) and ``layers``: a list whose entries name the
layer's mixer (``type``: ``latent_attention``, ``lightning`` or ``retention``), the mixer's sizes (``mixer``) and the
feed-forward (``mlp``: ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k, "groups": {"count": g,
"keep": m}}, "shared": {"ff": n}}``, or null for a layer without one).  Every size and constant of a model is one of
these numbers; the code holds only what the design fixes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError
from .famalorn import _float, _int

ARCHITECTURE = "Neruzen"


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float

    @staticmethod
    def from_dict(raw, where: str, most: int) -> "Rotation | None":
        if not raw:
            return None
        rot = Rotation(_int(raw, "dims", where), _float(raw, "base", where))
        if rot.dims % 2 or rot.dims > most:
            raise ConfigError(f"config.json: {where}: the rotated part must be even and at most {most}, got {rot.dims}")
        return rot

    def to_dict(self) -> dict:
        return {"base": self.base, "dims": self.dims}


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int                # unrotated query/key numbers per head
    rot_dim: int            # rotated query/key numbers per head; the key's are shared by all heads
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None      # mask.size: a position sees itself and the window - 1 before it; None: all
    rot: Rotation | None

    @staticmethod
    def from_dict(raw: dict, where: str) -> "LatentAttentionSizes":
        rot_dim = _int(raw, "rot_dim", where)
        mask = raw.get("mask")
        return LatentAttentionSizes(
            _int(raw, "heads", where), _int(raw, "dim", where), rot_dim, _int(raw, "vdim", where), _int(raw, "q_rank", where),
            _int(raw, "kv_rank", where), _float(raw, "scale", where), _int(mask, "size", where + ".mask") if mask else None,
            Rotation.from_dict(raw.get("rot"), where + ".rot", rot_dim))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        out["q_rank"] = self.q_rank
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out.update({"rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim})
        return out


@dataclass(frozen=True)
class LinearAttentionSizes:
    """Sizes of a ``lightning`` or ``retention`` mixer; ``rot`` belongs to retention only."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: Rotation | None = None

    @staticmethod
    def from_dict(raw: dict, where: str, rotates: bool = False) -> "LinearAttentionSizes":
        heads, dim = _int(raw, "heads", where), _int(raw, "dim", where)
        decay = raw.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {where} needs a list 'decay' with one number for each of its {heads} heads")
        return LinearAttentionSizes(heads, dim, _int(raw, "vdim", where), tuple(float(d) for d in decay),
                                    Rotation.from_dict(raw.get("rot"), where + ".rot", dim) if rotates else None)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out["vdim"] = self.vdim
        return out


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0      # 0: no shared expert
    grouped: bool = True    # whether config.json spells the groups out (one group of which one stays says the same)

    @staticmethod
    def from_dict(raw: dict, where: str) -> "MoeSizes":
        router, expert = raw.get("router"), raw.get("expert")
        if not isinstance(router, dict) or not isinstance(expert, dict):
            raise ConfigError(f"config.json: {where} needs 'router' and 'expert'")
        groups = router.get("groups") or {}
        shared = raw.get("shared") or {}
        sizes = MoeSizes(_int(router, "experts", where + ".router"), _int(router, "top", where + ".router"), _int(expert, "ff", where + ".expert"),
                         _int(groups, "count", where + ".router.groups") if groups else 1,
                         _int(groups, "keep", where + ".router.groups") if groups else 1,
                         _int(shared, "ff", where + ".shared") if shared else 0, bool(groups))
        if sizes.experts % sizes.groups or sizes.keep > sizes.groups:
            raise ConfigError(f"config.json: {where}: {sizes.experts} experts do not form {sizes.groups} equal groups of which {sizes.keep} stay")
        if sizes.top > sizes.keep * (sizes.experts // sizes.groups):
            raise ConfigError(f"config.json: {where}: top {sizes.top} is more than the experts of {sizes.keep} groups")
        return sizes

    def to_dict(self) -> dict:
        router: dict[str, Any] = {"experts": self.experts}
        if self.grouped:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        router["top"] = self.top
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXER_TYPES = ("latent_attention", "lightning", "retention")


@dataclass(frozen=True)
class NeruzenLayer:
    type: str
    mixer: Any              # LatentAttentionSizes or LinearAttentionSizes
    mlp: MoeSizes | None    # None: the layer has no feed-forward

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int

    def to_dict(self) -> dict:
        return {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev}


@dataclass(frozen=True)
class NeruzenConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[NeruzenLayer, ...]
    bigram: PairTable | None = None
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "NeruzenConfig":
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
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs the sizes of its mixer")
            if kind == "latent_attention":
                mixer = LatentAttentionSizes.from_dict(entry["mixer"], where + ".mixer")
            else:
                mixer = LinearAttentionSizes.from_dict(entry["mixer"], where + ".mixer", rotates=kind == "retention")
            mlp = entry.get("mlp")
            if mlp is not None and (not isinstance(mlp, dict) or mlp.get("kind") != "moe"):
                raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'moe'")
            layers.append(NeruzenLayer(kind, mixer, None if mlp is None else MoeSizes.from_dict(mlp, where + ".mlp")))
        pair = (raw.get("embedding") or {}).get("bigram")
        bigram = None
        if pair:
            bigram = PairTable(_int(pair, "buckets", "embedding.bigram"), _int(pair, "mul_prev", "embedding.bigram", 0),
                               _int(pair, "mul_cur", "embedding.bigram", 0))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return NeruzenConfig(_int(raw, "vocab", "the model"), _int(raw, "width", "the model"), _float(norm, "eps", "norm"),
                             tuple(layers), bigram, eos_ids)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture}
        if self.bigram is not None:
            out["embedding"] = {"bigram": self.bigram.to_dict()}
        out.update({"layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width})
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
