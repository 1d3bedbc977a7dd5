"""Typed configuration of the Fizadra decoder, read from config.json.

Keys: `vocab`, `width`, `norm` {`eps`, `groups`}, `layers` (a list; each entry has `type`, `mixer`, the mixer's
sizes, and `mlp`, {`kind`: "dense", `ff`} or null).

Layer types "latent_attention" and "latent_attention_2" (attention over a cached latent with one turned key part
shared by all heads): {`heads`, `dim`, `rot_dim`, `vdim`, `kv_rank`, `q_rank`, `scale`, `rot`: {`base`, `dims`,
`scaling`: {`factor`, `original`, `fast`, `slow`} or absent}, `kv_from`: an earlier layer whose cached latent and key
part this layer reads instead of making its own (absent: its own)}.
Layer type "attention" (grouped queries, biases, normed heads, mixed scores): {`heads`, `kv_heads`, `dim`, `vdim`,
`scale`, `rot`: {`base`, `dims`}}.

Every size and every constant that can differ between models comes from here.  A layer kind or a feed-forward kind
the engine does not know rejects the file (it would change what is computed); other keys it does not know are named
in a warning and left alone.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Optional

from .llama import ConfigError
from .mogevik import DEFAULT_CONTEXT, _number, _positive_int

_TOP_KEYS = {"architecture", "architectures", "model_type", "torch_dtype", "dtype", "vocab", "width", "layers", "norm",
             "eos_token_id", "max_context"}
LATENT_KINDS = ("latent_attention", "latent_attention_2")
LAYER_KINDS = LATENT_KINDS + ("attention",)


def _warn_unknown(where: str, have, known) -> None:
    unknown = sorted(set(have) - set(known))
    if unknown:
        print(f"[mdma_b200] {where} has keys the Fizadra reader does not know and leaves alone: {unknown}", file=sys.stderr)


def _object(where: str, v) -> dict:
    if not isinstance(v, dict):
        raise ConfigError(f"{where} must be an object")
    return v


@dataclass(frozen=True)
class FizadraRotation:
    """`dims` numbers of a head are turned; `scaling` None or (factor, original, fast, slow)."""
    base: float
    dims: int
    scaling: Optional[tuple] = None


@dataclass(frozen=True)
class FizadraLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: FizadraRotation
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class FizadraAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: FizadraRotation


@dataclass(frozen=True)
class FizadraLayer:
    type: str
    mixer: object                 # FizadraLatent | FizadraAttention
    ff: int = 0                   # 0: the layer has no feed-forward


@dataclass(frozen=True)
class FizadraConfig:
    vocab: int
    width: int
    layers: tuple
    eps: float
    groups: int = 1
    eos_token_id: tuple = ()
    max_context: int = DEFAULT_CONTEXT

    @classmethod
    def from_dict(cls, raw: dict) -> "FizadraConfig":
        _warn_unknown("config.json", raw, _TOP_KEYS)
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        vocab, width = _positive_int("vocab", raw["vocab"]), _positive_int("width", raw["width"])
        norm = _object("norm", raw["norm"])
        _warn_unknown("norm", norm, {"eps", "groups"})
        if "eps" not in norm:
            raise ConfigError("`norm` must have `eps`")
        eps = _number("norm.eps", norm["eps"])
        if eps < 0:
            raise ConfigError(f"norm.eps must be >= 0, got {eps!r}")
        groups = _positive_int("norm.groups", norm.get("groups", 1))
        if width % groups:
            raise ConfigError(f"a row of {width} numbers does not split into {groups} equal parts")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            layers.append(cls._layer(f"layers[{i}]", entry, i, layers))
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        max_context = _positive_int("max_context", raw.get("max_context", DEFAULT_CONTEXT))
        return cls(vocab, width, tuple(layers), eps, groups, eos, max_context)

    @staticmethod
    def _rotation(where: str, raw, head: int) -> FizadraRotation:
        rot = _object(where, raw)
        _warn_unknown(where, rot, {"base", "dims", "scaling"})
        dims = _positive_int(f"{where}.dims", rot.get("dims", head))
        base = _number(f"{where}.base", rot.get("base"))
        if dims % 2 or dims > head or base <= 0:
            raise ConfigError(f"{where}: {dims} turned numbers of a head of {head} with base {base}")
        scaling = None
        s = rot.get("scaling")
        if s is not None:
            _warn_unknown(f"{where}.scaling", _object(f"{where}.scaling", s), {"factor", "original", "fast", "slow"})
            scaling = tuple(_number(f"{where}.scaling.{k}", s.get(k)) for k in ("factor", "original", "fast", "slow"))
            if min(scaling) <= 0:
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        return FizadraRotation(base, dims, scaling)

    @staticmethod
    def _layer(where: str, entry, index: int, before: list) -> FizadraLayer:
        if not isinstance(entry, dict) or "type" not in entry or "mixer" not in entry:
            raise ConfigError(f"{where} must have `type`, `mixer` and `mlp`")
        _warn_unknown(where, entry, {"type", "mixer", "mlp"})
        kind = entry["type"]
        if kind not in LAYER_KINDS:
            raise ConfigError(f"{where}.type {kind!r} is not implemented (have {sorted(LAYER_KINDS)})")
        m = _object(f"{where}.mixer", entry["mixer"])
        w = f"{where}.mixer"
        heads, dim = _positive_int(f"{w}.heads", m.get("heads")), _positive_int(f"{w}.dim", m.get("dim"))
        vdim = _positive_int(f"{w}.vdim", m.get("vdim", dim))
        if kind == "attention":
            _warn_unknown(w, m, {"heads", "kv_heads", "dim", "vdim", "scale", "rot"})
            kv_heads = _positive_int(f"{w}.kv_heads", m.get("kv_heads", heads))
            if heads % kv_heads:
                raise ConfigError(f"{w}: {heads} heads do not divide over {kv_heads} kv heads")
            scale = _number(f"{w}.scale", m.get("scale", dim ** -0.5))
            mixer = FizadraAttention(heads, kv_heads, dim, vdim, scale,
                                     FizadraConfig._rotation(f"{w}.rot", m.get("rot"), dim))
        else:
            _warn_unknown(w, m, {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot", "kv_from"})
            rot_dim = _positive_int(f"{w}.rot_dim", m.get("rot_dim"))
            kv_rank, q_rank = _positive_int(f"{w}.kv_rank", m.get("kv_rank")), _positive_int(f"{w}.q_rank", m.get("q_rank"))
            scale = _number(f"{w}.scale", m.get("scale", (dim + rot_dim) ** -0.5))
            rot = FizadraConfig._rotation(f"{w}.rot", m.get("rot"), rot_dim)
            src = m.get("kv_from")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index:
                    raise ConfigError(f"{w}.kv_from must name an earlier layer, got {src!r}")
                other = before[src]
                if (other.type not in LATENT_KINDS or other.mixer.kv_from is not None
                        or (other.mixer.kv_rank, other.mixer.rot_dim) != (kv_rank, rot_dim)):
                    raise ConfigError(f"{w}.kv_from: layer {src} keeps no latent of {kv_rank} + {rot_dim} numbers of its own")
            mixer = FizadraLatent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot, src)
        ff = 0
        mlp = entry.get("mlp")
        if mlp is not None:
            _warn_unknown(f"{where}.mlp", _object(f"{where}.mlp", mlp), {"kind", "ff"})
            if mlp.get("kind") != "dense":
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not implemented (have ['dense'])")
            ff = _positive_int(f"{where}.mlp.ff", mlp.get("ff"))
        return FizadraLayer(kind, mixer, ff)
