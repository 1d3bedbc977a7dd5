"""Typed configuration of the Tubusun decoder, read from config.json.

Keys: `vocab`, `width`, `embedding.scale`, `norm.eps`, `logit_softcap`, `layers` (a list; each entry has
`type`, `mixer`, the mixer's sizes, and `mlp`, the feed-forward's description or null), `loop` (`start`,
`stop`, `times`: layers start..stop-1 run `times` times in a row; absent or null: no loop).

Mixer `parallel`: {`left`, `right`, `left_scale`, `right_scale`}, two mixers that read the same rows.
  left  (softmax attention over a sliding window): {`heads`, `kv_heads`, `dim`, `vdim`, `scale`,
        `mask`: {`size`} (absent or null: every earlier token is seen), `rot`: {`base`, `dims`} (absent or
        null, or dims 0: no rotation)}
  right (linear attention with a decay per head): {`heads`, `dim`, `vdim`, `decay`: one number per head}
Feed-forward: {`kind`: "dense", `ff`} or {`kind`: "moe", `expert`: {`ff`, `limit`}, `router`: {`experts`,
`top`, `groups`: {`count`, `keep`} or null}}.

Every size and every constant that can differ between models comes from here.  A layer kind or a
feed-forward kind the engine does not know rejects the file (it would change what is computed); other
keys it does not know are named in a warning and left alone.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Optional

from .llama import ConfigError
from .mogevik import DEFAULT_CONTEXT, _count, _number, _positive_int

_TOP_KEYS = {"architecture", "architectures", "model_type", "torch_dtype", "dtype", "vocab", "width", "layers", "loop",
             "norm", "embedding", "eos_token_id", "max_context", "logit_softcap"}


def _warn_unknown(where: str, have, known) -> None:
    unknown = sorted(set(have) - set(known))
    if unknown:
        print(f"[mdma_b200] {where} has keys the Tubusun reader does not know and leaves alone: {unknown}", file=sys.stderr)


def _object(where: str, v) -> dict:
    if not isinstance(v, dict):
        raise ConfigError(f"{where} must be an object")
    return v


@dataclass(frozen=True)
class TubusunWindowed:
    """The softmax attention of a pair: `window` 0 means none, `rot_dims` 0 no rotation."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class TubusunLinear:
    heads: int
    dim: int
    vdim: int
    decay: tuple


@dataclass(frozen=True)
class TubusunPair:
    left: TubusunWindowed
    right: TubusunLinear
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class TubusunFeedForward:
    """`kind` "dense": `ff`.  `kind` "moe": `experts` experts of `ff`, `top` per token, in `groups` groups of
    which `keep` can be chosen from; `limit` bounds the experts' two products."""
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class TubusunLayer:
    type: str
    mixer: TubusunPair
    mlp: Optional[TubusunFeedForward]


@dataclass(frozen=True)
class TubusunConfig:
    vocab: int
    width: int
    layers: tuple
    eps: float
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0    # 0: none
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0           # 0: no loop
    eos_token_id: tuple = ()
    max_context: int = DEFAULT_CONTEXT

    @classmethod
    def from_dict(cls, raw: dict) -> "TubusunConfig":
        _warn_unknown("config.json", raw, _TOP_KEYS)
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        vocab, width = _positive_int("vocab", raw["vocab"]), _positive_int("width", raw["width"])
        norm = raw["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("`norm` must be {\"eps\": number}")
        eps = _number("norm.eps", norm["eps"])
        if eps < 0:
            raise ConfigError(f"norm.eps must be >= 0, got {eps!r}")
        scale = 1.0
        emb = raw.get("embedding")
        if emb is not None:
            _warn_unknown("embedding", _object("embedding", emb), {"scale"})
            if emb.get("scale") is not None:
                scale = _number("embedding.scale", emb["scale"])
        cap = raw.get("logit_softcap")
        cap = 0.0 if cap is None else _number("logit_softcap", cap)
        if cap < 0:
            raise ConfigError(f"logit_softcap must be positive (or absent), got {cap!r}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        layers = tuple(cls._layer(f"layers[{i}]", entry) for i, entry in enumerate(raw["layers"]))
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not {"start", "stop", "times"} <= set(loop):
                raise ConfigError("`loop` must be null or have `start`, `stop` and `times`")
            start, stop, times = (_count(f"loop.{k}", loop[k]) for k in ("start", "stop", "times"))
            if not (0 <= start < stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop {loop} does not name a run of the {len(layers)} layers at least once")
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        max_context = _positive_int("max_context", raw.get("max_context", DEFAULT_CONTEXT))
        return cls(vocab, width, layers, eps, scale, cap, start, stop, times, eos, max_context)

    @staticmethod
    def _layer(where: str, entry) -> TubusunLayer:
        if not isinstance(entry, dict) or "type" not in entry or "mixer" not in entry:
            raise ConfigError(f"{where} must have `type`, `mixer` and `mlp`")
        _warn_unknown(where, entry, {"type", "mixer", "mlp"})
        kind = entry["type"]
        if kind != "parallel":
            raise ConfigError(f"{where}.type {kind!r} is not implemented (have ['parallel'])")
        m = _object(f"{where}.mixer", entry["mixer"])
        _warn_unknown(f"{where}.mixer", m, {"left", "right", "left_scale", "right_scale"})
        if "left" not in m or "right" not in m:
            raise ConfigError(f"{where}.mixer must have `left` and `right`")
        pair = TubusunPair(TubusunConfig._left(f"{where}.mixer.left", _object(f"{where}.mixer.left", m["left"])),
                           TubusunConfig._right(f"{where}.mixer.right", _object(f"{where}.mixer.right", m["right"])),
                           _number(f"{where}.mixer.left_scale", m.get("left_scale", 1.0)),
                           _number(f"{where}.mixer.right_scale", m.get("right_scale", 1.0)))
        return TubusunLayer(kind, pair, TubusunConfig._mlp(f"{where}.mlp", entry.get("mlp")))

    @staticmethod
    def _left(where: str, raw: dict) -> TubusunWindowed:
        _warn_unknown(where, raw, {"heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"})
        heads, dim = _positive_int(f"{where}.heads", raw.get("heads")), _positive_int(f"{where}.dim", raw.get("dim"))
        kv_heads = _positive_int(f"{where}.kv_heads", raw.get("kv_heads", heads))
        vdim = _positive_int(f"{where}.vdim", raw.get("vdim", dim))
        scale = _number(f"{where}.scale", raw.get("scale", dim ** -0.5))
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads do not divide over {kv_heads} kv heads")
        window = 0
        mask = raw.get("mask")
        if mask is not None:
            _warn_unknown(f"{where}.mask", _object(f"{where}.mask", mask), {"size"})
            if mask.get("size") is not None:
                window = _positive_int(f"{where}.mask.size", mask["size"])
        rot_dims, rot_base = 0, 10000.0
        rot = raw.get("rot")
        if rot is not None:
            _warn_unknown(f"{where}.rot", _object(f"{where}.rot", rot), {"base", "dims"})
            rot_dims = _count(f"{where}.rot.dims", rot.get("dims", dim))
            if rot_dims:
                rot_base = _number(f"{where}.rot.base", rot.get("base"))
                if rot_dims % 2 or rot_dims > dim or rot_base <= 0:
                    raise ConfigError(f"{where}.rot: {rot_dims} rotated numbers of a head of {dim} with base {rot_base}")
        return TubusunWindowed(heads, kv_heads, dim, vdim, scale, window, rot_dims, rot_base)

    @staticmethod
    def _right(where: str, raw: dict) -> TubusunLinear:
        _warn_unknown(where, raw, {"heads", "dim", "vdim", "decay"})
        heads, dim = _positive_int(f"{where}.heads", raw.get("heads")), _positive_int(f"{where}.dim", raw.get("dim"))
        vdim = _positive_int(f"{where}.vdim", raw.get("vdim", dim))
        decay = raw.get("decay")
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * heads
        if not isinstance(decay, list) or len(decay) != heads:
            raise ConfigError(f"{where}.decay must give one number per head ({heads})")
        return TubusunLinear(heads, dim, vdim, tuple(_number(f"{where}.decay[{i}]", d) for i, d in enumerate(decay)))

    @staticmethod
    def _mlp(where: str, raw) -> Optional[TubusunFeedForward]:
        if raw is None:
            return None
        kind = _object(where, raw).get("kind")
        if kind == "dense":
            _warn_unknown(where, raw, {"kind", "ff"})
            return TubusunFeedForward("dense", _positive_int(f"{where}.ff", raw.get("ff")))
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r} is not implemented (have ['dense', 'moe'])")
        _warn_unknown(where, raw, {"kind", "expert", "router"})
        expert, router = raw.get("expert"), raw.get("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise ConfigError(f"{where} must have `expert` and `router`")
        _warn_unknown(f"{where}.expert", expert, {"ff", "limit"})
        _warn_unknown(f"{where}.router", router, {"experts", "top", "groups"})
        ff = _positive_int(f"{where}.expert.ff", expert.get("ff"))
        limit = _number(f"{where}.expert.limit", expert.get("limit"))
        if limit <= 0:
            raise ConfigError(f"{where}.expert.limit must be positive, got {limit!r}")
        experts = _positive_int(f"{where}.router.experts", router.get("experts"))
        top = _positive_int(f"{where}.router.top", router.get("top"))
        if top > experts:
            raise ConfigError(f"{where}: top {top} of {experts} experts")
        count = keep = 1
        groups = router.get("groups")
        if groups is not None:
            _warn_unknown(f"{where}.router.groups", _object(f"{where}.router.groups", groups), {"count", "keep"})
            count = _positive_int(f"{where}.router.groups.count", groups.get("count"))
            keep = _positive_int(f"{where}.router.groups.keep", groups.get("keep", count))
            if experts % count or keep > count:
                raise ConfigError(f"{where}: {experts} experts do not form {count} groups of which {keep} are kept")
        return TubusunFeedForward("moe", ff, limit, experts, top, count, keep)
