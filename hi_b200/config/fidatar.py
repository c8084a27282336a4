"""Typed configuration of the Fidatar decoder: post-norm layers, each with one of two mixers (attention
over a chunked, paged cache with a sink term in its softmax, or the mLSTM matrix memory) and a dense or
routed feed-forward, or none.

config.json keys: ``architecture`` ("Fidatar"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``
(default 1), ``postln_alpha`` (default 1), ``logit_softcap`` (optional), and ``layers``: a list of
``{"type": "attention" | "mlstm", "mixer": {...}, "mlp": {...} | null}``.

Mixer keys. attention: ``heads, kv_heads, dim, vdim, scale``; optionally ``mask.size`` (a query sees the
keys of its own block of that many positions; absent: every earlier key) and ``rot`` with ``base, dims``
and optionally ``scaling`` = ``{factor, original, fast, slow}``. mlstm: ``heads, dim, vdim, gate_cap``.

mlp: ``{"kind": "dense", "ff": n}`` or ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts", "top",
"scale", "groups": {"count", "keep"}}}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, get_key, token_ids

MIXERS = ("attention", "mlstm")


@dataclass(frozen=True)
class FidatarRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow


@dataclass(frozen=True)
class FidatarFeedForward:
    kind: str                        # "dense" | "moe"
    ff: int                          # intermediate size (of every expert, for "moe")
    experts: int = 0
    top: int = 0
    score_scale: float = 1.0
    groups: Optional[Tuple[int, int]] = None      # (count, keep)


@dataclass(frozen=True)
class FidatarLayer:
    kind: str
    heads: int
    dim: int
    vdim: int
    mlp: Optional[FidatarFeedForward]
    # attention
    kv_heads: int = 0
    scale: float = 0.0
    chunk: Optional[int] = None
    rot: Optional[FidatarRotation] = None
    # mlstm
    gate_cap: float = 0.0


@dataclass(frozen=True)
class FidatarConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    alpha: float
    logit_softcap: Optional[float]
    layers: Tuple[FidatarLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = ("Fidatar",)

    @staticmethod
    def from_json(raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "FidatarConfig":
        def obj(parent, key, where, required=True):
            value = parent.get(key)
            if value is None and not required:
                return None
            if not isinstance(value, dict):
                raise ConfigError(f"config.json: required key '{where}' is missing or not an object")
            return value

        def need(parent, key, typ, where):
            try:
                return get_key(parent, key, typ, required=True)
            except ConfigError as e:
                raise ConfigError(str(e).replace("key '", f"key '{where}.")) from None

        vocab = get_key(raw, "vocab", int, required=True)
        width = get_key(raw, "width", int, required=True)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = need(obj(raw, "norm", "norm"), "eps", float, "norm")
        emb = obj(raw, "embedding", "embedding", required=False) or {}
        embedding_scale = get_key(emb, "scale", float, default=1.0)
        alpha = get_key(raw, "postln_alpha", float, default=1.0)
        softcap = get_key(raw, "logit_softcap", float)
        if softcap is not None and not softcap > 0:
            raise ConfigError("config.json: 'logit_softcap' must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and a 'mixer' object")
            kind, m = entry.get("type"), entry["mixer"]
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type is {kind!r}; known mixers: {MIXERS}")
            mw = f"{where}.mixer"
            heads, dim, vdim = (need(m, k, int, mw) for k in ("heads", "dim", "vdim"))
            if min(heads, dim, vdim) <= 0:
                raise ConfigError(f"config.json: {mw} sizes must be positive")
            mlp = _feed_forward(entry.get("mlp"), f"{where}.mlp", need, obj)
            if kind == "attention":
                kv_heads = need(m, "kv_heads", int, mw)
                if kv_heads <= 0 or heads % kv_heads:
                    raise ConfigError(f"config.json: {mw}.heads must be a multiple of kv_heads")
                scale = get_key(m, "scale", float)
                mask = obj(m, "mask", f"{mw}.mask", required=False)
                chunk = need(mask, "size", int, f"{mw}.mask") if mask else None
                if chunk is not None and chunk <= 0:
                    raise ConfigError(f"config.json: {mw}.mask.size must be positive")
                rot_raw, rot = obj(m, "rot", f"{mw}.rot", required=False), None
                if rot_raw:
                    rw = f"{mw}.rot"
                    dims, base = need(rot_raw, "dims", int, rw), need(rot_raw, "base", float, rw)
                    if dims <= 0 or dims % 2 or dims > dim or not base > 1.0:
                        raise ConfigError(f"config.json: {rw}.dims must be even and at most dim, base above 1")
                    sc_raw, scaling = obj(rot_raw, "scaling", f"{rw}.scaling", required=False), None
                    if sc_raw:
                        scaling = tuple(need(sc_raw, k, float, f"{rw}.scaling") for k in ("factor", "original", "fast", "slow"))
                        if min(scaling) <= 0:
                            raise ConfigError(f"config.json: {rw}.scaling values must be positive")
                    rot = FidatarRotation(base=base, dims=dims, scaling=scaling)
                layers.append(FidatarLayer(kind, heads, dim, vdim, mlp, kv_heads=kv_heads,
                                           scale=dim ** -0.5 if scale is None else scale, chunk=chunk, rot=rot))
            else:
                cap = need(m, "gate_cap", float, mw)
                if not cap > 0:
                    raise ConfigError(f"config.json: {mw}.gate_cap must be positive")
                layers.append(FidatarLayer(kind, heads, dim, vdim, mlp, gate_cap=cap))
        eos = token_ids(raw, "eos_token_id") or (token_ids(generation, "eos_token_id") if generation else [])
        return FidatarConfig(vocab=vocab, width=width, eps=eps, embedding_scale=embedding_scale, alpha=alpha,
                             logit_softcap=softcap, layers=tuple(layers), eos_token_ids=tuple(eos))


def _feed_forward(mlp, where, need, obj) -> Optional[FidatarFeedForward]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}.kind must be 'dense' or 'moe' (or mlp null)")
    if mlp["kind"] == "dense":
        ff = need(mlp, "ff", int, where)
        if ff <= 0:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return FidatarFeedForward("dense", ff)
    ff = need(obj(mlp, "expert", f"{where}.expert"), "ff", int, f"{where}.expert")
    router = obj(mlp, "router", f"{where}.router")
    rw = f"{where}.router"
    experts, top = need(router, "experts", int, rw), need(router, "top", int, rw)
    if ff <= 0 or experts <= 0 or not 0 < top <= experts:
        raise ConfigError(f"config.json: {where}: sizes must be positive and router.top at most router.experts")
    groups_raw, groups = obj(router, "groups", f"{rw}.groups", required=False), None
    if groups_raw:
        count, keep = need(groups_raw, "count", int, f"{rw}.groups"), need(groups_raw, "keep", int, f"{rw}.groups")
        if count <= 0 or experts % count or not 0 < keep <= count or top > keep * (experts // count):
            raise ConfigError(f"config.json: {rw}.groups: {experts} experts do not form {count} equal groups of which "
                              f"{keep} hold {top} choices")
        groups = (count, keep)
    return FidatarFeedForward("moe", ff, experts=experts, top=top, score_scale=get_key(router, "scale", float, default=1.0),
                              groups=groups)
