"""Typed configuration of the Vinurax decoder: a list of layers, each with one of two mixers
(latent attention over a cached low-rank latent, or the channel-wise gated delta rule) beside an
optional dense feed-forward, Dynamic Tanh norms, gated residuals and a depth-weighted average.

config.json keys: ``architecture`` ("Vinurax"), ``vocab``, ``width``, ``norm.eps``, and ``layers``: a list
of ``{"type": "latent_attention" | "channel_delta", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}``.
Mixer keys: latent attention ``heads, dim, vdim, kv_rank, scale`` and optionally ``kv_from`` (the layer
whose latents it reads); channel delta ``heads, kv_heads, dim, vdim, conv``. The inner sizes of the delta
mixer's two low-rank maps are not in config.json: the checkpoint's tensor shapes give them
(:func:`sizes_from_tensors`); a configuration without a checkpoint (random weights) may name them as
``decay_rank`` / ``gate_rank`` and otherwise gets ``dim``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, get_key

MIXERS = ("latent_attention", "channel_delta")


@dataclass(frozen=True)
class VinuraxLayer:
    kind: str
    heads: int
    dim: int
    vdim: int
    ff: Optional[int]                 # None: the layer has no feed-forward
    # latent attention
    kv_rank: int = 0
    scale: float = 0.0
    kv_from: Optional[int] = None
    # channel delta
    kv_heads: int = 0
    conv: int = 0
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class VinuraxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[VinuraxLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = ("Vinurax",)

    @staticmethod
    def from_json(raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "VinuraxConfig":
        vocab = get_key(raw, "vocab", int, required=True)
        width = get_key(raw, "width", int, required=True)
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: required key 'norm' (with 'eps') is missing")
        eps = get_key(norm, "eps", float, required=True)
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and a 'mixer' object")
            kind, m = entry.get("type"), entry["mixer"]
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type is {kind!r}; known mixers: {MIXERS}")

            def need(key, typ=int):
                try:
                    return get_key(m, key, typ, required=True)
                except ConfigError as e:
                    raise ConfigError(str(e).replace("key '", f"key '{where}.mixer.")) from None

            mlp, ff = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null)")
                ff = get_key(mlp, "ff", int, required=True)
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
            common = dict(kind=kind, heads=need("heads"), dim=need("dim"), vdim=need("vdim"), ff=ff)
            if min(common["heads"], common["dim"], common["vdim"]) <= 0:
                raise ConfigError(f"config.json: {where}.mixer sizes must be positive")
            if kind == "latent_attention":
                src = get_key(m, "kv_from", int)
                scale = get_key(m, "scale", float)          # the usual dim^-1/2 where the config names none
                layer = VinuraxLayer(**common, kv_rank=need("kv_rank"), kv_from=src,
                                     scale=common["dim"] ** -0.5 if scale is None else scale)
                if layer.kv_rank <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.kv_rank must be positive")
                if src is not None:
                    if not 0 <= src < i or layers[src].kind != "latent_attention" or layers[src].kv_from is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from = {src} must name an earlier "
                                          f"latent_attention layer that makes its own latents")
                    if layers[src].kv_rank != layer.kv_rank:
                        raise ConfigError(f"config.json: {where}.mixer.kv_rank differs from layer {src}'s, whose latents it reads")
            else:
                layer = VinuraxLayer(**common, kv_heads=need("kv_heads"), conv=need("conv"),
                                     decay_rank=get_key(m, "decay_rank", int), gate_rank=get_key(m, "gate_rank", int))
                if layer.kv_heads <= 0 or layer.heads % layer.kv_heads:
                    raise ConfigError(f"config.json: {where}.mixer.heads must be a multiple of kv_heads")
                if layer.conv < 1:
                    raise ConfigError(f"config.json: {where}.mixer.conv must be at least 1")
            layers.append(layer)
        from .base import token_ids

        eos = token_ids(raw, "eos_token_id") or (token_ids(generation, "eos_token_id") if generation else [])
        return VinuraxConfig(vocab=vocab, width=width, eps=eps, layers=tuple(layers), eos_token_ids=tuple(eos))


def sizes_from_tensors(cfg: VinuraxConfig, shapes: Dict[str, tuple]) -> VinuraxConfig:
    """The sizes that only the checkpoint gives: the inner sizes of each delta mixer's low-rank decay and
    gate maps, read off ``l<i>.mix.a1`` and ``l<i>.mix.g1`` ([rank, width])."""
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        if layer.kind != "channel_delta":
            continue
        a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
        layers[i] = replace(layer, decay_rank=int(a1[0]) if a1 else layer.decay_rank,
                            gate_rank=int(g1[0]) if g1 else layer.gate_rank)
    return replace(cfg, layers=tuple(layers))
