"""Vinurax as data: its configuration turned into a ModelSpec of registered parts.

Every layer is a ``parallel_gated`` block (two Dynamic Tanh norms of the same input, a mixer beside a
dense xIELU feed-forward, sigmoid-gated results, the depth-weighted average over all results so far);
the mixer is ``latent_attention`` or ``channel_delta``. A latent-attention layer with ``kv_from`` reads
the cache slot of the layer it names. The head is the embedding table, behind a last Dynamic Tanh.
Checkpoint names: ``embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.dwa``, ``final.norm`` (+ ``.b``, ``.alpha``).
"""
from __future__ import annotations

from typing import Optional

from ..config.vinurax import VinuraxConfig
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_vinurax_spec(cfg: VinuraxConfig) -> ModelSpec:
    n = len(cfg.layers)
    layers, schedule = [], []
    for i, l in enumerate(cfg.layers):
        if l.kind == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "name": "mix", "hidden_size": cfg.width, "heads": l.heads, "dim": l.dim, "vdim": l.vdim,
                "kv_rank": l.kv_rank, "scale": l.scale, "eps": cfg.eps, "own_latents": l.kv_from is None})
            schedule.append(ScheduleEntry(layer=i, cache=i if l.kv_from is None else l.kv_from,
                                          writes_cache=l.kv_from is None))
        else:
            mixer = PartSpec("channel_delta", {
                "name": "mix", "hidden_size": cfg.width, "heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim,
                "vdim": l.vdim, "conv": l.conv, "decay_rank": l.decay_rank or l.dim, "gate_rank": l.gate_rank or l.dim,
                "eps": cfg.eps})
            schedule.append(ScheduleEntry(layer=i, cache=i))
        norm = lambda name: PartSpec("dynamic_tanh", {"name": name, "size": cfg.width})
        ffn = None if l.ff is None else PartSpec("dense_mlp", {"name": "mlp", "hidden_size": cfg.width,
                                                              "intermediate_size": l.ff, "activation": "xielu"})
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=mixer, feed_forward=ffn, norm_mixer=norm("norm1"),
            norm_feed_forward=None if ffn is None else norm("norm2"),
            arrangement=PartSpec("parallel_gated", {"hidden_size": cfg.width, "gated": True, "depth_average": True,
                                                    "results_before": i + 1, "total_results": n + 1,
                                                    "feed_forward": ffn is not None})))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": cfg.vocab, "hidden_size": cfg.width}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("dynamic_tanh", {"name": "final.norm", "size": cfg.width}),
        head=PartSpec("linear_head", {"name": "head", "vocab_size": cfg.vocab, "hidden_size": cfg.width, "tie": True}),
        eos_token_ids=cfg.eos_token_ids, max_position_embeddings=None)


def normalize_vinurax_tensor_name(name: str) -> Optional[str]:
    """The parts ask for the checkpoint's own names, but for the embedding table (``embed`` is the
    token-embedding part's ``embed.weight``)."""
    return "embed.weight" if name == "embed" else name
