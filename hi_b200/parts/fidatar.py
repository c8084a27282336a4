"""Fidatar as data: its configuration turned into a ModelSpec of registered parts.

Every layer is a ``postnorm`` block (x <- norm(alpha x + sub-layer(x)) after the mixer and after the
feed-forward). The mixer is ``attention`` (grouped heads over a chunked paged cache, biases on q/k/v, a
weighted RMS norm of q and k before a partial rotation with ramped frequency scaling, a sink term in the
softmax) or ``mlstm``. The feed-forward is ``dense_mlp`` with the squared relu, or ``routed_experts``
without a gate branch or a shared expert, chosen within the best groups and weighted by scaled sigmoid
scores. The embedding is multiplied by a constant; the logits pass a soft cap.
Checkpoint names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from ..config.fidatar import FidatarConfig
from .spec import LayerSpec, ModelSpec, PartSpec


def build_fidatar_spec(cfg: FidatarConfig) -> ModelSpec:
    layers = []
    for i, l in enumerate(cfg.layers):
        if l.kind == "attention":
            position = None
            if l.rot is not None:
                scaling = None if l.rot.scaling is None else dict(zip(("factor", "original", "fast", "slow"), l.rot.scaling))
                position = PartSpec("rope_yarn", {"head_dim": l.dim, "dims": l.rot.dims, "base": l.rot.base,
                                                  "scaling": scaling})
            mixer = PartSpec("attention", {
                "name": "mix", "hidden_size": cfg.width, "num_heads": l.heads, "num_kv_heads": l.kv_heads,
                "head_dim": l.dim, "value_dim": l.vdim, "window": ("chunk", l.chunk) if l.chunk else None,
                "position": position, "qk_norm_weighted": True, "qk_norm_eps": cfg.eps, "scale": l.scale,
                "bias": "qkv", "sink": True, "names": "short"})
        else:
            mixer = PartSpec("mlstm", {"name": "mix", "hidden_size": cfg.width, "heads": l.heads, "dim": l.dim,
                                       "vdim": l.vdim, "gate_cap": l.gate_cap, "eps": cfg.eps})
        ffn = None
        if l.mlp is not None and l.mlp.kind == "dense":
            ffn = PartSpec("dense_mlp", {"name": "mlp", "hidden_size": cfg.width, "intermediate_size": l.mlp.ff,
                                         "activation": "relu2"})
        elif l.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "name": "mlp", "hidden_size": cfg.width, "num_experts": l.mlp.experts, "top_k": l.mlp.top,
                "intermediate_size": l.mlp.ff, "shared_expert": False, "score": "sigmoid", "renormalize": False,
                "scale": "output", "activation": "relu2", "groups": l.mlp.groups, "score_scale": l.mlp.score_scale,
                "names": "per_expert"})
        norm = lambda name: PartSpec("rmsnorm", {"name": name, "size": cfg.width, "eps": cfg.eps, "tensor": "bare"})
        layers.append(LayerSpec(prefix=f"l{i}", mixer=mixer, feed_forward=ffn, norm_mixer=norm("norm1"),
                                norm_feed_forward=None if ffn is None else norm("norm2"),
                                arrangement=PartSpec("postnorm", {"alpha": cfg.alpha})))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)),
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "size": cfg.width, "eps": cfg.eps, "tensor": "bare"}),
        head=PartSpec("linear_head", {"name": "head", "vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                      "softcap": cfg.logit_softcap, "tensor": "head"}),
        eos_token_ids=cfg.eos_token_ids, max_position_embeddings=None)


def normalize_fidatar_tensor_name(name: str) -> Optional[str]:
    """The parts ask for the checkpoint's own names, but for the embedding table (``embed`` is the
    token-embedding part's ``embed.weight``)."""
    return "embed.weight" if name == "embed" else name
