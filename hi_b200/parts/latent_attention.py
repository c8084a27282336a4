"""Latent attention: the cache holds one low-rank latent per token; every head's keys and values are
linear maps of it."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .attention import attend_over_pages
from .basic import Part
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "latent_attention")
class LatentAttentionMixer(Part):
    """q = W_q h [heads, dim];  c = rmsnorm(W_dkv h) * w_c  [rank], the only thing cached;
    per head a: k_a = U_a c, v_a = V_a c;  o_a = softmax_j(q_a . k_a(j) * scale) v_a(j) over j <= i;
    o_a *= sigmoid(W_g h)_a;  out = W_o concat(o_a).  No position encoding.

    Computed on the latents: q_a . (U_a c) = (U_a^T q_a) . c and sum_j p_j V_a c_j = V_a (sum_j p_j c_j), so
    the step's queries are mapped into latent space (one batched product), attention runs over the paged
    latents with one shared "kv head" whose keys and values are the same rows (the paged attention kernels
    of the other mixers), and the result is mapped out by V_a (another batched product). The cached rows are
    padded to a multiple of 16 elements with zeros, which changes no dot product.

    A mixer with ``kv_source`` makes no latents: its schedule entry reads the cache slot of the layer that
    does (``writes_cache=False``), with its own U, V, queries and everything else.

    params: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``, ``eps`` (of the latent's
    norm), ``own_latents`` (False for a layer that reads another's), ``window`` (None | ("sliding", W) |
    ("chunk", C): which earlier latents a query reads; default all).
    tensors: ``<prefix>.q`` [heads*dim, H], ``<prefix>.dkv`` [rank, H] and ``<prefix>.dkv.norm`` [rank] (own
    latents only), ``<prefix>.uk`` [heads*dim, rank], ``<prefix>.uv`` [heads*vdim, rank], ``<prefix>.g``
    [heads, H], ``<prefix>.o`` [H, heads*vdim].
    """

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.dim ** -0.5
        self.eps = float(p["eps"])
        self.own = bool(p.get("own_latents", True))
        self.window = tuple(p["window"]) if p.get("window") else None
        self.row_len = -(-self.rank // 16) * 16
        if self.row_len > 512:
            raise ValueError(f"{prefix}: kv_rank {self.rank} is not supported (up to 512)")
        self.w_in = self.w_c = self.w_uk_t = self.w_uv_t = self.w_o = None

    def cache_spec(self):
        return CacheSpec(kv_heads=1, head_dim=self.row_len, window=self.window, values=False)

    def tensor_specs(self):
        h, hd, hv, r = self.hidden, self.heads * self.dim, self.heads * self.vdim, self.rank
        specs = [TensorSpec(f"{self.prefix}.q", (hd, h))]
        if self.own:
            specs += [TensorSpec(f"{self.prefix}.dkv", (r, h)), TensorSpec(f"{self.prefix}.dkv.norm", (r,), init="ones")]
        return specs + [TensorSpec(f"{self.prefix}.uk", (hd, r)), TensorSpec(f"{self.prefix}.uv", (hv, r)),
                        TensorSpec(f"{self.prefix}.g", (self.heads, h)), TensorSpec(f"{self.prefix}.o", (h, hv))]

    def load(self, fetch):
        q, g = fetch(f"{self.prefix}.q"), fetch(f"{self.prefix}.g")
        parts = [q, g]
        if self.own:
            parts.append(fetch(f"{self.prefix}.dkv"))
            self.w_c = fetch(f"{self.prefix}.dkv.norm").to(q.dtype).contiguous()
        # one product for the queries, the gates and (own latents) the down projection: [q | g | dkv]
        self.w_in = torch.cat([t.to(q.dtype) for t in parts], dim=0).contiguous()
        pad = self.row_len - self.rank
        uk = fetch(f"{self.prefix}.uk").view(self.heads, self.dim, self.rank)
        uv = fetch(f"{self.prefix}.uv").view(self.heads, self.vdim, self.rank)
        if pad:
            uk = torch.nn.functional.pad(uk, (0, pad))
            uv = torch.nn.functional.pad(uv, (0, pad))
        self.w_uk = uk.contiguous()                              # [heads, dim, row_len]: q_a -> latent space
        self.w_uv_t = uv.transpose(1, 2).contiguous()            # [heads, row_len, vdim]: latent space -> o_a
        self.w_o = fetch(f"{self.prefix}.o").contiguous()

    def forward(self, normed, ctx, cache):
        n, hd = normed.shape[0], self.heads * self.dim
        proj = linear(normed, self.w_in)
        block_table = ctx.block_tables[cache.group]
        if self.own != cache.writes:
            raise RuntimeError(f"{self.prefix}: a layer with its own latents writes its cache slot, another reads one")
        if self.own:
            ops.latent_append(proj[:, hd + self.heads:], self.w_c, self.eps, ctx.positions, ctx.seq_of_token, block_table,
                              cache.k_pages)
        # queries into latent space, head by head: [heads, N, dim] x [heads, dim, row_len]
        q_lat = torch.empty((n, self.heads, self.row_len), dtype=proj.dtype, device=proj.device)
        torch.bmm(proj[:, :hd].view(n, self.heads, self.dim).transpose(0, 1), self.w_uk, out=q_lat.transpose(0, 1))
        chunk = self.window[1] if self.window and self.window[0] == "chunk" else 0
        sliding = self.window[1] if self.window and self.window[0] == "sliding" else 0
        o_lat = attend_over_pages(q_lat, cache.k_pages, cache.k_pages, block_table, ctx, self.heads, 1, self.row_len,
                                  chunk, sliding, self.scale)
        o = torch.empty((n, self.heads, self.vdim), dtype=proj.dtype, device=proj.device)
        torch.bmm(o_lat.transpose(0, 1), self.w_uv_t, out=o.transpose(0, 1))
        o = ops.head_gate(o, proj[:, hd: hd + self.heads])
        return linear(o.view(n, self.heads * self.vdim), self.w_o)
