"""The mLSTM mixer: a matrix memory per head with exponential gates, a fixed-size state per request
instead of a cache that grows."""
from __future__ import annotations

import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "mlstm")
class MLSTMMixer(Part):
    """Per head a matrix S [dim, vdim], a vector n [dim] and a running maximum m (all zero at a sequence's
    start), updated and read by every token:

        q = W_q h * dim^-1/2, k = W_k h [heads, dim];  v = W_v h [heads, vdim]
        i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))     per head
        m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' = e^(f + m - m') n + e^(i - m') k
        o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
        y = o / rms_vdim(o) * w_norm * sigmoid(W_g h);  out = W_o y

    The gates, the maximum, the state and the read-out are float32 in every mode (``ops.mlstm_gates``,
    ``ops.mlstm_recurrence``, ``ops.mlstm_out_norm``); the gates' pre-activations come out of their
    product in float32. State per request: one float32 row (S column by column, n, m).

    params: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``gate_cap``, ``eps`` (of the output norm).
    tensors: ``<prefix>.{q,k}`` [heads*dim, H], ``<prefix>.{v,g}`` [heads*vdim, H], ``<prefix>.{i,f}`` [heads, H]
    with ``.b`` [heads], ``<prefix>.norm`` [heads*vdim], ``<prefix>.o`` [H, heads*vdim]."""

    graph_safe = True
    ROWS_PER_LANE = 0            # tests: force a layout of the recurrence kernel (0: chosen by dim)

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        if min(self.heads, self.dim, self.vdim) <= 0 or not self.cap > 0:
            raise ValueError(f"{prefix}: heads, sizes and the gate cap must be positive")
        if self.dim > 1024:
            raise ValueError(f"{prefix}: a key size of {self.dim} is not supported (up to 1024)")
        self.w_in = self.w_gates = self.b_i = self.b_f = self.w_norm = self.w_o = None

    def cache_spec(self):
        return CacheSpec(state_shape=(ops.mlstm_state_floats(self.heads, self.dim, self.vdim),), state_dtype="float32")

    def tensor_specs(self):
        h, pre = self.hidden, self.prefix
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        return [TensorSpec(f"{pre}.q", (hd, h)), TensorSpec(f"{pre}.k", (hd, h)), TensorSpec(f"{pre}.v", (hv, h)),
                TensorSpec(f"{pre}.g", (hv, h)), TensorSpec(f"{pre}.o", (h, hv)),
                TensorSpec(f"{pre}.norm", (hv,), init="ones"),
                TensorSpec(f"{pre}.i", (self.heads, h)), TensorSpec(f"{pre}.i.b", (self.heads,)),
                TensorSpec(f"{pre}.f", (self.heads, h)), TensorSpec(f"{pre}.f.b", (self.heads,))]

    def load(self, fetch):
        pre = self.prefix
        rows = [fetch(f"{pre}.{n}") for n in ("q", "k", "v", "g")]
        dt = rows[0].dtype
        self.w_in = torch.cat([t.to(dt) for t in rows], dim=0).contiguous()     # one product: [q | k | v | gate]
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        self.off_k, self.off_v, self.off_g = hd, 2 * hd, 2 * hd + hv
        self.w_gates = torch.cat([fetch(f"{pre}.i").to(dt), fetch(f"{pre}.f").to(dt)], dim=0).contiguous()
        self.b_i = fetch(f"{pre}.i.b").to(torch.float32).contiguous()
        self.b_f = fetch(f"{pre}.f.b").to(torch.float32).contiguous()
        self.w_norm = fetch(f"{pre}.norm").to(dt).contiguous()
        self.w_o = fetch(f"{pre}.o").contiguous()

    def forward(self, normed, ctx, cache):
        if cache.state is None or not cache.writes:
            raise RuntimeError(f"{self.prefix}: the recurrent mixer needs a state slot of its own")
        proj = linear(normed, self.w_in)
        z = linear(normed, self.w_gates, out_dtype=torch.float32)
        keep, take, floor = ops.mlstm_gates(z, self.b_i, self.b_f, self.cap, cache.state, ctx.cu_seqlens, ctx.slots,
                                            self.heads, self.dim, self.vdim)
        o, nq = ops.mlstm_recurrence(proj, 0, self.off_k, self.off_v, self.dim ** -0.5, keep, take, cache.state,
                                     ctx.cu_seqlens, ctx.slots, self.heads, self.dim, self.vdim, self.ROWS_PER_LANE)
        y = ops.mlstm_out_norm(o, nq, floor, proj, self.off_g, self.w_norm, self.eps, proj.dtype)
        return linear(y, self.w_o)
