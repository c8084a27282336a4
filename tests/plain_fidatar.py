"""A plain, slow statement of the Fidatar decoder: one function per mechanism, written from the
equations, on the CPU in float64 (or float32). It shares no code with hi_b200's parts or kernels.

Notation: ``h`` [T, width] is what a sub-layer reads, ``w`` a dict of the checkpoint's tensors
(linear weights [out, in], applied as ``h @ W.T``), ``p`` a prefix such as ``l3.mix``, ``m`` the
layer's ``mixer`` object of config.json.

The layer is post-norm: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)).

Every function that carries something from one portion of a sequence to the next takes and returns it
explicitly, so token-by-token and portion-by-portion runs of the oracle can be held against its
whole-sequence run.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# --------------------------------------------------------------------------- rotary angles
def rotary_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """(frequency of every pair [dims/2], factor on cos and sin). Pair i turns by p * base^(-2i/dims) per
    position p; with ``scaling`` the slow pairs (long wavelengths) are slowed by ``factor``, the fast
    ones stay, a linear ramp over the pair index lies between, and cos/sin grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_index_of(turns):           # the (fractional) pair whose wavelength fits `turns` times into `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_index_of(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, dim]: element i of the first ``dims`` pairs with element i + dims/2; the rest pass."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f, grow = rotary_frequencies(rot)
    a = positions.to(torch.float64)[:, None] * f[None, :]                  # [T, half]
    c, s = (torch.cos(a) * grow).to(x.dtype)[:, None, :], (torch.sin(a) * grow).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- attention
def attention_keys_values(h, positions, w, p, m, eps):
    """Keys (normed, rotated) [T, G, dim] and values [T, G, vdim] of the tokens ``h`` at ``positions``."""
    g, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).view(t, g, dim)
    v = (h @ w[p + ".v"].T + w[p + ".v.b"]).view(t, g, vdim)
    k = rotate(rms(k, eps) * w[p + ".k.norm"], positions, m.get("rot"))
    return k, v


def sink_softmax_attention(q, k, v, q_pos, k_pos, scale: float, chunk: Optional[int]) -> torch.Tensor:
    """q [T, H, dim] at ``q_pos``; k [S, G, dim], v [S, G, vdim] at ``k_pos``. Query i sees key j iff
    j <= i and both lie in the same block of ``chunk`` positions. The weights are
    exp(s_j) / (1 + sum_j exp(s_j)): one more term of score 0 in the denominator, with no value."""
    t, heads, _ = q.shape
    g = k.shape[1]
    out = torch.zeros(t, heads, v.shape[2], dtype=q.dtype)
    for a in range(heads):
        b = a // (heads // g)
        s = (q[:, a] @ k[:, b].T) * scale                                   # [T, S]
        seen = k_pos[None, :] <= q_pos[:, None]
        if chunk:
            seen = seen & ((k_pos[None, :] // chunk) == (q_pos[:, None] // chunk))
        s = s.masked_fill(~seen, float("-inf"))
        top = torch.clamp(s.max(dim=1, keepdim=True).values, min=0.0)       # the sink's score is 0
        e = torch.exp(s - top)
        out[:, a] = (e / (torch.exp(-top) + e.sum(dim=1, keepdim=True))) @ v[:, b]
    return out


def attention_mixer(h, positions, kv_before, w, p, m, eps):
    """``kv_before``: (keys, values, positions) of the sequence's earlier tokens or None. Returns the
    mixer's output [T, width] and the keys, values and positions including this portion's."""
    heads, dim = m["heads"], m["dim"]
    t = h.shape[0]
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).view(t, heads, dim)
    q = rotate(rms(q, eps) * w[p + ".q.norm"], positions, m.get("rot"))
    k, v = attention_keys_values(h, positions, w, p, m, eps)
    k_pos = positions
    if kv_before is not None:
        k, v, k_pos = torch.cat([kv_before[0], k]), torch.cat([kv_before[1], v]), torch.cat([kv_before[2], positions])
    mask = m.get("mask")
    o = sink_softmax_attention(q, k, v, positions, k_pos, float(m["scale"]), int(mask["size"]) if mask else None)
    return o.reshape(t, -1) @ w[p + ".o"].T, (k, v, k_pos)


# --------------------------------------------------------------------------- mLSTM
def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm_mixer(h, state, w, p, m, eps):
    """The matrix memory, token after token. ``state``: None (a sequence's start: all zeros, the running
    maximum too) or (S [heads, dim, vdim], n [heads, dim], mx [heads]).

        i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))
        mx' = max(f + mx, i);  S' = e^(f + mx - mx') S + e^(i - mx') k v^T;  n' likewise with k
        o = S'^T q / (max(|n' . q|, e^(-mx')) + 1e-6),  q scaled by dim^-1/2
    then each head's o over its root mean square, the weight over all heads, the sigmoid gate, W_o."""
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    t = h.shape[0]
    q = (h @ w[p + ".q"].T).view(t, heads, dim) * dim ** -0.5
    k = (h @ w[p + ".k"].T).view(t, heads, dim)
    v = (h @ w[p + ".v"].T).view(t, heads, vdim)
    gi = capped(h @ w[p + ".i"].T + w[p + ".i.b"], cap)                              # [T, heads]
    gf = torch.nn.functional.logsigmoid(capped(h @ w[p + ".f"].T + w[p + ".f.b"], cap))
    if state is None:
        S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
        n = torch.zeros(heads, dim, dtype=h.dtype)
        mx = torch.zeros(heads, dtype=h.dtype)
    else:
        S, n, mx = (x.clone() for x in state)
    o = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for s in range(t):
        new = torch.maximum(gf[s] + mx, gi[s])
        keep, take = torch.exp(gf[s] + mx - new), torch.exp(gi[s] - new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[s][:, :, None] * v[s][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[s]
        mx = new
        den = torch.maximum((n * q[s]).sum(dim=1).abs(), torch.exp(-mx)) + 1e-6
        o[s] = torch.einsum("adv,ad->av", S, q[s]) / den[:, None]
    o = rms(o, eps).reshape(t, heads * vdim) * w[p + ".norm"] * torch.sigmoid(h @ w[p + ".g"].T)
    return o @ w[p + ".o"].T, (S, n, mx)


# --------------------------------------------------------------------------- feed-forward
def dense_ff(h, w, p):
    return relu_squared(h @ w[p + ".up"].T) @ w[p + ".down"].T


def route(h, w, p, router: dict, forced=None, record=None):
    """(expert ids [T, top], weights [T, top]): scores are sigmoids of the router's logits; the experts lie
    in ``groups.count`` equal groups of neighbours, a group counts as the sum of its two largest scores, only
    the ``groups.keep`` best groups stay open, the ``top`` best experts of those are taken, and each
    weighs its score times ``scale``.

    ``forced`` [T, top]: choices to take instead of the own ones (their weights are still the own scores).
    ``record(ids, gap)`` gets the own choices and how clear they were: the smaller of the distance between the
    last open and the first shut group's score and that between the last taken and the first left-out score."""
    s = torch.sigmoid(h @ w[p + ".router"].T)                                        # [T, E]
    t, e = s.shape
    top = int(router["top"])
    groups = router.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    gap = torch.full((t,), float("inf"), dtype=s.dtype)
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = e // count
        best_two = s.view(t, count, per).topk(min(2, per), dim=2).values.sum(dim=2)  # [T, count]
        ranked = best_two.sort(dim=1, descending=True)
        if keep < count:
            gap = ranked.values[:, keep - 1] - ranked.values[:, keep]
        allowed = torch.zeros(t, count, dtype=torch.bool)
        allowed.scatter_(1, ranked.indices[:, :keep], True)
        allowed = allowed[:, :, None].expand(t, count, per).reshape(t, e)
    ranked = s.masked_fill(~allowed, -1.0).sort(dim=1, descending=True)
    chosen = ranked.indices[:, :top]
    if top < int(allowed[0].sum()):
        gap = torch.minimum(gap, ranked.values[:, top - 1] - ranked.values[:, top])
    if record is not None:
        record(chosen, gap)
    if forced is not None:
        chosen = forced.long()
    return chosen, torch.gather(s, 1, chosen) * float(router.get("scale", 1.0))


def moe_ff(h, w, p, mlp: dict, forced=None, record=None):
    ids, weights = route(h, w, p, mlp["router"], forced, record)
    out = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t]):
            out[t] += g * (relu_squared(h[t] @ w[f"{p}.e{e}.up"].T) @ w[f"{p}.e{e}.down"].T)
    return out


def feed_forward(h, w, p, mlp: dict, forced=None, record=None):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else moe_ff(h, w, p, mlp, forced, record)


# --------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], first_pos: int = 0, carried=None,
            dtype=torch.float64, layers_out: Optional[list] = None, forced_routing=None, record=None):
    """Logits [T, vocab] of ``tokens`` at positions first_pos .., and what the next portion needs
    (``carried``: per layer the attention's keys/values/positions or the mLSTM's state).
    ``forced_routing`` {"l<i>.mlp": ids [T, top]} and ``record(name, ids, gap)``: see :func:`route`."""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg.get("postln_alpha", 1.0))
    positions = torch.arange(first_pos, first_pos + len(tokens))
    x = w["embed"][torch.tensor(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    carried = list(carried) if carried is not None else [None] * len(cfg["layers"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] == "attention":
            y, carried[i] = attention_mixer(x, positions, carried[i], w, p + ".mix", layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            y, carried[i] = mlstm_mixer(x, carried[i], w, p + ".mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = rms(alpha * x + y, eps) * w[p + ".norm1"]
        if layer.get("mlp"):
            name = p + ".mlp"
            y = feed_forward(x, w, name, layer["mlp"], (forced_routing or {}).get(name),
                             None if record is None else (lambda ids, gap, name=name: record(name, ids, gap)))
            x = rms(alpha * x + y, eps) * w[p + ".norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    z = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return (soft_cap(z, float(cap)) if cap else z), carried


def forward_in_portions(cfg, w, tokens: List[int], sizes: List[int], dtype=torch.float64) -> torch.Tensor:
    """The same logits with the sequence cut into portions of the given sizes (the last takes the rest)."""
    out, at, carried = [], 0, None
    sizes = list(sizes)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else len(tokens) - at
        n = min(n, len(tokens) - at)
        z, carried = forward(cfg, w, tokens[at: at + n], at, carried, dtype)
        out.append(z)
        at += n
    return torch.cat(out)
