"""A plain, slow statement of the Vinurax decoder: one function per mechanism, written from the
equations, on the CPU in float64 or float32. It shares no code with hi_b200's parts or kernels.

Notation: ``h`` [T, width] is what a sub-layer reads, ``w`` a dict of the checkpoint's tensors
(linear weights [out, in], applied as ``h @ W.T``), ``p`` a prefix such as ``l3.mix``.

Every function that has something to carry from one portion of a sequence to the next takes and
returns it explicitly (``state``), so token-by-token and portion-by-portion runs of the oracle itself
can be held against its whole-sequence run.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dynamic_tanh(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """tanh(alpha x) * weight + b: a norm without statistics."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def xielu(z: torch.Tensor, act: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2, (p, q) = act."""
    ap = F.softplus(act[0])
    an = 0.5 + F.softplus(act[1])
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return xielu(h @ w[p + ".up"].T, w[p + ".act"]) @ w[p + ".down"].T


# --------------------------------------------------------------------------- latent attention
def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """The cached latent of every token: RMS norm of the down projection, times its weight."""
    return rms(h @ w[p + ".dkv"].T, eps) * w[p + ".dkv.norm"]


def latent_attention(h: torch.Tensor, latents: torch.Tensor, first_pos: int, w: Dict[str, torch.Tensor], p: str,
                     mixer: dict) -> torch.Tensor:
    """``h`` holds the tokens at positions first_pos .. first_pos + T - 1; ``latents`` [first_pos + T, rank]
    the latents of positions 0 .. (its own layer's, or the layer's named by ``kv_from``). Keys and values
    of every head are expanded from the latents; query i reads keys 0 .. i; softmax; per-head sigmoid gate."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    t, total = h.shape[0], latents.shape[0]
    q = (h @ w[p + ".q"].T).view(t, heads, dim)
    k = (latents @ w[p + ".uk"].T).view(total, heads, dim)
    v = (latents @ w[p + ".uv"].T).view(total, heads, vdim)
    gate = torch.sigmoid(h @ w[p + ".g"].T)                       # [t, heads]
    out = torch.zeros(t, heads, vdim, dtype=h.dtype)
    for i in range(t):
        last = first_pos + i
        for a in range(heads):
            s = (k[: last + 1, a] @ q[i, a]) * mixer["scale"]
            out[i, a] = torch.softmax(s, dim=0) @ v[: last + 1, a]
    out = out * gate[:, :, None]
    return out.reshape(t, heads * vdim) @ w[p + ".o"].T


# --------------------------------------------------------------------------- gated delta rule
def short_conv(x: torch.Tensor, taps: torch.Tensor, carry: torch.Tensor):
    """Causal convolution over time per channel, then silu. ``x`` [T, C], ``taps`` [C, K] (the last
    column multiplies the current token), ``carry`` [K-1, C] the inputs before this portion (zeros at
    the start of a sequence). Returns (y [T, C], the new carry)."""
    k = taps.shape[1]
    full = torch.cat([carry, x], dim=0)                           # [K-1+T, C]
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + full[j: j + x.shape[0]] * taps[:, j]
    new_carry = full[full.shape[0] - (k - 1):] if k > 1 else carry
    return F.silu(y), new_carry


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def channel_delta(h: torch.Tensor, state: Optional[dict], w: Dict[str, torch.Tensor], p: str, mixer: dict, eps: float):
    """The recurrent mixer over a portion of one sequence. ``state`` = {"S": [heads, dim, vdim],
    "q"/"k"/"v": conv carries} or None at the start. Returns (output [T, width], new state)."""
    heads, kvh, dim, vdim, taps = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"], mixer["conv"]
    t = h.shape[0]
    if state is None:
        state = {"S": torch.zeros(heads, dim, vdim, dtype=h.dtype),
                 "q": torch.zeros(taps - 1, kvh * dim, dtype=h.dtype),
                 "k": torch.zeros(taps - 1, kvh * dim, dtype=h.dtype),
                 "v": torch.zeros(taps - 1, heads * vdim, dtype=h.dtype)}
    q, cq = short_conv(h @ w[p + ".q"].T, w[p + ".q.conv"], state["q"])
    k, ck = short_conv(h @ w[p + ".k"].T, w[p + ".k.conv"], state["k"])
    v, cv = short_conv(h @ w[p + ".v"].T, w[p + ".v.conv"], state["v"])
    q = unit(q.view(t, kvh, dim)) * dim ** -0.5
    k = unit(k.view(t, kvh, dim))
    v = v.view(t, heads, vdim)
    beta = torch.sigmoid(h @ w[p + ".b"].T)                                           # [t, heads]
    rate = torch.exp(w[p + ".A_log"])                                                 # [heads]
    step = F.softplus((h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"])      # [t, heads*dim]
    decay = torch.exp(-rate[None, :, None] * step.view(t, heads, dim))                # [t, heads, dim]
    S = state["S"].clone()
    o = torch.zeros(t, heads, vdim, dtype=h.dtype)
    per = heads // kvh
    for i in range(t):
        for a in range(heads):
            qa, ka = q[i, a // per], k[i, a // per]
            S[a] = decay[i, a][:, None] * S[a]
            u = beta[i, a] * (v[i, a] - S[a].T @ ka)
            S[a] = S[a] + torch.outer(ka, u)
            o[i, a] = S[a].T @ qa
    gate = torch.sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T).view(t, heads, vdim)
    o = rms(o, eps) * w[p + ".norm"] * gate
    return o.reshape(t, heads * vdim) @ w[p + ".o"].T, {"S": S, "q": cq, "k": ck, "v": cv}


# --------------------------------------------------------------------------- the model
class PlainVinurax:
    """Runs sequences portion by portion, keeping per sequence what the design keeps: the latents of
    every latent-attention layer that makes its own, and the recurrent mixers' states."""

    def __init__(self, config: dict, weights: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg = config
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]

    def new_sequence(self) -> dict:
        return {"pos": 0, "latents": {}, "state": {}}

    def forward(self, seq: dict, tokens: List[int], layer_outputs: Optional[list] = None) -> torch.Tensor:
        """Feed the next tokens of a sequence; returns logits [T, vocab] at every one of them."""
        w = self.w
        x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        first = seq["pos"]
        streams = [x]                                   # X_0 and every layer's result
        for i, layer in enumerate(self.layers):
            pre = f"l{i}"
            h1 = dynamic_tanh(x, w, pre + ".norm1")
            mixer = layer["mixer"]
            if layer["type"] == "latent_attention":
                src = mixer.get("kv_from")
                if src is None:
                    new = latent_of(h1, w, pre + ".mix", self.eps)
                    old = seq["latents"].get(i)
                    seq["latents"][i] = new if old is None else torch.cat([old, new], dim=0)
                    src = i
                m = latent_attention(h1, seq["latents"][src], first, w, pre + ".mix", mixer)
            elif layer["type"] == "channel_delta":
                m, seq["state"][i] = channel_delta(h1, seq["state"].get(i), w, pre + ".mix", mixer, self.eps)
            else:
                raise ValueError(layer["type"])
            total = m * torch.sigmoid(h1 @ w[pre + ".rg1"].T + w[pre + ".rg1.b"])
            if layer.get("mlp") is not None:
                h2 = dynamic_tanh(x, w, pre + ".norm2")
                f = dense_mlp(h2, w, pre + ".mlp")
                total = total + f * torch.sigmoid(h2 @ w[pre + ".rg2"].T + w[pre + ".rg2.b"])
            streams.append(x + total)
            mix = w[pre + ".dwa"]
            x = sum(mix[j] * streams[j] for j in range(i + 2))
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        seq["pos"] = first + len(tokens)
        return dynamic_tanh(x, w, "final.norm") @ w["embed"].T

    def logits(self, tokens: List[int]) -> torch.Tensor:
        return self.forward(self.new_sequence(), tokens)
