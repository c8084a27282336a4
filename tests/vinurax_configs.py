"""Small Vinurax configurations of the tests and a writer of weights with activations of order one
everywhere (fan-in scaled matrices, norm weights around 1, decays from fast to slow), so that a
mechanism that is left out or misplaced moves the logits."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch


def latent(heads, dim, vdim, rank, scale, ff=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, eps, layers):
    return {"architecture": "Vinurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# both mixers, a layer without feed-forward, a shared latent cache, a latent size that needs padding (40),
# one that the tensor-core attention kernels take (64), grouped q/k heads in the delta mixer
VX_A = config(131, 64, 1e-5, [
    delta(4, 2, 16, 24, 4, ff=96),
    latent(4, 16, 8, 64, 0.25, ff=80),
    latent(2, 24, 16, 64, 0.2, ff=72, kv_from=1),
    delta(2, 2, 32, 16, 2),
    latent(2, 8, 24, 40, 0.35, ff=64),
])
# starts with attention; one q/k head for three value heads; key size 48 (between the register kernels' sizes);
# a latent of 128; one tap (no convolution state); one head
VX_B = config(200, 96, 1e-6, [
    latent(6, 16, 16, 128, 0.25, ff=128),
    delta(3, 1, 48, 40, 3, ff=100),
    latent(3, 32, 8, 128, 0.18, kv_from=0),
    delta(1, 1, 8, 72, 1, ff=48),
    latent(1, 16, 16, 16, 0.3, ff=64),
])
# no attention at all: no page group
VX_C = config(64, 48, 1e-5, [delta(2, 2, 16, 16, 3, ff=64), delta(3, 3, 8, 20, 5)])
# attention only: no state
VX_D = config(90, 40, 1e-5, [latent(2, 8, 8, 32, 0.4, ff=40), latent(5, 8, 4, 32, 0.3, kv_from=0), latent(2, 4, 12, 24, 0.5)])


# sizes that no kernel's wide path takes: width, head sizes, latent size, feed-forward and vocabulary
# that are no multiples of four
VX_E = config(77, 50, 1e-5, [latent(3, 10, 6, 22, 0.3, ff=30), delta(2, 1, 18, 10, 3, ff=26), latent(1, 6, 14, 22, 0.4, kv_from=0),
                             delta(3, 3, 5, 7, 2)])


def peaked(cfg: dict, factor: float) -> dict:
    """The same model with every attention scale multiplied: the softmax then puts nearly all of its
    weight on one key, often a far one, so a key that is lost, doubled or shifted shows in the logits."""
    import copy

    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["type"] == "latent_attention":
            layer["mixer"]["scale"] *= factor
    return out


def make_weights(cfg: dict, seed: int, decay_rank: int = 6, gate_rank: int = 5) -> Dict[str, torch.Tensor]:
    """All tensors of a model, float32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    width = cfg["width"]

    def mat(name, rows, cols, gain=1.0):
        w[name] = torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = mean + std * torch.randn(n, generator=g)

    def dyt(name):
        vec(name, width, 1.0, 0.3)
        vec(name + ".b", width, 0.0, 0.3)
        w[name + ".alpha"] = torch.tensor(0.6) + 0.4 * torch.rand((), generator=g)

    w["embed"] = torch.randn(cfg["vocab"], width, generator=g)
    n_layers = len(cfg["layers"])
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        dyt(p + ".norm1")
        if layer["type"] == "latent_attention":
            hd, hv, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["kv_rank"]
            mat(p + ".mix.q", hd, width, 2.0)
            if "kv_from" not in m:
                mat(p + ".mix.dkv", r, width)
                vec(p + ".mix.dkv.norm", r, 1.0, 0.3)
            mat(p + ".mix.uk", hd, r, 2.0)
            mat(p + ".mix.uv", hv, r)
            mat(p + ".mix.g", m["heads"], width, 2.0)
            mat(p + ".mix.o", width, hv)
        else:
            qk, hv, hd = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"] * m["dim"]
            for n, rows in (("q", qk), ("k", qk), ("v", hv)):
                mat(f"{p}.mix.{n}", rows, width, 1.5)
                w[f"{p}.mix.{n}.conv"] = torch.randn(rows, m["conv"], generator=g) * 0.6
            mat(p + ".mix.b", m["heads"], width, 2.0)
            w[p + ".mix.A_log"] = torch.linspace(-4.0, 0.5, m["heads"])      # from slow to fast forgetting
            vec(p + ".mix.norm", m["vdim"], 1.0, 0.3)
            mat(p + ".mix.a1", decay_rank, width)
            mat(p + ".mix.a2", hd, decay_rank, 2.0)
            vec(p + ".mix.dt_bias", hd, -1.0, 1.0)
            mat(p + ".mix.g1", gate_rank, width)
            mat(p + ".mix.g2", hv, gate_rank, 2.0)
            mat(p + ".mix.o", width, hv)
        mat(p + ".rg1", width, width, 1.5)
        vec(p + ".rg1.b", width, 0.0, 0.5)
        if layer["mlp"] is not None:
            dyt(p + ".norm2")
            mat(p + ".mlp.up", layer["mlp"]["ff"], width, 1.5)
            mat(p + ".mlp.down", width, layer["mlp"]["ff"])
            w[p + ".mlp.act"] = torch.tensor([0.3, -0.4]) + 0.2 * torch.randn(2, generator=g)
            mat(p + ".rg2", width, width, 1.5)
            vec(p + ".rg2.b", width, 0.0, 0.5)
        mix = 0.25 * torch.randn(i + 2, generator=g) / math.sqrt(i + 1)
        mix[-1] += 0.8
        w[p + ".dwa"] = mix
    dyt("final.norm")
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def write_model(path: str, cfg: dict, seed: int, **sizes) -> Dict[str, torch.Tensor]:
    """A model folder (config.json + model.safetensors in bfloat16) with :func:`make_weights`; returns the weights."""
    import json
    import os

    from safetensors.torch import save_file

    weights = make_weights(cfg, seed, **sizes)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return weights
