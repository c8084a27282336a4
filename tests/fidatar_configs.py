"""Small Fidatar configurations of the tests and a writer of weights with activations of order one
everywhere (fan-in scaled matrices, norm weights around 1, gates that both keep and forget), so that a
mechanism that is left out or misplaced moves the logits."""
from __future__ import annotations

import copy
import math
from typing import Dict, Optional

import torch


def attention(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def mlstm(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale=None, groups=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(vocab, width, eps, layers, alpha=None, emb_scale=None, softcap=None):
    cfg = {"architecture": "Fidatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if alpha is not None:
        cfg["postln_alpha"] = alpha
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# both mixers and both feed-forwards; value heads narrower and wider than key heads; chunks that cut pages of 16
# anywhere; a layer without feed-forward; a rotation over part of a head with the ramped scaling, one over a whole
# head without; three query heads on a key head
FD_A = config(131, 64, 1e-5, [
    attention(4, 2, 16, 16, 0.5, chunk=24, rot=rot(8, 10000.0, (4.0, 64, 8.0, 1.0)), mlp=dense(96)),
    mlstm(2, 16, 24, 8.0, mlp=moe(8, 2, 32, scale=2.0, groups=(4, 2))),
    attention(3, 1, 24, 8, 0.4, chunk=10, rot=rot(24, 500.0)),
    mlstm(3, 8, 8, 15.0, mlp=dense(40)),
    attention(2, 2, 8, 40, 0.7, chunk=37, rot=rot(4, 100.0, (2.0, 16, 4.0, 0.5)), mlp=moe(6, 3, 24, scale=0.75, groups=(3, 2))),
], alpha=1.5, emb_scale=4.0, softcap=20.0)
# head sizes that the tensor-core attention kernels take in bfloat16 (64 and 128), with and without a chunk;
# experts without groups, one expert a token; a key size of the matrix memory that is no multiple of anything
FD_B = config(200, 96, 1e-6, [
    attention(4, 2, 64, 64, 0.22, chunk=100, rot=rot(32, 50000.0, (8.0, 128, 16.0, 2.0)), mlp=moe(6, 1, 48)),
    mlstm(1, 40, 12, 10.0),
    attention(2, 2, 128, 128, 0.15, mlp=dense(64)),
    mlstm(2, 24, 24, 6.0, mlp=moe(12, 4, 16, scale=1.25, groups=(2, 1))),
], alpha=2.5, emb_scale=9.0, softcap=30.0)
# no attention at all (no page group); a key size above 128 (another layout of the recurrence kernel);
# no multiplier on the embedding, no factor on the residual, no soft cap
FD_C = config(64, 48, 1e-5, [mlstm(2, 136, 20, 12.0, mlp=dense(64)), mlstm(4, 4, 36, 5.0)])
# attention only (no state); values that the other configurations do not make 1 or equal: one key head for all,
# as many key heads as query heads, a chunk of one position (a token sees itself only), every group kept,
# one group, no rotation, a rotation without mask
FD_D = config(90, 40, 1e-5, [
    attention(4, 1, 8, 8, 0.6, chunk=1, rot=rot(8, 10000.0), mlp=moe(4, 1, 24, scale=1.0, groups=(2, 2))),
    attention(5, 5, 8, 4, 0.5, chunk=33, mlp=moe(4, 2, 16, groups=(1, 1))),
    attention(2, 2, 16, 16, 0.45, rot=rot(16, 1000.0, (3.0, 40, 4.0, 1.0)), mlp=dense(40)),
], alpha=1.0, softcap=8.0)
# sizes that no kernel's wide path takes: width, head sizes, rotating pairs, feed-forward and vocabulary that are
# no multiples of four
FD_E = config(77, 50, 1e-5, [
    attention(3, 1, 10, 6, 0.5, chunk=13, rot=rot(6, 300.0, (2.0, 32, 8.0, 1.0)), mlp=dense(30)),
    mlstm(2, 5, 7, 9.0, mlp=moe(9, 2, 10, scale=1.5, groups=(3, 2))),
    attention(2, 2, 18, 22, 0.4, chunk=50, rot=rot(10, 10000.0), mlp=moe(5, 5, 6, scale=0.5)),
    mlstm(3, 18, 10, 12.0),
], alpha=2.0, emb_scale=3.0, softcap=12.0)


# more choices a token than the norm kernel sums in place (the experts' rows are then summed on their own first);
# one expert in all; sixteen query heads on one key head
FD_F = config(70, 32, 1e-5, [
    mlstm(1, 16, 16, 8.0, mlp=moe(12, 10, 8, scale=0.5, groups=(3, 3))),
    attention(16, 1, 16, 16, 0.3, chunk=48, rot=rot(16, 10000.0), mlp=moe(1, 1, 24)),
    attention(34, 2, 16, 16, 0.3, mlp=moe(16, 9, 8, scale=1.5, groups=(4, 3))),
], alpha=2.0, emb_scale=5.0, softcap=25.0)


def peaked(cfg: dict, factor: float) -> dict:
    """The same model with every attention scale multiplied: the softmax then puts nearly all of its
    weight on one key (or on the sink), so a key that is lost, doubled or shifted shows in the logits."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["scale"] *= factor
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """All tensors of a model, float32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    width = cfg["width"]

    def mat(name, rows, cols, gain=1.0):
        w[name] = torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = mean + std * torch.randn(n, generator=g)

    # the stream is normalised to about 1 per element before every sub-layer but the first
    w["embed"] = torch.randn(cfg["vocab"], width, generator=g) / float(cfg.get("embedding", {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        vec(p + ".norm1", width, 1.0, 0.3)
        hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
        if layer["type"] == "attention":
            kd, kv = m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            for n, rows in (("q", hd), ("k", kd), ("v", kv)):
                mat(f"{p}.mix.{n}", rows, width, 1.5)
                vec(f"{p}.mix.{n}.b", rows, 0.0, 0.3)
            vec(p + ".mix.q.norm", m["dim"], 1.0, 0.4)
            vec(p + ".mix.k.norm", m["dim"], 1.0, 0.4)
            mat(p + ".mix.o", width, hv, 2.0)
        else:
            for n, rows in (("q", hd), ("k", hd), ("v", hv), ("g", hv)):
                mat(f"{p}.mix.{n}", rows, width, 1.5)
            mat(p + ".mix.o", width, hv, 2.0)
            vec(p + ".mix.norm", hv, 1.0, 0.3)
            mat(p + ".mix.i", m["heads"], width, 2.0)
            vec(p + ".mix.i.b", m["heads"], 0.0, 1.0)
            mat(p + ".mix.f", m["heads"], width, 2.0)
            w[p + ".mix.f.b"] = torch.linspace(0.5, 4.0, m["heads"])          # from fast to slow forgetting
        mlp = layer["mlp"]
        if mlp is None:
            continue
        vec(p + ".norm2", width, 1.0, 0.3)
        if mlp["kind"] == "dense":
            mat(p + ".mlp.up", mlp["ff"], width, 1.5)
            mat(p + ".mlp.down", width, mlp["ff"], 1.5)
        else:
            mat(p + ".mlp.router", mlp["router"]["experts"], width, 2.5)
            for e in range(mlp["router"]["experts"]):
                mat(f"{p}.mlp.e{e}.up", mlp["expert"]["ff"], width, 1.5)
                mat(f"{p}.mlp.e{e}.down", width, mlp["expert"]["ff"], 1.5)
    vec("final.norm", width, 1.0, 0.3)
    mat("head", cfg["vocab"], width, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def write_model(path: str, cfg: dict, seed: int, weights: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """A model folder (config.json + model.safetensors in bfloat16) with :func:`make_weights` (or the given
    weights); returns the weights."""
    import json
    import os

    from safetensors.torch import save_file

    weights = make_weights(cfg, seed) if weights is None else weights
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return weights


class PlainFidatar:
    """The plain model with its per-sequence memory, for tests that decode with it."""

    def __init__(self, cfg, weights, dtype=torch.float64):
        import plain_fidatar as plain

        self.plain, self.cfg, self.w, self.dtype = plain, cfg, weights, dtype

    def logits(self, tokens):
        return self.plain.forward(self.cfg, self.w, list(tokens), dtype=self.dtype)[0]

    def new_sequence(self):
        return {"at": 0, "carried": None}

    def forward(self, seq, tokens):
        z, seq["carried"] = self.plain.forward(self.cfg, self.w, list(tokens), seq["at"], seq["carried"], self.dtype)
        seq["at"] += len(tokens)
        return z
