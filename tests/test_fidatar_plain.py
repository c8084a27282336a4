"""The plain Fidatar model against itself and against hand-made cases, on the CPU: cut into portions and
token by token it must give what it gives whole; each mechanism shows when it is left out; the
configuration reader names what is wrong; the parts ask for the checkpoint's tensor names."""
import copy
import math

import pytest
import torch

import plain_fidatar as plain
from fidatar_configs import FD_A, FD_B, FD_C, FD_D, FD_E, FD_F, make_weights, peaked

CONFIGS = {"A": FD_A, "B": FD_B, "C": FD_C, "D": FD_D, "E": FD_E, "F": FD_F}


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_and_single_tokens_equal_the_whole(name):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 3)
    toks = tokens(cfg, 75, 1)
    whole, _ = plain.forward(cfg, w, toks)
    assert torch.isfinite(whole).all() and float(whole.std()) > 0.1
    cut = plain.forward_in_portions(cfg, w, toks, [13, 2, 1, 30, 2, 5])
    one = plain.forward_in_portions(cfg, w, toks, [1] * 75)
    assert float((cut - whole).abs().max()) < 1e-9 and float((one - whole).abs().max()) < 1e-9


def test_every_mechanism_moves_the_logits():
    """Leaving a mechanism out of the configuration or the weights changes the result by far more than rounding."""
    cfg, w = FD_A, make_weights(FD_A, 5)
    toks = tokens(cfg, 60, 2)
    base, _ = plain.forward(cfg, w, toks)

    def moved(cfg2=None, w2=None):
        z, _ = plain.forward(cfg2 or cfg, w2 or w, toks)
        return float((z - base).abs().max())

    def with_cfg(edit):
        c = copy.deepcopy(cfg)
        edit(c)
        return c

    assert moved(with_cfg(lambda c: c.update(postln_alpha=1.0))) > 1e-2
    assert moved(with_cfg(lambda c: c.update(embedding={"scale": 1.0}))) > 1e-2
    assert moved(with_cfg(lambda c: c.pop("logit_softcap"))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][0]["mixer"].pop("mask"))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][0]["mixer"]["mask"].update(size=25))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][0]["mixer"].pop("rot"))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling"))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][1]["mlp"]["router"].pop("groups"))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][1]["mlp"]["router"].update(scale=1.0))) > 1e-3
    assert moved(with_cfg(lambda c: c["layers"][1]["mixer"].update(gate_cap=2.0))) > 1e-3
    for name in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l1.mix.i.b", "l1.mix.f.b"):
        assert moved(w2={**w, name: torch.zeros_like(w[name])}) > 1e-3, name
    for name in ("l0.mix.q.norm", "l0.mix.k.norm", "l1.mix.norm", "l0.norm2"):
        assert moved(w2={**w, name: torch.ones_like(w[name])}) > 1e-3, name


def test_sink_takes_weight_and_has_no_value():
    """One key with score s: the weight is e^s / (1 + e^s), not 1; with a very negative score the output vanishes."""
    q = torch.tensor([[[2.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.5, 0.0]]], dtype=torch.float64)
    v = torch.tensor([[[3.0, -1.0]]], dtype=torch.float64)
    pos = torch.tensor([0])
    o = plain.sink_softmax_attention(q, k, v, pos, pos, 1.0, None)
    assert torch.allclose(o[0, 0], v[0, 0] * (math.exp(3.0) / (1 + math.exp(3.0))))
    o = plain.sink_softmax_attention(q, -40 * k, v, pos, pos, 1.0, None)
    assert float(o.abs().max()) < 1e-40


def test_chunk_mask_counts_from_position_zero():
    """Query 7 with chunks of 4 sees keys 4..7, wherever the portion started."""
    t = 8
    q = torch.zeros(t, 1, 2, dtype=torch.float64)
    k = torch.zeros(t, 1, 2, dtype=torch.float64)
    v = torch.eye(t, dtype=torch.float64).view(t, 1, t)
    pos = torch.arange(t)
    o = plain.sink_softmax_attention(q, k, v, pos, pos, 1.0, 4)
    assert torch.allclose(o[7, 0], torch.tensor([0, 0, 0, 0, .2, .2, .2, .2], dtype=torch.float64))
    assert torch.allclose(o[4, 0], torch.tensor([0, 0, 0, 0, .5, 0, 0, 0], dtype=torch.float64))
    o2 = plain.sink_softmax_attention(q[6:], k, v, pos[6:], pos, 1.0, 4)       # a portion that starts at 6
    assert torch.allclose(o2, o[6:])


def test_rotary_table():
    f, grow = plain.rotary_frequencies({"dims": 8, "base": 10000.0})
    assert grow == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64))
    # original 64, fast 8, slow 1: pair index of `turns` = 8 ln(64 / (2 pi turns)) / (2 ln 10000)
    f2, grow2 = plain.rotary_frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert abs(grow2 - (0.1 * math.log(4.0) + 1)) < 1e-12
    lo, hi = 0, 2                                   # floor(0.104) = 0, ceil(1.008) = 2
    ramp = [min(max((i - lo) / (hi - lo), 0), 1) for i in range(4)]
    want = [fi / 4 * r + fi * (1 - r) for fi, r in zip(f.tolist(), ramp)]
    assert torch.allclose(f2, torch.tensor(want, dtype=torch.float64))
    # the framework's table is the same statement
    from hi_b200.parts.basic import yarn_inverse_frequencies
    for rot in (FD_A["layers"][0]["mixer"]["rot"], FD_B["layers"][0]["mixer"]["rot"], FD_E["layers"][0]["mixer"]["rot"],
                FD_A["layers"][2]["mixer"]["rot"]):
        have, mag = yarn_inverse_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        ref, grow = plain.rotary_frequencies(rot)
        assert abs(mag - grow) < 1e-12 and torch.allclose(torch.from_numpy(have).double(), ref, rtol=1e-6)
    # only the first dims of a head turn; position 0 turns nothing but still grows
    x = torch.randn(3, 2, 12, dtype=torch.float64)
    y = plain.rotate(x, torch.tensor([0, 5, 9]), {"dims": 8, "base": 100.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}})
    assert torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[0, :, :8], x[0, :, :8] * (0.1 * math.log(2.0) + 1))


def test_routing_by_groups():
    """Scores by expert: groups of two; the best single expert sits in a group whose pair is weak."""
    h = torch.eye(6, dtype=torch.float64)[:1]                      # picks the first column of the router
    logits = torch.tensor([2.0, -5.0, 1.0, 1.2, 0.9, 1.1], dtype=torch.float64)
    w = {"m.router": logits.view(6, 1) * torch.ones(1, 6, dtype=torch.float64) * torch.eye(6, dtype=torch.float64)[0]}
    s = torch.sigmoid(logits)
    ids, wt = plain.route(h, w, "m", {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}})
    # group sums: (0.88 + 0.007), (0.73 + 0.77), (0.71 + 0.75): groups 1 and 2 stay open, expert 0 is shut out
    assert sorted(ids[0].tolist()) == [3, 5]
    assert torch.allclose(wt[0].sort().values, (s[[3, 5]] * 1.5).sort().values)
    ids, _ = plain.route(h, w, "m", {"experts": 6, "top": 2, "scale": 1.5})
    assert sorted(ids[0].tolist()) == [0, 3]


def test_mlstm_against_the_unstabilised_sum():
    """With small gates the memory is the plain weighted sum: S_t = sum_s e^(i_s + f_(s+1) + .. + f_t) k_s v_s^T."""
    m = {"heads": 1, "dim": 3, "vdim": 2, "gate_cap": 30.0}
    g = torch.Generator().manual_seed(1)
    width, t = 5, 6
    w = {f"p.{n}": torch.randn(r, width, generator=g, dtype=torch.float64) for n, r in (("q", 3), ("k", 3), ("v", 2), ("g", 2), ("i", 1), ("f", 1))}
    w.update({"p.i.b": torch.tensor([0.3], dtype=torch.float64), "p.f.b": torch.tensor([1.0], dtype=torch.float64),
              "p.norm": torch.ones(2, dtype=torch.float64), "p.o": torch.eye(2, dtype=torch.float64)})
    h = torch.randn(t, width, generator=g, dtype=torch.float64)
    out, (S, n, mx) = plain.mlstm_mixer(h, None, w, "p", m, 1e-6)
    gi = 30 * torch.tanh((h @ w["p.i"].T + 0.3) / 30)[:, 0]
    gf = torch.nn.functional.logsigmoid(30 * torch.tanh((h @ w["p.f"].T + 1.0) / 30))[:, 0]
    k, v = h @ w["p.k"].T, h @ w["p.v"].T
    S_ref = sum(torch.exp(gi[s] + gf[s + 1:].sum()) * torch.outer(k[s], v[s]) for s in range(t))
    assert torch.allclose(S * torch.exp(mx), S_ref.unsqueeze(0), rtol=1e-9)
    assert float(mx) >= 0 or True      # the maximum starts at 0: it never drops below min(0 + sum f, ...)
    # carried state: two halves equal the whole
    a, st = plain.mlstm_mixer(h[:4], None, w, "p", m, 1e-6)
    b, _ = plain.mlstm_mixer(h[4:], st, w, "p", m, 1e-6)
    assert torch.allclose(torch.cat([a, b]), out, rtol=1e-9, atol=1e-12)


# --------------------------------------------------------------------------- configuration and tensor names
def test_config_reader_and_errors():
    from hi_b200.config.base import ConfigError
    from hi_b200.config.fidatar import FidatarConfig
    from hi_b200.config.registry import lookup

    assert lookup(FD_A).name == "fidatar"
    cfg = FidatarConfig.from_json(FD_A)
    assert (cfg.vocab, cfg.width, cfg.alpha, cfg.embedding_scale, cfg.logit_softcap) == (131, 64, 1.5, 4.0, 20.0)
    a, m = cfg.layers[0], cfg.layers[1]
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.scale) == ("attention", 4, 2, 16, 16, 24, 0.5)
    assert a.rot.dims == 8 and a.rot.scaling == (4.0, 64.0, 8.0, 1.0) and a.mlp.kind == "dense" and a.mlp.ff == 96
    assert (m.kind, m.gate_cap, m.mlp.experts, m.mlp.top, m.mlp.groups, m.mlp.score_scale) == ("mlstm", 8.0, 8, 2, (4, 2), 2.0)
    assert cfg.layers[2].mlp is None and cfg.layers[2].rot.scaling is None
    d = FidatarConfig.from_json(FD_D)
    assert d.alpha == 1.0 and d.embedding_scale == 1.0 and d.layers[1].rot is None and d.layers[2].chunk is None
    assert FidatarConfig.from_json(FD_C).logit_softcap is None

    def broken(edit, word):
        c = copy.deepcopy(FD_A)
        edit(c)
        with pytest.raises(ConfigError) as e:
            FidatarConfig.from_json(c)
        assert word in str(e.value), str(e.value)

    broken(lambda c: c.pop("width"), "width")
    broken(lambda c: c["layers"][0].update(type="conv"), "layers[0].type")
    broken(lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "layers[0].mixer.kv_heads")
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads")
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims")
    broken(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "rot.scaling.fast")
    broken(lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "layers[1].mixer.gate_cap")
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router.top")
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups")
    broken(lambda c: c["layers"][1]["mlp"].update(kind="glu"), "layers[1].mlp.kind")
    broken(lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size")


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_parts_ask_for_the_checkpoints_names(name):
    from hi_b200.config.registry import lookup
    from hi_b200.parts.model import Model

    cfg = CONFIGS[name]
    arch = lookup(cfg)
    model = Model(arch.build_spec(arch.parse_config(cfg, None)), torch.float32, "cpu")
    have = {arch.normalize_tensor_name(k): tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
    want = {s.name: tuple(s.shape) for s in model.tensor_specs() if s.init != "absent"}
    assert want == have
    paged = [s for s in model.cache_specs.values() if s is not None and s.paged]
    states = [s for s in model.cache_specs.values() if s is not None and s.state_shape]
    assert len(paged) == sum(l["type"] == "attention" for l in cfg["layers"])
    assert len(states) == sum(l["type"] == "mlstm" for l in cfg["layers"])
    for layer, spec in zip(cfg["layers"], model.cache_specs.values()):
        m = layer["mixer"]
        if layer["type"] == "attention":
            assert spec.head_dim % 16 == 0 and spec.head_dim >= max(m["dim"], m["vdim"]) and spec.kv_heads == m["kv_heads"]
            assert spec.window == (("chunk", m["mask"]["size"]) if "mask" in m else None)
        else:
            assert spec.state_shape == (m["heads"] * ((m["vdim"] + 1) * m["dim"] + 1),)


def test_peaked_configuration_is_another_model():
    w = make_weights(FD_D, 2)
    toks = tokens(FD_D, 40, 3)
    a, _ = plain.forward(FD_D, w, toks)
    b, _ = plain.forward(peaked(FD_D, 10.0), w, toks)
    assert float((a - b).abs().max()) > 1e-2
