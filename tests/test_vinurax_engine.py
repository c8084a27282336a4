"""The Vinurax parts in the engine against the plain implementation: each mixer alone, whole prompts,
decoding through the cache and the state, portions down to two tokens, mixed batches with pages and
slots used again, far keys under a peaked softmax, long decoding, models with one kind of mixer only,
generation through the entry point, and the trace replay as a user runs it."""
import math

import numpy as np
import pytest
import torch

import harness as h
import plain_vinurax as plain
from vinurax_configs import VX_A, VX_B, VX_C, VX_D, VX_E, make_weights, peaked, write_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
CONFIGS = {"A": VX_A, "B": VX_B, "C": VX_C, "D": VX_D, "E": VX_E}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("vinurax")
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(base / name)
        out[name] = (cfg, d, write_model(d, cfg, seed=20 + len(name) + ord(name)))
    return out


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def engine(mdir, dtype, **kw):
    from hi_b200.engine.core import Engine

    kw.setdefault("kv_page_size", 16)
    kw.setdefault("kv_cache_tokens", 2048)
    kw.setdefault("max_active_requests", 4)
    return Engine.from_dir(mdir, dtype=dtype, **kw)


def compare(cfg, weights, requests, got, tol, what):
    """Every wanted row against the plain model; names the first wrong token."""
    model = plain.PlainVinurax(cfg, weights)
    for rid, toks in requests.items():
        ref = model.logits(toks)
        scale = float(ref.abs().max())
        rows = got.get(rid, {})
        assert rows, f"{what}: no logits came back for request {rid!r}"
        for p in sorted(rows):
            err = float(np.abs(rows[p].astype(np.float64) - ref[p].numpy()).max()) / scale
            assert np.isfinite(err) and err <= tol, (
                f"{what}: request {rid!r} first differs at position {p} of {len(toks)}: rel err {err:.3e} > {tol:.1e}")


# --------------------------------------------------------------------------- each mixer alone
def _env(dt, hidden):
    from hi_b200.parts.linear import configure_matmul_precision
    from hi_b200.parts.registry import BuildEnv

    configure_matmul_precision()
    return BuildEnv(dtype=dt, device=torch.device(DEV), hidden_size=hidden)


def _ctx(lens, starts, page, table, slots):
    from hi_b200.parts.context import StepContext

    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    singles = [i for i, n in enumerate(lens) if n == 1]
    ctx = StepContext(n_tokens=sum(lens), n_seqs=len(lens), tokens=torch.zeros(sum(lens), dtype=torch.int32, device=DEV),
                      positions=pos.to(DEV), seq_of_token=sot.to(DEV), cu_seqlens=cu.to(DEV),
                      slots=torch.tensor(slots, dtype=torch.int32, device=DEV), start_pos=list(starts), n_new=list(lens),
                      slot_ids=list(slots), block_tables={0: table.to(DEV)}, page_size=page,
                      max_context=max(s + n for s, n in zip(starts, lens)))
    if singles and len(singles) < len(lens):
        ctx.decode_rows = cu[singles].to(torch.int64).to(DEV)
        ctx.decode_max_context = max(starts[i] + 1 for i in singles)
    return ctx


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("heads,dim,vdim,rank", [(4, 16, 8, 64), (3, 8, 20, 40), (2, 32, 32, 128), (20, 8, 8, 64), (2, 16, 16, 272)])
def test_latent_attention_mixer_alone(dt, tol, heads, dim, vdim, rank):
    """Two requests in two steps (a portion each, then a portion beside a single token) on scattered pages."""
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    width, page = 48, 8
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": 0.3}
    cfg = {"vocab": 8, "width": width, "norm": {"eps": 1e-5},
           "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": None}]}
    w = make_weights(cfg, rank)
    part = build("mixer", PartSpec("latent_attention", {"hidden_size": width, **mixer, "eps": 1e-5}), _env(dt, width), "l0.mix")
    part.load(lambda name: w[name].to(DEV).to(dt) if name in w else None)
    spec = part.cache_spec()
    pool = torch.zeros((12, 1, page, spec.head_dim), dtype=dt, device=DEV)
    view = CacheView(group=0, k_pages=pool, v_pages=None, writes=True)
    table = torch.tensor([[7, 2, 9, 4], [1, 11, 0, 5]], dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(21, width, generator=g), torch.randn(18, width, generator=g)]
    xs = [x.to(dt).float() for x in xs]
    cuts = [([13, 17], [0, 0]), ([8, 1], [13, 17])]
    got = [[], []]
    for lens, starts in cuts:
        x = torch.cat([xs[i][s: s + n] for i, (n, s) in enumerate(zip(lens, starts))])
        out = part.forward(x.to(DEV).to(dt), _ctx(lens, starts, page, table, [0, 1]), view)
        a = 0
        for i, n in enumerate(lens):
            got[i].append(out[a: a + n].float().cpu())
            a += n
    wd = {k: v.double() for k, v in w.items()}
    for i in range(2):
        lat = plain.latent_of(xs[i].double(), wd, "l0.mix", 1e-5)
        want = plain.latent_attention(xs[i].double(), lat, 0, wd, "l0.mix", mixer)
        err = float((torch.cat(got[i]).double() - want).abs().max() / want.abs().max())
        assert err <= tol, f"request {i}: rel err {err:.3e}"


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("heads,kvh,dim,vdim,taps,general", [(4, 2, 16, 24, 4, False), (3, 1, 48, 40, 3, False), (2, 2, 8, 8, 1, False),
                                                             (2, 1, 72, 20, 2, True), (1, 1, 136, 16, 3, False)])
def test_channel_delta_mixer_alone(dt, tol, heads, kvh, dim, vdim, taps, general):
    """Three requests in state slots 2, 0, 3, fed in steps of unequal portions (down to one token,
    shorter than the convolution reaches back); a slot that was used before starts from a zeroed state."""
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec

    width = 40
    mixer = {"heads": heads, "kv_heads": kvh, "dim": dim, "vdim": vdim, "conv": taps}
    cfg = {"vocab": 8, "width": width, "norm": {"eps": 1e-5}, "layers": [{"type": "channel_delta", "mixer": mixer, "mlp": None}]}
    w = make_weights(cfg, dim + taps)
    part = build("mixer", PartSpec("channel_delta", {"hidden_size": width, **mixer, "decay_rank": 6, "gate_rank": 5, "eps": 1e-5}),
                 _env(dt, width), "l0.mix")
    part.GENERAL_KERNEL = general
    part.load(lambda name: w[name].to(DEV).to(dt) if name in w else None)
    state = torch.randn((4, *part.cache_spec().state_shape), device=DEV)      # noise: slots are zeroed when taken
    view = CacheView(state=state, writes=True)
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, width, generator=g).to(dt).float() for n in (30, 17, 9)]
    steps = [([7, 1, 2], [0, 0, 0]), ([1, 5, 1], [7, 1, 2]), ([20, 11, 6], [8, 6, 3]), ([2], [28])]
    got = [[], [], []]
    table = torch.zeros((3, 1), dtype=torch.int32)
    for lens, starts in steps:
        ids = list(range(len(lens)))
        x = torch.cat([xs[i][s: s + n] for i, (n, s) in zip(ids, zip(lens, starts))])
        out = part.forward(x.to(DEV).to(dt), _ctx(lens, starts, 16, table, [slots[i] for i in ids]), view)
        a = 0
        for i, n in zip(ids, lens):
            got[i].append(out[a: a + n].float().cpu())
            a += n
    wd = {k: v.double() for k, v in w.items()}
    for i in range(3):
        want, _ = plain.channel_delta(xs[i].double(), None, wd, "l0.mix", mixer, 1e-5)
        have = torch.cat(got[i]).double()
        err = float((have - want[: have.shape[0]]).abs().max() / want.abs().max())
        assert err <= tol, f"request {i}: rel err {err:.3e}"
    assert float(state[1].abs().max()) > 0 and torch.isfinite(state).all()       # the unused slot kept its noise


# --------------------------------------------------------------------------- the model in the engine
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_ways_of_cutting(name, dtype, models):
    cfg, mdir, weights = models[name]
    requests = {"p": tokens(cfg, 150, 1), "q": tokens(cfg, 37, 2), "r": tokens(cfg, 1, 3), "s": tokens(cfg, 2, 4),
                "t": tokens(cfg, 64, 5), "u": tokens(cfg, 97, 6)}
    eng = engine(mdir, dtype, kv_cache_tokens=352, debug_poison=True)
    prompt = {r: min(len(t), max(2, len(t) - 24)) for r, t in requests.items()}      # the rest is decoded token by token
    for what, steps in (("whole", h.trace_whole(requests)), ("decode", h.trace_tail_decode(requests, tail=20)),
                        ("portions", h.trace_portions(requests)),
                        ("mixed", h.trace_mixed(requests, max_tokens=352, page=16, seed=7, max_live=4, prefill_len=prompt))):
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, TOL[dtype], f"{name} {dtype} {what}")
    assert len(eng.manager.requests) == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_use_pages_and_slots_again(name, models):
    """More requests than slots and than the pool holds at once, in two orders: every request's logits equal
    the plain model's whatever ran beside it and whichever pages and slot it got."""
    cfg, mdir, weights = models[name]
    requests = {i: tokens(cfg, n, 30 + i) for i, n in enumerate((70, 33, 48, 5, 90, 17, 64, 31, 2, 55))}
    for seed, live in ((1, 4), (2, 2)):
        eng = engine(mdir, "float32", kv_cache_tokens=272, max_active_requests=live, debug_poison=True)
        steps = h.trace_mixed(requests, max_tokens=272, page=16, seed=seed, max_live=live)
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, TOL["float32"], f"{name} mixed seed {seed}")
        assert eng.manager.snapshot()["groups"][0]["allocations"] > 272 // 16      # pages were handed out again


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_far_keys_under_a_peaked_softmax(name, models, tmp_path):
    """Attention scales times 12: nearly all weight on one key, which among hundreds is usually a far one.
    A prompt over many pages whole, in portions whose edges fall inside pages, and decoded at the end."""
    cfg = peaked(CONFIGS[name], 12.0)
    mdir = str(tmp_path / "peaked")
    weights = write_model(mdir, cfg, seed=77)
    requests = {"long": tokens(cfg, 700, 8), "short": tokens(cfg, 90, 9)}
    eng = engine(mdir, "float32", kv_cache_tokens=1024)
    for what, steps in (("whole", h.trace_whole(requests)), ("decode", h.trace_tail_decode(requests, tail=40)),
                        ("portions", h.trace_portions(requests, sizes=(100, 3, 61, 2, 129, 17, 2, 250, 5))),
                        ("mixed", h.trace_mixed(requests, max_tokens=1024, page=16, seed=3, max_live=2))):
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, 1e-4, f"{name} peaked {what}")


def test_long_decoding_and_first_tokens(models):
    """300 tokens decoded one by one after a two-token prompt (captured steps), beside a request that starts
    later; position 0 and 1 are compared too."""
    cfg, mdir, weights = models["A"]
    requests = {"a": tokens(cfg, 300, 11), "b": tokens(cfg, 120, 12)}
    for dtype in ("float32", "bfloat16"):
        eng = engine(mdir, dtype)
        steps = [([("a", requests["a"][:2], [0, 1])], [])]
        for i in range(2, 300):
            entries = [("a", [requests["a"][i]], [0])]
            j = i - 100
            if 0 <= j < 120:
                entries.append(("b", [requests["b"][j]], [0]))
            steps.append((entries, [r for r, n in (("a", 299), ("b", 219)) if i == n]))
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, TOL[dtype], f"long decoding {dtype}")
        assert len(eng._graphs) >= 1 and any(g.captured for g in eng._graphs.values())


def test_other_page_sizes_and_kernel_choices(models):
    """Page sizes 8 and 64; in bfloat16 the 64- and 128-wide latents go through the tensor-core attention
    kernels (single tokens, short portions, portions of 128 tokens and more), other sizes through the general one."""
    from hi_b200.kernels import ops

    for name, want in (("A", ("attention_decode", "attention_prefill")), ("B", ("attention_prefill_tc",))):
        cfg, mdir, weights = models[name]
        requests = {"x": tokens(cfg, 333, 14), "y": tokens(cfg, 40, 15)}
        for page in (8, 64):
            before = dict(ops.CALLS)
            eng = engine(mdir, "bfloat16", kv_page_size=page, kv_cache_tokens=1024)
            for steps in (h.trace_whole(requests), h.trace_tail_decode(requests, tail=8),
                          h.trace_portions(requests, sizes=(140, 5, 2, 150, 30))):
                got, _ = h.replay_in_process(eng, steps)
                compare(cfg, weights, requests, got, TOL["bfloat16"], f"{name} page {page}")
            used = {k for k, v in ops.CALLS.items() if v > before.get(k, 0)}
            if page == 64:
                assert any(k.startswith(w) for w in want for k in used), (name, sorted(used))
            assert {"gated_depth_dyt", "latent_append", "delta_recurrence", "xielu"} <= used


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(name, models):
    """hi_b200.generate (scheduler, sampler, launch-ahead) against greedy decoding of the plain model."""
    import hi_b200

    cfg, mdir, weights = models[name]
    prompts = [tokens(cfg, n, 40 + n) for n in (9, 1, 30, 17, 5)]
    model = plain.PlainVinurax(cfg, weights)
    outs = hi_b200.generate(mdir, prompts, hi_b200.SamplingParams(max_tokens=12, ignore_eos=True), dtype="float32",
                            kv_page_size=16, max_batch_size=3, kv_cache_tokens=512, max_batched_tokens=24)
    for prompt, out in zip(prompts, outs):
        seq = model.new_sequence()
        logits = model.forward(seq, prompt)[-1]
        for k, tok in enumerate(out.token_ids):
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(logits.abs().max()):
                assert tok == int(logits.argmax()), f"prompt of {len(prompt)}: token {k} is {tok}, plain model says {int(logits.argmax())}"
            logits = model.forward(seq, [tok])[-1]
        assert len(out.token_ids) == 12


def test_trace_replay_as_a_user_runs_it(models, tmp_path):
    cfg, mdir, weights = models["B"]
    requests = {"a": tokens(cfg, 80, 21), "b": tokens(cfg, 33, 22), "c": tokens(cfg, 3, 23), "d": tokens(cfg, 50, 24),
                "e": tokens(cfg, 20, 25)}
    steps = h.trace_mixed(requests, max_tokens=192, page=64, seed=5, max_live=4)
    for dtype in ("float32", "bfloat16"):
        got = h.replay_subprocess(mdir, dtype, steps, max_tokens=192, out_dir=str(tmp_path / dtype), vocab=cfg["vocab"],
                                  extra=["--max-live", "4"])
        compare(cfg, weights, requests, got, TOL[dtype], f"trace_run {dtype}")


def test_command_line_run(models, capsys):
    """``python -m hi_b200 run``: the next token, the top logits and greedy generation of a Vinurax folder."""
    import json

    from hi_b200.cli import main

    cfg, mdir, weights = models["D"]
    prompt = tokens(cfg, 12, 50)
    assert main(["run", mdir, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "5", "--top-k", "3",
                 "--dtype", "float32", "--kv-page-size", "16", "--include-logits"]) == 0
    report = json.loads(capsys.readouterr().out)
    model = plain.PlainVinurax(cfg, weights)
    ref = model.logits(prompt)[-1]
    assert report["next_token"] == int(ref.argmax()) and report["logit_count"] == cfg["vocab"]
    assert float((torch.tensor(report["logits"], dtype=torch.float64) - ref).abs().max()) <= 3e-5 * float(ref.abs().max())
    assert [t["token_id"] for t in report["top_logits"]] == torch.topk(ref, 3).indices.tolist()
    assert len(report["generated_tokens"]) == 5 and report["generated_tokens"][0] == report["next_token"]
