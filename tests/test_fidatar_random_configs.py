"""Fidatar configurations drawn at random (seeded): every size, constant and the order of layers move at once, small
odd sizes as well as sizes at which the tensor-core kernels take over, and each draw goes through the four ways
of cutting against the plain model, in 32-bit and in bfloat16."""
import random

import pytest

import harness as h
from fidatar_configs import attention, config, dense, mlstm, moe, rot, write_model
from test_fidatar_engine import TOL, compare, tokens

pytestmark = pytest.mark.gpu


def draw_ff(rng: random.Random, large: bool):
    kind = rng.choice(["dense", "moe", "moe", None])
    if kind is None:
        return None
    if kind == "dense":
        return dense(rng.choice([128, 192, 320]) if large else rng.choice([2, 8, 16]) * rng.randrange(3, 20))
    count = rng.choice([1, 2, 3, 4, 8])
    per = rng.choice([1, 2, 3, 4])
    keep = rng.randrange(1, count + 1)
    top = rng.randrange(1, min(keep * per, 9) + 1)
    ff = rng.choice([64, 96, 128]) if large else rng.choice([2, 8]) * rng.randrange(2, 12)
    return moe(count * per, top, ff, scale=rng.choice([None, 0.5, 1.5, 2.5]), groups=rng.choice([None, (count, keep)]) if top <= keep * per else None)


def draw(rng: random.Random, large: bool) -> dict:
    layers = []
    for _ in range(rng.randrange(1, 6)):
        if rng.random() < 0.55:
            nkv = rng.choice([1, 2, 3, 4])
            nh = nkv * rng.choice([1, 2, 3, 4, 6])
            dim = rng.choice([64, 64, 128]) if large else rng.choice([8, 12, 16, 24, 40, 48, 64, 80, 96])
            vdim = dim if (large or rng.random() < 0.5) else rng.choice([4, 8, 20, 32, 48, 72])
            dims = rng.choice([d for d in (2, 4, 6, 8, 12, 16, 24, 32, 64, dim) if d <= dim and d % 2 == 0])
            scaling = rng.choice([None, (rng.choice([2.0, 4.0, 8.0]), rng.choice([32, 64, 256]), rng.choice([8.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))])
            r = rng.choice([None, rot(dims, rng.choice([100.0, 10000.0, 1e6]), scaling)])
            chunk = rng.choice([None, 1, 7, 24, 64, 100, 112, 128, 200])
            layers.append(attention(nh, nkv, dim, vdim, rng.choice([0.5, 1.0, 2.0]) * dim ** -0.5, chunk=chunk, rot=r, mlp=draw_ff(rng, large)))
        else:
            dim = rng.choice([64, 128]) if large else rng.choice([3, 8, 16, 20, 48, 64, 100, 130])
            vdim = rng.choice([64, 128]) if large else rng.choice([4, 8, 16, 24, 48, 64, 90])
            layers.append(mlstm(rng.choice([1, 2, 3, 4]), dim, vdim, rng.choice([4.0, 10.0, 12.0, 30.0]), mlp=draw_ff(rng, large)))
    width = rng.choice([256, 320, 384]) if large else rng.choice([2, 4, 8, 16]) * rng.randrange(3, 20)
    return config(rng.randrange(60, 900), width, rng.choice([1e-5, 1e-6, 3e-4]), layers, alpha=rng.choice([None, 0.5, 2.0, 3.0]),
                  emb_scale=rng.choice([None, 2.0, 16.0]), softcap=rng.choice([None, 10.0, 30.0]))


@pytest.mark.parametrize("seed,large", [(1, False), (2, False), (3, False), (4, False), (5, False), (6, False), (7, False), (8, False),
                                        (101, True), (102, True), (103, True)])
def test_a_random_configuration_in_the_four_ways_of_cutting(seed, large, tmp_path):
    from hi_b200.engine.core import Engine

    rng = random.Random(seed)
    cfg = draw(rng, large)
    page = rng.choice([16, 64, 64, 128]) if large else rng.choice([8, 16, 64])
    lengths = [rng.randrange(1, 40), rng.randrange(20, 120), rng.randrange(60, 200)] + ([rng.randrange(200, 420)] if large else [rng.randrange(40, 260)])
    mdir = str(tmp_path / "m")
    weights = write_model(mdir, cfg, seed=seed)
    reqs = {f"r{i}": tokens(cfg, n, seed * 10 + i) for i, n in enumerate(lengths)}
    rounded = lambda n: -(-n // page) * page
    cap = max(rounded(n) for n in lengths) + 2 * page
    mixed_cap = max(cap, sum(sorted(rounded(n) for n in lengths)[-2:]) + page)
    prompt = {r: min(len(t), max(2, len(t) - 24)) for r, t in reqs.items()}       # the rest is decoded token by token
    for dtype in ("float32", "bfloat16"):
        for regime, steps, pool in (("whole", h.trace_whole(reqs), cap), ("tail", h.trace_tail_decode(reqs), cap),
                                    ("portions", h.trace_portions(reqs), cap),
                                    ("mixed", h.trace_mixed(reqs, max_tokens=mixed_cap, page=page, seed=seed, prefill_len=prompt), mixed_cap)):
            eng = Engine.from_dir(mdir, dtype=dtype, kv_page_size=page, kv_cache_tokens=pool, max_active_requests=4, debug_poison=True)
            got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
            compare(cfg, weights, reqs, got, TOL[dtype], f"seed {seed} {cfg} page {page}: {dtype} {regime}",
                    forced if dtype == "bfloat16" else None)
            assert not eng.manager.requests
            for p in eng.manager.pools:
                assert p.free == p.total, "pages were lost"
