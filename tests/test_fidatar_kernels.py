"""The kernels that the Fidatar parts added or extended, each alone against a plain float64 statement of
the same operation: the post-norm boundary, the embedding multiplier, the soft cap, the squared relu, the
encoding of q and k (weighted norm before a partial rotation with a magnitude factor), the sink term in
every attention kernel (chunk edges, far keys, splits), group-limited routing with a score factor, experts
without a gate branch, and the three kernels of the matrix memory."""
import math

import pytest
import torch

import plain_fidatar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(t, dt=None):
    t = t.to(DEV)
    return t if dt is None else t.to(dt)


def rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def rel_rms(got, want):
    """Root mean square of the difference over that of the expected values: what rounding does on average. (The
    largest difference of a long run is set by its worst-conditioned token: an output that is normalised after
    a sum that nearly cancels magnifies the rounding of its inputs a hundredfold.)"""
    d = got.double().cpu() - want.double()
    return float(d.pow(2).mean().sqrt() / want.double().pow(2).mean().sqrt().clamp_min(1e-30))


# --------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("hidden", [64, 50, 2048, 4100])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_post_norm_boundary(hidden, dt, tol):
    """stream <- rmsnorm(alpha * stream + delta (+ routed rows times weights)) * w, and its rounding."""
    from hi_b200.kernels import ops

    g = torch.Generator().manual_seed(hidden)
    n, k, alpha, eps = 7, 3, 1.75, 1e-5
    x = torch.randn(n, hidden, generator=g)
    delta = torch.randn(n, hidden, generator=g).to(dt).float()
    w = (1 + 0.3 * torch.randn(hidden, generator=g)).to(dt).float()
    want = plain.rms((alpha * x + delta).double(), eps) * w.double()
    xs = dev(x.clone())
    y = ops.add_rmsnorm(xs, dev(delta, dt), dev(w, dt), eps, dt, x_scale=alpha, post=True)
    assert rel(xs, want) <= 2e-6 and rel(y, want) <= tol and y.dtype == dt
    # with routed rows: slot_of_entry scatters, the weights multiply
    routed = torch.randn(n * k, hidden, generator=g)
    slot = torch.randperm(n * k, generator=g).to(torch.int32)
    wt = torch.rand(n * k, generator=g)
    summed = (routed[slot.long()] * wt[:, None]).view(n, k, hidden).sum(1)
    want = plain.rms((alpha * x + summed).double(), eps) * w.double()
    xs = dev(x.clone())
    y = ops.add_rmsnorm(xs, None, dev(w, dt), eps, dt, None, False, dev(routed), dev(slot), k, dev(wt), x_scale=alpha, post=True)
    assert rel(xs, want) <= 3e-6 and rel(y, want) <= tol
    # without a delta the stream is still replaced (a sub-layer that returned nothing would be a bug elsewhere)
    xs = dev(x.clone())
    ops.add_rmsnorm(xs, None, dev(w, dt), eps, dt, x_scale=1.0, post=True)
    assert rel(xs, plain.rms(x.double(), eps) * w.double()) <= 2e-6
    # the pre-norm use is untouched: the stream takes the sum
    xs = dev(x.clone())
    ops.add_rmsnorm(xs, dev(delta, dt), dev(w, dt), eps, dt)
    assert rel(xs, (x + delta).double()) <= 1e-7


def test_embedding_multiplier_soft_cap_and_squared_relu():
    from hi_b200.kernels import ops

    g = torch.Generator().manual_seed(1)
    for hidden in (48, 50):
        table = torch.randn(11, hidden, generator=g).to(torch.bfloat16)
        toks = torch.tensor([3, 0, 10, 3], dtype=torch.int32)
        out = ops.embed_gather(dev(table), dev(toks), scale=12.5)
        assert torch.equal(out.cpu(), table.float()[toks.long()] * 12.5)
        assert torch.equal(ops.embed_gather(dev(table), dev(toks)).cpu(), table.float()[toks.long()])
    for n in (64, 67, 5000):
        x = torch.randn(n, generator=g)
        assert torch.equal(ops.convert(dev(x), torch.bfloat16).cpu(), x.to(torch.bfloat16))
        assert torch.equal(ops.convert(dev(x.to(torch.bfloat16)), torch.float32).cpu(), x.to(torch.bfloat16).float())
    z = torch.randn(5, 77, generator=g) * 40
    got = ops.softcap_(dev(z.clone()), 18.0)
    assert rel(got, plain.soft_cap(z.double(), 18.0)) <= 2e-6
    for n in (64, 67, 5000):
        x = torch.randn(n, generator=g)
        assert torch.equal(ops.relu2(dev(x)).cpu(), torch.clamp(x, min=0) ** 2)
        xb = x.to(torch.bfloat16)
        assert torch.equal(ops.relu2(dev(xb)).cpu(), (torch.clamp(xb.float(), min=0) ** 2).to(torch.bfloat16))
        assert torch.equal(ops.relu2(dev(x), torch.bfloat16).cpu(), (torch.clamp(x, min=0) ** 2).to(torch.bfloat16))


# --------------------------------------------------------------------------- encoding of q and k
# float32: the angle position * frequency is itself a float32 (at position 700 it is known to about 4e-5)
@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("nh,nkv,dim,hd,rot", [
    (4, 2, 16, 16, {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}),
    (3, 1, 10, 16, {"dims": 6, "base": 300.0, "scaling": {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}}),
    (2, 2, 64, 64, {"dims": 32, "base": 50000.0}),
    (2, 1, 24, 32, {"dims": 24, "base": 500.0}),
    (2, 2, 128, 128, None),
    (1, 1, 72, 80, {"dims": 2, "base": 10.0, "scaling": {"factor": 16.0, "original": 8, "fast": 2.0, "slow": 1.0}}),
])
def test_weighted_norm_before_partial_rotation(dt, tol, nh, nkv, dim, hd, rot):
    """q and k: RMS over the head's own dims (the padding stays zero), weight, then the rotation; v is stored
    as it is; keys and values land on their pages."""
    from hi_b200.kernels import ops
    from hi_b200.parts.basic import yarn_inverse_frequencies

    g = torch.Generator().manual_seed(dim)
    n, page, eps = 9, 4, 1e-5
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 700, 701, 702], dtype=torch.int32)
    seq = torch.tensor([0] * 6 + [1] * 3, dtype=torch.int32)
    table = torch.full((2, 180), -1, dtype=torch.int32)
    table[0, :2] = torch.tensor([5, 2])
    table[1, 175] = 1
    heads = nh + 2 * nkv
    x = torch.zeros(n, heads, hd)
    x[..., :dim] = torch.randn(n, heads, dim, generator=g)
    x = x.to(dt).float()
    wq, wk = (torch.zeros(hd) for _ in range(2))
    wq[:dim], wk[:dim] = 1 + 0.4 * torch.randn(dim, generator=g), 1 + 0.4 * torch.randn(dim, generator=g)
    inv, mag = (None, 1.0) if rot is None else yarn_inverse_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    kp, vp = (torch.zeros(6, nkv, page, hd, dtype=dt, device=DEV) for _ in range(2))
    q = ops.qkv_post(dev(x.view(n, -1), dt), nh, nkv, hd, dev(positions), None if inv is None else dev(torch.from_numpy(inv)),
                     False, True, eps, None, dev(seq), dev(table), kp, vp, page, True, q_norm_weight=dev(wq),
                     k_norm_weight=dev(wk), norm_first=True, norm_dim=dim, rot_mul=mag)
    xd = x.double()
    want_q = plain.rotate(plain.rms(xd[:, :nh, :dim], eps) * wq[:dim].double(), positions, rot)
    want_k = plain.rotate(plain.rms(xd[:, nh: nh + nkv, :dim], eps) * wk[:dim].double(), positions, rot)
    assert rel(q[..., :dim], want_q) <= tol and float(q[..., dim:].abs().max() if hd > dim else 0) == 0
    for t in range(n):
        pg = int(table[int(seq[t]), int(positions[t]) // page])
        at = int(positions[t]) % page
        assert rel(kp[pg, :, at, :dim], want_k[t]) <= tol
        assert torch.equal(vp[pg, :, at].float().cpu(), x[t, nh + nkv:])


# --------------------------------------------------------------------------- the sink in every attention kernel
def _paged(k, v, page, n_pages, order_seed):
    """Scatter a sequence's keys and values [T, G, hd] over pages in a shuffled order."""
    t, g, hd = k.shape
    need = -(-t // page)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(order_seed))[:need]
    kp = torch.full((n_pages, g, page, hd), float("nan"))
    vp = torch.full((n_pages, g, page, hd), float("nan"))
    for i in range(t):
        kp[perm[i // page], :, i % page] = k[i]
        vp[perm[i // page], :, i % page] = v[i]
    return kp, vp, perm.to(torch.int32)


def _reference(q, k, v, q_pos, scale, chunk):
    t = k.shape[0]
    return plain.sink_softmax_attention(q.double(), k.double(), v.double(), q_pos, torch.arange(t), scale, chunk or None)


@pytest.mark.parametrize("dt,hd,chunk,tol", [
    (torch.float32, 16, 24, 3e-6), (torch.float32, 80, 0, 3e-6), (torch.float32, 64, 1, 3e-6),
    (torch.bfloat16, 64, 104, 1.5e-2), (torch.bfloat16, 128, 0, 1.5e-2), (torch.bfloat16, 64, 128, 1.5e-2), (torch.bfloat16, 48, 37, 1.5e-2)])
def test_sink_softmax_single_tokens(dt, hd, chunk, tol):
    """One decoded token per request at contexts that end just inside, on and just after a chunk's edge and far
    into a long context (splits). The same call without the sink differs: the sink is not a no-op."""
    from hi_b200.kernels import ops

    nh, nkv, page, t = 4, 2, 16, 900
    g = torch.Generator().manual_seed(hd + chunk)
    k = torch.randn(t, nkv, hd, generator=g).to(dt).float()
    v = torch.randn(t, nkv, hd, generator=g).to(dt).float()
    kp, vp, pages = _paged(k, v, page, 64, 3)
    edge = chunk if chunk > 1 else 100
    where = [0, 1, edge - 2, edge - 1, edge, edge + 1, 2 * edge - 1, 2 * edge, 511, 512, 899]
    where = [p for p in where if 0 <= p < t]
    q = (torch.randn(len(where), nh, hd, generator=g) * 0.5).to(dt).float()
    pos = torch.tensor(where, dtype=torch.int32)
    scale = 1.3 / math.sqrt(hd)
    table = pages.view(1, -1).repeat(len(where), 1).contiguous()       # every row is its own request on the same pages
    seq = torch.arange(len(where), dtype=torch.int32)
    want = _reference(q, k, v, pos, scale, chunk)
    args = (dev(q, dt), dev(kp, dt), dev(vp, dt), dev(table), dev(seq), dev(pos), chunk, 0, scale, t)
    got = ops.paged_attention(*args, sink=True)
    assert rel(got, want) <= tol
    assert rel(ops.paged_attention(*args), want) > 10 * tol
    if ops.decode_attention_supported(dt, nh, nkv, hd):
        got = ops.decode_attention(*args, sink=True)
        assert rel(got, want) <= tol
        assert rel(ops.decode_attention(*args), want) > 10 * tol


@pytest.mark.parametrize("hd,chunk,new,start", [(64, 104, 300, 0), (64, 104, 9, 210), (128, 0, 260, 40), (64, 64, 130, 62),
                                                (128, 200, 2, 199), (64, 0, 140, 700)])
def test_sink_softmax_portions_bfloat16(hd, chunk, new, start):
    """Portions of a prompt through the mma.sync kernel and, from 128 new tokens, the tcgen05 kernel, with and
    without key splits, beside the general kernel in float32; all against the plain statement."""
    from hi_b200.kernels import ops

    nh, nkv, page = 4, 2, 64
    t = start + new
    g = torch.Generator().manual_seed(hd + chunk + new)
    k = torch.randn(t, nkv, hd, generator=g).to(torch.bfloat16).float()
    v = torch.randn(t, nkv, hd, generator=g).to(torch.bfloat16).float()
    q = (torch.randn(new, nh, hd, generator=g) * 0.5).to(torch.bfloat16).float()
    kp, vp, pages = _paged(k, v, page, 24, 5)
    pos = torch.arange(start, t, dtype=torch.int32)
    scale = 1.3 / math.sqrt(hd)
    want = _reference(q, k, v, pos, scale, chunk)
    table, cu = pages.view(1, -1).contiguous(), torch.tensor([0, new], dtype=torch.int32)
    bf = torch.bfloat16
    common = (dev(table), dev(cu), dev(pos), 1, new, chunk, 0, scale)
    got = ops.prefill_attention(dev(q, bf), dev(kp, bf), dev(vp, bf), *common, sink=True)
    assert rel(got, want) <= 1.5e-2
    fewest = min(int(p) - (int(p) // chunk * chunk if chunk else 0) + 1 for p in pos)
    if fewest <= 8:       # among hundreds of keys the sink's share is small; among a few it is not
        assert rel(ops.prefill_attention(dev(q, bf), dev(kp, bf), dev(vp, bf), *common), want) > 0.1
    if new >= ops.PREFILL_TC_MIN_TOKENS:
        for splits in (1, 3):
            got = ops.prefill_attention_tc(dev(q, bf), dev(kp, bf), dev(vp, bf), *common, key_splits=splits, sink=True)
            torch.cuda.synchronize()
            ops.check_tc_status()
            assert rel(got, want) <= 1.5e-2, splits
    got = ops.paged_attention(dev(q), dev(kp), dev(vp), dev(table), dev(torch.zeros(new, dtype=torch.int32)), dev(pos), chunk, 0,
                              scale, t, sink=True)
    assert rel(got, want) <= 3e-6


def test_a_far_key_and_the_sink_under_a_peaked_softmax():
    """One key among 700 matches the query strongly: the output is that key's value times e^s / (1 + e^s + rest).
    With the matching key one position outside the chunk the output is what the others and the sink leave."""
    from hi_b200.kernels import ops

    nh = nkv = 1
    hd, page, t, chunk = 64, 16, 700, 300
    g = torch.Generator().manual_seed(4)
    k = torch.randn(t, nkv, hd, generator=g) * 0.1
    v = torch.randn(t, nkv, hd, generator=g)
    q = torch.zeros(1, nh, hd)
    q[0, 0, 5] = 1.0
    for far, inside in ((600, True), (599, False), (310, True)):
        kk = k.clone()
        kk[far, 0, 5] = 3.0                    # score 3 * scale stands out
        kp, vp, pages = _paged(kk, v, page, 48, 6)
        pos = torch.tensor([699 if far >= 600 or inside is False else 400], dtype=torch.int32)
        if not inside:
            pos = torch.tensor([899], dtype=torch.int32)      # chunk [600, 899] shuts 599 out; keys past 699 do not exist
            pos = torch.tensor([699], dtype=torch.int32)
            kk2 = kk.clone()
            kk2[far, 0, 5] = 0.0
        want = _reference(q, kk, v, pos, 4.0, chunk)
        got = ops.paged_attention(dev(q), dev(kp), dev(vp), dev(pages.view(1, -1).contiguous()), dev(torch.zeros(1, dtype=torch.int32)),
                                  dev(pos), chunk, 0, 4.0, t, sink=True)
        assert rel(got, want) <= 3e-6
        if inside:
            weight = math.exp(12.0) / (1 + math.exp(12.0))
            assert float((got.cpu()[0, 0] - v[far, 0] * weight).abs().max()) < 2e-2      # the rest shares e^-12
        else:
            assert rel(got, _reference(q, kk2, v, pos, 4.0, chunk)) <= 3e-6


# --------------------------------------------------------------------------- routing and experts
@pytest.mark.parametrize("experts,top,groups,n", [(8, 2, (4, 2), 5), (16, 5, (4, 2), 150), (6, 3, (3, 2), 33), (12, 4, (2, 1), 200),
                                                  (4, 1, (2, 2), 7), (4, 2, (1, 1), 9), (9, 2, (3, 2), 120), (5, 5, None, 11),
                                                  (64, 6, (8, 4), 40)])
def test_group_limited_routing(experts, top, groups, n):
    from hi_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * top)
    hidden = 48
    x = torch.randn(n, hidden, generator=g)
    w = (torch.randn(experts, hidden, generator=g) * 0.5).to(torch.bfloat16).float()
    router = {"experts": experts, "top": top, "scale": 1.5}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    want_ids, want_w = plain.route(x.double(), {"m.router": w.double()}, "m", router)
    mode = ops.router_groups(*groups) if groups else 0
    for wt in (dev(w), dev(w, torch.bfloat16)):
        ids, scores, plan = ops.router_plan(dev(x), wt, top, mode, 1.5)
        ids2, scores2, _ = ops.router_topk(dev(x), wt, top, mode=mode, score_scale=1.5)
        assert torch.equal(ids, ids2) and torch.equal(scores, scores2)
        order = ids.cpu().long().sort(dim=1)
        ref_order = want_ids.sort(dim=1)
        assert torch.equal(order.values, ref_order.values)
        assert rel(torch.gather(scores.cpu(), 1, order.indices), torch.gather(want_w, 1, ref_order.indices)) <= 2e-6
        # the plan groups every entry under its expert
        offs, sorted_entry = plan.offsets.cpu().tolist(), plan.sorted_entry.cpu().tolist()
        flat = ids.cpu().view(-1).tolist()
        assert offs[-1] == n * top
        for e in range(experts):
            assert all(flat[sorted_entry[s]] == e for s in range(offs[e], offs[e + 1]))


@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("n,hidden,inter,experts,top", [(3, 64, 32, 8, 2), (70, 64, 48, 6, 3), (300, 128, 64, 16, 3), (9, 50, 10, 5, 5),
                                                        (12, 64, 16, 12, 10)])
def test_experts_without_a_gate_branch(dt, tol, n, hidden, inter, experts, top):
    """W_down max(W_up x, 0)^2, weighted by the scores in the sum: the general kernels (few rows and many) and, in
    bfloat16 with many rows, the tensor-core path of the part."""
    from hi_b200.parts.context import StepContext
    from hi_b200.parts.registry import BuildEnv, build
    from hi_b200.parts.linear import configure_matmul_precision
    from hi_b200.parts.spec import PartSpec

    configure_matmul_precision()
    g = torch.Generator().manual_seed(n)
    w = {"m.router": torch.randn(experts, hidden, generator=g) * 0.4}
    for e in range(experts):
        w[f"m.e{e}.up"] = torch.randn(inter, hidden, generator=g) / math.sqrt(hidden)
        w[f"m.e{e}.down"] = torch.randn(hidden, inter, generator=g) / math.sqrt(inter)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    x = torch.randn(n, hidden, generator=g).to(dt).float()
    mlp = {"kind": "moe", "expert": {"ff": inter}, "router": {"experts": experts, "top": top, "scale": 1.25}}
    want = plain.moe_ff(x.double(), {k: v.double() for k, v in w.items()}, "m", mlp)
    part = build("feed_forward", PartSpec("routed_experts", {
        "hidden_size": hidden, "num_experts": experts, "top_k": top, "intermediate_size": inter, "shared_expert": False,
        "scale": "output", "activation": "relu2", "score_scale": 1.25, "names": "per_expert"}),
        BuildEnv(dtype=dt, device=torch.device(DEV), hidden_size=hidden), "m")
    part.load(lambda name: dev(w[name], dt))
    ctx = StepContext(n_tokens=n, n_seqs=1, tokens=None, positions=None, seq_of_token=None, cu_seqlens=None, slots=None,
                      start_pos=[0], n_new=[n], slot_ids=[0])
    pending = part.forward(dev(x, dt), ctx, normed_f32=dev(x))
    got = pending.materialize(n)
    torch.cuda.synchronize()
    assert rel(got, want) <= tol


# --------------------------------------------------------------------------- the matrix memory
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("heads,dim,vdim,cap,rows", [
    (2, 16, 24, 8.0, 0), (1, 40, 12, 10.0, 0), (3, 8, 8, 15.0, 0), (2, 136, 20, 12.0, 0), (2, 5, 7, 9.0, 0),
    (4, 4, 36, 5.0, 0), (2, 48, 48, 12.0, 16), (1, 128, 128, 6.0, 8), (1, 300, 4, 6.0, 0),
    # the staged kernel with 4 to 32 rows a lane, and a key size with padding rows (96 in 128)
    (2, 128, 128, 6.0, 0), (2, 64, 64, 9.0, 4), (1, 96, 64, 9.0, 4), (2, 64, 192, 12.0, 16), (1, 256, 64, 12.0, 32)])
def test_mlstm_mixer_alone(dt, tol, heads, dim, vdim, cap, rows):
    """Three requests in state slots 2, 0, 3, fed in steps of unequal portions down to one token; a long run so
    that the running maximum and the decays matter; the unused slot keeps its noise."""
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.registry import build
    from hi_b200.parts.spec import PartSpec
    from fidatar_configs import make_weights, mlstm
    from test_vinurax_engine import _ctx, _env

    width = 40
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    cfg = {"vocab": 8, "width": width, "norm": {"eps": 1e-5}, "layers": [mlstm(heads, dim, vdim, cap)]}
    w = make_weights(cfg, dim + vdim)
    part = build("mixer", PartSpec("mlstm", {"hidden_size": width, **mixer, "eps": 1e-5}), _env(dt, width), "l0.mix")
    part.ROWS_PER_LANE = rows
    part.load(lambda name: w[name].to(DEV).to(dt) if name in w else None)
    state = torch.randn((4, *part.cache_spec().state_shape), device=DEV)      # noise: slots are zeroed when taken
    view = CacheView(state=state, writes=True)
    slots = [2, 0, 3]
    for s in slots:
        state[s].zero_()
    g = torch.Generator().manual_seed(5)
    xs = [(1.5 * torch.randn(n, width, generator=g)).to(dt).float() for n in (230, 17, 9)]
    steps = [([7, 1, 2], [0, 0, 0]), ([1, 5, 1], [7, 1, 2]), ([20, 11, 6], [8, 6, 3]), ([2], [28]), ([199], [30]), ([1], [229])]
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
        want, (S, nvec, mx) = plain.mlstm_mixer(xs[i].double(), None, wd, "l0.mix", mixer, 1e-5)
        have = torch.cat(got[i]).double()
        assert have.shape[0] == want.shape[0]
        assert rel_rms(have, want) <= tol and rel(have, want) <= 100 * tol, f"request {i}"
        # the state row: S column by column, n, then the maximum per head
        row = state[slots[i]].cpu().double()
        body = row[: heads * (vdim + 1) * dim].view(heads, vdim + 1, dim)
        assert rel(body[:, :vdim].transpose(1, 2), S) <= max(tol, 1e-5) and rel(body[:, vdim], nvec) <= max(tol, 1e-5)
        assert (body[:, :vdim].transpose(1, 2) - S).abs().max() > 0 or dt == torch.float32
        assert float((row[heads * (vdim + 1) * dim:] - mx).abs().max()) <= (1e-4 if dt == torch.float32 else 0.2)
    assert float(state[1].abs().max()) > 0 and torch.isfinite(state).all()


def test_mlstm_gates_kernel():
    """keep, take and floor against the formulas over several blocks of tokens and a state that carries m."""
    from hi_b200.kernels import ops

    heads, dim, vdim, cap, n = 3, 4, 4, 7.0, 333
    g = torch.Generator().manual_seed(2)
    z = torch.randn(n, 2 * heads, generator=g) * 6
    bi, bf = torch.randn(heads, generator=g), torch.randn(heads, generator=g) + 2
    state = torch.zeros(2, ops.mlstm_state_floats(heads, dim, vdim), device=DEV)
    m0 = torch.tensor([0.5, -1.0, 3.0])
    state[1, -heads:] = dev(m0)
    cu = torch.tensor([0, n], dtype=torch.int32)
    keep, take, floor = ops.mlstm_gates(dev(z), dev(bi), dev(bf), cap, state, dev(cu), dev(torch.tensor([1], dtype=torch.int32)),
                                        heads, dim, vdim)
    zi = plain.capped(z[:, :heads].double() + bi.double(), cap)
    zf = torch.nn.functional.logsigmoid(plain.capped(z[:, heads:].double() + bf.double(), cap))
    m = m0.double()
    for t in range(n):
        new = torch.maximum(zf[t] + m, zi[t])
        assert float((keep[t].cpu() - torch.exp(zf[t] + m - new)).abs().max()) < 2e-5
        assert float((take[t].cpu() - torch.exp(zi[t] - new)).abs().max()) < 2e-5
        assert rel(floor[t], torch.exp(-new)) < 2e-5
        m = new
    assert float((state[1, -heads:].cpu() - m).abs().max()) < 1e-5 and float(state[0].abs().max()) == 0


# --------------------------------------------------------------------------- the one-launch decode form
@pytest.mark.parametrize("nh,nkv,hd,page,chunk,rot_dims,scaling", [(16, 4, 128, 64, 8192, 64, (4.0, 4096, 32.0, 1.0)), (8, 8, 64, 16, 0, 32, None),
                                                                  (12, 4, 64, 32, 512, 64, (2.0, 64, 8.0, 1.0)), (6, 2, 128, 128, 128, 0, None)])
def test_fused_decode_form_with_weighted_norm_and_sink(nh, nkv, hd, page, chunk, rot_dims, scaling):
    """Encoding (weighted norm before a partial rotation with a magnitude factor), append, attention with the
    sink and the merge of its splits in one launch, against the three kernels that the other tests hold
    against the plain statement: the appended keys and values are the same bits, the outputs agree to
    bfloat16 rounding. Requests of very different lengths in one batch; twice on the same buffers."""
    from hi_b200.kernels import ops
    from hi_b200.parts.basic import yarn_inverse_frequencies

    starts = [0, 1, 63, 64, 255, 256, 1030, 2500, 8191, 8192, 8200]
    S = len(starts)
    total = [s + 1 for s in starts]
    g = torch.Generator().manual_seed(nh * 7 + hd)
    n_pages = sum(-(-t // page) for t in total) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-t // page) for t in total)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    c = 0
    for s in range(S):
        for b in range(-(-total[s] // page)):
            bt[s, b] = perm[c]
            c += 1
    bf = torch.bfloat16
    kp = torch.randn(n_pages, nkv, page, hd, generator=g).to(bf)
    vp = torch.randn(n_pages, nkv, page, hd, generator=g).to(bf)
    qkv = dev((torch.randn(S, (nh + 2 * nkv) * hd, generator=g) * 1.5).to(bf))
    pos, sot, bt = dev(torch.tensor(starts, dtype=torch.int32)), dev(torch.arange(S, dtype=torch.int32)), dev(bt)
    inv, mag = None, 1.0
    if rot_dims:
        table, mag = yarn_inverse_frequencies(rot_dims, 1e5, None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling)))
        inv = dev(torch.from_numpy(table))
    wq, wk = dev(1 + 0.4 * torch.randn(hd, generator=g)), dev(1 + 0.4 * torch.randn(hd, generator=g))
    extra = dict(q_norm_weight=wq, k_norm_weight=wk, norm_first=True, rot_mul=mag)
    for _round in range(2):
        k1, v1, k2, v2 = dev(kp), dev(vp), dev(kp), dev(vp)
        q = ops.qkv_post(qkv, nh, nkv, hd, pos, inv, False, True, 1e-6, None, sot, bt, k1, v1, page, True, norm_dim=hd, **extra)
        want = ops.decode_attention(q, k1, v1, bt, sot, pos, chunk, 0, hd ** -0.5, max(total), sink=True)
        got = ops.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, False, True, 1e-6, None, sot, bt, k2, v2, chunk, 0,
                                         hd ** -0.5, max(total), sink=True, **extra)
        assert got is not None, "the fused kernel refused shapes it is written for"
        torch.cuda.synchronize()
        assert torch.equal(k1, k2) and torch.equal(v1, v2), "the appended keys or values differ"
        assert rel(got, want.double().cpu()) <= 1e-2
        no_sink = ops.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, False, True, 1e-6, None, sot, bt, dev(kp), dev(vp), chunk, 0,
                                             hd ** -0.5, max(total), sink=False, **extra)
        assert rel(no_sink[:2], want[:2].double().cpu()) > 5e-2          # among one or two keys the sink weighs
        assert int(ops._fused_counter_buffer(torch.device(DEV)).abs().sum()) == 0, "the counters were not left at zero"
    ops.check_tc_status()
