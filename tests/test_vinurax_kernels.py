"""Each kernel of the gated parallel block, the latent cache and the gated delta rule alone, against
plain float64 arithmetic written here (or in plain_vinurax.py)."""
import math

import pytest
import torch
import torch.nn.functional as F

import plain_vinurax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from hi_b200.kernels import ops
    return ops


def _close(got, want, tol, what=""):
    err = float((got.double().cpu() - want.double().cpu()).abs().max() / (want.double().abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol}"


@pytest.mark.parametrize("width", [192, 130, 1024, 4100])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gated_depth_dyt(width, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    n, entries, filled = 7, 5, 3
    x = torch.randn(n, width, generator=g) * 3
    d = [(torch.randn(n, width, generator=g)).to(dt) for _ in range(2)]
    gt = [(torch.randn(n, width, generator=g) * 2).to(dt) for _ in range(2)]
    hist = torch.randn(entries, n, width, generator=g)
    mix = torch.randn(filled + 1, generator=g)
    norms = [(torch.rand(1, generator=g) + 0.2, torch.randn(width, generator=g).to(dt), torch.randn(width, generator=g).to(dt))
             for _ in range(2)]
    s = x.double() + torch.sigmoid(gt[0].double()) * d[0].double() + torch.sigmoid(gt[1].double()) * d[1].double()
    z = sum(mix[j].double() * hist[j].double() for j in range(filled)) + mix[filled].double() * s
    ys = [torch.tanh(a.double() * z) * w.double() + b.double() for a, w, b in norms]
    hist_dev = hist.to(DEV)
    zz, got = ops.gated_depth_dyt(x.to(DEV), [(d[0].to(DEV), gt[0].to(DEV)), (d[1].to(DEV), gt[1].to(DEV))], hist_dev, filled,
                                  mix.to(DEV), [tuple(t.to(DEV) for t in nm) for nm in norms], dt)
    tol = 1e-5 if dt == torch.float32 else 1e-2
    _close(zz, z, 1e-5, "stream")
    _close(hist_dev[filled], s, 1e-6, "stored result")
    assert torch.equal(hist_dev[:filled].cpu(), hist[:filled]) and torch.equal(hist_dev[filled + 1:].cpu(), hist[filled + 1:])
    for k in range(2):
        _close(got[k], ys[k], tol, f"norm {k}")
    # only some rows, one norm, one ungated term, history read but not extended
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32)
    hist_dev = hist.to(DEV)
    _z, got = ops.gated_depth_dyt(x.to(DEV), [(d[0].to(DEV), None)], hist_dev, filled, mix.to(DEV),
                                  [tuple(t.to(DEV) for t in norms[1])], dt, row_map=rows.to(DEV), want_z=False)
    s1 = x.double() + d[0].double()
    z1 = sum(mix[j].double() * hist[j].double() for j in range(filled)) + mix[filled].double() * s1
    a, w, b = norms[1]
    _close(got[0], (torch.tanh(a.double() * z1) * w.double() + b.double())[rows.long()], tol, "wanted rows")
    assert torch.equal(hist_dev.cpu(), hist)
    # nothing pending, no average: the norms of x and x stored as result 0
    hist_dev = torch.zeros(2, n, width, device=DEV)
    _z, got = ops.gated_depth_dyt(x.to(DEV), [], hist_dev, 0, None, [tuple(t.to(DEV) for t in norms[0])], dt, want_z=False)
    a, w, b = norms[0]
    _close(got[0], torch.tanh(a.double() * x.double()) * w.double() + b.double(), tol, "first layer")
    assert torch.equal(hist_dev[0].cpu(), x)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_xielu(dt):
    ops = _ops()
    z = torch.cat([torch.linspace(-12, 12, 4001), torch.tensor([0.0, -0.0, 1e-4, -1e-4, 30.0, -60.0])]).to(dt)
    z = z if dt == torch.float32 else torch.cat([z, z[:1]])     # 4,008 elements: the eight-at-a-time bfloat16 kernel
    pq = torch.tensor([0.3, -1.1], dtype=torch.float64)
    want = plain.xielu(z.double(), pq)
    coef = torch.stack([F.softplus(pq[0]), 0.5 + F.softplus(pq[1])]).float()
    got = ops.xielu(z.to(DEV), coef.to(DEV))
    err = (got.double().cpu() - want).abs() / (want.abs() + z.double().abs() + 1e-3)    # y has a root near z = -2.5
    worst = int(err.argmax())
    assert float(err.max()) <= (2e-6 if dt == torch.float32 else 5e-3), (float(z[worst]), float(got[worst]), float(want[worst]))
    ragged = ops.xielu(z[:-3].contiguous().to(DEV), coef.to(DEV))          # a count that is no multiple of eight
    assert torch.equal(ragged.cpu(), got[:-3].cpu())


@pytest.mark.parametrize("rank,row_len", [(128, 128), (40, 48), (72, 80)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_latent_append_and_head_gate(rank, row_len, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(rank)
    n, page, pages = 9, 8, 6
    wide = torch.randn(n, 20 + rank + 3, generator=g).to(dt)
    w = torch.randn(rank, generator=g).to(dt)
    positions = torch.tensor([0, 1, 2, 13, 14, 15, 16, 7, 8], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1, 1, 2, 2], dtype=torch.int32)
    table = torch.tensor([[3, -1, -1], [5, 0, 2], [4, 1, -1]], dtype=torch.int32)
    pool = torch.full((pages, 1, page, row_len), 7.0, dtype=dt, device=DEV)
    dev = wide.to(DEV)
    ops.latent_append(dev[:, 20: 20 + rank], w.to(DEV), 1e-5, positions.to(DEV), seq.to(DEV), table.to(DEV), pool)
    want = plain.rms(wide[:, 20: 20 + rank].double(), 1e-5) * w.double()
    touched = set()
    for t in range(n):
        pg = int(table[seq[t], positions[t] // page])
        row = pool[pg, 0, int(positions[t]) % page].cpu()
        touched.add((pg, int(positions[t]) % page))
        _close(row[:rank], want[t], 1e-5 if dt == torch.float32 else 1e-2, f"latent {t}")
        assert float(row[rank:].abs().sum()) == 0.0
    for pg in range(pages):
        for r in range(page):
            if (pg, r) not in touched:
                assert float((pool[pg, 0, r].float() - 7.0).abs().max()) == 0.0
    heads, dim = 5, 12
    x = torch.randn(n, heads, dim, generator=g).to(dt)
    gate = torch.randn(n, heads + 4, generator=g).to(dt)
    got = ops.head_gate(x.to(DEV), gate.to(DEV)[:, 2: 2 + heads])
    _close(got, x.double() * torch.sigmoid(gate[:, 2: 2 + heads].double())[:, :, None], 1e-6 if dt == torch.float32 else 1e-2)


def _recurrence(q, k, v, beta, decay, S, heads, kvh, dim, vdim):
    """One request in float64: returns (o [T, heads*vdim], final S)."""
    t = q.shape[0]
    S = S.clone()
    o = torch.zeros(t, heads, vdim, dtype=torch.float64)
    per = heads // kvh
    for i in range(t):
        for a in range(heads):
            qa, ka = q[i].view(kvh, dim)[a // per], k[i].view(kvh, dim)[a // per]
            S[a] = decay[i].view(heads, dim)[a][:, None] * S[a]
            u = beta[i, a] * (v[i].view(heads, vdim)[a] - S[a].T @ ka)
            S[a] = S[a] + torch.outer(ka, u)
            o[i, a] = S[a].T @ qa
    return o.reshape(t, heads * vdim), S


@pytest.mark.parametrize("heads,kvh,dim,vdim", [(4, 4, 32, 32), (4, 2, 16, 24), (3, 1, 48, 70), (2, 2, 64, 16),
                                               (2, 1, 100, 40), (2, 2, 128, 128), (1, 1, 200, 33), (2, 1, 264, 20),
                                               (2, 1, 18, 10), (3, 3, 5, 7)])
@pytest.mark.parametrize("form", ["auto", "single", 16, 32, "general"])
def test_delta_recurrence(heads, kvh, dim, vdim, form):
    ops = _ops()
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lens = [1, 37, 2, 5]
    slots = [3, 0, 5, 1]
    n, n_slots = sum(lens), 6
    extra = 11                                   # the state rows hold more than S
    q = F.normalize(torch.randn(n, kvh, dim, generator=g, dtype=torch.float64), dim=-1).reshape(n, -1) * dim ** -0.5
    k = F.normalize(torch.randn(n, kvh, dim, generator=g, dtype=torch.float64), dim=-1).reshape(n, -1)
    v = torch.randn(n, heads * vdim, generator=g, dtype=torch.float64)
    beta = torch.rand(n, heads, generator=g, dtype=torch.float64)
    decay = torch.rand(n, heads * dim, generator=g, dtype=torch.float64) * 0.5 + 0.5
    state = torch.randn(n_slots, heads * dim * vdim + extra, generator=g, dtype=torch.float64).float()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    dev = state.to(DEV)
    f = lambda t: t.float().to(DEV).contiguous()
    got = ops.delta_recurrence(f(q), f(k), f(v), f(beta), f(decay), dev, cu.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV),
                               heads, kvh, dim, vdim, general=form == "general", single_tokens=form == "single",
                               rows=form if isinstance(form, int) else 0)
    after = dev.cpu()
    for s, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        S0 = state[slots[s], : heads * dim * vdim].double().view(heads, dim, vdim)
        o, S1 = _recurrence(q[a:b].float().double(), k[a:b].float().double(), v[a:b].float().double(),
                            beta[a:b].float().double(), decay[a:b].float().double(), S0, heads, kvh, dim, vdim)
        _close(got[a:b], o, 2e-5, f"request {s} output")
        _close(after[slots[s], : heads * dim * vdim], S1.reshape(-1), 2e-5, f"request {s} state")
        assert torch.equal(after[slots[s], heads * dim * vdim:], state[slots[s], heads * dim * vdim:])
    for other in set(range(n_slots)) - set(slots):
        assert torch.equal(after[other], state[other])


@pytest.mark.parametrize("heads,kvh,dim,vdim,taps", [(4, 4, 32, 32, 3), (4, 2, 16, 24, 4), (2, 1, 40, 20, 2), (2, 2, 8, 8, 1)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_delta_prep_conv_and_out_norm(heads, kvh, dim, vdim, taps, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(dim + taps)
    lens, slots = [1, 6, 2, 1], [2, 0, 3, 1]          # portions shorter than the taps reach back into the state
    n = sum(lens)
    qk, hv, hd = kvh * dim, heads * vdim, heads * dim
    C = 2 * qk + hv
    lead, s_len = 5, 13
    proj = torch.randn(n, lead + C + heads + 3, generator=g).to(dt)
    tap_w = torch.randn(C, taps, generator=g)
    state = torch.randn(4, s_len + (taps - 1) * C, generator=g)
    a_pre = (torch.randn(n, hd, generator=g) * 3).to(dt)
    dt_bias, a_log = torch.randn(hd, generator=g), torch.randn(heads, generator=g) * 0.5
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).to(torch.int32)
    dev_state = state.to(DEV)
    dproj = proj.to(DEV)
    sl = torch.tensor(slots, dtype=torch.int32, device=DEV)
    q, k, v, beta, decay = ops.delta_prep(dproj, lead, lead + C, tap_w.to(DEV), dev_state, s_len, a_pre.to(DEV), dt_bias.to(DEV),
                                          a_log.to(DEV), cu.to(DEV), seq.to(DEV), sl, heads, kvh, dim, vdim)
    ops.delta_conv_update(dproj, lead, C, taps, dev_state, s_len, cu.to(DEV), sl)
    after = dev_state.cpu()
    x = proj.double()
    for s, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        carry = state[slots[s], s_len:].double().view(taps - 1, C)
        y, new = plain.short_conv(x[a:b, lead: lead + C], tap_w.double(), carry)
        _close(q[a:b], plain.unit(y[:, :qk].reshape(-1, kvh, dim)).reshape(-1, qk) * dim ** -0.5, 1e-5, "q")
        _close(k[a:b], plain.unit(y[:, qk: 2 * qk].reshape(-1, kvh, dim)).reshape(-1, qk), 1e-5, "k")
        _close(v[a:b], y[:, 2 * qk:], 1e-5, "v")
        if taps > 1:
            _close(after[slots[s], s_len:], new.reshape(-1), 1e-6, "conv state")
        assert torch.equal(after[slots[s], :s_len], state[slots[s], :s_len])
    _close(beta, torch.sigmoid(x[:, lead + C: lead + C + heads]), 1e-6, "beta")
    want = torch.exp(-torch.exp(a_log.double())[None, :, None] * F.softplus(a_pre.double() + dt_bias.double()).view(n, heads, dim))
    _close(decay, want.reshape(n, hd), 1e-5, "decay")
    o = torch.randn(n, hv, generator=g)
    gate = torch.randn(n, hv, generator=g).to(dt)
    w = torch.randn(vdim, generator=g).to(dt)
    got = ops.delta_out_norm(o.to(DEV), gate.to(DEV), w.to(DEV), 1e-5, vdim, dt)
    want = (plain.rms(o.double().view(n, heads, vdim), 1e-5) * w.double() * torch.sigmoid(gate.double()).view(n, heads, vdim))
    _close(got, want.reshape(n, hv), 1e-5 if dt == torch.float32 else 1e-2, "output norm")
