"""The kernels that the Bumolix layers add, alone against the plain functions: the decaying matrix state of gated linear
attention, the selective scan, the causal convolution with bias and activation, the norm per head with a gate, attention
rows whose heads are divided by their own root mean square after a partial rotation, and the norm that adds a weighted
sum of several terms and norms the result twice."""
import math

import pytest
import torch

import kernel_utils as K
import plain_bumolix as PB

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rts():
    from atoma_infer_b200.engine.runtime import make_runtime

    return {"bfloat16": make_runtime("bfloat16", "cuda:0"), "float32": make_runtime("float32", "cuda:0")}


def _portions(lens, sizes):
    """Steps of a batch of requests: per step a list of (request, start, count); long and short portions side by side."""
    at, step, steps = [0] * len(lens), 0, []
    while any(a < n for a, n in zip(at, lens)):
        cur = []
        for k, n in enumerate(lens):
            c = min(sizes[(step + 2 * k) % len(sizes)], n - at[k])
            if c > 0:
                cur.append((k, at[k], c))
                at[k] += c
        steps.append(cur)
        step += 1
    return steps


def _context(rt, cur, slots):
    ctx, _ = K.make_context(rt, [(a, c) for _, a, c in cur], 16, [[1]] * len(cur))
    ctx.state_slots.copy_(torch.tensor([slots[k] for k, _, _ in cur], dtype=torch.int32))
    return ctx


# portions of 1 and 2 tokens, of a few, and long ones that the kernels cut into chunks of time (300, 170: with a ragged
# last chunk; 128: exactly two)
SIZES = (3, 1, 300, 2, 17, 128, 1, 170, 5, 64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,N,P", [(3, 24, 16), (2, 80, 128), (4, 8, 40), (1, 64, 64), (2, 48, 32), (1, 130, 20)])
def test_decaying_matrix_state_over_portions_and_slots(rts, dtype, H, N, P):
    """Three requests in portions of many sizes, in one batch, their states in scattered slots that are slices of a wider
    per-request state; every portion's output equals the plain recurrence over the whole sequence."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(N + P)
    lens, tau, scale = [470, 9, 331], 6.0, N ** -0.5
    mk = lambda n, w: torch.randn(n, H * w, generator=g).to(rt.dtype)  # noqa: E731
    qs, ks, vs = ([mk(n, w) for n in lens] for w in (N, N, P))
    zs = [4.0 * torch.randn(n, H * N, generator=g) for n in lens]       # decays from fast to almost none
    zb = torch.randn(H * N, generator=g)
    want = []
    for q, k, v, z in zip(qs, ks, vs, zs):
        a = (torch.sigmoid(z.double() + zb.double()) ** (1 / tau)).view(-1, H, N)
        qq, kk, vv = (q.double() * scale).view(-1, H, N), k.double().view(-1, H, N), v.double().view(-1, H, P)
        want.append(torch.stack([PB.decay_recurrence(qq[:, h], kk[:, h], vv[:, h], a[:, h]) for h in range(H)], 1).flatten(1))
    slots = [4, 0, 2]
    wide = torch.zeros((5, 4 + H * N * P + 2), device=rt.device)
    state = wide[:, 4:4 + H * N * P].unflatten(1, (H, N, P))
    zbd = zb.to(rt.device)
    worst = 0.0
    for cur in _portions(lens, SIZES):
        ctx = _context(rt, cur, slots)
        cat = lambda xs: torch.cat([xs[k][a:a + c] for k, a, c in cur]).to(rt.device)  # noqa: E731
        # q, k and v as slices of one wider row, as the fused projection leaves them
        row = torch.cat([cat(qs), cat(ks), cat(vs)], dim=1)
        o = torch.full((ctx.T, H * P), float("nan"), device=rt.device)
        rt.ops.gla_scan(row[:, :H * N], row[:, H * N:2 * H * N], row[:, 2 * H * N:], cat(zs), zbd, tau, scale, state, ctx, o,
                        heads=H, dim=N, vdim=P)
        r = 0
        for k, a, c in cur:
            exp = want[k][a:a + c]
            worst = max(worst, float((o[r:r + c].cpu().double() - exp).abs().max()) / float(want[k].abs().max()))
            r += c
    rt.ops.check_status()
    assert worst < 2e-5, worst  # the inputs are the same numbers in both types; the recurrence is float32 in both
    assert float(wide[1].abs().max()) == 0.0 and float(wide[:, :4].abs().max()) == 0.0 and float(wide[:, -2:].abs().max()) == 0.0


def test_a_far_key_is_kept_by_a_channel_that_does_not_decay(rts):
    """One key channel keeps everything (decay 1 to rounding), the others forget within a few tokens: after hundreds of
    tokens, in a long portion and then token by token, a query on that channel returns the first token's value."""
    rt = rts["float32"]
    H, N, P, T = 2, 16, 8, 700
    g = torch.Generator().manual_seed(0)
    k, v = torch.randn(T, H * N, generator=g) * 0.01, torch.randn(T, H * P, generator=g)
    k[0, 5], k[1:, 5] = 4.0, 0.0                     # head 0, channel 5: written once
    z = torch.full((T, H * N), -3.0)
    z[:, 5] = 60.0                                   # sigmoid(60)^(1/tau) = 1 in float32
    q = torch.zeros(T, H * N)
    q[:, 5] = 1.0
    state = torch.zeros((1, H, N, P), device=rt.device)
    outs = []
    for a, c in [(0, 650)] + [(p, 1) for p in range(650, T)]:
        ctx = _context(rt, [(0, a, c)], [0])
        o = torch.empty((c, H * P), device=rt.device)
        rt.ops.gla_scan(q[a:a + c].to(rt.device), k[a:a + c].to(rt.device), v[a:a + c].to(rt.device), z[a:a + c].to(rt.device),
                        None, 2.0, 1.0, state, ctx, o, heads=H, dim=N, vdim=P)
        outs.append(o.cpu())
    o = torch.cat(outs)
    assert torch.allclose(o[:, :P], (4.0 * v[0, :P]).expand(T, P), rtol=1e-5, atol=1e-6)
    assert float(o[:, P:].abs().max()) == 0.0        # the other head's query is zero


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,N", [(80, 24), (96, 5), (128, 40), (48, 16), (300, 64), (33, 1)])
def test_selective_scan_over_portions_and_slots(rts, dtype, C, N):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(C + N)
    lens = [470, 9, 331]
    us, zs = ([torch.randn(n, C, generator=g).to(rt.dtype) for n in lens] for _ in range(2))
    bcs = [torch.randn(n, 2 * N, generator=g).to(rt.dtype) for n in lens]
    dts = [torch.randn(n, C, generator=g) for n in lens]
    dt_bias, a_log, d_skip = torch.randn(C, generator=g) - 1.0, 1.5 * torch.randn(C, N, generator=g), torch.randn(C, generator=g)
    want = []
    for u, z, bc, dt in zip(us, zs, bcs, dts):
        step = PB.softplus(dt.double() + dt_bias.double())
        y = PB.selective_scan(u.double(), step, -torch.exp(a_log.double()), bc[:, :N].double(), bc[:, N:].double(), d_skip.double())
        want.append(y * PB.silu(z.double()))
    slots = [3, 1, 0]
    wide = torch.zeros((4, 8 + C * N + 4), device=rt.device)
    state = wide[:, 8:8 + C * N].unflatten(1, (C, N))
    dev = lambda t: t.to(rt.device)  # noqa: E731
    worst = 0.0
    for cur in _portions(lens, SIZES):
        ctx = _context(rt, cur, slots)
        cat = lambda xs: torch.cat([xs[k][a:a + c] for k, a, c in cur]).to(rt.device)  # noqa: E731
        row = torch.cat([cat(us), cat(zs), torch.zeros((ctx.T, 8), dtype=rt.dtype, device=rt.device), cat(bcs)], dim=1)
        out = torch.full((ctx.T, C), float("nan"), dtype=rt.dtype, device=rt.device)
        rt.ops.selective_scan(row[:, :C], cat(dts).contiguous(), dev(dt_bias), row[:, 2 * C + 8:], row[:, C:2 * C], dev(a_log),
                              dev(d_skip), state, ctx, out, inner=C, nstate=N)
        r = 0
        for k, a, c in cur:
            exp = want[k][a:a + c]
            worst = max(worst, float((out[r:r + c].cpu().double() - exp).abs().max()) / float(want[k].abs().max()))
            r += c
    rt.ops.check_status()
    assert worst < (3e-5 if dtype == "float32" else 8e-3), worst  # bfloat16: the output's own rounding
    assert float(wide[2].abs().max()) == 0.0 and float(wide[:, :8].abs().max()) == 0.0


def test_a_slow_state_keeps_a_far_input(rts):
    """Channel 3 has one state that decays by exp(-1e-4) a token and reads only the first token's B: its output after
    hundreds of tokens is that input times what is left of it."""
    rt = rts["float32"]
    C, N, T = 8, 4, 600
    u, z = torch.ones(T, C), torch.full((T, C), 30.0)           # silu(30) = 30
    bc = torch.zeros(T, 2 * N)
    bc[0, 2], bc[:, N + 2] = 1.0, 1.0                           # B_2 at the first token only, C_2 always
    a_log = torch.zeros(C, N)
    a_log[3, 2] = math.log(1e-4)
    dt_raw = torch.full((T, C), math.log(math.e - 1.0))         # softplus = 1
    state = torch.zeros((1, C, N), device=rt.device)
    outs = []
    for a, c in [(0, 520)] + [(p, 1) for p in range(520, T)]:
        ctx = _context(rt, [(0, a, c)], [0])
        out = torch.empty((c, C), device=rt.device)
        rt.ops.selective_scan(u[a:a + c].to(rt.device), dt_raw[a:a + c].to(rt.device), torch.zeros(C, device=rt.device),
                              bc[a:a + c].to(rt.device), z[a:a + c].to(rt.device), a_log.to(rt.device), torch.zeros(C, device=rt.device),
                              state, ctx, out, inner=C, nstate=N)
        outs.append(out.cpu())
    y = torch.cat(outs)
    t = torch.arange(T, dtype=torch.float64)
    assert torch.allclose(y[:, 3].double(), 30.0 * torch.exp(-1e-4 * t), rtol=2e-5)
    assert torch.allclose(y[:, 0].double(), 30.0 * torch.exp(-1.0 * t), rtol=2e-5, atol=1e-30)  # a fast channel forgets it


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,C", [(4, 80), (2, 48), (5, 1100), (1, 96), (3, 256)])
def test_causal_convolution_with_bias_and_activation(rts, dtype, taps, C):
    """Requests in portions of 1 to 9 rows, and in single rows (where the kernel that reads a channel's ring also turns
    it); zeros before the start, whatever the slot held before."""
    rt = rts[dtype]
    ops = rt.ops
    g = torch.Generator().manual_seed(taps)
    lens = [23, 9, 14]
    xs = [torch.randn(n, C, generator=g).to(rt.dtype) for n in lens]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = [PB.silu(PB.causal_conv(x.double(), w.double(), b.double())) for x in xs]
    R = taps - 1
    wide = torch.empty((3, 8 + R * C + 5), device=rt.device)
    state = wide[:, 8:8 + R * C].unflatten(1, (R, C)) if R else None
    wd, bd = w.t().contiguous().to(rt.device), b.to(rt.device)  # the kernels take [taps, channels]
    tol = 1e-5 if dtype == "float32" else 2e-2
    for sizes in ((1, 2, 9, 3, 1, 1, 4, 2), (1,)):
        wide.fill_(float("nan"))  # NaN: a row read before it was written shows
        for cur in _portions(lens, sizes):
            ctx = _context(rt, cur, [0, 1, 2])
            x = torch.cat([xs[k][a:a + c] for k, a, c in cur]).to(rt.device)
            out = torch.empty((ctx.T, C), dtype=rt.dtype, device=rt.device)
            if not ops.causal_conv_act(x, wd, bd, state, ctx, out, act="silu"):
                ops.causal_conv_save(x, state, ctx, taps)
            r = 0
            for k, a, c in cur:
                exp = want[k][a:a + c]
                assert torch.allclose(out[r:r + c].double().cpu(), exp, atol=tol * float(want[k].abs().max())), (sizes, k, a)
                r += c
    ops.check_status()


@pytest.mark.parametrize("H,P", [(3, 16), (2, 128), (4, 40), (5, 8), (1, 20)])
def test_norm_per_head_with_a_shared_weight_and_a_gate(rts, H, P):
    g = torch.Generator().manual_seed(H * P)
    o, w = torch.randn(7, H * P, generator=g) * torch.rand(7, 1, generator=g) * 1e-2, 1 + 0.3 * torch.randn(P, generator=g)
    for dtype in ("float32", "bfloat16"):
        rt = rts[dtype]
        ctx, _ = K.make_context(rt, [(0, 4), (9, 3)], 16, [[1]] * 2)
        wide = torch.randn(7, 3 * H * P, generator=g).to(rt.dtype)
        gate = wide[:, H * P:2 * H * P]
        out = torch.empty((7, H * P), dtype=rt.dtype, device=rt.device)
        rt.ops.head_norm_gate(o.to(rt.device), wide.to(rt.device)[:, H * P:2 * H * P], w.to(rt.device), 1e-5, out, ctx.meta, H)
        want = (PB.rms_divide(o.double().view(7, H, P), 1e-5) * w.double()).view(7, H * P) * PB.silu(gate.double())
        assert torch.allclose(out.cpu().double(), want, atol=(1e-5 if dtype == "float32" else 1e-2) * float(want.abs().max()))
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("entries", [[(0, 5), (13, 3), (4000, 1)], [(3, 2100), (0, 7)]])
@pytest.mark.parametrize("nq,nkv,d,dv,rot,factor", [(6, 2, 16, 24, 8, 3.0), (4, 4, 24, 8, 24, 1.0), (20, 1, 16, 16, 0, 1.0),
                                                    (2, 1, 64, 64, 32, 2.0), (4, 2, 32, 48, 16, 8.0), (8, 2, 16, 16, 4, 1.0)])
def test_attention_rows_with_heads_divided_by_their_own_size(rts, dtype, entries, nq, nkv, d, dv, rot, factor):
    """Biases, the rotation of a head's first dimensions (i with i + rot / 2, stretched positions), then every q and k
    head over its own root mean square; values untouched; all at their pages' places."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(d + dv)
    page, dp, eps, base = 8, -(-max(d, dv) // 16) * 16, 1e-3, 5000.0
    tables, num_pages = K.scrambled_tables([c + n for c, n in entries], page, seed=1)
    ctx, _ = K.make_context(rt, entries, page, tables)
    T, NQ, NK, NV = ctx.T, nq * d, nkv * d, nkv * dv
    qkv = (0.05 * torch.randn(T, NQ + NK + NV, generator=g)).to(rt.dtype)   # small rows: eps counts
    bias = (0.05 * torch.randn(NQ + NK + NV, generator=g)).bfloat16().float()
    inv_freq = (torch.tensor([base ** (-2.0 * i / rot) / factor for i in range(rot // 2)], dtype=torch.float64)).float() if rot else None
    cache = torch.full((num_pages, 2, nkv, page, dp), float("nan"), dtype=rt.dtype, device=rt.device)
    q_out = torch.full((T, nq * dp), float("nan"), dtype=rt.dtype, device=rt.device)
    dev = lambda t: t.to(rt.device) if t is not None else None  # noqa: E731
    rt.ops.qkv_prepare(dev(qkv), ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=dv, dp=dp, page_size=page, num_pages=num_pages,
                       store_kv=True, bias=dev(bias.to(rt.dtype if rot % 16 == 0 else torch.float32)), eps=eps, inv_freq=dev(inv_freq),
                       rot=rot, head_norm=True)
    rt.ops.check_status()
    rows = qkv.double() + bias.double()
    pos = torch.cat([torch.arange(c, c + n) for c, n in entries])
    q = PB.rms_divide(PB.rotate_leading(rows[:, :NQ].view(T, nq, d), pos, rot, base, factor), eps)
    k = PB.rms_divide(PB.rotate_leading(rows[:, NQ:NQ + NK].view(T, nkv, d), pos, rot, base, factor), eps)
    v = rows[:, NQ + NK:].view(T, nkv, dv)
    tol = (1e-5 + 2e-7 * max(c + n for c, n in entries)) if dtype == "float32" else 2e-2
    got_q = q_out.float().cpu().view(T, nq, dp)
    assert torch.allclose(got_q[..., :d].double(), q, atol=tol * float(q.abs().max())) and (got_q[..., d:] == 0).all()
    row = 0
    for (c, n), table in zip(entries, tables):
        for p in range(c, c + n):
            kk, vv = (cache[table[p // page], i, :, p % page].float().cpu() for i in (0, 1))
            assert torch.allclose(kk[:, :d].double(), k[row], atol=tol * float(k.abs().max())) and (kk[:, d:] == 0).all()
            assert torch.allclose(vv[:, :dv].double(), v[row], atol=tol * float(v.abs().max())) and (vv[:, dv:] == 0).all()
            row += 1


@pytest.mark.parametrize("H", [96, 1000, 2048])
def test_weighted_sum_into_the_stream_and_two_norms(rts, H):
    """stream += m * (f0 t0 + f1 t1 + t2) in float32, then the same rows through two norms with weights of their own."""
    from atoma_infer_b200.parts.base import PendingSum

    g = torch.Generator().manual_seed(H)
    x = torch.randn(6, H, generator=g)
    w1, w2 = 1 + 0.2 * torch.randn(H, generator=g), 1 + 0.2 * torch.randn(H, generator=g)
    for dtype in ("float32", "bfloat16"):
        rt = rts[dtype]
        ctx, _ = K.make_context(rt, [(0, 4), (5, 2)], 16, [[1]] * 2)
        terms = [torch.randn(6, H, generator=g).to(rt.dtype) for _ in range(3)]
        pend = PendingSum(tuple(t.to(rt.device) for t in terms), 0.7, factors=(0.55, 0.85, 1.0))
        resid = x.clone().to(rt.device)
        out, out2 = (torch.empty((6, H), dtype=rt.dtype, device=rt.device) for _ in range(2))
        rt.ops.sum_rmsnorm(resid, pend, w1.to(rt.device), 1e-5, out, ctx.meta, 6, second=(w2.to(rt.device), 1e-5, out2))
        s = x.double() + 0.7 * (0.55 * terms[0].double() + 0.85 * terms[1].double() + terms[2].double())
        assert torch.allclose(resid.cpu().double(), s, atol=3e-6)                    # the stream is float32 in both modes
        tol = 1e-5 if dtype == "float32" else 1e-2
        assert torch.allclose(out.cpu().double(), PB.rms_norm(s, w1.double(), 1e-5), atol=tol * 4)
        assert torch.allclose(out2.cpu().double(), PB.rms_norm(s, w2.double(), 1e-5), atol=tol * 4)
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,N,pad", [(32, 64, 0), (6, 24, 8), (3, 20, 0), (5, 8, 3)])
def test_output_gate_on_slices_of_wider_rows(rts, dtype, heads, N, pad):
    """y[t, h, :N] *= sigmoid(gate[t, h, :N]) in place, y a slice of heads padded to N + pad and the gate the last columns of
    wider rows: slices that start on 16 bytes (sixteen bytes a thread) and slices that do not (an element a thread)."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(N)
    T, lead = 37, 40 if pad != 3 else 5
    ctx, _ = K.make_context(rt, [(0, T)], 16, [[1, 2, 3]])
    y_full = torch.randn(T, heads, N + pad, generator=g).to(rt.dtype).to(rt.device)
    rows = (3 * torch.randn(T, lead + heads * N, generator=g)).to(rt.dtype).to(rt.device)
    before = y_full.clone()
    gate = rows[:, lead:].view(T, heads, N)
    rt.ops.sigmoid_gate(y_full[:, :, :N], gate, ctx.meta)
    rt.ops.check_status()
    want = before.double()
    want[:, :, :N] *= torch.sigmoid(gate.double())
    tol = 1e-6 if dtype == "float32" else 1e-2
    assert torch.allclose(y_full.double(), want, atol=tol, rtol=tol)
    assert torch.equal(y_full[:, :, N:], before[:, :, N:])
