"""The kernels that the Kulivik layers add or extend, alone against the plain functions: the norm with the row shifted
toward the token before (over portions and slots), the gated, normed sum into the stream, attention whose scores are
capped, biased by distance or masked by a window that keeps the first tokens (one key made to tower just inside or just
outside every edge), attention rows with a weighted norm per head before an interleaved rotation and a query temperature,
linear attention with constant decays, the clamped gated activation, the gate per head, the norm over the whole row with
a gate, the scaled soft cap, and the router with a bias and weights over the chosen experts."""
import math

import pytest
import torch

import kernel_utils as K
import plain_kulivik as PK
from atoma_infer_b200.parts.base import PendingSum

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rts():
    from atoma_infer_b200.engine.runtime import make_runtime

    return {"bfloat16": make_runtime("bfloat16", "cuda:0"), "float32": make_runtime("float32", "cuda:0")}


def _portions(lens, sizes):
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [72, 256, 1030])
def test_norm_and_shift_over_portions_and_slots(rts, dtype, H):
    """Three requests in portions of 1, 2 and more tokens in one batch; the kept row lives in scattered slots that are
    slices of a wider state and reaches them through the gated sum's kernel; a slot that held another request's row
    reads as zeros at position 0."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(H)
    lens = [37, 5, 60]
    xs = [torch.randn(n, H, generator=g) * 3 for n in lens]
    w, mu = 1 + 0.2 * torch.randn(H, generator=g), torch.rand(H, generator=g) * 1.2
    want_h = [PK.rms(x.double(), 1e-5) * w.double() for x in xs]
    want_s = [PK.token_shift(h, mu.double()) for h in want_h]
    slots = [3, 0, 1]
    wide = torch.full((4, 8 + H + 4), 7.0, device=rt.device)     # (whatever an earlier request left)
    state = wide[:, 8:8 + H]
    dev = lambda t: t.to(rt.device)  # noqa: E731
    tol = 1e-5 if dtype == "float32" else 1e-2
    for cur in _portions(lens, (3, 1, 2, 9, 1, 20)):
        ctx = _context(rt, cur, slots)
        resid = torch.cat([xs[k][a:a + c] for k, a, c in cur]).to(rt.device)
        h = torch.full((ctx.T, H), float("nan"), dtype=rt.dtype, device=rt.device)
        hs, last = torch.full_like(h, float("nan")), torch.full((ctx.S, H), float("nan"), device=rt.device)
        rt.ops.norm_shift(resid, dev(w), 1e-5, ctx, shift=dev(mu), state=state, h=h, hs=hs, last=last)
        # the sum's kernel moves the kept rows into the state (its terms here are zeros)
        zero = torch.zeros((ctx.T, H), dtype=rt.dtype, device=rt.device)
        rt.ops.gated_norm_add(resid.clone(), PendingSum((zero,)), torch.zeros((ctx.T, H), device=rt.device), None, dev(w), 1e-5, ctx,
                              keep=(last, state))
        r = 0
        for k, a, c in cur:
            assert torch.allclose(h[r:r + c].float().cpu().double(), want_h[k][a:a + c], atol=tol * 4)
            assert torch.allclose(hs[r:r + c].float().cpu().double(), want_s[k][a:a + c], atol=tol * 4), (k, a, c)
            assert torch.allclose(state[slots[k]].cpu().double(), want_h[k][a + c - 1], atol=1e-5 * 4)
            r += c
    rt.ops.check_status()
    assert float((wide[:, :8] - 7).abs().max()) == 0 and float((wide[:, -4:] - 7).abs().max()) == 0 and float((wide[2] - 7).abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,terms", [(72, 1), (256, 2), (1030, 3)])
def test_gated_normed_sum_into_the_stream(rts, dtype, H, terms):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(H + terms)
    T = 7
    ctx, _ = K.make_context(rt, [(0, 4), (9, 3)], 16, [[1], [2]])
    ts = [torch.randn(T, H, generator=g).to(rt.dtype) for _ in range(terms)]
    fs = [0.7, 0.45, -1.25][:terms]
    vec, gate, gb = torch.randn(H, generator=g), 2 * torch.randn(T, H, generator=g), torch.randn(H, generator=g)
    w, w2 = 1 + 0.2 * torch.randn(H, generator=g), 1 + 0.2 * torch.randn(H, generator=g)
    x = torch.randn(T, H, generator=g)
    y = 0.9 * sum(f * t.double() for f, t in zip(fs, ts)) + vec.double()
    y = y * torch.sigmoid(gate.double() + gb.double())
    want = x.double() + PK.rms(y, 1e-6) * w.double()
    want2 = PK.rms(want, 1e-4) * w2.double()
    dev = lambda t: t.to(rt.device)  # noqa: E731
    resid, out = dev(x.clone()), torch.full((T, H), float("nan"), dtype=rt.dtype, device=rt.device)
    rt.ops.gated_norm_add(resid, PendingSum(tuple(dev(t) for t in ts), 0.9, vector=dev(vec), factors=tuple(fs)), dev(gate), dev(gb),
                          dev(w), 1e-6, ctx, next_norm=(dev(w2), 1e-4, out))
    rt.ops.check_status()
    assert torch.allclose(resid.cpu().double(), want, atol=2e-5 * float(want.abs().max()))
    assert torch.allclose(out.float().cpu().double(), want2, atol=(2e-5 if dtype == "float32" else 1e-2) * float(want2.abs().max()))


def _scores_case(rt, entries, nq, nkv, d, page, *, window=0, keep_first=0, softcap=0.0, slopes=False, sink=False, seed=0,
                 stand_out=None, fast=True):
    """Attention of a step over a hand-filled cache; returns the largest difference from the plain attention."""
    g = torch.Generator().manual_seed(seed)
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page, seed)
    qs, ks, vs = ([torch.randn(L, h, d, generator=g) for L in lengths] for h in (nq, nkv, nkv))
    if stand_out is not None:  # (key, query): that key towers for that query, if the query may see it
        for q, k, (key, qi) in zip(qs, ks, stand_out):
            k[key] *= 3.0
            q[qi] = k[key].repeat_interleave(nq // nkv, dim=0) * 1.5
    qs, ks, vs = ([t.to(rt.dtype).float() for t in x] for x in (qs, ks, vs))
    cache = torch.full((num_pages, 2, nkv, page, d), float("nan"), dtype=rt.dtype, device=rt.device)
    K.fill_cache(cache, tables, ks, vs, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    q = torch.cat([x[c:c + n].reshape(n, nq * d) for (c, n), x in zip(entries, qs)]).to(rt.dtype).to(rt.device)
    out = torch.full((ctx.T, nq * d), float("nan"), dtype=rt.dtype, device=rt.device)
    sl = PK.slopes_of(nq) if slopes else None
    sk = torch.randn(nq, generator=g) if sink else None
    ops = rt.ops
    ops.scored_fast_attention = fast
    try:
        ops.attention(q, nq * d, cache, ctx, 0, out, nq, nkv, d, page, num_pages, window, 1 / math.sqrt(d),
                      sink=sk.to(rt.device) if sink else False, keep_first=keep_first, softcap=softcap,
                      slopes=sl.float().to(rt.device) if slopes else None)
    finally:
        ops.scored_fast_attention = True
    ops.check_status()
    worst, row = 0.0, 0
    for (c, n), qq, k, v in zip(entries, qs, ks, vs):
        L = c + n
        see = PK.visible(L, window or None, keep_first)
        want = PK.softmax_attention(qq.double(), k.double(), v.double(), 1 / math.sqrt(d), see, softcap=softcap or None, slopes=sl,
                                    sink=sk.double() if sink else None)[c:]
        worst = max(worst, float((out[row:row + n].float().cpu().view(n, nq, d).double() - want).abs().max()))
        row += n
    return worst


SCORE_KINDS = {"window+kept+cap": dict(softcap=3.0), "window+kept": dict(), "slopes": dict(slopes=True),
               "cap+slopes+sink": dict(softcap=5.0, slopes=True, sink=True)}


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,nkv,page,window,keep", [(48, 6, 2, 16, 36, 5), (64, 4, 1, 8, 64, 9), (32, 6, 3, 4, 21, 30), (128, 2, 2, 16, 100, 1),
                                                        (16, 8, 8, 16, 7, 0), (64, 4, 2, 16, 50, 0)])
def test_scores_in_prompt_portions(rts, dtype, fast, d, nq, nkv, page, window, keep):
    """Portions that start and end anywhere, beside single tokens; for the last query of each request one key towers: the
    newest key outside its window, the oldest inside, the last kept token, and the first token that is not kept."""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    entries = [(0, 3 * window + 5), (window - 2, 7), (2 * window - 1, 1), (window + 3, 2), (5, 2 * window), (0, 1), (1, 2)]
    for kind, opts in SCORE_KINDS.items():
        windowed = kind.startswith("window")
        for which in ("outside", "inside", "last kept", "first not kept"):
            marks = []
            for c, n in entries:
                last = c + n - 1
                edge = {"outside": last - window, "inside": last - window + 1, "last kept": keep - 1, "first not kept": keep}[which]
                marks.append((min(max(edge, 0), last), last))
            # head sizes 64 and 128 with pages of 8 and more, nothing kept: the tcgen05 kernel, and the mma.sync kernel in its place
            for tc in ((True, False) if dtype == "bfloat16" and fast and d in (64, 128) else (True,)):
                rt.ops.tc_attention = tc
                try:
                    err = _scores_case(rt, entries, nq, nkv, d, page, window=window if windowed else 0, keep_first=keep if windowed else 0,
                                       seed=window, stand_out=marks, fast=fast, **opts)
                finally:
                    rt.ops.tc_attention = True
                assert err < tol, (kind, which, tc, err)


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,nkv,page,window,keep", [(48, 6, 2, 16, 36, 5), (64, 8, 1, 8, 512, 20), (32, 6, 3, 4, 21, 30), (128, 4, 2, 16, 300, 3)])
def test_scores_in_decode_steps(rts, dtype, fast, d, nq, nkv, page, window, keep):
    """Every request brings one token: at the start of a sequence, while the window still holds everything, when it has
    just begun to pass over the kept tokens' neighbours, and far beyond."""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    ctxs = [0, 1, keep, window - 1, window, window + keep, window + keep + 1, 3 * window + 7, 2000]
    entries = [(p, 1) for p in ctxs]
    for kind, opts in SCORE_KINDS.items():
        windowed = kind.startswith("window")
        for which in ("outside", "inside", "last kept", "first not kept"):
            marks = []
            for p, _ in entries:
                edge = {"outside": p - window, "inside": p - window + 1, "last kept": keep - 1, "first not kept": keep}[which]
                marks.append((min(max(edge, 0), p), p))
            err = _scores_case(rt, entries, nq, nkv, d, page, window=window if windowed else 0, keep_first=keep if windowed else 0,
                               seed=window + 1, stand_out=marks, fast=fast, **opts)
            assert err < tol, (kind, which, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("entries", [[(0, 5), (13, 3), (40, 1)], [(3, 2100), (0, 7)]])
@pytest.mark.parametrize("nq,nkv,d,dv,rot,qt", [(6, 2, 48, 48, 48, None), (6, 2, 24, 16, 8, (0.4, 7)), (4, 4, 16, 32, 16, None),
                                                (3, 1, 40, 40, 0, (0.3, 64)), (2, 2, 18, 10, 6, (0.7, 3)), (2, 1, 20, 20, 12, None)])
def test_rows_with_a_weighted_norm_per_head_before_an_interleaved_rotation(rts, dtype, entries, nq, nkv, d, dv, rot, qt):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(d + dv)
    page, dp = 8, -(-max(d, dv) // 16) * 16
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page, 1)
    ctx, _ = K.make_context(rt, entries, page, tables)
    T, NQ, NK, NV = ctx.T, nq * d, nkv * d, nkv * dv
    qkv = torch.randn(T, NQ + NK + NV, generator=g).to(rt.dtype)
    bias = torch.randn(NQ + NK + NV, generator=g).bfloat16().float()
    qn, kn = (1 + 0.3 * torch.randn(d, generator=g)).bfloat16().float(), (1 + 0.3 * torch.randn(d, generator=g)).bfloat16().float()
    inv_freq = (100.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float() if rot else None
    cache = torch.full((num_pages, 2, nkv, page, dp), float("nan"), dtype=rt.dtype, device=rt.device)
    q_out = torch.full((T, nq * dp), float("nan"), dtype=rt.dtype, device=rt.device)
    dev = lambda t: t.to(rt.device) if t is not None else None  # noqa: E731
    rt.ops.qkv_prepare(dev(qkv), ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=dv, dp=dp, page_size=page, num_pages=num_pages,
                       store_kv=True, bias=dev(bias), q_norm=dev(qn), k_norm=dev(kn), eps=1e-5, inv_freq=dev(inv_freq), rot=rot,
                       head_norm=True, interleaved=True, q_temp=qt)
    rt.ops.check_status()
    rows = qkv.double() + bias.double()
    pos = torch.cat([torch.arange(c, c + n) for c, n in entries])
    q = PK.rms(rows[:, :NQ].view(T, nq, d), 1e-5) * qn.double()
    k = PK.rms(rows[:, NQ:NQ + NK].view(T, nkv, d), 1e-5) * kn.double()

    if rot:
        # rotate_pairs counts positions from 0: each entry's rows are placed in a sequence as long as its last position
        qo, ko, r = [], [], 0
        for c, n in entries:
            p = torch.arange(c, c + n)
            fq = torch.zeros((c + n, nq, d), dtype=q.dtype)
            fk = torch.zeros((c + n, nkv, d), dtype=k.dtype)
            fq[p], fk[p] = q[r:r + n], k[r:r + n]
            qo.append(PK.rotate_pairs(fq, rot, 100.0)[p])
            ko.append(PK.rotate_pairs(fk, rot, 100.0)[p])
            r += n
        q, k = torch.cat(qo), torch.cat(ko)
    if qt:
        q = q * (1.0 + qt[0] * torch.log(torch.floor((pos.double() + 1) / qt[1]) + 1.0))[:, None, None]
    v = rows[:, NQ + NK:].view(T, nkv, dv)
    tol = (1e-5 + 2e-7 * max(lengths)) if dtype == "float32" else 2e-2
    got_q = q_out.float().cpu().view(T, nq, dp)
    assert torch.allclose(got_q[..., :d].double(), q, atol=tol * float(q.abs().max())) and (got_q[..., d:] == 0).all()
    row = 0
    for (c, n), table in zip(entries, tables):
        for p in range(c, c + n):
            kk, vv = (cache[table[p // page], i, :, p % page].float().cpu() for i in (0, 1))
            assert torch.allclose(kk[:, :d].double(), k[row], atol=tol * float(k.abs().max())) and (kk[:, d:] == 0).all()
            assert torch.allclose(vv[:, :dv].double(), v[row], atol=tol * float(v.abs().max())) and (vv[:, dv:] == 0).all()
            row += 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,N,P", [(3, 32, 32), (2, 24, 16), (3, 16, 8), (1, 40, 24), (4, 8, 40), (2, 128, 64)])
def test_constant_decays_over_portions_and_slots(rts, dtype, H, N, P):
    """Three requests in portions of many sizes in one batch (long ones run as chunks of time side by side), one head that
    never forgets: every portion's output equals the plain recurrence over the whole sequence."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(N + P)
    lens = [470, 9, 331]
    mk = lambda n, w: torch.randn(n, H * w, generator=g).to(rt.dtype)  # noqa: E731
    qs, ks, vs = ([mk(n, w) for n in lens] for w in (N, N, P))
    decay = [1.0, 0.6, 0.97, 0.995][:H]
    want = []
    for q, k, v in zip(qs, ks, vs):
        qq, kk, vv = (PK.silu(x.double()) for x in (q, k, v))
        want.append(PK.decaying_state(qq.view(-1, H, N), kk.view(-1, H, N), vv.view(-1, H, P), decay).flatten(1))
    slots = [4, 0, 2]
    wide = torch.zeros((5, 4 + H * N * P + 2), device=rt.device)
    state = wide[:, 4:4 + H * N * P].unflatten(1, (H, N, P))
    dec = torch.tensor(decay, dtype=torch.float32, device=rt.device)
    worst = 0.0
    for cur in _portions(lens, (3, 1, 300, 2, 17, 128, 1, 170, 5, 64)):
        ctx = _context(rt, cur, slots)
        cat = lambda xs: torch.cat([xs[k][a:a + c] for k, a, c in cur]).to(rt.device)  # noqa: E731
        row = torch.cat([cat(qs), cat(ks), cat(vs)], dim=1)
        o = torch.full((ctx.T, H * P), float("nan"), device=rt.device)
        rt.ops.gla_scan(row[:, :H * N], row[:, H * N:2 * H * N], row[:, 2 * H * N:], None, None, 1.0, 1.0, state, ctx, o,
                        heads=H, dim=N, vdim=P, head_decay=dec, silu=True)
        r = 0
        for k, a, c in cur:
            worst = max(worst, float((o[r:r + c].cpu().double() - want[k][a:a + c]).abs().max()) / float(want[k].abs().max()))
            r += c
    rt.ops.check_status()
    assert worst < 2e-5, worst
    assert float(wide[1].abs().max()) == 0.0 and float(wide[:, :4].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_maps(rts, dtype):
    """The clamped gated activation, the gate per head, the norm over the whole row with a gate, the scaled soft cap."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(5)
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    dev = lambda t: t.to(rt.device)  # noqa: E731
    ctx, rows = K.make_context(rt, [(0, 4), (9, 3)], 16, [[1], [2]], rows=[1, 3, 6])
    T = 7
    for F in (24, 257, 1024):
        gu = (3 * torch.randn(T, 2 * F, generator=g)).to(rt.dtype)
        out = torch.full((T, F), float("nan"), dtype=rt.dtype, device=rt.device)
        rt.ops.clamped_glu(dev(gu), out, 1.25, 1.702, ctx.meta)
        gg, uu = gu[:, :F].double().clamp(max=1.25), gu[:, F:].double().clamp(-1.25, 1.25)
        assert torch.allclose(out.float().cpu().double(), gg * torch.sigmoid(1.702 * gg) * (uu + 1), atol=tol * 4)
    for heads, n, pad in ((5, 48, 64), (3, 10, 16), (8, 128, 128)):
        y = torch.randn(T, heads, pad, generator=g).to(rt.dtype)
        gate = torch.randn(T, heads + 5, generator=g).to(rt.dtype)
        yd, gd = dev(y), dev(gate)
        rt.ops.head_gate(yd[:, :, :n], gd[:, 2:2 + heads], ctx.meta)
        want = y.double()
        want[:, :, :n] = want[:, :, :n] * torch.sigmoid(gate[:, 2:2 + heads].double())[:, :, None]
        assert torch.allclose(yd.float().cpu().double(), want, atol=tol * 4)
    for n in (96, 128, 1030):
        o = 2 * torch.randn(T, n, generator=g)
        gate = torch.randn(T, n + 8, generator=g).to(rt.dtype)
        w = 1 + 0.2 * torch.randn(n, generator=g)
        out = torch.full((T, n), float("nan"), dtype=rt.dtype, device=rt.device)
        rt.ops.row_norm_gate(dev(o), dev(gate)[:, 8:], dev(w), 1e-5, out, ctx.meta, kind="sigmoid")
        want = PK.rms(o.double(), 1e-5) * w.double() * torch.sigmoid(gate[:, 8:].double())
        assert torch.allclose(out.float().cpu().double(), want, atol=tol * 4)
    z = 20 * torch.randn(3, 515, generator=g)
    for scale, cap in ((2.5, 20.0), (1.0, 0.0), (0.5, 4.0)):
        zd = dev(z.clone())
        rt.ops.scale_softcap(zd, scale, cap, ctx.meta)
        want = cap * torch.tanh(z.double() * scale / cap) if cap else z.double() * scale
        assert torch.allclose(zd.cpu().double(), want, atol=1e-5 * float(want.abs().max()))
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,H", [(12, 3, 192), (5, 1, 96), (3, 3, 72), (64, 8, 130)])
def test_router_with_a_bias_and_weights_over_the_chosen(rts, dtype, E, top, H):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(E + H)
    T = 9
    ctx, _ = K.make_context(rt, [(0, T)], 16, [[1]])
    h = torch.randn(T, H, generator=g).to(rt.dtype)
    w, b = torch.randn(E, H, generator=g) * 0.3, 2 * torch.randn(E, generator=g)
    ids = torch.full((T, top), -1, dtype=torch.int32, device=rt.device)
    wts = torch.full((T, top), float("nan"), device=rt.device)
    rt.ops.moe_route(h.to(rt.device), w.to(rt.device), ids, wts, ctx.meta, bias=b.to(rt.device), over_chosen=True)
    rt.ops.check_status()
    idx, wt = PK.route(h.double() @ w.double().T + b.double(), top)
    assert ids.cpu().tolist() == idx.tolist()
    assert torch.allclose(wts.cpu().double(), wt, atol=1e-5)
