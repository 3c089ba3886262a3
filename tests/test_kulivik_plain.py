"""The plain Kulivik implementation's mechanisms, each against what it must do."""
import math

import torch

import plain_kulivik as PK

F = torch.float64


def g(seed):
    return torch.Generator().manual_seed(seed)


def test_norm_has_eps_inside_the_root_and_a_weight_around_zero():
    x = torch.randn(3, 8, generator=g(0), dtype=F)
    w = torch.randn(8, generator=g(1), dtype=F) * 0.1
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 0.5) * (1 + w)
    assert torch.allclose(PK.norm_one_plus(x, w, 0.5), want)
    assert torch.allclose(PK.norm_one_plus(x, torch.zeros(8), 0.0), x / x.pow(2).mean(-1, keepdim=True).sqrt())


def test_token_shift_reads_the_row_before_and_zeros_before_the_first():
    h = torch.randn(5, 4, generator=g(2), dtype=F)
    mu = torch.tensor([0.0, 1.0, 0.25, 2.0], dtype=F)
    s = PK.token_shift(h, mu)
    assert torch.equal(s[:, 0], h[:, 0])                                  # mu 0: the row itself
    assert torch.allclose(s[1:, 1], h[:-1, 1]) and s[0, 1] == 0           # mu 1: the row before; zeros before the first
    assert torch.allclose(s[2, 2], 0.75 * h[2, 2] + 0.25 * h[1, 2])
    assert torch.allclose(s[0], h[0] * (1 - mu))


def test_gate_reads_the_unshifted_input():
    r, h = torch.randn(2, 3, generator=g(3), dtype=F), torch.randn(2, 3, generator=g(4), dtype=F)
    wg, bg = torch.randn(3, 3, generator=g(5), dtype=F), torch.randn(3, generator=g(6), dtype=F)
    assert torch.allclose(PK.gated(r, h, wg, bg), r / (1 + torch.exp(-(h @ wg.T + bg))))


def test_rotation_pairs_neighbours_keeps_the_tail_and_depends_on_distance():
    x = torch.randn(6, 2, 10, generator=g(7), dtype=F)
    y = PK.rotate_pairs(x, 6, 100.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    a = 3 * 100.0 ** (-2.0 / 6)   # position 3, pair 1 = dimensions (2, 3)
    assert torch.allclose(y[3, 0, 2], x[3, 0, 2] * math.cos(a) - x[3, 0, 3] * math.sin(a))
    assert torch.allclose(y[3, 0, 3], x[3, 0, 3] * math.cos(a) + x[3, 0, 2] * math.sin(a))
    q = torch.randn(1, 1, 6, generator=g(8), dtype=F).expand(6, 1, 6)
    k = torch.randn(1, 1, 6, generator=g(9), dtype=F).expand(6, 1, 6)
    rq, rk = PK.rotate_pairs(q.clone(), 6, 100.0), PK.rotate_pairs(k.clone(), 6, 100.0)
    assert torch.allclose((rq[4, 0] * rk[1, 0]).sum(), (rq[5, 0] * rk[2, 0]).sum())


def test_window_with_kept_first_tokens():
    see = PK.visible(12, window=4, keep_first=2)
    assert see[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]      # i - j < 4, or j < 2
    assert see[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert PK.visible(5)[4].all() and not PK.visible(5)[2, 3]
    assert PK.visible(12, window=4)[9].nonzero().flatten().tolist() == [6, 7, 8, 9]


def test_attention_cap_slopes_sink_and_key_head():
    T, H, G, d = 7, 4, 2, 6
    q, k = torch.randn(T, H, d, generator=g(10), dtype=F) * 3, torch.randn(T, G, d, generator=g(11), dtype=F) * 3
    v = torch.randn(T, G, 5, generator=g(12), dtype=F)
    see = PK.visible(T)
    # a cap far above every score changes nothing; a small one bounds what a towering key can take
    base = PK.softmax_attention(q, k, v, 0.3, see)
    assert torch.allclose(PK.softmax_attention(q, k, v, 0.3, see, softcap=1e6), base, atol=1e-9)
    i, h = 5, 3
    s = (q[i, h] @ k[:i + 1, h // 2].T) * 0.3
    p = torch.softmax(2.0 * torch.tanh(s / 2.0), 0)
    assert torch.allclose(PK.softmax_attention(q, k, v, 0.3, see, softcap=2.0)[i, h], p @ v[:i + 1, h // 2])
    # slopes take slope * distance off; the sink adds exp(sink) to the denominator only
    sl = PK.slopes_of(H)
    assert torch.allclose(sl, torch.tensor([2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8], dtype=F))
    p = torch.softmax(s - sl[h] * (i - torch.arange(i + 1, dtype=F)), 0)
    assert torch.allclose(PK.softmax_attention(q, k, v, 0.3, see, slopes=sl)[i, h], p @ v[:i + 1, h // 2])
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=F)
    e = torch.exp(s)
    assert torch.allclose(PK.softmax_attention(q, k, v, 0.3, see, sink=sink)[i, h], (e / (e.sum() + math.exp(0.0))) @ v[:i + 1, h // 2])
    e2 = torch.exp((q[i, 2] @ k[:i + 1, 1].T) * 0.3)
    assert torch.allclose(PK.softmax_attention(q, k, v, 0.3, see, sink=sink)[i, 2], (e2 / (e2.sum() + math.exp(2.0))) @ v[:i + 1, 1])


def test_query_temperature_steps_with_whole_stretches():
    t = PK.query_temperature(9, 0.5, 4)
    assert torch.allclose(t[:3], torch.ones(3, dtype=F))                   # floor((p + 1) / 4) = 0 for p < 3
    assert torch.allclose(t[3:7], torch.full((4,), 1 + 0.5 * math.log(2.0), dtype=F))
    assert torch.allclose(t[7], torch.tensor(1 + 0.5 * math.log(3.0), dtype=F))


def test_decaying_state_against_its_unrolled_sum():
    T, H, n, p = 6, 2, 3, 4
    q, k = torch.randn(T, H, n, generator=g(13), dtype=F), torch.randn(T, H, n, generator=g(14), dtype=F)
    v = torch.randn(T, H, p, generator=g(15), dtype=F)
    decay = [0.5, 1.0]
    o = PK.decaying_state(q, k, v, decay)
    for h in range(H):
        want = sum(decay[h] ** (5 - j) * (q[5, h] @ k[j, h]) * v[j, h] for j in range(6))
        assert torch.allclose(o[5, h], want)


def test_convolution_is_causal_starts_from_zeros_and_ends_on_the_newest():
    u = torch.randn(7, 3, generator=g(16), dtype=F)
    w = torch.randn(3, 4, generator=g(17), dtype=F)
    y = PK.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0])
    assert torch.allclose(y[5], w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4] + w[:, 3] * u[5])
    u2 = u.clone()
    u2[6] += 1
    assert torch.equal(PK.causal_conv(u2, w)[:6], y[:6])


def test_value_mixing_and_router():
    v, f = torch.randn(2, 3, generator=g(18), dtype=F), torch.randn(2, 3, generator=g(19), dtype=F)
    assert torch.allclose(PK.mix_values(v, f, 0.25), 0.75 * v + 0.25 * f)
    z = torch.tensor([[0.1, 2.0, -1.0, 1.5]], dtype=F)
    idx, wt = PK.route(z, 2)
    assert idx.tolist() == [[1, 3]]
    assert torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 1.5]], dtype=F), -1))   # over the chosen logits only


def test_dense_feed_forward_clamps_both_branches():
    h = torch.eye(2, dtype=F)
    w = {"gate": torch.tensor([[5.0, -5.0]], dtype=F).T.contiguous().T, "up": torch.tensor([[9.0, -9.0]], dtype=F),
         "down": torch.ones(1, 1, dtype=F)}
    y = PK.dense_ff({"limit": 2.0}, {"p.gate": w["gate"], "p.up": w["up"], "p.down": w["down"]}, "p.", h)
    sig = lambda x: 1 / (1 + math.exp(-x))  # noqa: E731
    assert torch.allclose(y[0, 0], torch.tensor(2.0 * sig(1.702 * 2.0) * (2.0 + 1.0), dtype=F))      # both clamped from above
    assert torch.allclose(y[1, 0], torch.tensor(-5.0 * sig(1.702 * -5.0) * (-2.0 + 1.0), dtype=F))   # gate unclamped below, up at -limit
