"""The plain Bumolix implementation against what each mechanism must do, without the engine."""
import math

import torch

import plain_bumolix as PB

torch.manual_seed(0)
F64 = torch.float64


def test_rotation_pairs_halves_keeps_the_tail_stretches_positions_and_depends_on_distance():
    q, k = torch.randn(1, 1, 10, dtype=F64), torch.randn(1, 1, 10, dtype=F64)
    r = PB.rotate_leading(q, torch.tensor([3]), 6, 100.0, 2.0)
    assert torch.equal(r[..., 6:], q[..., 6:])
    a = 3 * 100.0 ** (-2.0 / 6) / 2.0                                                 # i = 1 pairs dimensions 1 and 4
    assert torch.allclose(r[0, 0, 1], q[0, 0, 1] * math.cos(a) - q[0, 0, 4] * math.sin(a))
    assert torch.allclose(r[0, 0, 4], q[0, 0, 4] * math.cos(a) + q[0, 0, 1] * math.sin(a))
    assert torch.equal(PB.rotate_leading(q, torch.tensor([3]), 0, 100.0), q)          # no rotation at all
    # a stretch by f is the unstretched rotation at position p / f
    assert torch.allclose(PB.rotate_leading(q, torch.tensor([8]), 10, 50.0, 4.0), PB.rotate_leading(q, torch.tensor([2]), 10, 50.0))
    dot = lambda pq, pk: float((PB.rotate_leading(q, torch.tensor([pq]), 10, 1e4, 3.0)  # noqa: E731
                                * PB.rotate_leading(k, torch.tensor([pk]), 10, 1e4, 3.0)).sum())
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9


def test_chunk_edges_the_sink_and_the_key_head_of_a_query_head():
    T, H, G, C = 11, 4, 2, 4
    q, k = torch.zeros(T, H, 3, dtype=F64), torch.zeros(T, G, 3, dtype=F64)           # every score 0: weights 1 / (1 + keys)
    v = torch.zeros(T, G, T, dtype=F64)
    for t in range(T):
        v[t, :, t] = 1.0                                                              # the output lists the weights by key
    v[:, 1] *= 2.0
    o = PB.chunk_sink_attention(q, k, v, 1.0, C)
    assert torch.allclose(o[6, 0, 4:7], torch.full((3,), 1 / 4, dtype=F64)) and float(o[6, 0, :4].abs().sum()) == 0.0
    assert float(o[6, 0, 7:].abs().sum()) == 0.0
    assert torch.allclose(o[8, 0, 8], torch.tensor(1 / 2, dtype=F64)) and float(o[8, 0, :8].abs().sum()) == 0.0  # a chunk's first token
    assert torch.allclose(o[7, 0, 4:8], torch.full((4,), 1 / 5, dtype=F64))           # a chunk's last token sees all of it
    assert torch.allclose(o[6, 1], o[6, 0]) and torch.allclose(o[6, 2], 2 * o[6, 0]) and torch.allclose(o[6, 3], o[6, 2])
    full = PB.chunk_sink_attention(q, k, v, 1.0, 0)                                    # no chunks: every earlier key
    assert torch.allclose(full[6, 0, :7], torch.full((7,), 1 / 8, dtype=F64))
    nosink = PB.chunk_sink_attention(q, k, v, 1.0, C, sink=False)
    assert torch.allclose(nosink[6, 0, 4:7], torch.full((3,), 1 / 3, dtype=F64))
    q2 = q.clone()
    q2[6, 0, 0], k2 = 1.0, k.clone()
    k2[5, 0, 0] = math.log(3.0) / 0.5                                                  # one score log 3 after the scale
    o2 = PB.chunk_sink_attention(q2, k2, v, 0.5, C)
    assert torch.allclose(o2[6, 0, 5], torch.tensor(3 / 6, dtype=F64)) and torch.allclose(o2[6, 0, 4], torch.tensor(1 / 6, dtype=F64))


def test_unit_heads_have_no_weight_and_eps_inside_the_root():
    x = torch.randn(2, 3, 8, dtype=F64)
    y = PB.rms_divide(x, 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(2, 3, dtype=F64))
    z = PB.rms_divide(torch.zeros(1, 4, dtype=F64), 0.25)
    assert torch.equal(z, torch.zeros(1, 4, dtype=F64))
    one = PB.rms_divide(torch.full((1, 4), 1.5, dtype=F64), 4.0)
    assert torch.allclose(one, torch.full((1, 4), 1.5 / math.sqrt(1.5 ** 2 + 4.0), dtype=F64))


def test_decay_recurrence_equals_its_unrolled_sum_and_decays_key_rows():
    T, N, P = 7, 4, 3
    q, k, v = torch.randn(T, N, dtype=F64), torch.randn(T, N, dtype=F64), torch.randn(T, P, dtype=F64)
    a = torch.rand(T, N, dtype=F64)
    o = PB.decay_recurrence(q, k, v, a)
    t = T - 1
    want = torch.zeros(P, dtype=F64)
    for s in range(t + 1):  # o_t = sum_s (sum_n q_t[n] k_s[n] prod_{s < r <= t} a_r[n]) v_s
        w = (q[t] * k[s] * a[s + 1:t + 1].prod(0)).sum()
        want += w * v[s]
    assert torch.allclose(o[t], want)
    assert torch.allclose(o[0], (q[0] @ k[0]) * v[0])                                  # the first token's own decay meets a zero state
    a2 = a.clone()
    a2[3, 1] = 0.0                                                                     # key channel 1 forgets at t = 3 ...
    q1 = torch.zeros(T, N, dtype=F64)
    q1[:, 1] = 1.0                                                                     # ... and a query on that channel alone
    o2 = PB.decay_recurrence(q1, k, v, a2)
    assert torch.allclose(o2[3], k[3, 1] * v[3])                                       # sees only what came since


def test_selective_scan_equals_its_unrolled_sum():
    T, C, N = 6, 3, 4
    u, dt = torch.randn(T, C, dtype=F64), torch.rand(T, C, dtype=F64) + 0.1
    A, B, Cm, D = -torch.rand(C, N, dtype=F64), torch.randn(T, N, dtype=F64), torch.randn(T, N, dtype=F64), torch.randn(C, dtype=F64)
    y = PB.selective_scan(u, dt, A, B, Cm, D)
    t, c = T - 1, 1
    want = D[c] * u[t, c]
    for s in range(t + 1):
        for n in range(N):
            want = want + Cm[t, n] * B[s, n] * dt[s, c] * u[s, c] * torch.exp(A[c, n] * dt[s + 1:t + 1, c].sum())
    assert torch.allclose(y[t, c], want)


def test_convolution_is_causal_starts_from_zeros_and_ends_on_the_current_token():
    u, w, b = torch.randn(9, 5, dtype=F64), torch.randn(5, 3, dtype=F64), torch.randn(5, dtype=F64)
    y = PB.causal_conv(u, w, b)
    assert torch.allclose(y[0], b + w[:, 2] * u[0])
    assert torch.allclose(y[4], b + w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4])
    one = PB.causal_conv(u, w[:, :1], b)
    assert torch.allclose(one, b + w[:, 0] * u)                                        # one tap: no neighbours


def test_activations():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.7, 40.0], dtype=F64)
    assert torch.allclose(PB.relu_squared(z), torch.tensor([0.0, 0.0, 0.0, 0.49, 1600.0], dtype=F64))
    assert torch.allclose(PB.softplus(z), torch.tensor([math.log1p(math.exp(v)) if v < 30 else v for v in z.tolist()], dtype=F64))
    assert torch.allclose(PB.silu(z), torch.tensor([v / (1 + math.exp(-v)) for v in z.tolist()], dtype=F64))


def test_a_layer_reads_one_stream_through_two_norms_and_scales_the_sum():
    cfg = {"norm": {"eps": 1e-5}, "residual_mult": 0.25,
           "layers": [{"type": "mamba1", "mixer": {"inner": 6, "state": 3, "dt_rank": 2, "conv": 2}, "mlp": {"kind": "dense", "ff": 5}}]}
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)  # noqa: E731
    W = {"l0.norm1": r(4), "l0.norm2": r(4), "l0.mix.in": r(12, 4), "l0.mix.conv": r(6, 2), "l0.mix.conv.b": r(6), "l0.mix.x": r(8, 6),
         "l0.mix.dt": r(6, 2), "l0.mix.dt.b": r(6), "l0.mix.A_log": r(6, 3), "l0.mix.D": r(6), "l0.mix.o": r(4, 6),
         "l0.mlp.up": r(5, 4), "l0.mlp.down": r(4, 5)}
    x = r(5, 4)
    ly = cfg["layers"][0]
    out = PB.layer(x, W, 0, ly, cfg)
    mix = PB.mamba1_mixer(PB.rms_norm(x, W["l0.norm1"], 1e-5), W, "l0.mix", ly["mixer"])
    ff = PB.feed_forward(PB.rms_norm(x, W["l0.norm2"], 1e-5), W, "l0.mlp")
    assert torch.allclose(out, x + 0.25 * (mix + ff))
    alone = PB.layer(x, W, 0, dict(ly, mlp=None), cfg)
    assert torch.allclose(alone, x + 0.25 * mix)
