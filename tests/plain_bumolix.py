"""Plain, slow implementation of the Bumolix design, one function per mechanism, float64 by default.

It is the oracle of the tests: written from the design's equations in this file's own notation, over whole sequences,
with no cache, no pages and no state slots, and it shares no code with the package.  A model is a dict ``cfg`` (the
parsed config.json) and a dict ``W`` of tensors by checkpoint name.

Notation.  A layer reads the stream x [T, width]:  x <- x + m (mixer(n1(x)) + ff(n2(x))), n(x) = x / rms(x) * w with
rms(x) = sqrt(mean(x^2) + eps).  A ``parallel`` mixer is a_L * left(h) + a_R * right(h):
  left   grouped-query attention: biased q, k, v; rotation of the first R dims of a head (i pairs with i + R/2, angle
         p * base^(-2i/R) / factor); q and k divided by their own rms per head; scores scale * q.k inside the chunk
         floor(i / C) = floor(j / C), j <= i; weights e^s / (1 + sum e^s); heads times sigmoid(W_g h); W_o.
  right  gated linear attention: per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q scaled by
         dim^(-1/2) and a_t = sigmoid(W_a2 W_a1 h + b)^(1/tau); o / rms(o) * w per head, times silu(W_g h), W_o.
A ``mamba1`` mixer: [u | z] = W_in h; u <- silu(conv(u) + b); [d | B | C] = W_x u; dt = softplus(W_dt d + b_dt);
S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n with A = -exp(A_log); y_c = sum_n S[c, n] C_n + D_c u_c;
out = W_o (y silu(z)).  Feed-forward: W_down relu(W_up h)^2.  Logits: embed n_final(x).
"""
from __future__ import annotations

import math

import torch

DT = torch.float64

# A yardstick for reduced precision, not a second oracle: with ROUND set to a narrower type, what a matrix product reads
# and what it writes (and what is stored between a product and the next) is rounded to that type, everything else stays
# as it is.  The difference from the exact run says how much a position's logits amplify such roundings.
ROUND = None


def rnd(x):
    return x.to(ROUND).to(x.dtype) if ROUND is not None else x


def lin(x, w, b=None, keep=False):
    """w x (+ b) row by row; ``keep``: the result is not rounded (it stays wide in every mode)."""
    y = rnd(x) @ w.T
    if b is not None:
        y = y + b
    return y if keep else rnd(y)


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_divide(x, eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def relu_squared(x):
    return torch.relu(x) ** 2


def rotate_leading(x, positions, dims, base, factor=1.0):
    """x [T, heads, D]: the first ``dims`` dimensions of every head turn, dimension i with i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None, None] * freq
    cs, sn = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cs - v * sn, v * cs + u * sn, x[..., dims:]], -1)


def chunk_sink_attention(q, k, v, scale, chunk, sink=True):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence from position 0.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        lo = (i // chunk) * chunk if chunk else 0
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            e = torch.exp(s)
            p = e / ((1.0 if sink else 0.0) + e.sum())
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def left_mixer(h, W, pre, c, eps):
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = torch.arange(T)
    q = lin(h, W[pre + ".q"], W[pre + ".q.b"]).view(T, H, D)
    k = lin(h, W[pre + ".k"], W[pre + ".k.b"]).view(T, G, D)
    v = lin(h, W[pre + ".v"], W[pre + ".v.b"]).view(T, G, Dv)
    rot = c.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_leading(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_leading(k, pos, rot["dims"], rot["base"], factor)
    q, k = rnd(rms_divide(q, eps)), rnd(rms_divide(k, eps))
    chunk = (c.get("mask") or {}).get("size", 0)
    o = chunk_sink_attention(q, k, v, c["scale"], chunk).reshape(T, H * Dv)
    o = rnd(o) * torch.sigmoid(lin(h, W[pre + ".g"]))
    return lin(o, W[pre + ".o"])


def decay_recurrence(q, k, v, a):
    """One head: q, k, a [T, N], v [T, P]; S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, N = k.shape
    S = torch.zeros(N, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = a[t][:, None] * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def right_mixer(h, W, pre, c, eps):
    T = h.shape[0]
    H, N, P = c["heads"], c["dim"], c["vdim"]
    q = lin(h, W[pre + ".q"]).view(T, H, N) * N ** -0.5
    k = lin(h, W[pre + ".k"]).view(T, H, N)
    v = lin(h, W[pre + ".v"]).view(T, H, P)
    z = lin(lin(h, W[pre + ".a1"]), W[pre + ".a2"], W[pre + ".a2.b"], keep=True)
    a = (torch.sigmoid(z) ** (1.0 / c["tau"])).view(T, H, N)
    o = torch.stack([decay_recurrence(q[:, i], k[:, i], v[:, i], a[:, i]) for i in range(H)], 1)   # [T, H, P]
    o = rms_divide(o, eps) * W[pre + ".norm"]
    return lin(o.reshape(T, H * P) * silu(lin(h, W[pre + ".g"])), W[pre + ".o"])


def parallel_mixer(h, W, pre, c, eps):
    return (c["left_scale"] * left_mixer(h, W, pre + ".left", c["left"], eps)
            + c["right_scale"] * right_mixer(h, W, pre + ".right", c["right"], eps))


def causal_conv(u, w, b):
    """u [T, C], w [C, taps] (last column: the current token), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u])
    return sum(padded[j:j + T] * w[:, j] for j in range(taps)) + b


def selective_scan(u, dt, A, B, C, D):
    """u, dt [T, C]; A [C, N]; B, C [T, N]; D [C]."""
    S = torch.zeros_like(A)
    ys = []
    for t in range(u.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + D * u[t])
    return torch.stack(ys)


def mamba1_mixer(h, W, pre, c):
    inner, N, R = c["inner"], c["state"], c["dt_rank"]
    xz = lin(h, W[pre + ".in"])
    u, z = xz[:, :inner], xz[:, inner:]
    u = rnd(silu(causal_conv(u, W[pre + ".conv"], W[pre + ".conv.b"])))
    low = lin(u, W[pre + ".x"])
    d, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:]
    dt = softplus(lin(d, W[pre + ".dt"], W[pre + ".dt.b"], keep=True))
    y = selective_scan(u, dt, -torch.exp(W[pre + ".A_log"]), B, C, W[pre + ".D"])
    return lin(y * silu(z), W[pre + ".o"])


def feed_forward(h, W, pre):
    return lin(relu_squared(lin(h, W[pre + ".up"])), W[pre + ".down"])


def layer(x, W, i, ly, cfg):
    eps, m, pre = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0), f"l{i}"
    h1 = rms_norm(x, W[pre + ".norm1"], eps)
    if ly["type"] == "parallel":
        a = parallel_mixer(h1, W, pre + ".mix", ly["mixer"], eps)
    elif ly["type"] == "mamba1":
        a = mamba1_mixer(h1, W, pre + ".mix", ly["mixer"])
    else:
        raise ValueError(ly["type"])
    if ly.get("mlp"):
        a = a + feed_forward(rms_norm(x, W[pre + ".norm2"], eps), W, pre + ".mlp")
    return x + m * a


def forward(cfg, W, tokens, dtype=DT, streams=None, round_to=None):
    """Logits [T, vocab] of one whole sequence; ``streams``: a list that receives the stream after every layer;
    ``round_to``: the yardstick run (see ``ROUND``)."""
    global ROUND
    W = {k: v.to(dtype) if v.is_floating_point() else v for k, v in W.items()}
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    ROUND = round_to
    try:
        for i, ly in enumerate(cfg["layers"]):
            x = layer(x, W, i, ly, cfg)
            if streams is not None:
                streams.append(x.clone())
        return lin(rms_norm(x, W["final.norm"], cfg["norm"]["eps"]), W["embed"], keep=True)
    finally:
        ROUND = None
