"""Kulivik, plainly: one function per mechanism, float64, whole sequences at once, written from the design's equations.

Shares no code with the engine.  ``forward(cfg, w, tokens)`` runs one request's tokens and returns the logits at every
position (and, on request, the stream after every layer).  ``cfg`` is the configuration as config.json has it (a
dict), ``w`` a dict of tensors by checkpoint name.

Notation.  A layer: h = N1(x); m = mixer(shift(h)); x <- x + N1b(m * sigmoid(R1 h + r1)); then h2 = N2(x);
x <- x + N2b(ff(h2) * sigmoid(R2 h2 + r2)).  N(u) = u / sqrt(mean(u^2) + eps) * (1 + w).  shift(h)_t = h_t + (h_(t-1) -
h_t) * mu with h_(-1) = 0.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


_ROUND = None  # a storage type that matrix products read and write through (None: exact), see ``forward``


def t64(x):
    return x.to(F)


def lin(x, w):
    """x W^T; with a storage type set, what the product reads and what it writes is rounded to that type first."""
    if _ROUND is None:
        return x @ t64(w).T
    return (x.to(_ROUND).to(F) @ t64(w).T).to(_ROUND).to(F)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + t64(w))


def token_shift(h, mu):
    """h [T, W]: every row moves toward the row before it (zeros before the first) by ``mu`` per channel."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * t64(mu)


def gated(result, h, wg, bg):
    return result * torch.sigmoid(lin(h, wg) + t64(bg))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros((taps - 1, C), dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + t64(w)[:, j] * pad[j:j + T]
    return y


def rotate_pairs(x, dims, base):
    """x [T, heads, dim]: the first ``dims`` dimensions of every head rotate, (2i, 2i + 1) by the angle p * base^(-2i / dims)."""
    T = x.shape[0]
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F)
    ang = torch.arange(T, dtype=F)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(T, window=None, keep_first=0):
    """[T, T] bool: position i sees j <= i, and with a window only i - j < window or j < keep_first."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, scale, mask, softcap=None, slopes=None, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  score = q.k * scale, capped by cap * tanh(score / cap), less
    slope_h * (i - j); softmax over the visible keys, whose denominator also holds exp(sink_h) if a sink is given."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(~mask, -math.inf)
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].reshape(1, 1))
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - top)
        out[:, h] = (e / den) @ v[:, g]
    return out


def decaying_state(q, k, v, decay):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        S = torch.zeros((d, v.shape[2]), dtype=F)
        for t in range(T):
            S = decay[h] * S + k[t, h][:, None] * v[t, h][None, :]
            out[t, h] = S.T @ q[t, h]
    return out


def query_temperature(T, coef, every):
    p = torch.arange(T, dtype=F)
    return 1.0 + coef * torch.log(torch.floor((p + 1) / every) + 1.0)


def slopes_of(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F)


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


# ---------------------------------------------------------------------------------------------- mixers
def attention_rotary(m, w, pre, hs, eps, shared):
    """The windowed, rotated kind: biases, norm per head with one weight for all heads, rotation, cap, window with
    kept first tokens, value mixing."""
    T = hs.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (lin(hs, w[pre + "q"]) + t64(w[pre + "q.b"])).view(T, H, d)
    k = (lin(hs, w[pre + "k"]) + t64(w[pre + "k.b"])).view(T, G, d)
    v = (lin(hs, w[pre + "v"]) + t64(w[pre + "v.b"])).view(T, G, dv)
    q = rms(q, eps) * t64(w[pre + "q.norm"])
    k = rms(k, eps) * t64(w[pre + "k.norm"])
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, rot["dims"], rot["base"]), rotate_pairs(k, rot["dims"], rot["base"])
    v = _value_mix(m, w, pre, v, shared)
    mask = m.get("mask")
    see = visible(T, mask["size"], mask.get("keep_first", 0)) if mask else visible(T)
    o = softmax_attention(q, k, v, m["scale"], see, softcap=m.get("softcap"))
    return lin(o.reshape(T, H * dv), w[pre + "o"]) + t64(w[pre + "o.b"])


def _value_mix(m, w, pre, v, shared):
    if m.get("v_mix"):
        if "v_first" in shared:
            v = mix_values(v, shared["v_first"], t64(w[pre + "vmix"]))
        else:
            shared["v_first"] = v
    return v


def attention_conv(m, w, pre, hs, eps, shared):
    """The convolved kind: short convolution on q, k, v, norm over the whole projection, sink, value mixing, a gate per head."""
    T = hs.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (lin(hs, w[pre + n]) for n in ("q", "k", "v"))
    if m.get("conv", 0) > 1:
        q, k, v = (causal_conv(u, w[pre + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = (rms(q, eps) * t64(w[pre + "q.norm"])).view(T, H, d)
    k = (rms(k, eps) * t64(w[pre + "k.norm"])).view(T, G, d)
    v = _value_mix(m, w, pre, v.view(T, G, dv), shared)
    o = softmax_attention(q, k, v, m["scale"], visible(T), sink=t64(w[pre + "sink"]))
    o = o * torch.sigmoid(lin(hs, w[pre + "g"]))[:, :, None]
    return lin(o.reshape(T, H * dv), w[pre + "o"])


def side_by_side(m, w, pre, hs, eps):
    T = hs.shape[0]
    a, pl = m["left"], pre + "left."
    H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    q = (lin(hs, w[pl + "q"])).view(T, H, d)
    k = (lin(hs, w[pl + "k"])).view(T, G, d)
    v = (lin(hs, w[pl + "v"])).view(T, G, dv)
    qt = a.get("q_temp")
    if qt:
        q = q * query_temperature(T, qt["coef"], qt["every"])[:, None, None]
    left = softmax_attention(q, k, v, a["scale"], visible(T), slopes=slopes_of(H)).reshape(T, H * dv)
    left = lin(left, w[pl + "o"])
    r, pr = m["right"], pre + "right."
    H2, n, p = r["heads"], r["dim"], r["vdim"]
    q2 = silu(lin(hs, w[pr + "q"])).view(T, H2, n)
    k2 = silu(lin(hs, w[pr + "k"])).view(T, H2, n)
    v2 = silu(lin(hs, w[pr + "v"])).view(T, H2, p)
    o2 = decaying_state(q2, k2, v2, r["decay"]).reshape(T, H2 * p)
    o2 = rms(o2, eps) * t64(w[pr + "norm"]) * torch.sigmoid(lin(hs, w[pr + "g"]))
    right = lin(o2, w[pr + "o"])
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(f, w, pre, h):
    lim = f["limit"]
    g = torch.clamp(lin(h, w[pre + "gate"]), max=lim)
    u = torch.clamp(lin(h, w[pre + "up"]), -lim, lim)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[pre + "down"])


def route(z, top):
    """z [T, E] logits: the ``top`` largest choose; weights = softmax over the chosen logits."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def route_margin(z, top):
    """Per row: how far the last chosen logit leads the first one that is not chosen, relative to the largest |logit|
    (infinite when every expert is chosen): a small lead is a close call that any rounding may turn."""
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], math.inf, dtype=F)
    val = torch.topk(z, top + 1, dim=-1).values
    return (val[..., top - 1] - val[..., top]) / z.abs().max(-1).values


def moe_ff(f, w, pre, h, margins=None):
    z = lin(h, w[pre + "router"]) + t64(w[pre + "router.b"])
    idx, wt = route(z, f["router"]["top"])
    if margins is not None:
        margins.append(route_margin(z, f["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = pre + f"e{int(idx[t, c])}."
            y = silu(lin(h[t], w[e + "gate"])) * (lin(h[t], w[e + "up"]))
            out[t] = out[t] + wt[t, c] * (lin(y, w[e + "down"]))
    return out


# ---------------------------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None, margins=None, round_to=None):
    """``layers_out``: a list that receives the stream after every layer; ``margins``: a list that receives every routed
    layer's ``route_margin`` per position; ``round_to``: a storage type through which every matrix product reads and
    writes (to see how far rounding alone moves a position)."""
    global _ROUND
    _ROUND = round_to
    try:
        return _forward(cfg, w, tokens, layers_out, margins)
    finally:
        _ROUND = None


def _forward(cfg, w, tokens, layers_out, margins):
    eps = cfg["norm"]["eps"]
    x = t64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    shared = {}
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, w[p + "norm1"], eps)
        hs = token_shift(h, w[p + "shift"])
        kind, m = ly["type"], ly["mixer"]
        if kind == "attention_2":
            a = attention_rotary(m, w, p + "mix.", hs, eps, shared)
        elif kind == "attention":
            a = attention_conv(m, w, p + "mix.", hs, eps, shared)
        elif kind == "parallel":
            a = side_by_side(m, w, p + "mix.", hs, eps)
        else:
            raise ValueError(kind)
        x = x + norm_one_plus(gated(a, h, w[p + "rg1"], w[p + "rg1.b"]), w[p + "norm1b"], eps)
        f = ly.get("mlp")
        if f is not None:
            h2 = norm_one_plus(x, w[p + "norm2"], eps)
            y = dense_ff(f, w, p + "mlp.", h2) if f["kind"] == "dense" else moe_ff(f, w, p + "mlp.", h2, margins)
            x = x + norm_one_plus(gated(y, h2, w[p + "rg2"], w[p + "rg2.b"]), w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = norm_one_plus(x, w["final.norm"], eps)
    z = (lin(h, w["embed"])) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
