"""Gated linear attention: a matrix of dim x vdim per head that decays row by row.

q = W_q x * dim^(-1/2), k = W_k x (heads x dim), v = W_v x (heads x vdim).  The decay of key channel n of a head is
a = sigmoid(z)^(1 / tau) with z = W_a2 (W_a1 x) + b, a low-rank map laid out heads x dim.  Per head
S_t = diag(a_t) S_(t-1) + k_t v_t^T and o_t = S_t^T q_t.  Each head's o is divided by its root mean square over vdim and
multiplied by a weight of vdim elements that all heads share; the heads side by side are multiplied by silu(W_g x) and
projected out.

State per request (float32, fixed size, ``cache.state[slot]``): the heads' matrices [heads, dim, vdim], zero at the start;
no pages.  The decay (its logits, sigmoid, power), the recurrence, the norm and the gate are float32 in every mode; the
projections run in the compute dtype (the decay's logits leave their projection as float32).

Parameters: ``hidden``, ``heads``, ``dim``, ``vdim``, ``tau``, ``rank`` (of the decay's map; None: whatever the
checkpoint's tensors have, 16 in random-weights mode), ``eps``, ``names`` (suffixes of the tensors: q, k, v, g, o, norm, a1, a2, a2_bias).
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import FreeDim, TensorDecl
from .base import Mixer

_NAMES = {"q": ".q", "k": ".k", "v": ".v", "g": ".g", "o": ".o", "norm": ".norm", "a1": ".a1", "a2": ".a2", "a2_bias": ".a2.b"}


class GatedLinearAttention(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.tau, self.eps = float(p["tau"]), float(p["eps"])
        self.rank = int(p["rank"]) if p.get("rank") is not None else FreeDim(prefix + ":decay rank", 16)
        if self.tau <= 0:
            raise ValueError("tau must be positive")
        self.names = {**_NAMES, **(p.get("names") or {})}
        self.qk, self.vg = self.heads * self.dim, self.heads * self.vdim

    def state_bytes(self):
        return self.heads * self.dim * self.vdim * 4

    def activation_width(self):
        return 2 * self.qk + 2 * self.vg + 2 * self.qk

    def declare(self):
        pre, n = self.prefix, self.names
        return [
            TensorDecl(pre + n["q"], (self.qk, self.hidden)), TensorDecl(pre + n["k"], (self.qk, self.hidden)),
            TensorDecl(pre + n["v"], (self.vg, self.hidden)), TensorDecl(pre + n["g"], (self.vg, self.hidden)),
            TensorDecl(pre + n["o"], (self.hidden, self.vg)), TensorDecl(pre + n["norm"], (self.vdim,), init="ones"),
            TensorDecl(pre + n["a1"], (self.rank, self.hidden)), TensorDecl(pre + n["a2"], (self.qk, self.rank)),
            TensorDecl(pre + n["a2_bias"], (self.qk,)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n = self.prefix, self.names
        t = lambda name: tensors[pre + n[name]]  # noqa: E731
        # one matrix for everything that reads the mixer's input but the decay's low-rank map: [q; k; v; g]
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], dim=0).contiguous()
        self.w_a1, self.w_a2, self.w_out = t("a1").contiguous(), t("a2").contiguous(), t("o").contiguous()
        self.a_bias = t("a2_bias").to(torch.float32).contiguous()  # widened exactly
        self.norm_w = t("norm").to(torch.float32).contiguous()

    def streamed_weights(self):
        return [self.w_in, self.w_a1, self.w_a2, self.w_out]

    def matrices(self, state):
        """The per-request state as float32 [slots, heads, dim, vdim]."""
        return state[:, :self.state_bytes()].view(torch.float32).view(state.shape[0], self.heads, self.dim, self.vdim)

    def forward(self, x, ctx, cache):
        ops, T, qk, vg = self.rt.ops, ctx.T, self.qk, self.vg
        proj = ops.linear(x, self.w_in, meta=ctx.meta)
        low = ops.linear(x, self.w_a1, meta=ctx.meta)
        z = ops.linear(low, self.w_a2, out_dtype=torch.float32, meta=ctx.meta)
        o = torch.empty((T, vg), dtype=torch.float32, device=x.device)
        ops.gla_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vg], z, self.a_bias, self.tau,
                     float(self.dim) ** -0.5, self.matrices(cache.state), ctx, o, heads=self.heads, dim=self.dim, vdim=self.vdim)
        y = torch.empty((T, vg), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, proj[:, 2 * qk + vg:], self.norm_w, self.eps, y, ctx.meta, self.heads)
        return ops.linear(y, self.w_out, meta=ctx.meta)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)


class DecayLinearAttention(Mixer):
    """Linear attention whose state decays by a constant per head.

    q = act(W_q x), k = act(W_k x) (heads x dim), v = act(W_v x) (heads x vdim), act = SiLU.  Per head
    S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t (times ``q_scale``, 1 by default).  The heads side by side are
    divided by their root mean square over the whole row, multiplied by a weight of the row's size and by sigmoid(W_g x),
    and projected out.

    State per request (float32, ``cache.state[slot]``): the heads' matrices [heads, dim, vdim], zero at the start; no pages.
    The recurrence, the norm and the gate are float32 in every mode (the activations are taken in float32 from the
    projections' outputs); it runs on the kernel of ``GatedLinearAttention`` with the decay as a constant.

    Parameters: ``hidden``, ``heads``, ``dim``, ``vdim``, ``decay`` (one number per head), ``eps``, ``q_scale``, ``names``
    (suffixes of the tensors: q, k, v, g, o, norm).
    """

    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps, self.q_scale = float(p["eps"]), float(p.get("q_scale", 1.0))
        self.decay = [float(a) for a in p["decay"]]
        if len(self.decay) != self.heads:
            raise ValueError(f"{prefix}: {len(self.decay)} decays for {self.heads} heads")
        self.names = {"q": ".q", "k": ".k", "v": ".v", "g": ".g", "o": ".o", "norm": ".norm", **(p.get("names") or {})}
        self.qk, self.vg = self.heads * self.dim, self.heads * self.vdim

    def state_bytes(self):
        return self.heads * self.dim * self.vdim * 4

    def activation_width(self):
        return 2 * self.qk + 2 * self.vg + 2 * self.vg

    def declare(self):
        pre, n = self.prefix, self.names
        return [
            TensorDecl(pre + n["q"], (self.qk, self.hidden)), TensorDecl(pre + n["k"], (self.qk, self.hidden)),
            TensorDecl(pre + n["v"], (self.vg, self.hidden)), TensorDecl(pre + n["g"], (self.vg, self.hidden)),
            TensorDecl(pre + n["o"], (self.hidden, self.vg)), TensorDecl(pre + n["norm"], (self.vg,), init="ones"),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n = self.prefix, self.names
        t = lambda name: tensors[pre + n[name]]  # noqa: E731
        self.w_in = torch.cat([t("q"), t("k"), t("v"), t("g")], dim=0).contiguous()  # everything that reads the input
        self.w_out = t("o").contiguous()
        self.norm_w = t("norm").to(torch.float32).contiguous()  # widened exactly
        self.head_decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(rt.device).contiguous()

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def matrices(self, state):
        """The per-request state as float32 [slots, heads, dim, vdim]."""
        return state[:, :self.state_bytes()].view(torch.float32).view(state.shape[0], self.heads, self.dim, self.vdim)

    def forward(self, x, ctx, cache):
        ops, T, qk, vg = self.rt.ops, ctx.T, self.qk, self.vg
        proj = ops.linear(x, self.w_in, meta=ctx.meta)
        o = torch.empty((T, vg), dtype=torch.float32, device=x.device)
        ops.gla_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vg], None, None, 1.0, self.q_scale,
                     self.matrices(cache.state), ctx, o, heads=self.heads, dim=self.dim, vdim=self.vdim,
                     head_decay=self.head_decay, silu=True)
        y = torch.empty((T, vg), dtype=x.dtype, device=x.device)
        ops.row_norm_gate(o, proj[:, 2 * qk + vg:], self.norm_w, self.eps, y, ctx.meta, kind="sigmoid")
        return ops.linear(y, self.w_out, meta=ctx.meta)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
