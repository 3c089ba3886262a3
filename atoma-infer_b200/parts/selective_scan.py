"""Selective-scan mixer of the Mamba kind: a recurrence per channel with input-dependent step sizes.

The input projection's rows are [u: inner | z: inner].  u passes a causal convolution over time on each channel (weights
[inner, taps], the last column the current token's, a bias, zeros before the request's start) and SiLU.  W_x u is
[d: dt_rank | B: state | C: state]; dt = softplus(W_dt d + b_dt), one step size per channel; A = -exp(A_log), inner x state.
Per channel c and state n: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n; y_c = sum_n S[c, n] C_n + D_c u_c.  The
output is W_o (y * silu(z)).

State per request (float32, fixed size, ``cache.state[slot]``): the convolution's last taps - 1 input rows as a ring (the
row of position p at place p mod (taps - 1), so a row's place does not depend on how the prompt was cut), then the
channels' states [inner, state]; no pages.  Step sizes (their projection's output, softplus), decays, the recurrence and
the gate are float32 in every mode; the projections, the convolution and its activation run in the compute dtype.

The step-size projection reads the whole row [d | B | C] through a matrix whose columns behind dt_rank are zero (built
once at load time): the same sums, and no copy of the row's first part.

Parameters: ``hidden``, ``inner``, ``state``, ``dt_rank``, ``taps``, ``names`` (suffixes of the tensors: in, conv,
conv_bias, x, dt, dt_bias, a_log, d, out).
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Mixer

_NAMES = {"in": ".in", "conv": ".conv", "conv_bias": ".conv.b", "x": ".x", "dt": ".dt", "dt_bias": ".dt.b", "a_log": ".A_log",
          "d": ".D", "out": ".o"}


class SelectiveScanMixer(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.inner, self.nstate = int(p["hidden"]), int(p["inner"]), int(p["state"])
        self.dt_rank, self.taps = int(p["dt_rank"]), int(p["taps"])
        self.low = self.dt_rank + 2 * self.nstate
        self.names = {**_NAMES, **(p.get("names") or {})}
        self.ring_bytes = -(-(self.taps - 1) * self.inner * 4 // 16) * 16
        self.matrix_bytes = self.inner * self.nstate * 4

    def state_bytes(self):
        return self.ring_bytes + self.matrix_bytes

    def activation_width(self):
        return 5 * self.inner + self.low

    def declare(self):
        pre, n = self.prefix, self.names
        return [
            TensorDecl(pre + n["in"], (2 * self.inner, self.hidden)),
            TensorDecl(pre + n["conv"], (self.inner, self.taps)),
            TensorDecl(pre + n["conv_bias"], (self.inner,)),
            TensorDecl(pre + n["x"], (self.low, self.inner)),
            TensorDecl(pre + n["dt"], (self.inner, self.dt_rank)),
            TensorDecl(pre + n["dt_bias"], (self.inner,)),
            TensorDecl(pre + n["a_log"], (self.inner, self.nstate)),
            TensorDecl(pre + n["d"], (self.inner,), init="ones"),
            TensorDecl(pre + n["out"], (self.hidden, self.inner)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n = self.prefix, self.names
        t = lambda name: tensors[pre + n[name]]  # noqa: E731
        f32 = lambda name: t(name).to(torch.float32).contiguous()  # noqa: E731  (exact widening)
        self.w_in, self.w_x, self.w_out = t("in").contiguous(), t("x").contiguous(), t("out").contiguous()
        w_dt = t("dt")
        self.w_dt = w_dt.new_zeros((self.inner, self.low))
        self.w_dt[:, :self.dt_rank] = w_dt
        # [taps, channels]: neighbouring threads of the kernels read neighbouring weights
        self.conv_w = t("conv").to(torch.float32).t().contiguous()
        self.conv_b, self.dt_bias, self.a_log, self.d_skip = (f32(k) for k in ("conv_bias", "dt_bias", "a_log", "d"))

    def streamed_weights(self):
        return [self.w_in, self.w_x, self.w_dt, self.w_out]

    def ring(self, state):
        """The convolution's share of the state: float32 [slots, taps - 1, inner] (None with one tap)."""
        if state is None or self.taps == 1:
            return None
        return state[:, :(self.taps - 1) * self.inner * 4].view(torch.float32).view(state.shape[0], self.taps - 1, self.inner)

    def matrices(self, state):
        """The recurrence's share of the state: float32 [slots, inner, state]."""
        return state[:, self.ring_bytes:self.ring_bytes + self.matrix_bytes].view(torch.float32).view(
            state.shape[0], self.inner, self.nstate)

    def forward(self, x, ctx, cache):
        ops, T, inner = self.rt.ops, ctx.T, self.inner
        proj = ops.linear(x, self.w_in, meta=ctx.meta)
        u_in, z = proj[:, :inner], proj[:, inner:]
        ring = self.ring(cache.state)
        u = torch.empty((T, inner), dtype=x.dtype, device=x.device)
        if not ops.causal_conv_act(u_in, self.conv_w, self.conv_b, ring, ctx, u, act="silu"):
            ops.causal_conv_save(u_in, ring, ctx, self.taps)  # after the convolution has read the ring
        low = ops.linear(u, self.w_x, meta=ctx.meta)
        dt_raw = ops.linear(low, self.w_dt, out_dtype=torch.float32, meta=ctx.meta)
        y = torch.empty((T, inner), dtype=x.dtype, device=x.device)
        ops.selective_scan(u, dt_raw, self.dt_bias, low[:, self.dt_rank:], z, self.a_log, self.d_skip,
                           self.matrices(cache.state), ctx, y, inner=inner, nstate=self.nstate)
        return ops.linear(y, self.w_out, meta=ctx.meta)


register_part("mixer", "selective_scan", SelectiveScanMixer)
