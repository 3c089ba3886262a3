"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(models/src/llama.rs:362-366, 370-374).  Gate and up are one stacked matrix here.

Parameters: ``hidden``, ``intermediate``.  Checkpoint tensors:
``<prefix>.{gate,up,down}_proj.weight``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import FeedForward


class SwiGLU(FeedForward):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])

    def activation_width(self):
        return 2 * self.intermediate

    def declare(self):
        pre = self.prefix
        return [
            TensorDecl(pre + ".gate_proj.weight", (self.intermediate, self.hidden)),
            TensorDecl(pre + ".up_proj.weight", (self.intermediate, self.hidden)),
            TensorDecl(pre + ".down_proj.weight", (self.hidden, self.intermediate)),
        ]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre = self.prefix
        self.w_gate_up = torch.cat([tensors[pre + ".gate_proj.weight"], tensors[pre + ".up_proj.weight"]], 0).contiguous()
        self.w_down = tensors[pre + ".down_proj.weight"].contiguous()

    def streamed_weights(self):
        return [self.w_gate_up, self.w_down]

    def fused(self):
        return {"kind": "swiglu", "w_gate_up": self.w_gate_up, "w_down": self.w_down, "hidden": self.hidden,
                "intermediate": self.intermediate}

    def forward(self, x, ctx):
        ops = self.rt.ops
        act = ops.linear(x, self.w_gate_up, silu_mul=True, meta=ctx.meta)
        return ops.linear(act, self.w_down, meta=ctx.meta)


register_part("feed_forward", "swiglu", SwiGLU)


class PolyNormFF(FeedForward):
    """Dense feed-forward with a polynomial activation of normalised powers: down(act(up(x))),
    act(z) = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(u) = u / sqrt(mean(u^2) + eps) over
    the row's ``intermediate`` values, taken in float32.

    Parameters: ``hidden``, ``intermediate``, ``eps``, ``names`` (suffixes of up, down and the four coefficients;
    default ``.up``, ``.down``, ``.act``).
    """

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.eps = float(params["eps"])
        names = {"up": ".up", "down": ".down", "coef": ".act", **(params.get("names") or {})}
        self.t_up, self.t_down, self.t_coef = (prefix + names[k] for k in ("up", "down", "coef"))

    def activation_width(self):
        return self.intermediate

    def declare(self):
        return [TensorDecl(self.t_up, (self.intermediate, self.hidden)), TensorDecl(self.t_down, (self.hidden, self.intermediate)),
                TensorDecl(self.t_coef, (4,))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_up, self.w_down = tensors[self.t_up].contiguous(), tensors[self.t_down].contiguous()
        self.coef = tensors[self.t_coef].to(torch.float32).contiguous()

    def streamed_weights(self):
        return [self.w_up, self.w_down]

    def forward(self, x, ctx):
        ops = self.rt.ops
        z = ops.linear(x, self.w_up, meta=ctx.meta)
        act = torch.empty_like(z)
        ops.polynorm(z, self.coef, self.eps, act, ctx.meta)
        return ops.linear(act, self.w_down, meta=ctx.meta)


register_part("feed_forward", "polynorm", PolyNormFF)


class DenseActFF(FeedForward):
    """Dense feed-forward with an elementwise activation: down(act(up(x))), no biases.

    Parameters: ``hidden``, ``intermediate``, ``activation`` (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715
    z^3))); ``relu2``: max(z, 0)^2), ``names`` (suffixes of up and down; default ``.up``, ``.down``).
    """

    ACTIVATIONS = ("gelu_tanh", "relu2")

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.activation = str(params.get("activation", "gelu_tanh"))
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not known (known: {self.ACTIVATIONS})")
        names = {"up": ".up", "down": ".down", **(params.get("names") or {})}
        self.t_up, self.t_down = prefix + names["up"], prefix + names["down"]

    def activation_width(self):
        return self.intermediate

    def declare(self):
        return [TensorDecl(self.t_up, (self.intermediate, self.hidden)), TensorDecl(self.t_down, (self.hidden, self.intermediate))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_up, self.w_down = tensors[self.t_up].contiguous(), tensors[self.t_down].contiguous()

    def streamed_weights(self):
        return [self.w_up, self.w_down]

    def forward(self, x, ctx):
        ops = self.rt.ops
        z = ops.linear(x, self.w_up, meta=ctx.meta)
        act = torch.empty_like(z)
        ops.activation(z, act, self.activation, ctx.meta)
        return ops.linear(act, self.w_down, meta=ctx.meta)


register_part("feed_forward", "dense_act", DenseActFF)


class ClampedGLU(FeedForward):
    """Gated feed-forward with clamped branches: g = min(gate(x), limit), u = clamp(up(x), -limit, limit),
    down(g * sigmoid(alpha * g) * (u + 1)); no biases.  Gate and up are one stacked matrix.

    Parameters: ``hidden``, ``intermediate``, ``limit``, ``alpha`` (default 1.702), ``names`` (suffixes of gate, up, down;
    default ``.gate``, ``.up``, ``.down``).
    """

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.limit, self.alpha = float(params["limit"]), float(params.get("alpha", 1.702))
        if self.limit <= 0:
            raise ValueError("limit must be positive")
        names = {"gate": ".gate", "up": ".up", "down": ".down", **(params.get("names") or {})}
        self.t_gate, self.t_up, self.t_down = (prefix + names[k] for k in ("gate", "up", "down"))

    def activation_width(self):
        return 3 * self.intermediate

    def declare(self):
        return [TensorDecl(self.t_gate, (self.intermediate, self.hidden)), TensorDecl(self.t_up, (self.intermediate, self.hidden)),
                TensorDecl(self.t_down, (self.hidden, self.intermediate))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_gate_up = torch.cat([tensors[self.t_gate], tensors[self.t_up]], 0).contiguous()
        self.w_down = tensors[self.t_down].contiguous()

    def streamed_weights(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, x, ctx):
        ops = self.rt.ops
        gu = ops.linear(x, self.w_gate_up, meta=ctx.meta)
        act = torch.empty((gu.shape[0], self.intermediate), dtype=gu.dtype, device=gu.device)
        ops.clamped_glu(gu, act, self.limit, self.alpha, ctx.meta)
        return ops.linear(act, self.w_down, meta=ctx.meta)


register_part("feed_forward", "clamped_glu", ClampedGLU)
