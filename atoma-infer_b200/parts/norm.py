"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in float32, rounded once.

The reference uses candle's RmsNorm for input_layernorm, post_attention_layernorm
and model.norm (models/src/llama.rs:402, 408, 416-421, 474, 487).  Parameters:
``size`` and ``eps`` (config.json's rms_norm_eps); ``weight_offset`` (default 0): the
stored weight is w - offset, i.e. 1.0 for weights kept around zero; ``tensor_suffix``
(default ".weight"): the checkpoint tensor is ``<prefix><suffix>``.

``forward_post`` is the norm AFTER the sum: resid <- norm(alpha * resid + delta), the
normed rows being the new residual stream (float32, in place).
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import Norm, PendingSum


class RMSNorm(Norm):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("weight_offset", 0.0))
        self.tensor = self.prefix + str(params.get("tensor_suffix", ".weight"))

    def declare(self):
        return [TensorDecl(self.tensor, (self.size,), init="jitter" if self.offset == 1.0 else "ones")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = (tensors[self.tensor].to(torch.float32) + self.offset).contiguous()  # widened exactly, then the offset

    def forward_post(self, resid, delta, alpha, ctx, keep=None, conv=None):
        """resid <- rmsnorm(alpha * resid + delta) * weight.  ``keep`` / ``conv``: see ``scaled_add_rmsnorm``."""
        self.rt.ops.scaled_add_rmsnorm(resid, delta, alpha, self.weight, self.eps, ctx, keep=keep, conv=conv)

    def forward(self, resid, delta, ctx, rows=None, num_rows=0):
        n = num_rows if rows is not None else ctx.T
        out = torch.empty((n, self.size), dtype=self.rt.dtype, device=resid.device)
        if isinstance(delta, PendingSum):  # several terms, a factor, rows and a vector: one pass all the same
            self.rt.ops.sum_rmsnorm(resid, delta, self.weight, self.eps, out, ctx.meta, n, rows=rows)
        else:
            self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, ctx.meta, n, rows=rows)
        return out

    def forward_pair(self, resid, delta, ctx, other: "RMSNorm"):
        """Adds ``delta`` into the stream once and returns the rows normed by this norm and by ``other`` (same size):
        two sublayers that read the same stream, each through a norm of its own."""
        if other.size != self.size:
            raise ValueError("two norms of one stream have one size")
        if not isinstance(delta, PendingSum):
            delta = PendingSum((delta,) if delta is not None else ())
        out = torch.empty((ctx.T, self.size), dtype=self.rt.dtype, device=resid.device)
        out2 = torch.empty_like(out)
        self.rt.ops.sum_rmsnorm(resid, delta, self.weight, self.eps, out, ctx.meta, ctx.T, second=(other.weight, other.eps, out2))
        return out, out2

    def fused(self):
        return {"kind": "rmsnorm", "weight": self.weight, "eps": self.eps, "size": self.size}


register_part("norm", "rmsnorm", RMSNorm)
