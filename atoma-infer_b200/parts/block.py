"""Residual blocks.

Pre-norm: h = x + mixer(norm1(x)); out = h + ff(norm2(h)) (models/src/llama.rs:393-410).  The residual stream
is float32 and each addition happens inside the norm that follows it.  Parameters: ``norm`` (spec of both norms),
``mixer``, ``feed_forward`` (specs), and the names of the four parts inside the layer's prefix (``names``).

Post-norm: x <- norm1(alpha x + mixer(f1(x))); x <- norm2(alpha x + ff(f2(x))): the norm comes after the sum and
what it leaves IS the residual stream (float32); the sublayers read the stream itself, optionally through a
sequence filter (f1, f2: a short convolution over time, whose state the block keeps per request).  Parameters:
``norm``, ``mixer``, ``feed_forward`` (None: the layer has no second sublayer), ``alpha``, ``filter`` (spec or
None), ``names``.

Parallel and sandwich arrangements: see ``ParallelBlock`` and ``SandwichBlock``.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Optional

import torch

from ..config.registry import part_class, register_part
from ..weights.loader import TensorDecl
from .base import Block, PendingSum, apply_pending, join_terms

_DEFAULT_NAMES = {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                  "feed_forward": "mlp"}


class PreNormBlock(Block):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {**_DEFAULT_NAMES, **(params.get("names") or {})}
        mk = lambda fam, spec, name: part_class(fam, spec["kind"])(spec, f"{prefix}.{name}")  # noqa: E731
        self.norm1 = mk("norm", params["norm"], names["norm1"])
        self.mixer = mk("mixer", params["mixer"], names["mixer"])
        self.norm2 = mk("norm", params["norm"], names["norm2"])
        self.feed_forward = mk("feed_forward", params["feed_forward"], names["feed_forward"])

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def streamed_weights(self):
        return self.mixer.streamed_weights() + self.feed_forward.streamed_weights()

    def activation_width(self):
        return max(p.activation_width() for p in self.parts())

    def declare(self):
        return [d for p in self.parts() for d in p.declare()]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for p in self.parts():
            p.bind(tensors, rt)

    def decode_fusion(self):
        parts = {"norm1": self.norm1.fused(), "mixer": self.mixer.fused(), "norm2": self.norm2.fused(),
                 "feed_forward": self.feed_forward.fused()}
        if any(v is None for v in parts.values()):
            return None
        return {"kind": "prenorm", **parts}

    def forward(self, resid, delta, ctx, cache):
        h = self.norm1.forward(resid, delta, ctx)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm2.forward(resid, a, ctx)
        return self.feed_forward.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock)


_POST_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp", "filter1": "canon1",
               "filter2": "canon2"}


class PostNormBlock(Block):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {**_POST_NAMES, **(params.get("names") or {})}
        mk = lambda fam, spec, name: part_class(fam, spec["kind"])(spec, f"{prefix}.{name}")  # noqa: E731
        self.alpha = float(params.get("alpha", 1.0))
        self.norm1 = mk("norm", params["norm"], names["norm1"])
        self.mixer = mk("mixer", params["mixer"], names["mixer"])
        ff, flt = params.get("feed_forward"), params.get("filter")
        self.feed_forward = mk("feed_forward", ff, names["feed_forward"]) if ff else None
        self.norm2 = mk("norm", params["norm"], names["norm2"]) if ff else None
        self.filter1 = mk("filter", flt, names["filter1"]) if flt else None
        self.filter2 = mk("filter", flt, names["filter2"]) if flt and ff else None

    def parts(self):
        return [p for p in (self.filter1, self.mixer, self.norm1, self.filter2, self.feed_forward, self.norm2) if p is not None]

    def streamed_weights(self):
        return self.mixer.streamed_weights() + (self.feed_forward.streamed_weights() if self.feed_forward else [])

    def activation_width(self):
        return max(p.activation_width() for p in self.parts())

    def declare(self):
        return [d for p in self.parts() for d in p.declare()]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for p in self.parts():
            p.bind(tensors, rt)

    def _layout(self):
        """Shares of the per-request state: the mixer's, then the two filters', each starting on 16 bytes."""
        shares, at = {}, 0
        for name in ("mixer", "filter1", "filter2"):
            part = getattr(self, name)
            n = part.state_bytes() if part is not None else 0
            shares[name] = (at, n)
            at += -(-n // 16) * 16
        return shares, at

    def state_bytes(self):
        return self._layout()[1]

    def _share(self, state: Optional[torch.Tensor], name: str) -> Optional[torch.Tensor]:
        at, n = self._layout()[0][name]
        return state[:, at:at + n] if state is not None and n else None

    def forward(self, resid, delta, ctx, cache):
        ops = self.rt.ops
        apply_pending(ops, resid, delta, ctx)  # a block before this one left its addition pending
        mixer_cache = cache
        if self.mixer.state_bytes() != self.state_bytes() and cache.state is not None:
            mixer_cache = replace(cache, state=self._share(cache.state, "mixer"))
        s1, s2 = self._share(cache.state, "filter1"), self._share(cache.state, "filter2")
        # decode steps: the norm kernel also leaves the next sublayer's input (new row + its short convolution)
        f2 = self.filter2.fused() if self.filter2 is not None else None
        decode = ctx.decode_only and ctx.T == ctx.S and getattr(ops, "fused_post_norm", True)
        fuse = decode and f2 is not None and f2["kind"] == "short_conv" and f2["add_input"]
        ready = ctx.shared.pop("prepared_input", None)  # the block before may have left this block's input
        if ready is not None and ready[0] is self:
            h = ready[1]
        else:
            h = self.filter1.forward(resid, ctx, s1) if self.filter1 is not None else self._plain_input(resid)
        a = self.mixer.forward(h, ctx, mixer_cache)
        keep1 = (self.filter1.ring(s1), self.filter1.taps) if self.filter1 is not None else None
        h2 = None
        if self.feed_forward is not None and fuse:
            h2 = torch.empty((ctx.T, resid.shape[1]), dtype=self.rt.dtype, device=resid.device)
            self.norm1.forward_post(resid, a, self.alpha, ctx, keep=keep1,
                                    conv=(f2["weight"], self.filter2.ring(s2), h2))
        else:
            self.norm1.forward_post(resid, a, self.alpha, ctx, keep=keep1)
        if self.feed_forward is None:
            return None  # (a layer with one sum leaves the next block's input to that block)
        if h2 is None:
            h2 = self.filter2.forward(resid, ctx, s2) if self.filter2 is not None else self._plain_input(resid)
        f = self.feed_forward.forward(h2, ctx)
        keep2 = (self.filter2.ring(s2), self.filter2.taps) if self.filter2 is not None else None
        conv = None
        nxt = ctx.shared.get("next_run")
        if decode and nxt is not None and isinstance(nxt[0], PostNormBlock) and nxt[0].filter1 is not None:
            # decode steps: this norm also leaves the next block's input, the new row + that block's first convolution
            blk, view = nxt
            f1 = blk.filter1.fused()
            if f1["kind"] == "short_conv" and f1["add_input"] and view.state is not None:
                hn = torch.empty((ctx.T, resid.shape[1]), dtype=self.rt.dtype, device=resid.device)
                conv = (f1["weight"], blk.filter1.ring(blk._share(view.state, "filter1")), hn)
                ctx.shared["prepared_input"] = (blk, hn)
        self.norm2.forward_post(resid, f, self.alpha, ctx, keep=keep2, conv=conv)
        return None

    def _plain_input(self, resid):
        """Without a filter a sublayer reads the stream itself, in the compute type."""
        return self.rt.ops.narrow(resid, self.rt.dtype)


register_part("block", "postnorm", PostNormBlock)


class ParallelBlock(Block):
    """x <- x + mult * (mixer(h1) + ff(h2)), both sublayers reading the same x: through one norm (h2 = h1 = norm1(x)) or,
    with ``two_norms``, each through a norm of its own (h2 = norm2(x)), both taken in the pass that adds what the block
    before left pending.  The sum is left pending as a ``PendingSum`` (the terms, their weights if the mixer gives a
    weighted sum, the factor), which the next norm adds into the float32 stream term by term.  Parameters: ``norm``,
    ``mixer``, ``feed_forward`` (None: the mixer alone), ``mult``, ``two_norms``, ``names``."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {"norm1": "norm1", "norm2": "norm2", "mixer": "mix", "feed_forward": "mlp", **(params.get("names") or {})}
        mk = lambda fam, spec, name: part_class(fam, spec["kind"])(spec, f"{prefix}.{name}")  # noqa: E731
        self.mult = float(params.get("mult", 1.0))
        self.norm1 = mk("norm", params["norm"], names["norm1"])
        self.mixer = mk("mixer", params["mixer"], names["mixer"])
        ff = params.get("feed_forward")
        self.feed_forward = mk("feed_forward", ff, names["feed_forward"]) if ff else None
        self.norm2 = mk("norm", params["norm"], names["norm2"]) if ff and params.get("two_norms") else None

    def parts(self):
        return [p for p in (self.norm1, self.norm2, self.mixer, self.feed_forward) if p is not None]

    def streamed_weights(self):
        return self.mixer.streamed_weights() + (self.feed_forward.streamed_weights() if self.feed_forward else [])

    def activation_width(self):
        return max(p.activation_width() for p in self.parts())

    def declare(self):
        return [d for p in self.parts() for d in p.declare()]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for p in self.parts():
            p.bind(tensors, rt)

    def forward(self, resid, delta, ctx, cache):
        if self.norm2 is not None:
            h, h2 = self.norm1.forward_pair(resid, delta, ctx, self.norm2)
        else:
            h = h2 = self.norm1.forward(resid, delta, ctx)
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return join_terms((a,), self.mult)
        return join_terms((a, self.feed_forward.forward(h2, ctx)), self.mult)


register_part("block", "parallel", ParallelBlock)


class SandwichBlock(Block):
    """Norms before AND after each sublayer, a gate on each result, the mixer's input shifted toward the token before:

        h = norm1(x);  x <- x + norm1b(mixer(shift(h)) * sigmoid(R1 h + r1))
        h2 = norm2(x); x <- x + norm2b(ff(h2) * sigmoid(R2 h2 + r2))

    shift(h)_t = h_t + (h_(t-1) - h_t) * mu per channel, h_(t-1) the normed row of the request's token before (zeros before
    its first token); a request's last normed row is per-request state (float32, the first share of the block's state,
    the mixer's share behind it).  The gates read the normed rows as they are, before the shift.  Every sum into the
    stream is taken by the kernel that norms the gated result, in float32, so the block leaves nothing pending.  A
    mixer may hand back a ``PendingSum`` (weighted terms, a vector): gate and norm see its float32 value.
    Parameters: ``norm``, ``mixer``, ``feed_forward`` (None: the mixer alone), ``shift`` (default True), ``names``."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {"norm1": "norm1", "norm1b": "norm1b", "norm2": "norm2", "norm2b": "norm2b", "mixer": "mix", "feed_forward": "mlp",
                 "shift": ".shift", "gate1": ".rg1", "gate2": ".rg2", "gate_bias": ".b", **(params.get("names") or {})}
        self.names = names
        mk = lambda fam, spec, name: part_class(fam, spec["kind"])(spec, f"{prefix}.{name}")  # noqa: E731
        self.norm1, self.norm1b = mk("norm", params["norm"], names["norm1"]), mk("norm", params["norm"], names["norm1b"])
        self.mixer = mk("mixer", params["mixer"], names["mixer"])
        ff = params.get("feed_forward")
        self.feed_forward = mk("feed_forward", ff, names["feed_forward"]) if ff else None
        self.norm2 = mk("norm", params["norm"], names["norm2"]) if ff else None
        self.norm2b = mk("norm", params["norm"], names["norm2b"]) if ff else None
        self.shift = bool(params.get("shift", True))
        self.width = self.norm1.size

    def parts(self):
        return [p for p in (self.norm1, self.norm1b, self.mixer, self.norm2, self.norm2b, self.feed_forward) if p is not None]

    def streamed_weights(self):
        return ([self.w_gate1] + self.mixer.streamed_weights()
                + ([self.w_gate2] + self.feed_forward.streamed_weights() if self.feed_forward else []))

    def activation_width(self):
        return max(p.activation_width() for p in self.parts())

    def declare(self):
        pre, n, W = self.prefix, self.names, self.width
        decls = [d for p in self.parts() for d in p.declare()]
        decls += [TensorDecl(pre + n["gate1"], (W, W)), TensorDecl(pre + n["gate1"] + n["gate_bias"], (W,))]
        if self.feed_forward is not None:
            decls += [TensorDecl(pre + n["gate2"], (W, W)), TensorDecl(pre + n["gate2"] + n["gate_bias"], (W,))]
        if self.shift:
            decls.append(TensorDecl(pre + n["shift"], (W,)))
        return decls

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for p in self.parts():
            p.bind(tensors, rt)
        pre, n = self.prefix, self.names
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()  # noqa: E731  (exact widening)
        self.w_gate1, self.b_gate1 = tensors[pre + n["gate1"]].contiguous(), f32(pre + n["gate1"] + n["gate_bias"])
        if self.feed_forward is not None:
            self.w_gate2, self.b_gate2 = tensors[pre + n["gate2"]].contiguous(), f32(pre + n["gate2"] + n["gate_bias"])
        self.mu = f32(pre + n["shift"]) if self.shift else None

    def _kept_bytes(self):
        return -(-self.width * 4 // 16) * 16 if self.shift else 0

    def state_bytes(self):
        return self._kept_bytes() + self.mixer.state_bytes()

    def forward(self, resid, delta, ctx, cache):
        ops, dt, dev, T, W = self.rt.ops, self.rt.dtype, resid.device, ctx.T, self.width
        apply_pending(ops, resid, delta, ctx)  # a block of another kind before this one may have left its addition pending
        kept, mixer_cache = None, cache
        if cache.state is not None:
            nk = self._kept_bytes()
            if nk:
                kept = cache.state[:, :W * 4].view(torch.float32)
            mixer_cache = replace(cache, state=cache.state[:, nk:] if self.mixer.state_bytes() else None)
        h = torch.empty((T, W), dtype=dt, device=dev)
        hs, last = h, None
        if self.shift:
            hs = torch.empty_like(h)
            last = torch.empty((ctx.S, W), dtype=torch.float32, device=dev)
        ops.norm_shift(resid, self.norm1.weight, self.norm1.eps, ctx, shift=self.mu, state=kept, h=h,
                       hs=hs if self.shift else None, last=last)
        a = self.mixer.forward(hs, ctx, mixer_cache)
        if not isinstance(a, PendingSum):
            a = PendingSum((a,))
        g = ops.linear(h, self.w_gate1, out_dtype=torch.float32, meta=ctx.meta)
        keep = (last, kept) if self.shift and kept is not None else None
        if self.feed_forward is None:
            ops.gated_norm_add(resid, a, g, self.b_gate1, self.norm1b.weight, self.norm1b.eps, ctx, keep=keep)
            return None
        h2 = torch.empty((T, W), dtype=dt, device=dev)
        ops.gated_norm_add(resid, a, g, self.b_gate1, self.norm1b.weight, self.norm1b.eps, ctx, keep=keep,
                           next_norm=(self.norm2.weight, self.norm2.eps, h2))
        f = self.feed_forward.forward(h2, ctx)
        if not isinstance(f, PendingSum):
            f = PendingSum((f,))
        g2 = ops.linear(h2, self.w_gate2, out_dtype=torch.float32, meta=ctx.meta)
        ops.gated_norm_add(resid, f, g2, self.b_gate2, self.norm2b.weight, self.norm2b.eps, ctx)
        return None


register_part("block", "sandwich", SandwichBlock)
