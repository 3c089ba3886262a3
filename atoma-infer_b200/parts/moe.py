"""Routed experts: every token runs ``top`` of ``experts`` small gated feed-forward layers, chosen by a router, and
optionally one shared expert.

Router: logits z = W_router h in float32, scores s = softmax(z) over all experts; the ``top`` largest scores choose
the experts (ties go to the lower index), and their weights are those scores divided by their sum (+ 1e-20).
Expert: down(silu(gate(h)) * up(h)), no biases.  The output is the weighted sum of the chosen experts' outputs, taken
in float32 in the order of the choice, plus the shared expert's.  A token's result does not depend on what else is in
the batch: routing is per token and every product's order of summation depends on the output element alone.

How it runs: one kernel routes; one sorts the (token, choice) pairs by expert on the device (a stable order, no host
round trip, so a decode step can be captured in a graph); the experts' two linears run as grouped products over
that order (gate and up stacked, SiLU * up in the epilogue); a last kernel weighs, sums and adds the shared expert.

Parameters: ``hidden``, ``experts``, ``top``, ``intermediate``, ``shared_intermediate`` (0: none), ``names``,
``router_bias`` (the logits get a learned bias, ``<prefix>.router.b``), ``weights`` (``"all"``, the default: as above;
``"chosen"``: the softmax over the chosen experts' logits alone).
Checkpoint tensors: ``<prefix>.router`` [experts, hidden], ``<prefix>.e<j>.{gate,up,down}``,
``<prefix>.shared.{gate,up,down}``.
"""
from __future__ import annotations

import torch

from ..config.registry import register_part
from ..weights.loader import TensorDecl
from .base import FeedForward


class RoutedExperts(FeedForward):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden, self.experts, self.top = int(p["hidden"]), int(p["experts"]), int(p["top"])
        self.intermediate, self.shared = int(p["intermediate"]), int(p.get("shared_intermediate") or 0)
        self.router_bias, self.over_chosen = bool(p.get("router_bias", False)), p.get("weights", "all") == "chosen"
        if p.get("weights", "all") not in ("all", "chosen"):
            raise ValueError(f"weights {p.get('weights')!r} is not known (known: 'all', 'chosen')")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"top ({self.top}) must lie in 1 .. experts ({self.experts})")
        self.names = {"router": ".router", "router_bias": ".router.b", "expert": ".e{}", "shared": ".shared", "gate": ".gate", "up": ".up", "down": ".down",
                      **(p.get("names") or {})}

    def activation_width(self):
        return max(self.top * (2 * self.intermediate + 2 * self.hidden), 2 * self.shared)

    def _expert(self, j):
        n = self.names
        stem = self.prefix + (n["shared"] if j is None else n["expert"].format(j))
        return stem + n["gate"], stem + n["up"], stem + n["down"]

    def declare(self):
        decls = [TensorDecl(self.prefix + self.names["router"], (self.experts, self.hidden))]
        if self.router_bias:
            decls.append(TensorDecl(self.prefix + self.names["router_bias"], (self.experts,)))
        for j in list(range(self.experts)) + ([None] if self.shared else []):
            f = self.shared if j is None else self.intermediate
            g, u, d = self._expert(j)
            decls += [TensorDecl(g, (f, self.hidden)), TensorDecl(u, (f, self.hidden)), TensorDecl(d, (self.hidden, f))]
        return decls

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_router = tensors[self.prefix + self.names["router"]].to(torch.float32).contiguous()  # widened exactly
        self.b_router = (tensors[self.prefix + self.names["router_bias"]].to(torch.float32).contiguous()
                         if self.router_bias else None)
        gu, dn = [], []
        for j in range(self.experts):
            g, u, d = self._expert(j)
            gu.append(torch.cat([tensors[g], tensors[u]], 0))
            dn.append(tensors[d])
        self.w_gate_up = torch.stack(gu).contiguous()   # [experts, 2 * intermediate, hidden]
        self.w_down = torch.stack(dn).contiguous()      # [experts, hidden, intermediate]
        if self.shared:
            g, u, d = self._expert(None)
            self.ws_gate_up = torch.cat([tensors[g], tensors[u]], 0).contiguous()
            self.ws_down = tensors[d].contiguous()

    def streamed_weights(self):
        return [self.ws_gate_up, self.ws_down] if self.shared else []

    def forward(self, x, ctx):
        ops, T = self.rt.ops, ctx.T
        ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        wts = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        if self.router_bias or self.over_chosen:
            ops.moe_route(x, self.w_router, ids, wts, ctx.meta, bias=self.b_router, over_chosen=self.over_chosen)
        else:
            ops.moe_route(x, self.w_router, ids, wts, ctx.meta)
        shared = None
        if self.shared:
            shared = ops.linear(ops.linear(x, self.ws_gate_up, silu_mul=True, meta=ctx.meta), self.ws_down, meta=ctx.meta)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        ops.moe_experts(x, ids, wts, self.w_gate_up, self.w_down, shared, out, ctx.meta)
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
