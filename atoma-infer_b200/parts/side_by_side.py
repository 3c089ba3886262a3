"""Two mixers side by side: both read the same input, the result is the weighted sum of their outputs.

``forward`` returns the two outputs as a ``PendingSum`` of terms and weights, so that the sum is taken in float32 by the
norm that adds the block's result into the stream; nothing is rounded in between.  Each mixer keeps what it needs: at
most one of them pages (its need is the pair's), and each a share of the per-request state, the left one's first, every
share starting on 16 bytes.

Parameters: ``left``, ``right`` (mixer specs), ``left_scale``, ``right_scale``, ``names`` (suffixes of the two prefixes;
default ``.left``, ``.right``).
"""
from __future__ import annotations

from dataclasses import replace

from ..config.registry import part_class, register_part
from .base import Mixer, PendingSum


class SideBySide(Mixer):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        names = {"left": ".left", "right": ".right", **(params.get("names") or {})}
        mk = lambda side: part_class("mixer", params[side]["kind"])(params[side], prefix + names[side])  # noqa: E731
        self.left, self.right = mk("left"), mk("right")
        self.scales = (float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0)))
        needs = [m.cache_need() for m in (self.left, self.right)]
        if all(n is not None for n in needs):
            raise ValueError(f"{prefix}: only one of two mixers side by side may keep pages")
        self.pager = 0 if needs[0] is not None else (1 if needs[1] is not None else -1)

    def sides(self):
        return (self.left, self.right)

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m in self.sides())

    def cache_need(self):
        return self.sides()[self.pager].cache_need() if self.pager >= 0 else None

    def _shares(self):
        at, out = 0, []
        for m in self.sides():
            n = m.state_bytes()
            out.append((at, n))
            at += -(-n // 16) * 16
        return out, at

    def state_bytes(self):
        return self._shares()[1]

    def activation_width(self):
        return max(m.activation_width() for m in self.sides())

    def streamed_weights(self):
        return self.left.streamed_weights() + self.right.streamed_weights()

    def declare(self):
        return self.left.declare() + self.right.declare()

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for m in self.sides():
            m.bind(tensors, rt)

    def forward(self, x, ctx, cache):
        shares, _ = self._shares()
        outs = []
        for i, m in enumerate(self.sides()):
            at, n = shares[i]
            state = cache.state[:, at:at + n] if cache.state is not None and n else None
            view = replace(cache, state=state) if i == self.pager else replace(
                cache, group=-1, pages=None, num_pages=0, writes=False, state=state, tensors={})
            outs.append(m.forward(x, ctx, view))
        terms, factors, vector = [], [], None
        for out, scale in zip(outs, self.scales):
            if isinstance(out, PendingSum):
                if out.rows is not None:
                    raise ValueError(f"{self.prefix}: a side's result has terms, weights and a vector only")
                terms += list(out.terms)
                factors += [scale * out.mult * f for f in out.weights()]
                if out.vector is not None:  # (a bias of the side's output projection)
                    vector = scale * out.vector if vector is None else vector + scale * out.vector
            else:
                terms.append(out)
                factors.append(scale)
        return PendingSum(tuple(terms), 1.0, vector=vector, factors=tuple(factors))


register_part("mixer", "side_by_side", SideBySide)
