"""Grouped-query attention over the paged cache.

q, k, v projections without bias (one fused matrix here, three in the reference,
models/src/llama.rs:269-271), position encoding of q and k, keys and values written
to the request's pages, then for the query at position p of a request: scores
scale * q.k_j for j <= p (and p - j < window if the layer has one) over everything
the request has cached, softmax in float32, weighted sum of values; query head h
reads key/value head h // (heads / kv_heads) (csrc/kernels/flash_fwd_kernel.h:153,
159).  Output projection (models/src/llama.rs:310-311).  A portion of a prompt
attends to the portions before it through the block table; the reference's glue
misses that case (models/src/flash_attention.rs:384-410).

Parameters: ``hidden``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
``window`` (None: all keys), ``position`` (spec of the position encoding).
Checkpoint tensors: ``<prefix>.{q,k,v,o}_proj.weight`` (other suffixes: ``names``).

Further options, all off by default:
``chunk``: a query sees only keys of its own chunk of that many positions, counted from position 0;
``sink``: one more term in the softmax's denominator, a key of score 0 without a value;
``v_head_dim``: values of another size than queries and keys;
``bias``: q, k and v projections have biases;
``qk_norm`` ``{"eps": e}``: the whole q projection, and the whole k projection, is divided by its root mean square
and multiplied by a weight of its size, before the rotation;
``v_mix`` ``{"key": name}``: the first layer with this key leaves its values for the step, every later one caches
(1 - lambda) v + lambda v_first with its own learned scalar lambda;
``head_norm`` ``{"eps": e}``: after the rotation every q head and every k head is divided by its own root mean square
over the head's size (no weight);
``gate``: the heads' outputs side by side are multiplied by sigmoid(W_g x), W_g a matrix of their size that reads the
mixer's input like the projections (it joins their fused matrix), before the output projection.
``head_norm`` ``{"eps": e, "weight": True}``: every q head and every k head is divided by its own root mean square
BEFORE the rotation and multiplied by a weight of the head's size that all heads share (one for q, one for k);
``out_bias``: the output projection has a bias (handed on as the vector of a ``PendingSum``, which the kernel that adds
the mixer's result into the stream takes in float32);
``softcap``: a score s becomes softcap * tanh(s / softcap) before the mask;
``keep_first`` (beside ``window``): the first so many tokens of a request stay visible behind the window;
``distance_bias``: slope_h * (i - j) is taken off the score of query i and key j, slope_h = 2^(-8 (h + 1) / heads);
``q_temp`` ``{"coef": c, "every": n}``: the query at position p is multiplied by 1 + c ln(floor((p + 1) / n) + 1);
``conv``: taps of a causal convolution over time on every channel of q, k and v, directly after the projection (weights
``<tensor>.conv`` [channels, taps], no bias); the last taps - 1 projected rows are per-request state;
``sink: "learned"``: the sink's score is a learned number per head (``.sink``), not 0;
``head_gate``: head h's output is multiplied by sigmoid(W_g x)_h, one number per head (W_g [heads, hidden] joins the fused
matrix).
The position encoding's ``interleaved`` pairs dimension 2i with 2i + 1.
With any of ``v_head_dim``, ``bias``, ``qk_norm``, ``v_mix``, ``head_norm`` (and the options above that touch the rows) the rows are prepared by one kernel (``qkv_prepare``) that writes queries, keys and values
as heads of one padded size, the next multiple of 16 above both sizes, which the tensor-core kernels read like any
other head size; the output projection's matrix gets zero columns to match.
"""
from __future__ import annotations

import torch

from ..cache.spec import CacheNeed
from ..config.registry import part_class, register_part
from ..weights.loader import TensorDecl
from .base import Mixer, PendingSum


class Attention(Mixer):
    graph_safe = True  # reads the step's metadata on the device only

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = params
        self.hidden = int(p["hidden"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.v_head_dim = int(p.get("v_head_dim") or self.head_dim)
        self.chunk = int(p.get("chunk") or 0)
        self.sink = bool(p.get("sink", False))
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.v_mix = p.get("v_mix")
        self.head_norm = p.get("head_norm")
        self.gate = bool(p.get("gate", False))
        if self.head_norm is not None and self.qk_norm is not None:
            raise ValueError("qk_norm and head_norm exclude each other")
        self.head_norm_weight = bool((self.head_norm or {}).get("weight", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.softcap = float(p.get("softcap") or 0.0)
        self.keep_first = int(p.get("keep_first") or 0)
        self.distance_bias = bool(p.get("distance_bias", False))
        self.q_temp = p.get("q_temp")
        self.taps = int(p.get("conv") or 0)
        self.head_gate = bool(p.get("head_gate", False))
        self.learned_sink = p.get("sink") == "learned"
        if self.gate and self.head_gate:
            raise ValueError("gate and head_gate exclude each other")
        if self.keep_first and not self.window:
            raise ValueError("keep_first goes with a window")
        interleaved = bool((p.get("position") or {}).get("interleaved", False))
        self.prepared = bool(self.bias or self.qk_norm is not None or self.v_mix is not None or self.head_norm is not None
                             or self.gate or self.v_head_dim != self.head_dim or interleaved or self.q_temp or self.taps
                             or self.head_gate)
        self.padded_dim = -(-max(self.head_dim, self.v_head_dim) // 16) * 16 if self.prepared else self.head_dim
        self.names = {"q": ".q_proj.weight", "k": ".k_proj.weight", "v": ".v_proj.weight", "o": ".o_proj.weight",
                      "q_bias": ".q_proj.bias", "k_bias": ".k_proj.bias", "v_bias": ".v_proj.bias",
                      "q_norm": ".q_norm.weight", "k_norm": ".k_norm.weight", "v_mix": ".v_mix", "gate": ".g_proj.weight",
                      "o_bias": ".o_proj.bias", "sink": ".sink", "conv": ".conv", **(p.get("names") or {})}
        pos = dict(p.get("position") or {"kind": "none"})
        pos.setdefault("head_dim", self.head_dim)
        self.position = part_class("position", pos["kind"])(pos, prefix)

    @property
    def q_size(self):
        return self.num_heads * self.head_dim

    @property
    def kv_size(self):
        return self.num_kv_heads * self.head_dim

    @property
    def v_size(self):
        return self.num_kv_heads * self.v_head_dim

    def activation_width(self):
        gate = self.num_heads * self.v_head_dim if self.gate else (self.num_heads if self.head_gate else 0)
        rows = self.q_size + self.kv_size + self.v_size
        return max(rows + gate + (rows if self.taps else 0), 2 * self.num_heads * self.padded_dim)

    def state_bytes(self):
        """The convolution's ring: the last taps - 1 projected rows [q | k | v] of a request, float32."""
        return (self.taps - 1) * (self.q_size + self.kv_size + self.v_size) * 4 if self.taps > 1 else 0

    def ring(self, state):
        if state is None or self.taps <= 1:
            return None
        n = self.q_size + self.kv_size + self.v_size
        return state[:, :self.state_bytes()].view(torch.float32).view(state.shape[0], self.taps - 1, n)

    def streamed_weights(self):
        return [self.w_qkv, self.w_o]

    def cache_need(self):
        # (a window that keeps the first tokens gives no pages back: the kept pages would leave a hole in the live range)
        return CacheNeed.kv(self.num_kv_heads, self.padded_dim, None if self.keep_first else self.window, self.chunk or None)

    def declare(self):
        pre, n = self.prefix, self.names
        decls = [
            TensorDecl(pre + n["q"], (self.q_size, self.hidden)),
            TensorDecl(pre + n["k"], (self.kv_size, self.hidden)),
            TensorDecl(pre + n["v"], (self.v_size, self.hidden)),
            TensorDecl(pre + n["o"], (self.hidden, self.num_heads * self.v_head_dim)),
        ]
        if self.bias:
            decls += [TensorDecl(pre + n["q_bias"], (self.q_size,)), TensorDecl(pre + n["k_bias"], (self.kv_size,)),
                      TensorDecl(pre + n["v_bias"], (self.v_size,))]
        if self.qk_norm is not None:
            decls += [TensorDecl(pre + n["q_norm"], (self.q_size,), init="ones"),
                      TensorDecl(pre + n["k_norm"], (self.kv_size,), init="ones")]
        if self.head_norm_weight:
            decls += [TensorDecl(pre + n["q_norm"], (self.head_dim,), init="ones"),
                      TensorDecl(pre + n["k_norm"], (self.head_dim,), init="ones")]
        if self.out_bias:
            decls.append(TensorDecl(pre + n["o_bias"], (self.hidden,)))
        if self.learned_sink:
            decls.append(TensorDecl(pre + n["sink"], (self.num_heads,)))
        if self.head_gate:
            decls.append(TensorDecl(pre + n["gate"], (self.num_heads, self.hidden)))
        if self.taps:
            decls += [TensorDecl(pre + n[x] + n["conv"], (size, self.taps))
                      for x, size in (("q", self.q_size), ("k", self.kv_size), ("v", self.v_size))]
        if self.v_mix is not None:
            decls.append(TensorDecl(pre + n["v_mix"], ()))
        if self.gate:
            decls.append(TensorDecl(pre + n["gate"], (self.num_heads * self.v_head_dim, self.hidden)))
        return decls + self.position.declare()

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        pre, n = self.prefix, self.names
        # One matrix [q; k; v]: each output element is the same dot product as before.
        self.w_qkv = torch.cat([tensors[pre + n["q"]], tensors[pre + n["k"]], tensors[pre + n["v"]]]
                               + ([tensors[pre + n["gate"]]] if self.gate or self.head_gate else []), dim=0).contiguous()
        self.w_o = tensors[pre + n["o"]].contiguous()
        self.position.bind(tensors, rt)
        f32 = lambda name: tensors[pre + n[name]].to(torch.float32).contiguous()  # noqa: E731  (exact widening)
        self.b_o = f32("o_bias") if self.out_bias else None
        self.sinks = f32("sink") if self.learned_sink else None
        # slope_h = 2^(-8 (h + 1) / heads), taken in float64 and rounded once
        self.slopes = (torch.tensor([2.0 ** (-8.0 * (h + 1) / self.num_heads) for h in range(self.num_heads)], dtype=torch.float64)
                       .to(torch.float32).to(rt.device).contiguous() if self.distance_bias else None)
        if not self.prepared:
            return
        # Biases and norm weights stay as the loader left them when that is one type for all (bfloat16 from a bfloat16
        # checkpoint: the kernel widens them, exactly, as it reads them); else all are widened here.
        normed = self.qk_norm is not None or self.head_norm_weight
        names = (["q_bias", "k_bias", "v_bias"] if self.bias else []) + (["q_norm", "k_norm"] if normed else [])
        same = len({tensors[pre + n[x]].dtype for x in names}) <= 1
        get = (lambda name: tensors[pre + n[name]].contiguous()) if same else f32  # noqa: E731
        self.b_qkv = torch.cat([get("q_bias"), get("k_bias"), get("v_bias")]).contiguous() if self.bias else None
        self.w_q_norm, self.w_k_norm = (get("q_norm"), get("k_norm")) if normed else (None, None)
        self.v_lambda = f32("v_mix").reshape(1) if self.v_mix is not None else None
        # [taps, channels] over the fused [q | k | v] rows: neighbouring threads read neighbouring weights
        self.conv_w = (torch.cat([tensors[pre + n[x] + n["conv"]] for x in ("q", "k", "v")], 0).to(torch.float32).t().contiguous()
                       if self.taps else None)
        if self.padded_dim != self.v_head_dim:  # the attention's output has heads of the padded size: zero columns for the tail
            w = self.w_o.new_zeros((self.hidden, self.num_heads, self.padded_dim))
            w[:, :, :self.v_head_dim] = self.w_o.view(self.hidden, self.num_heads, self.v_head_dim)
            self.w_o = w.view(self.hidden, self.num_heads * self.padded_dim).contiguous()

    def fused(self):
        rotary = self.position.rotary()
        if rotary is None or self.prepared or self.chunk or self.sink:
            return None
        return {"kind": "attention", "w_qkv": self.w_qkv, "w_o": self.w_o, "hidden": self.hidden,
                "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "scale": self.scale, "window": int(self.window or 0), "inv_freq": rotary[0], "rotary_dim": rotary[1]}

    def _score_options(self):
        """What changes a score or the mask beyond window, chunk and sink, as keyword arguments of ``ops.attention``."""
        return {k: v for k, v in (("keep_first", self.keep_first), ("softcap", self.softcap), ("slopes", self.slopes))
                if v is not None and (torch.is_tensor(v) or v)}

    def _forward_prepared(self, x, ctx, cache):
        ops = self.rt.ops
        H, G, dp = self.num_heads, self.num_kv_heads, self.padded_dim
        qkv = ops.linear(x, self.w_qkv, meta=ctx.meta)
        gate = None
        n = self.q_size + self.kv_size + self.v_size
        if self.gate:  # the fused projection's last columns
            qkv, gate = qkv[:, :n], qkv[:, n:].view(ctx.T, H, self.v_head_dim)
        elif self.head_gate:
            qkv, gate = qkv[:, :n], qkv[:, n:]
        if self.taps:  # the convolution over time, directly after the projection
            ring, rows = self.ring(cache.state), qkv
            qkv = torch.empty((ctx.T, n), dtype=x.dtype, device=x.device)
            if not ops.causal_conv_act(rows, self.conv_w, None, ring, ctx, qkv, act="none"):
                ops.causal_conv_save(rows, ring, ctx, self.taps)  # after the convolution has read the ring
        q = torch.empty((ctx.T, H * dp), dtype=x.dtype, device=x.device)
        v_first = v_out = None
        if self.v_mix is not None:
            key = "v_mix:" + str(self.v_mix.get("key", ""))
            v_first = ctx.shared.get(key)
            if v_first is None:  # the first such layer of the step: its values are what later layers mix in
                v_out = ctx.shared[key] = torch.empty((ctx.T, self.v_size), dtype=x.dtype, device=x.device)
            elif tuple(v_first.shape) != (ctx.T, self.v_size):
                raise ValueError(f"{self.prefix}: mixes values of {v_first.shape[1]} elements a token into {self.v_size}")
        rotary = self.position.rotary()
        ops.qkv_prepare(qkv, ctx, cache.pages, cache.group, q, nq=H, nkv=G, d=self.head_dim, dv=self.v_head_dim, dp=dp,
                        page_size=cache.page_size, num_pages=cache.num_pages,
                        store_kv=cache.writes and cache.pages is not None, bias=self.b_qkv, q_norm=self.w_q_norm,
                        k_norm=self.w_k_norm, eps=float((self.qk_norm or self.head_norm or {}).get("eps", 0.0)),
                        inv_freq=rotary[0] if rotary else None, rot=rotary[1] if rotary else 0, v_first=v_first,
                        v_lambda=self.v_lambda if v_first is not None else None, v_out=v_out,
                        **({"head_norm": True} if self.head_norm is not None else {}),
                        **({"interleaved": True} if getattr(self.position, "interleaved", False) else {}),
                        **({"q_temp": (float(self.q_temp["coef"]), int(self.q_temp["every"]))} if self.q_temp else {}))
        out = torch.empty((ctx.T, H * dp), dtype=x.dtype, device=x.device)
        scores = self._score_options()
        ops.attention(q, H * dp, cache.pages, ctx, cache.group, out, H, G, dp, cache.page_size, cache.num_pages,
                      int(self.window or 0), self.scale, chunk=self.chunk, sink=self.sinks if self.learned_sink else self.sink,
                      **scores)
        if self.gate:
            ops.sigmoid_gate(out.view(ctx.T, H, dp)[:, :, :self.v_head_dim], gate, ctx.meta)
        elif self.head_gate:
            ops.head_gate(out.view(ctx.T, H, dp)[:, :, :self.v_head_dim], gate, ctx.meta)
        y = ops.linear(out, self.w_o, meta=ctx.meta)
        return PendingSum((y,), vector=self.b_o) if self.out_bias else y

    def forward(self, x, ctx, cache):
        if self.prepared:
            return self._forward_prepared(x, ctx, cache)
        ops = self.rt.ops
        qkv = ops.linear(x, self.w_qkv, meta=ctx.meta)
        # In a decode step the attention kernel can rotate q and write the new key and value itself.
        rope = None
        fast = getattr(ops, "fast_attention", None)
        scores = self._score_options()
        if self.chunk or self.sink or scores:
            fast = None  # the fused rotation is the plain decode kernel's
        if ctx.decode_only and getattr(ops, "fused_rope", True) and fast and fast(qkv.dtype, self.head_dim, self.num_heads, self.num_kv_heads, qkv.shape[1]):
            rotary = self.position.rotary()
            if rotary is not None:
                rope = (rotary[0], rotary[1], cache.writes and cache.pages is not None)
        if rope is None:
            self.position.encode_and_store(qkv, ctx, cache, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                                           head_dim=self.head_dim)
        out = torch.empty((ctx.T, self.q_size), dtype=x.dtype, device=x.device)
        ops.attention(qkv, qkv.shape[1], cache.pages, ctx, cache.group, out, self.num_heads, self.num_kv_heads,
                      self.head_dim, cache.page_size, cache.num_pages, int(self.window or 0), self.scale, rope=rope,
                      **({"chunk": self.chunk, "sink": self.sinks if self.learned_sink else self.sink} if self.chunk or self.sink else {}),
                      **scores)
        y = ops.linear(out, self.w_o, meta=ctx.meta)
        return PendingSum((y,), vector=self.b_o) if self.out_bias else y


register_part("mixer", "attention", Attention)
