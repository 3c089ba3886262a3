"""Kulivik as a model spec: sandwich blocks (a norm before and after each sublayer, the mixer's input shifted toward the
token before, every result gated by a sigmoid of the sublayer's input) around one of three mixers: rotated attention
inside a sliding window that keeps the first tokens, with biases, a norm per head, capped scores and value mixing;
attention behind a short convolution on q, k and v, with norms over the whole projections, a learned sink, value mixing
and a gate per head; or two mixers side by side, attention with a bias by distance and a query temperature beside linear
attention with a constant decay per head.  Feed-forwards are dense with clamped branches or routed experts.  The head is
the embedding matrix, its logits scaled and capped.

Tensor names: ``embed``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``shift``,
``rg1``, ``rg1.b``, ``rg2``, ``rg2.b``; mixers ``mix.{q,k,v,o}`` with ``.b``, ``.conv``, ``mix.{q,k}.norm``, ``mix.vmix``,
``mix.sink``, ``mix.g``; side by side ``mix.left.{q,k,v,o}``, ``mix.right.{q,k,v,g,o,norm}``; feed-forwards
``mlp.{gate,up,down}`` or ``mlp.router``, ``mlp.router.b``, ``mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

from ..config.kulivik_config import ConvSinkAttention, DenseFF, KulivikConfig, RotaryWindowAttention, SideBySideSizes
from ..config.registry import register_architecture
from ..parts.model import LayerSpec, ModelSpec

_NAMES = {"q": ".q", "k": ".k", "v": ".v", "o": ".o", "q_bias": ".q.b", "k_bias": ".k.b", "v_bias": ".v.b", "o_bias": ".o.b",
          "q_norm": ".q.norm", "k_norm": ".k.norm", "v_mix": ".vmix", "gate": ".g", "sink": ".sink", "conv": ".conv"}
_V_MIX = {"key": "kulivik"}  # every layer that mixes values reads the first such layer's, whatever its kind


def _sizes(cfg, s):
    return {"kind": "attention", "hidden": cfg.width, "num_heads": s.heads, "num_kv_heads": s.kv_heads, "head_dim": s.dim,
            "v_head_dim": s.vdim, "scale": s.scale, "window": None, "names": _NAMES,
            "position": {"kind": "none", "head_dim": s.dim}}


def _mixer(cfg: KulivikConfig, m):
    if isinstance(m, RotaryWindowAttention):
        spec = _sizes(cfg, m.sizes)
        spec.update(bias=True, out_bias=True, head_norm={"eps": cfg.eps, "weight": True}, softcap=m.softcap, window=m.window,
                    keep_first=m.keep_first if m.window else 0, v_mix=_V_MIX if m.v_mix else None)
        if m.rot_dims:
            spec["position"] = {"kind": "rope", "head_dim": m.sizes.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                "exact_frequencies": True, "interleaved": True}
        return spec
    if isinstance(m, ConvSinkAttention):
        spec = _sizes(cfg, m.sizes)
        spec.update(qk_norm={"eps": cfg.eps}, conv=m.conv if m.conv > 1 else 0, sink="learned", head_gate=True,
                    v_mix=_V_MIX if m.v_mix else None)
        return spec
    assert isinstance(m, SideBySideSizes)
    left = _sizes(cfg, m.left.sizes)
    left.update(distance_bias=True, q_temp={"coef": m.left.q_temp[0], "every": m.left.q_temp[1]} if m.left.q_temp else None)
    r = m.right
    right = {"kind": "decay_linear_attention", "hidden": cfg.width, "heads": r.heads, "dim": r.dim, "vdim": r.vdim,
             "decay": list(r.decay), "eps": cfg.eps}
    return {"kind": "side_by_side", "left": left, "right": right, "left_scale": m.left_scale, "right_scale": m.right_scale}


def _feed_forward(cfg: KulivikConfig, f):
    if f is None:
        return None
    if isinstance(f, DenseFF):
        return {"kind": "clamped_glu", "hidden": cfg.width, "intermediate": f.ff, "limit": f.limit, "alpha": 1.702}
    return {"kind": "routed_experts", "hidden": cfg.width, "experts": f.experts, "top": f.top, "intermediate": f.ff,
            "router_bias": True, "weights": "chosen"}


def kulivik_spec(cfg: KulivikConfig) -> ModelSpec:
    norm = {"kind": "rmsnorm", "size": cfg.width, "eps": cfg.eps, "weight_offset": 1.0, "tensor_suffix": ""}
    layers, ignored = [], []
    for i, ly in enumerate(cfg.layers):
        layers.append(LayerSpec(f"l{i}", {"kind": "sandwich", "norm": norm, "mixer": _mixer(cfg, ly.mixer),
                                          "feed_forward": _feed_forward(cfg, ly.mlp)}))
        if ly.mlp is None:  # a layer without a feed-forward has no use for what surrounds one
            ignored += [f"l{i}.norm2", f"l{i}.norm2b", f"l{i}.rg2", f"l{i}.rg2.b"]
        if isinstance(ly.mixer, ConvSinkAttention) and ly.mixer.conv <= 1:
            ignored += [f"l{i}.mix.{x}.conv" for x in "qkv"]
        if not isinstance(ly.mixer, SideBySideSizes) and not ly.mixer.v_mix:
            ignored.append(f"l{i}.mix.vmix")
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, final_norm=norm, final_norm_prefix="final.norm",
        embedding={"kind": "token", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed"},
        head={"kind": "linear", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": None, "scale": cfg.logit_scale,
              "softcap": cfg.logit_softcap or 0.0},
        ignored_tensors=tuple(ignored),
    )


register_architecture("Kulivik", KulivikConfig.from_dict, kulivik_spec, model_type="kulivik")
