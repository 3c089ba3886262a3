"""Bumolix as a model spec: parallel blocks with two norms (the mixer and the feed-forward read the same stream, each
through a norm of its own; their sum times a constant is added to the stream) whose mixers are either two mixers side by
side (grouped-query attention with biases, a partial rotation with stretched positions, a norm per head after the
rotation, a chunk mask, a softmax sink and an output gate; beside it gated linear attention with a decay per key
channel) or a selective scan of the Mamba kind, and whose feed-forward is dense with the square of relu.  The head is
the embedding matrix.

Tensor names: ``embed``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm2``; side by side
``mix.left.{q,k,v,g,o}``, ``mix.left.{q,k,v}.b``, ``mix.right.{q,k,v,g,o,norm,a1,a2}``, ``mix.right.a2.b``; selective scan
``mix.{in,conv,conv.b,x,dt,dt.b,A_log,D,o}``; feed-forward ``mlp.{up,down}``.
"""
from __future__ import annotations

from ..config.bumolix_config import BumolixConfig, Mamba1Sizes, SideBySideSizes
from ..config.registry import register_architecture
from ..parts.model import LayerSpec, ModelSpec

_ATTENTION_NAMES = {"q": ".q", "k": ".k", "v": ".v", "o": ".o", "q_bias": ".q.b", "k_bias": ".k.b", "v_bias": ".v.b", "gate": ".g"}


def _mixer(cfg: BumolixConfig, m):
    if isinstance(m, Mamba1Sizes):
        return {"kind": "selective_scan", "hidden": cfg.width, "inner": m.inner, "state": m.state, "dt_rank": m.dt_rank,
                "taps": m.conv}
    assert isinstance(m, SideBySideSizes)
    a, g = m.left, m.right
    scaling = {"rope_type": "linear", "factor": a.rot_factor} if a.rot_factor != 1.0 else None
    position = ({"kind": "rope", "head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base, "scaling": scaling,
                 "exact_frequencies": True} if a.rot_dims else {"kind": "none", "head_dim": a.dim})
    left = {"kind": "attention", "hidden": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
            "v_head_dim": a.vdim, "scale": a.scale, "window": None, "chunk": a.chunk, "sink": True, "bias": True,
            "head_norm": {"eps": cfg.eps}, "gate": True, "position": position, "names": _ATTENTION_NAMES}
    right = {"kind": "gated_linear_attention", "hidden": cfg.width, "heads": g.heads, "dim": g.dim, "vdim": g.vdim,
             "tau": g.tau, "eps": cfg.eps, "rank": None}  # the decay map's width is the checkpoint's
    return {"kind": "side_by_side", "left": left, "right": right, "left_scale": m.left_scale, "right_scale": m.right_scale}


def bumolix_spec(cfg: BumolixConfig) -> ModelSpec:
    norm = {"kind": "rmsnorm", "size": cfg.width, "eps": cfg.eps, "tensor_suffix": ""}
    layers, ignored = [], []
    for i, ly in enumerate(cfg.layers):
        ff = ({"kind": "dense_act", "hidden": cfg.width, "intermediate": ly.mlp.ff, "activation": "relu2"} if ly.mlp else None)
        layers.append(LayerSpec(f"l{i}", {"kind": "parallel", "norm": norm, "mixer": _mixer(cfg, ly.mixer),
                                          "feed_forward": ff, "mult": cfg.residual_mult, "two_norms": True}))
        if ly.mlp is None:  # a layer without a feed-forward has no use for its second norm
            ignored.append(f"l{i}.norm2")
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, final_norm=norm, final_norm_prefix="final.norm",
        embedding={"kind": "token", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": "embed"},
        head={"kind": "linear", "vocab": cfg.vocab, "hidden": cfg.width, "tensor": None},
        ignored_tensors=tuple(ignored),
    )


register_architecture("Bumolix", BumolixConfig.from_dict, bumolix_spec, model_type="bumolix")
