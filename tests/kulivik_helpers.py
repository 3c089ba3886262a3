"""Small Kulivik configurations for the tests, their model folders, and the plain logits of token lists.

The configurations differ in every size and constant and pick values that tell mechanisms apart: windows that are no
multiple of a page with kept first tokens that end inside a page (and a window without kept tokens, whose pages come
back, and no window at all); a rotation over part of a head, over all of it and none, with sizes that are no multiple of
four; heads of keys larger and smaller than heads of values; one key/value head for all query heads and one for each;
convolutions of two to four taps and none; the first value-mixing layer of either kind; a query temperature whose
stretches are a few positions long; decays from fast to none; experts of which one, some or all are chosen; a layer
without a feed-forward; every kind of layer first; logits with and without scale and cap.
"""
from __future__ import annotations

from typing import Dict, List

import torch

import helpers
import plain_kulivik as PK


def rotary(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot=None, base=1e4, softcap=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    if softcap:
        m["softcap"] = softcap
    if v_mix:
        m["v_mix"] = True
    return m


def convolved(heads, kv_heads, dim, vdim, scale, conv=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if v_mix:
        m["v_mix"] = True
    return m


def pair(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def biased(heads, kv_heads, dim, vdim, scale, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def decaying(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5, logit_scale=None, logit_softcap=None):
    c = {"architecture": "Kulivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    if logit_softcap is not None:
        c["logit_softcap"] = logit_softcap
    return c


# name -> (config, page size)
CONFIGS = {
    # the convolved kind first (it leaves the values the later layer mixes in), four taps, keys of 32 and values of 16;
    # side by side: a key/value head per query head, stretches of 5 positions, one expert of five; a window of 9 over pages
    # of 4 that keeps 3 tokens, half a head rotated; no feed-forward in the last layer
    "U": (config(96, 131, [layer("attention", convolved(6, 3, 32, 16, 0.2, conv=4, v_mix=True), dense(160, 1.25)),
                           layer("parallel", pair(biased(4, 4, 16, 24, 0.3, q_temp=(0.7, 5)),
                                                  decaying(2, 24, 16, (0.5, 0.97)), 0.55, 0.85), moe(40, 5, 1)),
                           layer("attention_2", rotary(6, 3, 16, 16, 0.4, window=9, keep_first=3, rot=8, base=200.0, softcap=5.0,
                                                       v_mix=True))],
                 logit_scale=1.5, logit_softcap=12.0), 4),
    # the rotated kind first: no window, no cap, a whole head rotated, no value mixing; one key/value head for eight query
    # heads without a temperature; no convolution; all experts chosen; logits as they are
    "V": (config(128, 300, [layer("attention_2", rotary(4, 2, 32, 48, 0.15, rot=32, base=1e6), moe(24, 3, 3)),
                            layer("parallel", pair(biased(8, 1, 16, 16, 0.25), decaying(4, 8, 40, (1.0, 0.9, 0.3, 0.995)),
                                                   1.0, 1.0), dense(72, 3.0)),
                            layer("attention", convolved(2, 1, 64, 64, 0.125, v_mix=True), moe(64, 4, 2))], eps=1e-6), 16),
    # sizes that are no multiple of four (heads of 18 with 6 rotated, values of 10); a window of 20 that keeps nothing (its
    # pages come back) and one of 5 that keeps more than it spans; two taps; the side-by-side kind first and last
    "W": (config(72, 97, [layer("parallel", pair(biased(2, 2, 24, 8, 0.3, q_temp=(0.25, 3)), decaying(3, 16, 8, (0.8, 0.95, 0.6)),
                                                 0.8, 1.1), dense(48, 0.75)),
                          layer("attention_2", rotary(4, 2, 18, 10, 0.3, window=20, rot=6, base=50.0, softcap=2.0, v_mix=True),
                                moe(32, 6, 2)),
                          layer("attention", convolved(4, 2, 18, 10, 0.3, conv=2, v_mix=True)),
                          layer("attention_2", rotary(4, 4, 16, 16, 0.25, window=5, keep_first=7, softcap=25.0), dense(80, 1.75)),
                          layer("parallel", pair(biased(6, 3, 16, 16, 0.2), decaying(1, 40, 24, (0.99,)), 0.4, 1.3),
                                moe(16, 2, 1))], logit_softcap=8.0), 8),
}

# stds that make every mechanism matter and leave the stream near 1: biases and sinks of order one, shifts and mixing
# weights well inside (0, 1), convolutions far from zero, gates that open and close, routers that choose clearly.  A key
# counts wherever it is part of a name, and the factors of all keys that match multiply.
SCALES = {".q.b": 12.0, ".k.b": 12.0, ".v.b": 12.0, ".o.b": 6.0, "sink": 30.0, "shift": 7.0, "vmix": 8.0, ".conv": 8.0,
          "rg1": 4.0, "rg2": 4.0, "router": 6.0, "mix.o": 2.0, "mix.left.o": 2.0, "mix.right.o": 2.0, "down": 2.0}


def make_model(path: str, name: str, seed: int = 0, decisive: bool = False) -> str:
    """``decisive``: router biases far apart, so that few choices hang on a lead that rounding to bfloat16 can turn (the
    choice still depends on the token where two biases lie close)."""
    cfg, _ = CONFIGS[name]
    scales = dict(SCALES, **{"router.b": 30.0}) if decisive else SCALES
    return helpers.make_model(path, cfg, seed=seed, scales=scales, norm_jitter=0.2)


def plain_logits(model_dir: str, cfg: dict, seqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    w = helpers.read_weights(model_dir)
    return {k: PK.forward(cfg, w, v) for k, v in seqs.items()}


def plain_greedy(model_dir: str, cfg: dict, prompt: List[int], n: int) -> List[int]:
    w = helpers.read_weights(model_dir)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(PK.forward(cfg, w, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out


def first_close_call(model_dir: str, cfg: dict, seqs: Dict[str, List[int]], lead: float = 0.01) -> Dict[str, int]:
    """Per request the first position at which a router's choice hangs on a lead of less than ``lead`` of its largest
    logit (the length of the request if there is none).  From there on a reduced-precision engine may rightly choose
    another expert, and every later position of the request reads what that choice left in the caches."""
    w = helpers.read_weights(model_dir)
    out = {}
    for k, v in seqs.items():
        margins: list = []
        PK.forward(cfg, w, v, margins=margins)
        worst = torch.stack(margins).min(0).values if margins else torch.full((len(v),), float("inf"))
        close = (worst < lead).nonzero().flatten()
        out[k] = int(close[0]) if len(close) else len(v)
    return out


def want_before(steps, limit: Dict[str, int], strip: int = 1):
    """The steps with every wanted place at or after its request's limit taken out (the tokens still run)."""
    pos: Dict[str, int] = {}
    out = []
    for s in steps:
        entries = []
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            entries.append(dict(e, want=[x for x in e["want"] if start + x < limit[e["id"][strip:]]]))
            pos[e["id"]] = start + len(e["tokens"])
        out.append(dict(s, entries=entries))
    return out


def rounding_errors(model_dir: str, cfg: dict, seqs: Dict[str, List[int]], ref: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per position, how far the plain implementation itself moves (largest logit difference over the largest logit of
    the sequence) when what its matrix products read and write is rounded to bfloat16: the measure of how much a
    position amplifies roundings that no implementation in that type can avoid."""
    w = helpers.read_weights(model_dir)
    return {k: (PK.forward(cfg, w, v, round_to=torch.bfloat16) - ref[k]).abs().max(-1).values / ref[k].abs().max()
            for k, v in seqs.items()}
