"""Small Bumolix configurations for the tests, their model folders, and the plain logits of token lists.

The configurations differ in every size and constant, and pick values that make mechanisms distinguishable: chunks that
are no multiple of a page (and one that is, and none), heads of keys larger and smaller than heads of values and sizes
that are no multiple of 16, one key/value head for all query heads and one for each, a rotation over part of a head, over
all of it and none, stretched positions and unstretched; linear attention with one head and several, key channels that
two and four threads share, decay maps of several widths; selective scans with states of 5 to 40 values, two to five
taps and one; layers without a feed-forward; the first layer of either kind; scales and factors other than 1.
"""
from __future__ import annotations

from typing import Dict, List

import torch

import helpers
import plain_bumolix as PB


def attention(heads, kv_heads, dim, vdim, scale, chunk=None, rot_dims=None, base=10000.0, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def linear(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def parallel(left, right, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def mamba(inner, state, dt_rank, conv, mlp=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, mult, eps=1e-5):
    return {"architecture": "Bumolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": layers}


# name -> (config, page size)
CONFIGS = {
    # chunks of 21 over pages of 4; keys of 16 and values of 24; a state of 24 values; a layer without feed-forward;
    # the scan comes first
    "P": (config(96, 131, [mamba(80, 24, 6, 4, dense(160)),
                           parallel(attention(6, 2, 16, 24, 0.3, chunk=21, rot_dims=8, base=2e5, factor=3.0),
                                    linear(3, 24, 16, 8.0), 0.55, 0.85, dense(72)),
                           parallel(attention(4, 4, 24, 8, 0.25, chunk=21, rot_dims=24, base=100.0),
                                    linear(1, 40, 24, 2.0), 1.3, 0.4)], mult=0.6), 4),
    # no chunk at all and chunks of one page; one key/value head for twenty query heads (the plain kernel in both modes);
    # no rotation; one tap; five states; factor and scales 1
    "Q": (config(128, 300, [parallel(attention(20, 1, 16, 16, 0.5), linear(4, 8, 40, 12.0), 1.0, 1.0, dense(192)),
                            mamba(96, 5, 3, 1),
                            parallel(attention(2, 1, 64, 64, 0.125, chunk=16, rot_dims=32, base=1e4, factor=2.0),
                                     linear(2, 64, 64, 4.0), 0.5, 2.0, dense(64))], mult=1.0, eps=1e-6), 16),
    # two scans in a row with 40 and 16 states, five and two taps; chunks of 64 = 8 pages and of 9; key channels that
    # four threads share (80) and heads of 128 values
    "R": (config(64, 97, [parallel(attention(4, 2, 32, 48, 0.2, chunk=64, rot_dims=16, base=1e6, factor=8.0),
                                   linear(2, 80, 128, 32.0), 0.8, 1.1, dense(80)),
                          mamba(128, 40, 10, 5, dense(48)),
                          mamba(48, 16, 4, 2),
                          parallel(attention(8, 2, 16, 16, 0.4, chunk=9, rot_dims=4, base=50.0),
                                   linear(5, 16, 8, 1.0), 1.0, 0.7, dense(96))], mult=0.5), 8),
}

# stds that make every mechanism matter and leave the stream near 1, so that no layer hides the others: biases of order
# one, decays from fast to nearly none (so that far tokens count), step sizes that differ from channel to channel and
# decay rates over three orders of magnitude, convolutions far from zero.  A key counts wherever it is part of a name, and
# the factors of all keys that match multiply ("mix.conv" also scales the convolution's bias).
SCALES = {".q.b": 20.0, ".k.b": 20.0, ".v.b": 20.0, "a1": 3.0, "a2": 6.0, "a2.b": 6.0, "A_log": 30.0, "mix.conv": 8.0,
          "conv.b": 0.75, "mix.dt": 10.0, "dt.b": 2.0, "mix.x": 4.0, "mix.o": 3.0, "mix.in": 1.4}


def make_model(path: str, name: str, seed: int = 0) -> str:
    cfg, _ = CONFIGS[name]
    return helpers.make_model(path, cfg, seed=seed, scales=SCALES, norm_jitter=0.2)


def plain_logits(model_dir: str, cfg: dict, seqs: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    w = helpers.read_weights(model_dir)
    return {k: PB.forward(cfg, w, v) for k, v in seqs.items()}


def rounding_errors(model_dir: str, cfg: dict, seqs: Dict[str, List[int]], ref: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per position, how far the plain implementation itself moves (largest logit difference over the largest logit of
    the sequence) when what its matrix products read and write is rounded to bfloat16: the measure of how much a
    position amplifies roundings that no implementation in that type can avoid."""
    w = helpers.read_weights(model_dir)
    return {k: (PB.forward(cfg, w, v, round_to=torch.bfloat16) - ref[k]).abs().max(-1).values / ref[k].abs().max()
            for k, v in seqs.items()}


def plain_greedy(model_dir: str, cfg: dict, prompt: List[int], n: int) -> List[int]:
    w = helpers.read_weights(model_dir)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(PB.forward(cfg, w, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
