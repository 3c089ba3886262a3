"""Kulivik through the engine's host side without a GPU: configuration, weights by name, the sandwich block and its
share of a request's state beside the mixer's, pages and slots used again, the scheduler.  The kernels are the torch
stand-ins of host_ops.py; what the CUDA kernels compute is tested on the GPU."""
import io
import json

import pytest
import torch

import helpers
import kulivik_helpers as KH
from host_ops import HostOps


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, name in enumerate(KH.CONFIGS):
        d = str(tmp_path_factory.mktemp("kulivik" + name))
        KH.make_model(d, name, seed=20 + i)
        out[name] = (d,) + KH.CONFIGS[name]
    return out


def _replay(d, steps, out_dir, max_tokens, page):
    from atoma_infer_b200.engine.trace import replay

    steps = helpers.number(steps)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    replay(d, "float32", out_dir, max_tokens, stream=io.StringIO(text), out=io.StringIO(), page_size=page, device="cpu",
           ops=HostOps())
    return steps


@pytest.mark.parametrize("name", list(KH.CONFIGS))
def test_every_cutting_matches_plain(name, models, tmp_path):
    d, cfg, page = models[name]
    seqs = helpers.random_tokens(cfg["vocab"], (1, 2, 9, 30, 47), seed=5)
    ref = KH.plain_logits(d, cfg, seqs)
    steps = (helpers.trace_whole(seqs) + helpers.trace_tail(seqs, tail=12) + helpers.trace_chunks(seqs, sizes=(5, 2, 7, 3, 2, 11, 1, 4))
             + helpers.trace_mixed(seqs, sizes=(6, 2, 9, 3, 5)))
    steps = _replay(d, steps, str(tmp_path), 192, page)  # four live requests at most, 64 tokens each: pages come back
    worst, where, agree, _ = helpers.compare_trace(steps, str(tmp_path), cfg["vocab"], ref)
    assert worst <= helpers.FP32_TOL, (worst, where)
    assert agree == 1.0


def test_config_is_read_key_by_key():
    from atoma_infer_b200.config import ConfigError
    from atoma_infer_b200.config.kulivik_config import (ConvSinkAttention, DenseFF, ExpertsFF, KulivikConfig, RotaryWindowAttention,
                                                        SideBySideSizes)

    cfg = KH.CONFIGS["U"][0]
    c = KulivikConfig.from_dict(cfg)
    assert (c.width, c.vocab, c.eps, c.logit_scale, c.logit_softcap) == (96, 131, 1e-5, 1.5, 12.0)
    conv, both, rot = (ly.mixer for ly in c.layers)
    assert isinstance(conv, ConvSinkAttention) and (conv.conv, conv.v_mix, conv.sizes.dim, conv.sizes.vdim) == (4, True, 32, 16)
    assert isinstance(both, SideBySideSizes) and (both.left_scale, both.right_scale, both.left.q_temp) == (0.55, 0.85, (0.7, 5))
    assert (both.right.heads, both.right.dim, both.right.vdim, both.right.decay) == (2, 24, 16, (0.5, 0.97))
    assert isinstance(rot, RotaryWindowAttention)
    assert (rot.window, rot.keep_first, rot.rot_dims, rot.rot_base, rot.softcap, rot.v_mix) == (9, 3, 8, 200.0, 5.0, True)
    assert isinstance(c.layers[0].mlp, DenseFF) and (c.layers[0].mlp.ff, c.layers[0].mlp.limit) == (160, 1.25)
    assert isinstance(c.layers[1].mlp, ExpertsFF) and (c.layers[1].mlp.ff, c.layers[1].mlp.experts, c.layers[1].mlp.top) == (40, 5, 1)
    assert c.layers[2].mlp is None
    # what an entry does not mention is off
    v = KulivikConfig.from_dict(KH.CONFIGS["V"][0])
    first = v.layers[0].mixer
    assert (first.window, first.keep_first, first.softcap, first.v_mix, first.rot_dims) == (None, 0, None, False, 32)
    assert v.layers[1].mixer.left.q_temp is None and v.layers[2].mixer.conv == 0
    assert (v.logit_scale, v.logit_softcap) == (1.0, None)

    def broken(edit, match):
        bad = json.loads(json.dumps(cfg))
        edit(bad)
        with pytest.raises(ConfigError, match=match):
            KulivikConfig.from_dict(bad)

    broken(lambda b: b["layers"][0].update(type="attention_3"), "attention_3")
    broken(lambda b: b["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay")
    broken(lambda b: b["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads")
    broken(lambda b: b["layers"][2]["mixer"]["rot"].update(dims=7), "rot.dims")
    broken(lambda b: b["layers"][0]["mlp"].update(kind="experts"), "experts")
    broken(lambda b: b["layers"][1]["mlp"]["router"].update(top=6), "top")
    broken(lambda b: b["layers"][0]["mlp"].pop("limit"), "limit")


def test_the_spec_puts_each_mechanism_where_the_configuration_says(models):
    from atoma_infer_b200.engine.runtime import load_model

    d, cfg, page = models["U"]
    lm = load_model(d, dtype="float32", device="cpu", ops=HostOps(), num_pages=16, page_size=page, max_seqs=2)
    blocks = lm.model.blocks
    assert [type(b).__name__ for b in blocks] == ["SandwichBlock"] * 3
    assert [type(b.mixer).__name__ for b in blocks] == ["Attention", "SideBySide", "Attention"]
    conv, both, rot = (b.mixer for b in blocks)
    assert (conv.taps, conv.learned_sink, conv.head_gate, conv.qk_norm is not None) == (4, True, True, True)
    assert (rot.window, rot.keep_first, rot.softcap, rot.head_norm_weight, rot.out_bias, rot.position.interleaved) == (9, 3, 5.0, True, True, True)
    assert both.left.distance_bias and both.left.q_temp == {"coef": 0.7, "every": 5} and both.scales == (0.55, 0.85)
    assert blocks[2].feed_forward is None and type(blocks[1].feed_forward).__name__ == "RoutedExperts"
    # the state of a request: the kept normed row, then the mixer's (a ring of three projected rows; two matrices)
    assert blocks[0].state_bytes() == 96 * 4 + 3 * (6 * 32 + 3 * 32 + 3 * 16) * 4
    assert blocks[1].state_bytes() == 96 * 4 + 2 * 24 * 16 * 4 and blocks[2].state_bytes() == 96 * 4
    # a window that keeps first tokens holds on to its pages; one that keeps none gives them back
    assert rot.cache_need().window is None
    dw, _, pw = models["W"]
    lw = load_model(dw, dtype="float32", device="cpu", ops=HostOps(), num_pages=16, page_size=pw, max_seqs=2)
    assert lw.model.blocks[1].mixer.cache_need().window == 20 and lw.model.blocks[3].mixer.cache_need().window is None


def test_a_missing_tensor_is_named(models, tmp_path):
    from atoma_infer_b200.engine.runtime import load_model
    from atoma_infer_b200.weights.loader import WeightError
    from atoma_infer_b200.weights.safetensors_io import write_safetensors

    d, cfg, page = models["U"]
    w = {k: v.to(torch.bfloat16) for k, v in helpers.read_weights(d).items()}
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    for name in ("l0.mix.k.conv", "l1.shift", "l2.mix.o.b", "l1.mlp.router.b", "l0.mix.sink", "l0.rg2.b"):
        gone = dict(w)
        del gone[name]
        write_safetensors(str(tmp_path / "model.safetensors"), gone, {})
        with pytest.raises(WeightError, match=name):
            load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)


def test_greedy_generation_through_the_scheduler(models):
    """Few pages and a small token budget: prompts are cut, requests preempted and recomputed, slots used again."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = models["U"]
    prompts = list(helpers.random_tokens(cfg["vocab"], (3, 26, 9, 17, 5), seed=8).values())
    want = [KH.plain_greedy(d, cfg, p, 10) for p in prompts]
    eng = Engine(d, dtype="float32", block_size=page, cuda_graphs=False, ops=HostOps(), num_gpu_blocks_override=22,
                 max_num_sequences=3, max_num_batched_tokens=11)
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=10, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
