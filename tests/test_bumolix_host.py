"""Bumolix through the engine's host side without a GPU: configuration, weights by name, the block with two norms, two
mixers' shares of a request's state, pages and slots used again, the scheduler.  The kernels are the torch stand-ins of
host_ops.py; what the CUDA kernels compute is tested on the GPU."""
import io
import json

import pytest
import torch

import bumolix_helpers as BH
import helpers
from host_ops import HostOps


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, name in enumerate(BH.CONFIGS):
        d = str(tmp_path_factory.mktemp("bumolix" + name))
        BH.make_model(d, name, seed=10 + i)
        out[name] = (d,) + BH.CONFIGS[name]
    return out


def _replay(d, steps, out_dir, max_tokens, page):
    from atoma_infer_b200.engine.trace import replay

    steps = helpers.number(steps)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    replay(d, "float32", out_dir, max_tokens, stream=io.StringIO(text), out=io.StringIO(), page_size=page, device="cpu",
           ops=HostOps())
    return steps


@pytest.mark.parametrize("name", list(BH.CONFIGS))
def test_every_cutting_matches_plain(name, models, tmp_path):
    d, cfg, page = models[name]
    seqs = helpers.random_tokens(cfg["vocab"], (1, 2, 9, 30, 47), seed=5)
    ref = BH.plain_logits(d, cfg, seqs)
    steps = (helpers.trace_whole(seqs) + helpers.trace_tail(seqs, tail=12) + helpers.trace_chunks(seqs, sizes=(5, 2, 7, 3, 2, 11, 1, 4))
             + helpers.trace_mixed(seqs, sizes=(6, 2, 9, 3, 5)))
    steps = _replay(d, steps, str(tmp_path), 192, page)  # four live requests at most, 64 tokens each: pages come back
    worst, where, agree, _ = helpers.compare_trace(steps, str(tmp_path), cfg["vocab"], ref)
    assert worst <= helpers.FP32_TOL, (worst, where)
    assert agree == 1.0


def test_config_is_read_key_by_key():
    from atoma_infer_b200.config import ConfigError
    from atoma_infer_b200.config.bumolix_config import BumolixConfig, Mamba1Sizes, SideBySideSizes

    cfg = BH.CONFIGS["P"][0]
    c = BumolixConfig.from_dict(cfg)
    assert (c.width, c.vocab, c.eps, c.residual_mult) == (96, 131, 1e-5, 0.6)
    scan, pair, last = (ly.mixer for ly in c.layers)
    assert isinstance(scan, Mamba1Sizes) and (scan.inner, scan.state, scan.dt_rank, scan.conv) == (80, 24, 6, 4)
    assert isinstance(pair, SideBySideSizes) and (pair.left_scale, pair.right_scale) == (0.55, 0.85)
    assert (pair.left.heads, pair.left.kv_heads, pair.left.dim, pair.left.vdim, pair.left.chunk) == (6, 2, 16, 24, 21)
    assert (pair.left.rot_dims, pair.left.rot_base, pair.left.rot_factor, pair.left.scale) == (8, 2e5, 3.0, 0.3)
    assert (pair.right.heads, pair.right.dim, pair.right.vdim, pair.right.tau) == (3, 24, 16, 8.0)
    assert last.left.rot_factor == 1.0 and c.layers[2].mlp is None and c.layers[0].mlp.ff == 160
    q = BumolixConfig.from_dict(BH.CONFIGS["Q"][0])
    assert q.layers[0].mixer.left.chunk is None and q.layers[0].mixer.left.rot_dims == 0

    def broken(edit, match):
        bad = json.loads(json.dumps(cfg))
        edit(bad)
        with pytest.raises(ConfigError, match=match):
            BumolixConfig.from_dict(bad)

    broken(lambda b: b["layers"][0].update(type="mamba3"), "mamba3")
    broken(lambda b: b["layers"][1]["mixer"]["right"].pop("tau"), "tau")
    broken(lambda b: b["layers"][1]["mixer"]["left"].update(kv_heads=4), "kv_heads")
    broken(lambda b: b["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims")
    broken(lambda b: b["layers"][0]["mlp"].update(kind="experts"), "experts")
    broken(lambda b: b["layers"][0]["mixer"].update(state=0), "state")


def test_the_spec_puts_each_mechanism_where_the_configuration_says(models):
    from atoma_infer_b200.engine.runtime import load_model

    d, cfg, page = models["P"]
    lm = load_model(d, dtype="float32", device="cpu", ops=HostOps(), num_pages=16, page_size=page, max_seqs=2)
    blocks = lm.model.blocks
    kinds = [type(b.mixer).__name__ for b in blocks]
    assert kinds == ["SelectiveScanMixer", "SideBySide", "SideBySide"]
    pair = blocks[1].mixer
    assert (pair.left.chunk, pair.left.sink, pair.scales) == (21, True, (0.55, 0.85))
    assert blocks[2].feed_forward is None and blocks[0].feed_forward is not None
    # the state of a request: the scan's ring and matrices; the pair's linear-attention matrices (the attention keeps pages)
    assert blocks[0].mixer.state_bytes() == (3 * 80 * 4) + 80 * 24 * 4
    assert pair.state_bytes() == 3 * 24 * 16 * 4 and pair.cache_need() is not None and blocks[0].mixer.cache_need() is None


def test_a_missing_tensor_is_named_and_free_sizes_come_from_the_checkpoint(models, tmp_path):
    from atoma_infer_b200.engine.runtime import load_model
    from atoma_infer_b200.weights.loader import WeightError
    from atoma_infer_b200.weights.safetensors_io import write_safetensors

    d, cfg, page = models["P"]
    w = {k: v.to(torch.bfloat16) for k, v in helpers.read_weights(d).items()}
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    gone = dict(w)
    del gone["l1.mix.right.a2.b"]
    write_safetensors(str(tmp_path / "model.safetensors"), gone, {})
    with pytest.raises(WeightError, match="l1.mix.right.a2.b"):
        load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)
    # a decay map of another width loads as long as its two matrices agree, and is refused when they do not
    g = torch.Generator().manual_seed(1)
    wide = dict(w)
    wide["l1.mix.right.a1"] = (torch.randn(5, 96, generator=g) * 0.05).to(torch.bfloat16)
    wide["l1.mix.right.a2"] = (torch.randn(72, 5, generator=g) * 0.05).to(torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), wide, {})
    lm = load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)
    assert lm.model.blocks[1].mixer.right.w_a1.shape == (5, 96)
    wide["l1.mix.right.a2"] = w["l1.mix.right.a2"]
    write_safetensors(str(tmp_path / "model.safetensors"), wide, {})
    with pytest.raises(WeightError, match="l1.mix.right.a"):
        load_model(str(tmp_path), dtype="float32", device="cpu", ops=HostOps(), num_pages=8, page_size=page, max_seqs=2)


def test_greedy_generation_through_the_scheduler(models):
    """Few pages and a small token budget: prompts are cut, requests preempted and recomputed, slots used again."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, page = models["P"]
    prompts = list(helpers.random_tokens(cfg["vocab"], (3, 26, 9, 17, 5), seed=8).values())
    want = [BH.plain_greedy(d, cfg, p, 10) for p in prompts]
    eng = Engine(d, dtype="float32", block_size=page, cuda_graphs=False, ops=HostOps(), num_gpu_blocks_override=22,
                 max_num_sequences=3, max_num_batched_tokens=11)
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=10, ignore_eos_token=True))
    assert [o.token_ids for o in outs] == want
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
