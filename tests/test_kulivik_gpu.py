"""Kulivik on the GPU through the replay program and the engine: every cutting of the work against the plain
implementation, in both number formats, for configurations that differ in every size and option."""
import pytest
import torch

import helpers
import kulivik_helpers as KH

pytestmark = pytest.mark.gpu

BF16_TOP1 = 0.9


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per configuration and number format a model folder: bfloat16 runs get routers whose biases lie far apart."""
    out = {}
    for i, name in enumerate(KH.CONFIGS):
        for dtype in ("float32", "bfloat16"):
            d = str(tmp_path_factory.mktemp("kulivik" + name + dtype))
            # (W in bfloat16: a seed whose first positions do not happen to amplify every rounding several times over)
            seed = 62 if (name, dtype) == ("W", "bfloat16") else 30 + i
            KH.make_model(d, name, seed=seed, decisive=dtype == "bfloat16")
            out[name, dtype] = (d,) + KH.CONFIGS[name]
    return out


# lengths around the windows (9 with 3 kept; none; 20, and 5 with 7 kept), the pages' edges, the query temperature's
# stretches and the length from which a long portion's recurrence runs as chunks of time side by side (128); more requests
# than state slots, so that slots come back
LENGTHS = {"U": (1, 2, 9, 10, 13, 43, 90, 131, 64), "V": (3, 15, 17, 33, 160, 48), "W": (5, 19, 21, 26, 65, 130, 200, 8)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(KH.CONFIGS))
def test_every_cutting_matches_plain(name, dtype, models, tmp_path):
    d, cfg, page = models[name, dtype]
    seqs = helpers.random_tokens(cfg["vocab"], LENGTHS[name], seed=3)
    ref = KH.plain_logits(d, cfg, seqs)
    families = {
        "w": helpers.trace_whole(seqs, tag="w"),
        "t": helpers.trace_tail(seqs, tail=48, tag="t"),           # decoding passes windows' edges
        "c": helpers.trace_chunks(seqs, tag="c"),                  # portions of 1 to 11 tokens
        "m": helpers.trace_mixed(seqs, tag="m"),
        "n": helpers.trace_mixed(seqs, sizes=(140, 2, 37, 1, 64), tag="n", seed=1),  # long portions beside single tokens
    }
    steps = [s for f in families.values() for s in f]
    if dtype == "bfloat16":  # a router's close call may rightly go the other way: nothing is asked from there on
        steps = KH.want_before(steps, KH.first_close_call(d, cfg, seqs))
    longest = sorted((len(v) for v in seqs.values()), reverse=True)[:4]
    max_tokens = sum(-(-n // 64) * 64 for n in longest)             # pages and slots are used again
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), max_tokens, page)
    tol = helpers.FP32_TOL if dtype == "float32" else helpers.BF16_TOL
    # bfloat16: a place that amplifies every rounding is judged by what rounding does to the plain implementation there
    rounding = KH.rounding_errors(d, cfg, seqs, ref) if dtype == "bfloat16" else None
    for tag in families:
        sub = [s for s in steps if s["entries"][0]["id"].startswith(tag)]
        worst, where, agree, clear = helpers.compare_trace(sub, out, cfg["vocab"], ref, rounding=rounding)
        assert worst <= tol, f"family {tag!r}: error {worst:.3g} of the logit scale at (step, request, position) {where}"
        if dtype == "float32":
            assert agree == 1.0, f"family {tag!r}: greedy tokens differ from the plain implementation"
        else:
            assert agree >= BF16_TOP1 and clear == 1.0, f"family {tag!r}: top-1 agreement {agree:.3f} ({clear:.3f} where clear)"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_one_token_at_a_time(dtype, models, tmp_path):
    """A short prompt, then hundreds of single-token steps through the captured decode graph: the window passes over
    decoded tokens while the kept ones stay, the convolution's ring turns over a hundred times, the kept normed row and
    the decaying states are carried through every step."""
    d, cfg, page = models["U", dtype]
    seq = helpers.random_tokens(cfg["vocab"], (330,), seed=11)
    ref = KH.plain_logits(d, cfg, seq)
    steps = helpers.trace_tail(seq, tail=322)
    if dtype == "bfloat16":
        steps = KH.want_before(steps, KH.first_close_call(d, cfg, seq))
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), 384, page)
    worst, where, agree, clear = helpers.compare_trace(steps, out, cfg["vocab"], ref)
    assert worst <= (helpers.FP32_TOL if dtype == "float32" else helpers.BF16_TOL), (worst, where)
    assert agree == 1.0 if dtype == "float32" else agree > 0.95


def test_a_long_prompt_in_one_step_and_in_two(models, tmp_path):
    """Seven hundred tokens at once (the recurrence in eleven chunks of time, attention over dozens of pages), and the same
    cut at a place that is no edge of anything."""
    d, cfg, page = models["W", "float32"]
    seq = helpers.random_tokens(cfg["vocab"], (700,), seed=5)
    ref = KH.plain_logits(d, cfg, seq)
    v = seq["r0"]
    steps = helpers.trace_whole(seq, tag="w") + [
        {"entries": [{"id": "cr0", "tokens": v[:389], "want": list(range(0, 389, 7))}], "end": []},
        {"entries": [{"id": "cr0", "tokens": v[389:], "want": list(range(311))}], "end": ["cr0"]}]
    steps, out = helpers.run_trace(d, "float32", steps, str(tmp_path), 1536, page)
    worst, where, agree, _ = helpers.compare_trace(steps, out, cfg["vocab"], ref)
    assert worst <= helpers.FP32_TOL and agree == 1.0, (worst, where, agree)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_through_the_engine(dtype, models):
    """Greedy tokens through the entry point and the scheduler, with few pages and a small token budget (prompts in
    portions, preemption and recomputation, slots used again), against the plain loop."""
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams
    import plain_kulivik as PK

    d, cfg, page = models["W", dtype]
    prompts = list(helpers.random_tokens(cfg["vocab"], (3, 70, 9, 130, 21), seed=8).values())
    eng = Engine(d, dtype=dtype, block_size=page, num_gpu_blocks_override=40, max_num_sequences=3, max_num_batched_tokens=48)
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=12, ignore_eos_token=True))
    eng.lm.rt.ops.check_status()
    assert eng.lm.manager.audit() == "" and eng.lm.manager.num_requests() == 0
    w = helpers.read_weights(d)
    for p, o in zip(prompts, outs):
        got = o.token_ids
        if dtype == "float32":
            assert got == KH.plain_greedy(d, cfg, p, 12)
            continue
        logits = PK.forward(cfg, w, list(p) + list(got))  # each token judged on the engine's own history
        for i, tok in enumerate(got):
            row = logits[len(p) - 1 + i]
            lead = float(row.max() - row[tok]) / float(row.abs().max())
            assert lead <= 2 * helpers.BF16_TOL, (i, tok, lead)


def test_the_command_line_serves_the_design(tmp_path):
    """``random-model`` writes a Kulivik folder from its configuration, ``generate`` decodes greedily from it; both as
    child processes, the tokens against the plain loop (float32)."""
    import json
    import os
    import subprocess
    import sys

    cli = os.path.join(helpers.ROOT, "bin", "atoma-infer")
    cfg, page = KH.CONFIGS["V"]
    (tmp_path / "config_in.json").write_text(json.dumps(cfg))
    out = tmp_path / "model"

    def run(args):
        p = subprocess.run([sys.executable, cli, *args], capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, f"atoma-infer {' '.join(args)} failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
        return p

    run(["random-model", "--config", str(tmp_path / "config_in.json"), "--seed", "7", "--out", str(out), "--std", "0.05",
         "--norm-jitter", "0.1"])
    prompts = [[3, 14, 15, 92, 65, 35, 89, 79], list(range(40, 95))]
    args = ["generate", "--model", str(out), "--dtype", "f32", "--block-size", str(page), "--num-gpu-blocks-override", "16",
            "--max-num-batched-tokens", "24", "--max-num-sequences", "2", "--no-do-sample", "--max-new-tokens", "8",
            "--ignore-eos-token"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    recs = [json.loads(line) for line in run(args).stdout.splitlines() if line.startswith("{")]
    assert [r["token_ids"] for r in recs] == [KH.plain_greedy(str(out), cfg, p, 8) for p in prompts]
