"""Benchmark: decode and prefill throughput of Llama 3.2 1B (random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token prompt
in the cache (context up to 4,096).  ``value`` is decoded tokens a second over exactly
K steps, timed on the device; ``e2e`` is the same through ``Engine.step()``, with the
step's inputs copied from pinned host memory and the sampled tokens read back every
step.  Also: prefill of 2,048 tokens, decode at batch 1 and 64, and the decode step's
fraction of the measured HBM bandwidth.  Prints ONE JSON line.

``--designs`` instead of the benchmark: prefill and decode throughput of the Dosovik design beside Llama at equal
layer sizes, and the design's own kernels beside Llama's like kernels with their fractions of the copy bandwidth.
``--kulivik``: the same for the Kulivik design (windowed, biased and convolved attention, linear attention with constant
decays, routed experts), beside Llama and Bumolix.  ``--bumolix``: the same for the Bumolix design (attention beside gated linear attention, selective-scan layers), beside
Llama and Tutezen.  ``--tutezen``: the same for the Tutezen design (state-space and latent-attention layers, routed experts) at Llama's width
and as many layer runs.

Tables for profiles/ instead of the JSON line: ``--linears [--model 1b|3b|8b]`` (the two few-row linear
kernels on the four matrices of a layer) and ``--layer-kernel-phases`` (the persistent layer kernel's time
per phase); ``--model 3b|8b`` alone runs that configuration's serving workload through ``Engine.generate``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = {  # Llama 3.2 1B
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "vocab_size": 128256,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": 128001,
}
PROMPT_LEN, PREFILL_TOKENS, PAGE = 2048, 2048, 16

_LLAMA3 = {"architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "num_key_value_heads": 8, "head_dim": 128,
           "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072, "bos_token_id": 128000,
           "eos_token_id": 128001}
# The larger configurations with their serving workloads: requests, prompt lengths and new tokens (uniform, both
# ends included), seed, temperature, token budget of a step.
WORKLOADS = {
    "3b": {"config": dict(_LLAMA3, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
                          tie_word_embeddings=True,
                          rope_scaling={"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192, "rope_type": "llama3"}),
           "name": "Llama-3.2-3B", "requests": 16, "prompt": (256, 2048), "new": (256, 256), "seed": 3,
           "temperature": None, "budget": 2048},
    "8b": {"config": dict(_LLAMA3, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                          tie_word_embeddings=False,
                          rope_scaling={"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192, "rope_type": "llama3"}),
           "name": "Llama-3.1-8B", "requests": 64, "prompt": (128, 4096), "new": (128, 512), "seed": 4,
           "temperature": 0.7, "budget": 2048},
}


def serving_workload(which: str) -> int:
    """A larger configuration with its serving workload through ``Engine.generate`` (random weights drawn on the
    device; scheduler, chunked prefill, mixed steps, decode graphs).  Run twice: once as a user would, for the
    end-to-end rate; once with a synchronisation after every step, to split the time into decode-only steps
    (bytes they must read against the copy bandwidth) and steps that carry prompt tokens (flops against the
    tensor peak).  Prints one JSON line."""
    import tempfile
    import time

    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    wl = WORKLOADS[which]
    cfg = wl["config"]
    hbm_gbs, bf16_tflops, peak_kind = peaks()
    g = torch.Generator().manual_seed(wl["seed"])
    n = wl["requests"]
    plens = torch.randint(wl["prompt"][0], wl["prompt"][1] + 1, (n,), generator=g).tolist()
    news = torch.randint(wl["new"][0], wl["new"][1] + 1, (n,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (p,), generator=g).tolist() for p in plens]
    params = [SamplingParams(do_sample=wl["temperature"] is not None, temperature=wl["temperature"], random_seed=100 + i,
                             max_new_tokens=m, ignore_eos_token=True) for i, m in enumerate(news)]
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lin_params = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    head_params = V * H
    weight_bytes = 2 * (lin_params + head_params)  # decode reads every linear once and the head; no embedding rows to speak of
    kv_bytes_per_token = 2 * L * nkv * d * 2
    pages = sum(-(-(p + m) // PAGE) for p, m in zip(plens, news)) + 64
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "config.json"), "w") as f:
            json.dump(cfg, f)
        eng = Engine(tmp, dtype="bfloat16", block_size=PAGE, num_gpu_blocks_override=pages, max_num_sequences=n,
                     max_num_batched_tokens=wl["budget"], random_weights_seed=0)
    lm = eng.lm
    eng.generate([prompts[0][:64]], SamplingParams(do_sample=False, max_new_tokens=4, ignore_eos_token=True))  # libraries load
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    steps_e2e, launches = eng.num_steps, lm.rt.ops.launches
    generated = sum(len(o.token_ids) for o in outs)
    assert [len(o.token_ids) for o in outs] == news
    # second run, a synchronisation after every step
    rec = {"decode": [0, 0.0, 0.0, 0], "mixed": [0, 0.0, 0.0, 0]}  # steps, seconds, bytes or flops, tokens
    run = lm.step.run

    def timed(entries):
        ctx = [lm.manager.num_tokens(e.req) if lm.manager.has_request(e.req) else 0 for e in entries]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        out = run(entries)
        b.record()
        torch.cuda.synchronize()
        dt = a.elapsed_time(b) * 1e-3  # device time of the step, launch gaps of prompt steps included
        toks = sum(len(e.tokens) for e in entries)
        if all(len(e.tokens) == 1 for e in entries):
            r = rec["decode"]
            r[2] += weight_bytes + kv_bytes_per_token * sum(c + 1 for c in ctx)
        else:
            r = rec["mixed"]
            attn = sum(4 * d * nq * L * (len(e.tokens) * c + len(e.tokens) * (len(e.tokens) + 1) // 2) for e, c in zip(entries, ctx))
            r[2] += 2 * toks * lin_params + attn + 2 * head_params * sum(1 for e in entries if e.want)
        r[0] += 1
        r[1] += dt
        r[3] += toks
        return out

    lm.step.run = timed
    eng.generate(prompts, params)
    lm.step.run = run
    clock_rec = clocks.stop()
    dec, mix = rec["decode"], rec["mixed"]
    out = {
        "metric": f"generated tok/s through Engine.generate ({wl['name']} sizes, {n} requests)", "value": generated / wall,
        "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "vs_baseline": None, "seconds": wall, "total_tok_s": (generated + sum(plens)) / wall, "steps": steps_e2e,
        "prompt_tokens": sum(plens), "generated_tokens": generated, "preemptions": eng.scheduler.num_preemptions,
        "gpu_launches": launches,
        "config": {"model": f"{wl['name']} (random weights N(0,0.02), seed 0)", "layers": L, "hidden": H, "heads": nq,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V, "requests": n,
                   "prompt_lengths": f"uniform {wl['prompt']}, seed {wl['seed']}", "new_tokens": f"uniform {wl['new']}",
                   "temperature": wl["temperature"], "token_budget": wl["budget"], "page_size": PAGE, "parallelism": "1 GPU"},
        "decode_steps": {"steps": dec[0], "ms_per_step": dec[1] / max(dec[0], 1) * 1e3, "tokens_per_step": dec[3] / max(dec[0], 1),
                         "achieved": dec[2] / max(dec[1], 1e-9) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": dec[2] / max(dec[1], 1e-9) / 1e9 / hbm_gbs, "of": peak_kind},
        "prompt_steps": {"steps": mix[0], "ms_per_step": mix[1] / max(mix[0], 1) * 1e3, "tokens_per_step": mix[3] / max(mix[0], 1),
                         "achieved": mix[2] / max(mix[1], 1e-9) / 1e12, "peak": bf16_tflops, "unit": "TFLOP/s",
                         "frac": mix[2] / max(mix[1], 1e-9) / 1e12 / bf16_tflops, "of": f"{peak_kind} bf16 burst"},
        "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


def few_row_linears(which: str) -> int:
    """Times the two few-row linear kernels on the four matrices of a layer: 32 calls in one CUDA graph that cycle
    through as many weight sets as fit 2.5 GB (so no weight is found in L2), CUDA events around three replays."""
    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine.runtime import make_runtime

    H, I, nq, nkv, d = {"1b": (2048, 8192, 32, 8, 64), "3b": (3072, 8192, 24, 8, 128), "8b": (4096, 14336, 32, 8, 128)}[which]
    shapes = {"q/k/v": ((nq + 2 * nkv) * d, H, False), "output": (H, nq * d, False), "gate/up + SwiGLU": (2 * I, H, True),
              "down": (H, I, False)}
    rt = make_runtime("bfloat16", "cuda:0")
    ops, dev = rt.ops, rt.device
    hbm = peaks()[0]

    def graph_us(fn, n=32):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(3):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (3 * n) * 1e3

    print(f"few-row linears, Llama sizes {which}: us a call, direct | streamed (at the copy bandwidth {hbm:.0f} GB/s: ideal)")
    for name, (N, K, silu) in shapes.items():
        sets = max(2, min(16, int(2.5e9 // (N * K * 2))))
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
        row = []
        for M in (1, 8, 16):
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            cell = []
            for streamed in (False, True):
                ops.stream_linear = streamed
                if streamed and not ops._stream_linear(2, N, K):
                    cell.append(float("nan"))
                    continue
                calls = [0]

                def call():
                    if streamed:  # whatever the policy for this row count says
                        ops.linear_streamed(x, ws[calls[0] % sets], silu_mul=silu)
                    else:
                        ops.linear(x, ws[calls[0] % sets], silu_mul=silu)
                    calls[0] += 1
                cell.append(graph_us(call))
            row.append(f"{M:2d} rows {cell[0]:6.1f} | {cell[1]:6.1f}")
        print(f"  {name:18s} {N:6d} x {K:5d} ({N * K * 2 / 1e6:6.1f} MB, ideal {N * K * 2 / hbm / 1e3:5.1f}):  " + "   ".join(row))
        del ws
    ops.check_status()
    return 0


# Layer sizes that resemble real models, used for both designs: (width, feed-forward, heads, key/value heads, head size)
DESIGN_SIZES = {"w2048-h64": (2048, 8192, 32, 8, 64), "w3072-h128": (3072, 8192, 24, 8, 128), "w4096-h128": (4096, 14336, 32, 8, 128)}


def design_configs(size: str, layers: int, vocab: int = 32768, chunk: int = 1024, value_dim: int = 0):
    """(Llama config, Dosovik config) of equal width, heads, head size, feed-forward size, layers and vocabulary."""
    import math

    H, I, nq, nkv, d = DESIGN_SIZES[size]
    llama = {"architectures": ["LlamaForCausalLM"], "hidden_size": H, "intermediate_size": I, "vocab_size": vocab,
             "num_hidden_layers": layers, "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d,
             "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072, "tie_word_embeddings": False}
    mixer = {"heads": nq, "kv_heads": nkv, "dim": d, "vdim": value_dim or d, "scale": 1 / math.sqrt(d), "v_mix": True,
             "mask": {"size": chunk}, "rot": {"dims": d // 2, "base": 500000.0}}
    dosovik = {"architecture": "Dosovik", "vocab": vocab, "width": H, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
               "embedding": {"scale": math.sqrt(H)}, "canon": {"taps": 4},
               "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": I}} for _ in range(layers)]}
    return llama, dosovik


def tutezen_config(size: str, layers: int, vocab: int = 32768, window: int = 1024):
    """A Tutezen configuration of the width and feed-forward size of ``size``: state-space layers with a dense
    feed-forward alternate with latent-attention layers with routed experts (a quarter of the dense size each, two of
    sixteen chosen, one shared), the middle two layers run twice.  The state-space layers are twice the width inside
    (heads of 64, a state of 128 rows, 8 groups, 4 taps); latent attention caches 224 + 32 elements a token."""
    H, I, nq, _, d = DESIGN_SIZES[size]
    ssm = {"heads": 2 * H // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}
    att = {"heads": 16, "dim": d, "rot_dim": 32, "vdim": d, "q_rank": H // 4, "kv_rank": 224, "scale": (d + 32) ** -0.5,
           "mask": {"size": window}, "rot": {"dims": 32, "base": 500000.0}}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": I // 4}, "shared": {"ff": I // 4}}
    pair = [{"type": "mamba2", "mixer": ssm, "mlp": {"kind": "dense", "ff": I}}, {"type": "latent_attention", "mixer": att, "mlp": moe}]
    cfg = {"architecture": "Tutezen", "vocab": vocab, "width": H, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
           "layers": [pair[i % 2] for i in range(layers)]}
    if layers >= 4:
        cfg["loop"] = {"start": layers // 2 - 1, "stop": layers // 2 + 1, "times": 2}
    return cfg


def bumolix_config(size: str, layers: int, vocab: int = 32768, chunk: int = 1024):
    """A Bumolix configuration of the width, heads and feed-forward size of ``size``: layers whose mixer is attention
    (chunks of ``chunk``, half of a head rotated, positions stretched by 8) beside gated linear attention (width / 256
    heads of 128 key channels and 256 value channels) alternate with selective-scan layers (twice the width inside, 16
    states a channel, 4 taps, step sizes through width / 16); every layer has the dense feed-forward."""
    H, I, nq, nkv, d = DESIGN_SIZES[size]
    left = {"heads": nq, "kv_heads": nkv, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": chunk},
            "rot": {"dims": d // 2, "base": 1000000.0, "scaling": {"factor": 8.0}}}
    right = {"heads": H // 256, "dim": 128, "vdim": 256, "tau": 8.0}
    mlp = {"kind": "dense", "ff": I}
    pair = [{"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.5, "right_scale": 1.25}, "mlp": mlp},
            {"type": "mamba1", "mixer": {"inner": 2 * H, "state": 16, "dt_rank": H // 16, "conv": 4}, "mlp": mlp}]
    return {"architecture": "Bumolix", "vocab": vocab, "width": H, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "layers": [pair[i % 2] for i in range(layers)]}


def kulivik_config(size: str, layers: int, vocab: int = 32768, window: int = 1024):
    """A Kulivik configuration of the width, heads and feed-forward size of ``size``, its three kinds of layer in turn:
    rotated attention inside a window of ``window`` that keeps 8 tokens (capped scores, value mixing) with the dense
    clamped feed-forward; attention with a bias by distance and a query temperature beside linear attention with constant
    decays (width / 128 heads of 128 key and 128 value channels) with routed experts (a quarter of the dense size each,
    two of sixteen chosen); attention behind a convolution of 4 taps with a learned sink and a gate per head, with routed
    experts."""
    H, I, nq, nkv, d = DESIGN_SIZES[size]
    sizes = {"heads": nq, "kv_heads": nkv, "dim": d, "vdim": d, "scale": d ** -0.5}
    gh = H // 128
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": I // 4}}
    kinds = [
        {"type": "attention_2", "mixer": dict(sizes, mask={"size": window, "keep_first": 8}, rot={"dims": d, "base": 500000.0},
                                              softcap=50.0, v_mix=True), "mlp": {"kind": "dense", "ff": I, "limit": 7.0}},
        {"type": "parallel", "mixer": {"left": dict(sizes, q_temp={"coef": 0.25, "every": 128}), "left_scale": 0.7, "right_scale": 0.4,
                                       "right": {"heads": gh, "dim": 128, "vdim": 128,
                                                 "decay": [1.0 - 0.5 ** (1 + 8 * i / gh) for i in range(gh)]}}, "mlp": moe},
        {"type": "attention", "mixer": dict(sizes, conv=4, v_mix=True), "mlp": moe},
    ]
    return {"architecture": "Kulivik", "vocab": vocab, "width": H, "norm": {"eps": 1e-5}, "logit_scale": 1.5, "logit_softcap": 40.0,
            "layers": [kinds[i % 3] for i in range(layers)]}


def design_comparison(args, other: str = "dosovik") -> int:
    """Prefill (one prompt of 2,048 tokens) and decode (8 requests, 2,048 tokens cached each, captured graphs)
    through the step function for both designs at each size; then single kernels.  Timing: CUDA events, the median
    of five regions after three warm-up runs; weights and activations of a step exceed the L2 at every size."""
    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine import StepEntry
    from atoma_infer_b200.engine.runtime import load_model, make_runtime

    hbm, tflops, kind = peaks()
    g = torch.Generator().manual_seed(5)
    layers, batch, ctx_len, prefill = args.layers if args.layers != MODEL["num_hidden_layers"] else 8, args.batch, 2048, PREFILL_TOKENS

    def median_ms(fn, n=5):
        out = []
        for i in range(3 + n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= 3:
                out.append(a.elapsed_time(b))
        return statistics.median(out)

    rows = []
    for size in DESIGN_SIZES:
        pairs = design_configs(size, layers)
        names = ("llama", other)
        if other == "tutezen":  # two layers fewer: the middle two run twice, so a step runs as many layers as Llama's
            pairs = (pairs[0], tutezen_config(size, max(layers - 2, 2)))
        if other == "bumolix":  # beside Llama (equal sizes) and Tutezen (the other design with recurrent layers)
            names = ("llama", "tutezen", other)
            pairs = (pairs[0], tutezen_config(size, max(layers - 2, 2)), bumolix_config(size, layers))
        if other == "kulivik":  # beside Llama (equal sizes) and Bumolix (the closest design: two mixers side by side)
            names = ("llama", "bumolix", other)
            pairs = (pairs[0], bumolix_config(size, layers), kulivik_config(size, layers))
        for name, cfg in zip(names, pairs):
            with tempfile.TemporaryDirectory() as d:
                with open(os.path.join(d, "config.json"), "w") as f:
                    json.dump(cfg, f)
                pages = (batch + 1) * (-(-(ctx_len + 512) // PAGE)) + 64
                lm = load_model(d, dtype="bfloat16", page_size=PAGE, num_pages=pages, max_seqs=batch + 1, cuda_graphs=True,
                                random_weights_seed=1, max_batched_tokens=prefill)
            vocab = lm.model.spec.vocab_size
            toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()  # noqa: E731
            before = lm.rt.ops.launches
            nid = [0]

            def one_prefill():
                nid[0] += 1
                lm.step.run([StepEntry(1000 + nid[0], toks(prefill), [prefill - 1])])
                lm.step.finish(1000 + nid[0])
            pre_ms = median_ms(one_prefill)
            for r in range(batch):
                lm.step.run([StepEntry(r, toks(ctx_len), [])])
            cur = [toks(1) for _ in range(batch)]
            steps = 16

            def decode_steps():
                for _ in range(steps):
                    lm.step.run([StepEntry(r, cur[r], [0]) for r in range(batch)])
            dec_ms = median_ms(decode_steps) / steps
            lm.rt.ops.check_status()
            weights = sum(w.numel() * w.element_size() for r in lm.model.runs for w in lm.model.blocks[r.layer].streamed_weights())
            weights += lm.model.head.weight.numel() * 2
            for r in lm.model.runs:  # routed experts: a step streams what its tokens choose, at most every expert
                ff = getattr(lm.model.blocks[r.layer], "feed_forward", None)
                if hasattr(ff, "w_gate_up") and ff.w_gate_up.dim() == 3:
                    per = (ff.w_gate_up[0].numel() + ff.w_down[0].numel()) * 2
                    weights += per * min(ff.experts, batch * ff.top)
            row = {"size": size, "design": name, "layers": layers, "prefill_tokens": prefill, "prefill_ms": round(pre_ms, 3),
                   "prefill_tok_s": round(prefill / pre_ms * 1e3), "decode_batch": batch, "context": ctx_len,
                   "decode_ms_per_step": round(dec_ms, 4), "decode_tok_s": round(batch / dec_ms * 1e3),
                   "decode_weight_bytes_over_copy_bandwidth": round(weights / (dec_ms * 1e-3) / (hbm * 1e9), 3),
                   "launches": lm.rt.ops.launches - before}
            rows.append(row)
            print(json.dumps(row), flush=True)
            del lm
            torch.cuda.empty_cache()
    kernels = {"tutezen": tutezen_kernels, "bumolix": bumolix_kernels, "kulivik": kulivik_kernels}.get(other, design_kernels)
    kernels(make_runtime("bfloat16", "cuda:0"), hbm, median_ms)
    return 0


def design_kernels(rt, hbm, median_ms) -> None:
    """The Dosovik layers' own kernels beside Llama's like kernels, alone, at width 2048 / 32 heads of 64 / 8 key heads /
    feed-forward 8192: microseconds a call and the fraction of the copy bandwidth that the bytes each must move give.
    Rows of 16,384 tokens (every kernel's inputs and outputs together exceed the L2) and of 8 tokens (a decode step:
    the time of a launch inside a captured graph).  Each figure: 16 calls captured in one CUDA graph, CUDA events
    around three replays, after three warm-up calls."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import kernel_utils as K

    ops, dev = rt.ops, rt.device
    H, I, nq, nkv, d, taps = 2048, 8192, 32, 8, 64, 4
    bf = torch.bfloat16
    print(f"kernels alone (copy bandwidth {hbm:.0f} GB/s): name, rows, us, bytes moved / time / copy bandwidth")
    def graph_us(fn, n=16):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(n):
                fn()
        gr.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(3):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (3 * n) * 1e3

    for T in (16384, 8):
        entries = [(0, T)] if T > 64 else [(100 + i, 1) for i in range(T)]
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 0)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        resid, delta = torch.randn(T, H, device=dev), torch.randn(T, H, device=dev).to(bf)
        w = torch.ones(H, device=dev)
        cw, state = torch.randn(taps, H, device=dev), torch.zeros(max(len(entries), 1), taps - 1, H, device=dev)
        out = torch.empty(T, H, device=dev, dtype=bf)
        qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev).to(bf)
        cache = torch.zeros(num_pages, 2, nkv, PAGE, d, device=dev, dtype=bf)
        q_out = torch.empty(T, nq * d, device=dev, dtype=bf)
        bias, qn, kn = (torch.ones(n, device=dev, dtype=bf) for n in ((nq + 2 * nkv) * d, nq * d, nkv * d))
        inv_freq = torch.ones(d // 2, device=dev)
        v_first, lam = torch.randn(T, nkv * d, device=dev).to(bf), torch.tensor([0.3], device=dev)
        z, gu = torch.randn(T, I, device=dev).to(bf), torch.randn(T, 2 * I, device=dev).to(bf)
        act, coef = torch.empty(T, I, device=dev, dtype=bf), torch.tensor([0.5, 0.2, 0.1, 0.0], device=dev)
        cases = [
            ("dosovik: short convolution", lambda: ops.short_conv(resid, cw, state, ctx, out), T * H * (4 + 2)),
            ("dosovik: norm after the sum (+ state rows)", lambda: ops.scaled_add_rmsnorm(resid, delta, 1.0, w, 1e-5, ctx, keep=(state, taps)), T * H * (4 + 2 + 4)),
            ("llama:   add + RMSNorm", lambda: ops.add_rmsnorm(resid, delta, w, 1e-5, out, ctx.meta, T), T * H * (4 + 2 + 4 + 2)),
            ("dosovik: attention rows (bias, norms, rotation, mix, pages)",
             lambda: ops.qkv_prepare(qkv, ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=d, dp=d, page_size=PAGE, num_pages=num_pages,
                                     store_kv=True, bias=bias, q_norm=qn, k_norm=kn, eps=1e-5, inv_freq=inv_freq, rot=d // 2,
                                     v_first=v_first, v_lambda=lam), T * ((nq + 2 * nkv) * d * 2 * 2 + nkv * d * 2)),
            ("llama:   rotation + pages", lambda: ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, 0, inv_freq, cache, num_pages,
                                                                    T, nq, nkv, d, d, PAGE, True), T * (nq + 2 * nkv) * d * 2 * 2),
            ("dosovik: polynomial activation", lambda: ops.polynorm(z, coef, 1e-5, act, ctx.meta), T * I * 2 * 2),
            ("llama:   SiLU * up", lambda: ops.silu_mul(gu, act, ctx.meta, T, I), T * I * 2 * 3),
        ]
        if T <= 64:
            h2 = torch.empty(T, H, device=dev, dtype=bf)
            cases.insert(2, ("dosovik: norm after the sum + next input (decode)",
                             lambda: ops.scaled_add_rmsnorm(resid, delta, 1.0, w, 1e-5, ctx, keep=(state, taps), conv=(cw, state, h2)),
                             T * H * (4 + 2 + 4 + 2)))
        for name, fn, nbytes in cases:
            us = graph_us(fn)
            print(f"  {name:62s} {T:5d} rows {us:8.1f} us  {nbytes / (us * 1e-6) / (hbm * 1e9):5.2f}")
        # attention: a prompt of T tokens (or T decode tokens over 2,048 cached ones), plain and with chunk mask + sink
        entries = [(0, T)] if T > 64 else [(2047, 1)] * T
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 1)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        cache = torch.randn(num_pages, 2, nkv, PAGE, d, device=dev).to(bf)
        q, o = torch.randn(T, nq * d, device=dev).to(bf), torch.empty(T, nq * d, device=dev, dtype=bf)
        for name, kw in (("llama:   attention", {}), ("dosovik: attention, chunks of 1024 + sink", {"chunk": 1024, "sink": True}),
                         ("dosovik: attention, sink alone", {"sink": True})):
            us = graph_us(lambda: ops.attention(q, nq * d, cache, ctx, 0, o, nq, nkv, d, PAGE, num_pages, 0, 0.125, **kw), n=4)
            print(f"  {name:62s} {T:5d} rows {us:8.1f} us")
    ops.check_status()


def _graph_us(fn, n=16):
    """Microseconds a call: n calls captured in one CUDA graph, CUDA events around three replays, after three warm-up calls."""
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        for _ in range(n):
            fn()
    gr.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(3):
        gr.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (3 * n) * 1e3


def tutezen_kernels(rt, hbm, median_ms) -> None:
    """The Tutezen layers' own kernels beside the framework's like kernels, alone, at width 2048 (the sizes of
    ``tutezen_config("w2048-h64", ...)``): microseconds a call and, for kernels that move bytes, the fraction of the copy
    bandwidth that the bytes each must move give; for the recurrence and the experts' products, which compute, the rate
    of their arithmetic.  Rows of 16,384 tokens and of 8 tokens (a decode step: the time of a launch inside a graph)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import kernel_utils as K
    from atoma_infer_b200.parts.base import PendingSum

    ops, dev, bf = rt.ops, rt.device, torch.bfloat16
    H, I, taps = 2048, 8192, 4
    heads, P, N, G = 64, 64, 128, 8
    inner, C = heads * P, heads * P + 2 * G * N
    lh, rank, rdim, D = 16, 224, 32, 256
    E, top, F = 16, 2, 2048
    print(f"kernels alone (copy bandwidth {hbm:.0f} GB/s): name, rows, us, bytes moved / time / copy bandwidth, or the rate")
    for T in (16384, 8):
        entries = [(0, T)] if T > 64 else [(100 + i, 1) for i in range(T)]
        S = len(entries)
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 0)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        rnd = lambda *shape: torch.randn(*shape, device=dev)  # noqa: E731
        resid, a, b, w = rnd(T, H), rnd(T, H).to(bf), rnd(T, H).to(bf), torch.ones(H, device=dev)
        out = torch.empty(T, H, device=dev, dtype=bf)
        proj = (rnd(T, 2 * inner + 2 * G * N + heads) * 0.5).to(bf)
        cw, cb, ring = rnd(taps, C), rnd(C), torch.zeros(S, taps - 1, C, device=dev)
        xbc = torch.empty(T, C, device=dev, dtype=bf)
        mats = torch.zeros(S, heads, N, P, device=dev)
        y = torch.empty(T, inner, device=dev)
        hv = torch.ones(heads, device=dev)
        g_out, nw = torch.empty(T, inner, device=dev, dtype=bf), torch.ones(inner, device=dev)
        gu, act = rnd(T, 2 * I).to(bf), torch.empty(T, I, device=dev, dtype=bf)
        z_up = gu[:, :I].contiguous()
        qkv = rnd(T, (32 + 16) * 64).to(bf)
        cache_l = torch.zeros(num_pages, 2, 8, PAGE, 64, device=dev, dtype=bf)
        inv_freq = torch.ones(32, device=dev)
        q_rot, q_abs, dkv = rnd(T, lh, 64 + rdim).to(bf), rnd(T, lh, rank).to(bf), rnd(T, rank + rdim).to(bf)
        cache_t = torch.zeros(num_pages, 2, 1, PAGE, D, device=dev, dtype=bf)
        q_full = torch.empty(T, lh * D, device=dev, dtype=bf)
        nrm, fr = torch.ones(rank, device=dev), torch.ones(rdim // 2, device=dev)
        x = rnd(T, H).to(bf)
        wr = rnd(E, H) * 0.1
        ids, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
        wgu, wdn = (rnd(E, 2 * F, H) * 0.02).to(bf), (rnd(E, H, F) * 0.02).to(bf)
        dense_gu, dense_dn = (rnd(2 * F * top, H) * 0.02).to(bf), (rnd(H, F * top) * 0.02).to(bf)
        moe_out = torch.empty(T, H, device=dev, dtype=bf)
        ops.moe_route(x, wr, ids, wts, ctx.meta)
        scan_flops = 6.0 * T * heads * N * P * (2 if T >= 128 else 1)  # (chunks of time run twice)
        ff_flops = 6.0 * T * top * H * F
        cases = [
            ("tutezen: pending sum of two + RMSNorm", lambda: ops.sum_rmsnorm(resid, PendingSum((a, b), 0.5), w, 1e-5, out, ctx.meta, T),
             T * H * (4 + 2 + 2 + 4 + 2), None),
            ("llama:   add + RMSNorm", lambda: ops.add_rmsnorm(resid, a, w, 1e-5, out, ctx.meta, T), T * H * (4 + 2 + 4 + 2), None),
            ("tutezen: convolution + bias + SiLU (+ ring)", lambda: (ops.causal_conv_act(proj[:, inner:inner + C], cw, cb, ring, ctx, xbc) or
                                                                   ops.causal_conv_save(proj[:, inner:inner + C], ring, ctx, taps)),
             T * C * (2 + 2), None),
            ("dosovik: short convolution", lambda: ops.short_conv(resid, cw[:, :H].contiguous(), ring[:, :, :H].contiguous(), ctx, out),
             T * H * (4 + 2), None),
            ("tutezen: recurrence (float32 FMA)", lambda: ops.ssm_scan(xbc, proj[:, inner + C:], hv, hv * 0, hv, mats, ctx, y, heads=heads,
                                                                       head_dim=P, nstate=N, groups=G),
             T * (C * 2 + inner * 4) + 2 * S * heads * N * P * 4, scan_flops),
            ("tutezen: gate, norm in 8 parts", lambda: ops.gated_group_norm(y, proj[:, :inner], nw, 8, 1e-5, g_out, ctx.meta),
             T * inner * (4 + 2 + 2), None),
            ("llama:   SiLU * up", lambda: ops.silu_mul(gu, act, ctx.meta, T, I), T * I * 2 * 3, None),
            ("tutezen: GELU", lambda: ops.activation(z_up, act, "gelu_tanh", ctx.meta), T * I * 2 * 2, None),
            ("tutezen: latent rows (norm, rotation, pages, queries)",
             lambda: ops.latent_rows(q_rot[:, :, 64:], q_abs, dkv, nrm, 1e-5, ctx, cache_t, 0, q_full, heads=lh, kv_rank=rank, rot_dim=rdim,
                                     padded=D, page_size=PAGE, num_pages=num_pages, store=True, inv_freq=fr, rotary_dims=rdim),
             T * (lh * (rank + rdim) * 2 + (rank + rdim) * 2 + lh * D * 2 + 2 * D * 2), None),
            ("llama:   rotation + pages", lambda: ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, 0, inv_freq, cache_l, num_pages,
                                                                    T, 32, 8, 64, 64, PAGE, True), T * 48 * 64 * 2 * 2, None),
            ("tutezen: linear per head, 64 -> 224 (queries)", lambda: ops.head_linear(q_rot[:, :, :64], wgu[0, :lh * rank, :64].reshape(lh, rank, 64).contiguous(),
                                                                                  q_abs, ctx.meta), T * lh * (64 + rank) * 2, 2.0 * T * lh * 64 * rank),
            ("tutezen: router (float32)", lambda: ops.moe_route(x, wr, ids, wts, ctx.meta), T * H * 2, None),
            ("tutezen: experts (sort, two grouped products, weighted sum)",
             lambda: ops.moe_experts(x, ids, wts, wgu, wdn, None, moe_out, ctx.meta),
             min(E, T * top) * 3 * F * H * 2 + T * H * 4, ff_flops),
            ("llama:   gate/up + SiLU * up, down, at the experts' sizes (dense)",
             lambda: ops.linear(ops.linear(x, dense_gu, silu_mul=True, meta=ctx.meta), dense_dn, meta=ctx.meta),
             3 * top * F * H * 2 + T * H * 4, ff_flops),
        ]
        for name, fn, nbytes, flops in cases:
            us = _graph_us(fn, n=16 if T <= 64 else 2)
            rate = f"  {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s" if flops else ""
            print(f"  {name:68s} {T:5d} rows {us:9.1f} us  {nbytes / (us * 1e-6) / (hbm * 1e9):5.2f}{rate}")
        # attention: a prompt of T tokens (or T decode tokens over 2,048 cached ones)
        entries = [(0, T)] if T > 64 else [(2047, 1)] * T
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 1)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        sinks = torch.zeros(lh, device=dev)
        for name, nq, nkv, d, kw in (("llama:   attention, 32 x 64 over 8 x 64", 32, 8, 64, {}),
                                     ("llama:   attention, window 1024", 32, 8, 64, {"window": 1024}),
                                     ("tutezen: latent attention, 16 x 256 over 1 x 256, window 1024 + sinks", lh, 1, D, {"window": 1024, "sink": sinks})):
            cache = torch.randn(num_pages, 2, nkv, PAGE, d, device=dev).to(bf)
            q, o = torch.randn(T, nq * d, device=dev).to(bf), torch.empty(T, nq * d, device=dev, dtype=bf)
            window = kw.pop("window", 0)
            us = _graph_us(lambda: ops.attention(q, nq * d, cache, ctx, 0, o, nq, nkv, d, PAGE, num_pages, window, 0.125, **kw), n=4)
            keys = min(window, T) if window else T
            flops = 4.0 * T * nq * d * (keys / (1 if window and T > window else 2) if T > 64 else min(window or 2048, 2048))
            print(f"  {name:68s} {T:5d} rows {us:9.1f} us         {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s")
    ops.check_status()


def bumolix_kernels(rt, hbm, median_ms) -> None:
    """The Bumolix layers' own kernels beside the framework's like kernels, alone, at width 2048 (the sizes of
    ``bumolix_config("w2048-h64", ...)``): microseconds a call and the fraction of the copy bandwidth that the bytes each
    must move give; for the recurrences, which compute in float32, the rate of their arithmetic too.  Rows of 16,384
    tokens and of 8 tokens (a decode step: the time of a launch inside a graph)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import kernel_utils as K
    from atoma_infer_b200.parts.base import PendingSum

    ops, dev, bf = rt.ops, rt.device, torch.bfloat16
    H, I, taps = 2048, 8192, 4
    nq, nkv, d = 32, 8, 64
    gh, gN, gP = 8, 128, 256          # gated linear attention: heads, key channels, value channels
    inner, N, dt_rank = 4096, 16, 128  # selective scan
    th, tP, tN, tG = 64, 64, 128, 8    # Tutezen's state-space layer at this width
    t_inner, tC = th * tP, th * tP + 2 * tG * tN
    print(f"kernels alone (copy bandwidth {hbm:.0f} GB/s): name, rows, us, bytes moved / time / copy bandwidth, or the rate")
    for T in (16384, 8):
        entries = [(0, T)] if T > 64 else [(100 + i, 1) for i in range(T)]
        S = len(entries)
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 0)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        rnd = lambda *shape: torch.randn(*shape, device=dev)  # noqa: E731
        resid, w = rnd(T, H), torch.ones(H, device=dev)
        a, b, c = (rnd(T, H).to(bf) for _ in range(3))
        out, out2 = (torch.empty(T, H, device=dev, dtype=bf) for _ in range(2))
        # attention rows
        qkv = rnd(T, (nq + 2 * nkv) * d).to(bf)
        cache = torch.zeros(num_pages, 2, nkv, PAGE, d, device=dev, dtype=bf)
        q_out = torch.empty(T, nq * d, device=dev, dtype=bf)
        bias, inv_freq = torch.ones((nq + 2 * nkv) * d, device=dev, dtype=bf), torch.ones(d // 4, device=dev)
        att, gate = rnd(T, nq, d).to(bf), rnd(T, nq, d).to(bf)
        # gated linear attention
        g_proj = (rnd(T, 2 * gh * gN + 2 * gh * gP) * 0.5).to(bf)
        g_z, g_bias = rnd(T, gh * gN), torch.zeros(gh * gN, device=dev)
        g_state, g_o = torch.zeros(S, gh, gN, gP, device=dev), torch.empty(T, gh * gP, device=dev)
        g_y, g_w = torch.empty(T, gh * gP, device=dev, dtype=bf), torch.ones(gP, device=dev)
        # selective scan
        s_proj = (rnd(T, 2 * inner) * 0.5).to(bf)
        s_cw, s_cb, s_ring = rnd(taps, inner), rnd(inner), torch.zeros(S, taps - 1, inner, device=dev)
        s_u = torch.empty(T, inner, device=dev, dtype=bf)
        s_low, s_dt = (rnd(T, dt_rank + 2 * N) * 0.5).to(bf), rnd(T, inner)
        s_dtb, s_alog, s_d = torch.zeros(inner, device=dev), torch.zeros(inner, N, device=dev), torch.ones(inner, device=dev)
        s_state, s_y = torch.zeros(S, inner, N, device=dev), torch.empty(T, inner, device=dev, dtype=bf)
        # Tutezen's state-space layer
        t_proj = (rnd(T, 2 * t_inner + 2 * tG * tN + th) * 0.5).to(bf)
        t_cw, t_cb, t_ring = rnd(taps, tC), rnd(tC), torch.zeros(S, taps - 1, tC, device=dev)
        t_xbc = torch.empty(T, tC, device=dev, dtype=bf)
        t_state, t_y, hv = torch.zeros(S, th, tN, tP, device=dev), torch.empty(T, t_inner, device=dev), torch.ones(th, device=dev)
        t_out, t_nw = torch.empty(T, t_inner, device=dev, dtype=bf), torch.ones(t_inner, device=dev)
        ops.causal_conv_act(t_proj[:, t_inner:t_inner + tC], t_cw, t_cb, t_ring, ctx, t_xbc)
        # feed-forward activations
        z_up, act = rnd(T, I).to(bf), torch.empty(T, I, device=dev, dtype=bf)
        gu = rnd(T, 2 * I).to(bf)
        twice = 2 if T >= 128 else 1  # (chunks of time run twice)
        cases = [
            ("bumolix: weighted pending sum of three + two RMSNorms",
             lambda: ops.sum_rmsnorm(resid, PendingSum((a, b, c), 0.5, factors=(0.5, 1.25, 1.0)), w, 1e-5, out, ctx.meta, T, second=(w, 1e-5, out2)),
             T * H * (4 + 3 * 2 + 4 + 2 * 2), None),
            ("tutezen: pending sum of two + RMSNorm", lambda: ops.sum_rmsnorm(resid, PendingSum((a, b), 0.5), w, 1e-5, out, ctx.meta, T),
             T * H * (4 + 2 + 2 + 4 + 2), None),
            ("llama:   add + RMSNorm", lambda: ops.add_rmsnorm(resid, a, w, 1e-5, out, ctx.meta, T), T * H * (4 + 2 + 4 + 2), None),
            ("bumolix: attention rows (bias, half rotation, norm per head, pages)",
             lambda: ops.qkv_prepare(qkv, ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=d, dp=d, page_size=PAGE, num_pages=num_pages,
                                     store_kv=True, bias=bias, eps=1e-5, inv_freq=inv_freq, rot=d // 2, head_norm=True),
             T * (nq + 2 * nkv) * d * 2 * 2, None),
            ("llama:   rotation + pages", lambda: ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, 0, torch.ones(d // 2, device=dev),
                                                                    cache, num_pages, T, nq, nkv, d, d, PAGE, True),
             T * (nq + 2 * nkv) * d * 2 * 2, None),
            ("bumolix: output gate (sigmoid, in place)", lambda: ops.sigmoid_gate(att, gate, ctx.meta), T * nq * d * 2 * 3, None),
            ("bumolix: gated linear attention, 8 x 128 x 256 (float32 FMA)",
             lambda: ops.gla_scan(g_proj[:, :gh * gN], g_proj[:, gh * gN:2 * gh * gN], g_proj[:, 2 * gh * gN:2 * gh * gN + gh * gP], g_z, g_bias,
                                  8.0, gN ** -0.5, g_state, ctx, g_o, heads=gh, dim=gN, vdim=gP),
             T * (2 * gh * gN * 2 + gh * gP * 2 + gh * gN * 4 + gh * gP * 4) + 2 * S * gh * gN * gP * 4, 6.0 * T * gh * gN * gP * twice),
            ("tutezen: recurrence, 64 x 128 x 64 (float32 FMA)",
             lambda: ops.ssm_scan(t_xbc, t_proj[:, t_inner + tC:], hv, hv * 0, hv, t_state, ctx, t_y, heads=th, head_dim=tP, nstate=tN, groups=tG),
             T * (tC * 2 + t_inner * 4) + 2 * S * th * tN * tP * 4, 6.0 * T * th * tN * tP * twice),
            ("bumolix: norm per head, shared weight, SiLU gate", lambda: ops.head_norm_gate(g_o, g_proj[:, 2 * gh * gN + gh * gP:], g_w, 1e-5, g_y, ctx.meta, gh),
             T * gh * gP * (4 + 2 + 2), None),
            ("tutezen: gate, norm in 8 parts", lambda: ops.gated_group_norm(t_y, t_proj[:, :t_inner], t_nw, 8, 1e-5, t_out, ctx.meta),
             T * t_inner * (4 + 2 + 2), None),
            ("bumolix: convolution + bias + SiLU (+ ring), 4096 channels",
             lambda: (ops.causal_conv_act(s_proj[:, :inner], s_cw, s_cb, s_ring, ctx, s_u) or ops.causal_conv_save(s_proj[:, :inner], s_ring, ctx, taps)),
             T * inner * (2 + 2), None),
            ("bumolix: selective scan, 4096 x 16, + skip, SiLU gate (float32 FMA)",
             lambda: ops.selective_scan(s_u, s_dt, s_dtb, s_low[:, dt_rank:], s_proj[:, inner:], s_alog, s_d, s_state, ctx, s_y, inner=inner, nstate=N),
             T * (inner * (2 + 4 + 2 + 2) + 2 * N * 2) + 2 * S * inner * N * 4, 7.0 * T * inner * N * twice),
            ("bumolix: square of relu", lambda: ops.activation(z_up, act, "relu2", ctx.meta), T * I * 2 * 2, None),
            ("llama:   SiLU * up", lambda: ops.silu_mul(gu, act, ctx.meta, T, I), T * I * 2 * 3, None),
        ]
        for name, fn, nbytes, flops in cases:
            us = _graph_us(fn, n=16 if T <= 64 else 2)
            rate = f"  {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s" if flops else ""
            print(f"  {name:72s} {T:5d} rows {us:9.1f} us  {nbytes / (us * 1e-6) / (hbm * 1e9):5.2f}{rate}")
        # attention: a prompt of T tokens (or T decode tokens over 2,048 cached ones)
        entries = [(0, T)] if T > 64 else [(2047, 1)] * T
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 1)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        cache = torch.randn(num_pages, 2, nkv, PAGE, d, device=dev).to(bf)
        q, o = torch.randn(T, nq * d, device=dev).to(bf), torch.empty(T, nq * d, device=dev, dtype=bf)
        for name, window, kw in (("llama:   attention, 32 x 64 over 8 x 64", 0, {}), ("llama:   attention, window 1024", 1024, {}),
                                 ("bumolix: attention, chunks of 1024 + sink", 0, {"chunk": 1024, "sink": True})):
            us = _graph_us(lambda: ops.attention(q, nq * d, cache, ctx, 0, o, nq, nkv, d, PAGE, num_pages, window, 0.125, **kw), n=4)
            chunk = kw.get("chunk", 0)
            keys = (min(chunk, T) / 2 if chunk else (min(window, T) if window and T > window else T / 2)) if T > 64 else min(window or chunk or 2048, 2048)
            flops = 4.0 * T * nq * d * keys
            print(f"  {name:72s} {T:5d} rows {us:9.1f} us         {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s")
    ops.check_status()


def kulivik_kernels(rt, hbm, median_ms) -> None:
    """The Kulivik layers' own kernels beside the framework's like kernels, alone, at width 2048 (the sizes of
    ``kulivik_config("w2048-h64", ...)``): microseconds a call and the fraction of the copy bandwidth that the bytes each
    must move give; for the recurrence and the attention kernels the rate of their arithmetic.  Rows of 16,384 tokens and
    of 8 tokens (a decode step: the time of a launch inside a graph)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import kernel_utils as K
    from atoma_infer_b200.parts.base import PendingSum

    ops, dev, bf = rt.ops, rt.device, torch.bfloat16
    H, I, taps = 2048, 8192, 4
    nq, nkv, d = 32, 8, 64
    kh, kN, kP = 16, 128, 128          # linear attention with constant decays: heads, key channels, value channels
    gh, gN, gP = 8, 128, 256           # Bumolix's gated linear attention at this width
    E, top = 16, 2
    print(f"kernels alone (copy bandwidth {hbm:.0f} GB/s): name, rows, us, bytes moved / time / copy bandwidth, or the rate")
    for T in (16384, 8):
        entries = [(0, T)] if T > 64 else [(100 + i, 1) for i in range(T)]
        S = len(entries)
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 0)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        rnd = lambda *shape: torch.randn(*shape, device=dev)  # noqa: E731
        resid, w = rnd(T, H), torch.ones(H, device=dev)
        a, b, c = (rnd(T, H).to(bf) for _ in range(3))
        out, out2 = (torch.empty(T, H, device=dev, dtype=bf) for _ in range(2))
        mu, kept, last = torch.rand(H, device=dev), torch.zeros(S, H, device=dev), torch.empty(S, H, device=dev)
        gate32, gbias = rnd(T, H), torch.zeros(H, device=dev)
        qkv = rnd(T, (nq + 2 * nkv) * d).to(bf)
        cache = torch.zeros(num_pages, 2, nkv, PAGE, d, device=dev, dtype=bf)
        q_out = torch.empty(T, nq * d, device=dev, dtype=bf)
        bias, inv_freq = torch.ones((nq + 2 * nkv) * d, device=dev, dtype=bf), torch.ones(d // 2, device=dev)
        hw = torch.ones(d, device=dev, dtype=bf)
        att, gate, hgate = rnd(T, nq, d).to(bf), rnd(T, nq, d).to(bf), rnd(T, nq).to(bf)
        k_proj = (rnd(T, 2 * kh * kN + 2 * kh * kP) * 0.5).to(bf)
        k_state, k_o = torch.zeros(S, kh, kN, kP, device=dev), torch.empty(T, kh * kP, device=dev)
        k_dec, k_y, k_w = torch.full((kh,), 0.97, device=dev), torch.empty(T, kh * kP, device=dev, dtype=bf), torch.ones(kh * kP, device=dev)
        g_proj = (rnd(T, 2 * gh * gN + 2 * gh * gP) * 0.5).to(bf)
        g_z, g_bias = rnd(T, gh * gN), torch.zeros(gh * gN, device=dev)
        g_state, g_o = torch.zeros(S, gh, gN, gP, device=dev), torch.empty(T, gh * gP, device=dev)
        g_y, g_w = torch.empty(T, gh * gP, device=dev, dtype=bf), torch.ones(gP, device=dev)
        c_w, c_ring = rnd(taps, (nq + 2 * nkv) * d), torch.zeros(S, taps - 1, (nq + 2 * nkv) * d, device=dev)
        c_out = torch.empty(T, (nq + 2 * nkv) * d, device=dev, dtype=bf)
        gu, act = rnd(T, 2 * I).to(bf), torch.empty(T, I, device=dev, dtype=bf)
        x, wr, rb = rnd(T, H).to(bf), rnd(E, H), rnd(E)
        ids, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, device=dev)
        twice = 2 if T >= 128 else 1  # (chunks of time run twice)
        rows_b = T * (nq + 2 * nkv) * d * 2 * 2
        cases = [
            ("kulivik: norm + row shifted toward the token before", lambda: ops.norm_shift(resid, w, 1e-6, ctx, shift=mu, state=kept, h=out, hs=out2, last=last),
             T * H * (4 + 2 + 2), None),
            ("llama:   add + RMSNorm", lambda: ops.add_rmsnorm(resid, a, w, 1e-5, out, ctx.meta, T), T * H * (4 + 2 + 4 + 2), None),
            ("kulivik: gate, norm of two weighted terms, sum into the stream + next norm",
             lambda: ops.gated_norm_add(resid, PendingSum((a, b), 1.0, factors=(0.7, 0.4)), gate32, gbias, w, 1e-6, ctx, next_norm=(w, 1e-6, out), keep=(last, kept)),
             T * H * (2 * 2 + 4 + 4 + 4 + 2), None),
            ("bumolix: weighted pending sum of three + two RMSNorms",
             lambda: ops.sum_rmsnorm(resid, PendingSum((a, b, c), 0.5, factors=(0.5, 1.25, 1.0)), w, 1e-5, out, ctx.meta, T, second=(w, 1e-5, out2)),
             T * H * (4 + 3 * 2 + 4 + 2 * 2), None),
            ("kulivik: attention rows (bias, weighted norm per head, interleaved rotation, pages)",
             lambda: ops.qkv_prepare(qkv, ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=d, dp=d, page_size=PAGE, num_pages=num_pages,
                                     store_kv=True, bias=bias, q_norm=hw, k_norm=hw, eps=1e-6, inv_freq=inv_freq, rot=d, head_norm=True, interleaved=True),
             rows_b, None),
            ("kulivik: attention rows (query temperature, pages; no rotation)",
             lambda: ops.qkv_prepare(qkv, ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=d, dp=d, page_size=PAGE, num_pages=num_pages,
                                     store_kv=True, eps=1e-6, q_temp=(0.25, 128)), rows_b, None),
            ("bumolix: attention rows (bias, half rotation, norm per head, pages)",
             lambda: ops.qkv_prepare(qkv, ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=d, dp=d, page_size=PAGE, num_pages=num_pages,
                                     store_kv=True, bias=bias, eps=1e-5, inv_freq=inv_freq[:d // 4], rot=d // 2, head_norm=True), rows_b, None),
            ("llama:   rotation + pages", lambda: ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, 0, inv_freq,
                                                                    cache, num_pages, T, nq, nkv, d, d, PAGE, True), rows_b, None),
            ("kulivik: convolution of 4 taps on q, k, v (+ ring)",
             lambda: (ops.causal_conv_act(qkv, c_w, None, c_ring, ctx, c_out, act="none") or ops.causal_conv_save(qkv, c_ring, ctx, taps)),
             rows_b, None),
            ("kulivik: one gate per head (sigmoid, in place)", lambda: ops.head_gate(att, hgate, ctx.meta), T * nq * d * 2 * 2, None),
            ("bumolix: output gate (sigmoid, in place)", lambda: ops.sigmoid_gate(att, gate, ctx.meta), T * nq * d * 2 * 3, None),
            ("kulivik: linear attention, constant decays, SiLU, 16 x 128 x 128 (float32 FMA)",
             lambda: ops.gla_scan(k_proj[:, :kh * kN], k_proj[:, kh * kN:2 * kh * kN], k_proj[:, 2 * kh * kN:2 * kh * kN + kh * kP], None, None,
                                  1.0, 1.0, k_state, ctx, k_o, heads=kh, dim=kN, vdim=kP, head_decay=k_dec, silu=True),
             T * (2 * kh * kN * 2 + kh * kP * 2 + kh * kP * 4) + 2 * S * kh * kN * kP * 4, 6.0 * T * kh * kN * kP * twice),
            ("bumolix: gated linear attention, 8 x 128 x 256 (float32 FMA)",
             lambda: ops.gla_scan(g_proj[:, :gh * gN], g_proj[:, gh * gN:2 * gh * gN], g_proj[:, 2 * gh * gN:2 * gh * gN + gh * gP], g_z, g_bias,
                                  8.0, gN ** -0.5, g_state, ctx, g_o, heads=gh, dim=gN, vdim=gP),
             T * (2 * gh * gN * 2 + gh * gP * 2 + gh * gN * 4 + gh * gP * 4) + 2 * S * gh * gN * gP * 4, 6.0 * T * gh * gN * gP * twice),
            ("kulivik: norm over the whole row, weight, sigmoid gate", lambda: ops.row_norm_gate(k_o, k_proj[:, 2 * kh * kN + kh * kP:], k_w, 1e-6, k_y, ctx.meta),
             T * kh * kP * (4 + 2 + 2), None),
            ("bumolix: norm per head, shared weight, SiLU gate", lambda: ops.head_norm_gate(g_o, g_proj[:, 2 * gh * gN + gh * gP:], g_w, 1e-5, g_y, ctx.meta, gh),
             T * gh * gP * (4 + 2 + 2), None),
            ("kulivik: clamped gated activation", lambda: ops.clamped_glu(gu, act, 7.0, 1.702, ctx.meta), T * I * 2 * 3, None),
            ("llama:   SiLU * up", lambda: ops.silu_mul(gu, act, ctx.meta, T, I), T * I * 2 * 3, None),
            ("kulivik: router (bias, weights over the chosen)", lambda: ops.moe_route(x, wr, ids, wts, ctx.meta, bias=rb, over_chosen=True), T * H * 2, None),
            ("tutezen: router", lambda: ops.moe_route(x, wr, ids, wts, ctx.meta), T * H * 2, None),
        ]
        for name, fn, nbytes, flops in cases:
            us = _graph_us(fn, n=16 if T <= 64 else 2)
            rate = f"  {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s" if flops else ""
            print(f"  {name:84s} {T:5d} rows {us:9.1f} us  {nbytes / (us * 1e-6) / (hbm * 1e9):5.2f}{rate}")
        # attention: a prompt of T tokens (or T decode tokens over 2,048 cached ones)
        entries = [(0, T)] if T > 64 else [(2047, 1)] * T
        tables, num_pages = K.scrambled_tables([c + n for c, n in entries], PAGE, 1)
        ctx, _ = K.make_context(rt, entries, PAGE, tables)
        cache = torch.randn(num_pages, 2, nkv, PAGE, d, device=dev).to(bf)
        q, o = torch.randn(T, nq * d, device=dev).to(bf), torch.empty(T, nq * d, device=dev, dtype=bf)
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)], device=dev)
        sinks = torch.zeros(nq, device=dev)
        for name, window, kw in (("llama:   attention, 32 x 64 over 8 x 64, all keys", 0, {}), ("llama:   attention, window 1024", 1024, {}),
                                 ("bumolix: attention, chunks of 1024 + sink", 0, {"chunk": 1024, "sink": True}),
                                 ("kulivik: attention, window 1024 that keeps 8, capped scores", 1024, {"keep_first": 8, "softcap": 50.0}),
                                 ("kulivik: attention, window 1024 that keeps 8", 1024, {"keep_first": 8}),
                                 ("kulivik: attention, all keys, bias by distance", 0, {"slopes": slopes}),
                                 ("kulivik: attention, all keys, learned sink", 0, {"sink": sinks})):
            us = _graph_us(lambda: ops.attention(q, nq * d, cache, ctx, 0, o, nq, nkv, d, PAGE, num_pages, window, 0.125, **kw), n=4)
            chunk = kw.get("chunk", 0)
            keys = (min(chunk, T) / 2 if chunk else (min(window, T) if window and T > window else T / 2)) if T > 64 else min(window or chunk or 2048, 2048)
            flops = 4.0 * T * nq * d * keys
            print(f"  {name:84s} {T:5d} rows {us:9.1f} us         {flops / (us * 1e-6) / 1e12:7.1f} TFLOP/s")
    ops.check_status()


def layer_kernel_phases(eng, args, prompt, greedy, cfg) -> int:
    """Decode steps through the persistent layer kernel (csrc/kernels/decode_stack.cu), eagerly, with every block
    writing the global clock after each phase and each barrier of each layer; prints the mean, the slowest and the
    fastest block per slot.  The clock reads themselves cost about 0.3 us a slot."""
    import torch

    lm, ops = eng.lm, eng.lm.rt.ops
    ops.fused_layers = True
    lm.step.cuda_graphs = False
    d, H, L = cfg["head_dim"], cfg["hidden_size"], cfg["num_hidden_layers"]
    ids = [eng.add_request(prompt(), greedy) for _ in range(args.batch)]
    while any(eng.scheduler.num_computed(i) < args.context for i in ids):
        eng.step()
    for _ in range(max(args.warmup, 3)):
        eng.step()
    blocks = ops.decode_stack_blocks(d, args.batch, max(H, cfg["num_attention_heads"] * d))
    if not blocks:
        print("the layer kernel does not take this geometry")
        return 1
    clocks = torch.zeros((blocks, L, 10), dtype=torch.int64, device=lm.rt.device)
    ops.decode_stack_record_clocks(d, clocks)
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    ops.decode_stack_record_clocks(d, None)
    t = clocks.cpu().double()
    begin = torch.cat([t[:, :-1, 9:10], t[:, 1:, :9]], dim=2)  # a slot begins where the one before it ended
    dur = (t[:, 1:, :] - begin) / 1000.0                      # us; layers 1 .. L-1
    names = ["norm scales + q/k/v", "barrier", "attention", "barrier", "output projection", "barrier",
             "norm scales + gate/up", "barrier", "down projection", "barrier"]
    print(f"layer kernel, batch {args.batch}, context {args.context}, {L} layers, {blocks} blocks: us per slot "
          f"(mean over blocks and layers | slowest block | fastest block)")
    for j, name in enumerate(names):
        per_block = dur[:, :, j].mean(1)
        print(f"  {name:24s} {dur[:, :, j].mean().item():6.2f} | {per_block.max().item():6.2f} | {per_block.min().item():6.2f}")
    print(f"  a layer (block 0): {((t[0, -1, 9] - t[0, 0, 9]) / 1000.0 / (L - 1)).item():.2f} us")
    return 0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                    help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="1b", choices=["1b", "3b", "8b"],
                    help="1b: the headline benchmark; 3b / 8b: the larger configurations with their serving workloads")
    ap.add_argument("--context", type=int, default=PROMPT_LEN,
                    help="prompt length of the decode measurements (default 2,048; 8,192 and 32,768 for long contexts)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--layer-kernel-phases", action="store_true",
                    help="instead of the benchmark: decode steps with the persistent layer kernel switched on, and the "
                         "time its blocks spend in every phase and at every barrier of a layer (a table, for profiles/)")
    ap.add_argument("--linears", action="store_true",
                    help="instead of the benchmark: the four linears of a layer (sizes of --model) at 1, 8 and 16 rows on the "
                         "direct and on the streamed few-row kernel, weights cold (a table, for profiles/)")
    ap.add_argument("--designs", action="store_true",
                    help="instead of the benchmark: prefill and decode throughput of the Dosovik design beside Llama at equal "
                         "layer sizes (a JSON line each), then the design's kernels alone beside Llama's like kernels")
    ap.add_argument("--tutezen", action="store_true",
                    help="instead of the benchmark: prefill and decode throughput of the Tutezen design beside Llama at equal "
                         "width and as many layer runs (a JSON line each), then the design's kernels alone beside like kernels")
    ap.add_argument("--kulivik", action="store_true",
                    help="the Kulivik design beside Llama and Bumolix at equal layer sizes through the step function, then its kernels alone")
    ap.add_argument("--bumolix", action="store_true",
                    help="instead of the benchmark: prefill and decode throughput of the Bumolix design beside Llama and Tutezen "
                         "at equal width and as many layer runs (a JSON line each), then the design's kernels alone beside like kernels")
    ap.add_argument("--phase", default="all", choices=["all", "prefill", "decode"],
                    help="measure only one phase (for profiling); the JSON line then lacks the other")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is Rust (candle, cudarc) with no toolchain or vendored crates here, its "
                          "CUTLASS submodule is empty and its kernels reject sm_100 (csrc/src/lib.rs:2216-2231)"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py measures a one-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.linears:
        return few_row_linears(args.model)
    if args.designs:
        return design_comparison(args)
    if args.tutezen:
        return design_comparison(args, other="tutezen")
    if args.bumolix:
        return design_comparison(args, other="bumolix")
    if args.kulivik:
        return design_comparison(args, other="kulivik")
    if args.model != "1b":
        return serving_workload(args.model)

    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine import Engine, StepEntry
    from atoma_infer_b200.sampling import SamplingParams
    from atoma_infer_b200.weights import write_random_model

    hbm_gbs, bf16_tflops, peak_kind = peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    import atexit
    import shutil

    tmp = tempfile.mkdtemp(prefix="bench_model_")
    atexit.register(shutil.rmtree, tmp, ignore_errors=True)  # 2.5 GB of random weights: do not leave them behind
    write_random_model(tmp, cfg, seed=0, std=0.02, device="cuda")
    L, H, I, V = args.layers, cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lin_params = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    weight_bytes = 2 * (lin_params + V * H)  # every weight once; the tied embedding matrix is the head
    kv_bytes_per_token = 2 * L * nkv * d * 2

    max_batch = 64 if not args.skip_points else args.batch
    prompt_len = args.context
    tokens_per_req = prompt_len + 5 * args.steps + args.warmup + 64
    pages = max_batch * (-(-tokens_per_req // PAGE)) + 256
    eng = Engine(tmp, dtype="bfloat16", block_size=PAGE, num_gpu_blocks_override=pages,
                 max_num_sequences=max(max_batch, 8), max_num_batched_tokens=max(PREFILL_TOKENS, max_batch))
    lm, ops = eng.lm, eng.lm.rt.ops
    g = torch.Generator().manual_seed(2)
    greedy = SamplingParams(do_sample=False, max_new_tokens=10 ** 6, ignore_eos_token=True)

    def prompt():
        return torch.randint(0, V, (prompt_len,), generator=g).tolist()

    def event_ms(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    if args.layer_kernel_phases:
        return layer_kernel_phases(eng, args, prompt, greedy, cfg)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    toks = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(3 + 5 if args.phase != "decode" else 0):
        req = 10 ** 6 + i
        ms = event_ms(lambda: lm.step.run([StepEntry(req, toks, [PREFILL_TOKENS - 1])]))
        lm.step.finish(req)
        if i >= 3:
            times.append(ms)
    prefill_ms = statistics.median(times) if times else float("nan")
    prefill_flops = 2 * PREFILL_TOKENS * lin_params + 4 * (PREFILL_TOKENS ** 2 // 2) * d * nq * L + 2 * V * H
    prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12), "peak": f"{peak_kind} bf16 burst"}

    # ------------------------------------------------------------------ decode
    REPEATS = 5

    def decode_run(batch, steps, warmup, through_engine):
        """Prefills ``batch`` requests, warms up, then times ``steps`` decode steps REPEATS times over (the
        context grows from one repeat to the next).  Returns a record of the median repeat."""
        ids = [eng.add_request(prompt(), greedy) for _ in range(batch)]
        while any(eng.scheduler.num_computed(i) < prompt_len for i in ids):
            eng.step()  # prompts in portions under the token budget; the last portion samples
        for _ in range(warmup):
            eng.step()
        runs = []
        for rep in range(REPEATS):
            launches0 = ops.launches
            h2d0, d2h0 = lm.step.h2d_bytes + eng.sampler.h2d_bytes, eng.sampler.d2h_bytes
            ctx0 = lm.manager.num_tokens(ids[0])  # tokens in the cache when the region starts
            if through_engine:
                ms = event_ms(lambda: [eng.step() for _ in range(steps)])
            else:
                # device-timed: the same decode step with the tokens already on the host side
                # (synthetic ids), no read-back between steps
                fake = torch.randint(0, V, (steps, batch), generator=g).tolist()
                out = torch.empty(batch, dtype=torch.int32, device=lm.rt.device)

                def loop():
                    for s in range(steps):
                        logits = lm.step.run([StepEntry(i, [fake[s][k]], [0]) for k, i in enumerate(ids)])
                        ops.sample(logits, None, None, None, None, None, out)
                ms = event_ms(loop)
            ctx_mid = ctx0 + steps / 2
            nbytes = weight_bytes + batch * ctx_mid * kv_bytes_per_token
            runs.append({"ms": ms, "launches": ops.launches - launches0, "ctx_mid": ctx_mid, "bytes": nbytes,
                         "h2d": (lm.step.h2d_bytes + eng.sampler.h2d_bytes - h2d0) / steps,
                         "d2h": (eng.sampler.d2h_bytes - d2h0) / steps})
        for i in ids:
            eng.abort_request(i)
        runs.sort(key=lambda r: r["ms"])
        med = dict(runs[len(runs) // 2])
        med["ms_min"], med["ms_max"] = runs[0]["ms"], runs[-1]["ms"]
        return med

    def roofline_of(run, batch, steps):
        ms_step = run["ms"] / steps
        achieved = run["bytes"] / (ms_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "of": peak_kind, "ms_per_step": ms_step, "ms_per_step_min": run["ms_min"] / steps,
                "ms_per_step_max": run["ms_max"] / steps, "bytes": run["bytes"], "context": run["ctx_mid"],
                "tok_s": batch * steps / run["ms"] * 1e3}

    if args.phase == "prefill":
        print(json.dumps({"impl": "ours", "phase": "prefill", "prefill": prefill}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    run = decode_run(args.batch, args.steps, args.warmup, through_engine=False)
    roofline = roofline_of(run, args.batch, args.steps)
    e2e = None
    if args.phase == "all":
        e2e = decode_run(args.batch, args.steps, args.warmup, through_engine=True)
    points, points_roofline = {}, {f"decode_b{args.batch}": roofline}
    if not args.skip_points and args.phase == "all":
        for b in (1, 64):
            r = roofline_of(decode_run(b, args.steps, args.warmup, through_engine=False), b, args.steps)
            points[f"decode_b{b}"] = r["tok_s"]
            points_roofline[f"decode_b{b}"] = r
    clock_rec = clocks.stop()

    rec = {
        "metric": f"decode tok/s (Llama 3.2 1B, batch {args.batch}, {prompt_len:,}-token prompts)", "value": roofline["tok_s"],
        "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": roofline["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B (random weights N(0,0.02), seed 0)", "layers": L,
            "layers_full": MODEL["num_hidden_layers"], "hidden": H, "heads": nq, "kv_heads": nkv, "head_dim": d,
            "intermediate": I, "vocab": V, "global_batch": args.batch, "seq_len": prompt_len,
            "context": 4096 if prompt_len == PROMPT_LEN else prompt_len + 5 * args.steps + args.warmup,
            "page_size": PAGE, "parallelism": "1 GPU", "repeats": f"median of {REPEATS} regions of --steps steps each",
            "l2": "inputs larger than L2 (2.47 GB of weights read every step)", "prompt_ids": "uniform, seed 2",
        },
        "e2e": None if e2e is None else {
            "value": args.batch * args.steps / e2e["ms"] * 1e3, "unit": "tok/s",
            "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
            "bytes_counted": "from the pinned buffers copied each step (metadata, sampler parameters; tokens back)"},
        "gpu_launches": run["launches"],
        "prefill": prefill,
        "roofline": {k: roofline[k] for k in ("bound", "achieved", "peak", "unit", "frac", "of")},
        "points": points,
        "points_roofline": points_roofline,
        "clocks": clock_rec,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
