"""Benchmark: decode tokens per second of the Qwen2.5-0.5B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the 0.5B configuration
(24 layers, hidden 896, 14/2 heads of 64, feed-forward 4864, vocabulary 151936, tied head)
with random weights in bfloat16, a batch of 8 requests with 512-token random prompts and a
4096-token context limit.  One JSON line is printed:

* ``value``: decoded tokens per second with the step running wholly on the device (sampled
  tokens fed back by a kernel, the step replayed as a CUDA graph), timed with CUDA events
  over exactly K steps after W warm-up steps;
* ``e2e``: the same through the Python entry point (``Engine.step``): every step copies the
  batch's arrays from pinned host memory to the device and reads the new token ids back;
* ``prefill``: one 2,048-token prompt in one step, tokens per second and the fraction of the
  bfloat16 tensor-core peak its floating-point work reaches;
* ``roofline``: bytes a decode step must read (every weight once, the cache of the live
  requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens per second at batch 1 and 64;
* ``clocks``: SM clock and throttle reasons sampled during the timed region.

Inputs are larger than the L2 cache (988 MB of weights are read every step), so no flush is
needed between timed iterations.  ``--gpus N`` with N > 1 is refused with exit code 2: this
engine runs on one GPU.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIG_05B = dict(hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                  num_key_value_heads=2, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, tie_word_embeddings=True, eos_token_id=151645)
# the 7B shape of the reference's second workload (continuous batching over mixed prompt lengths)
CONFIG_7B = dict(hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                 num_key_value_heads=4, vocab_size=152064, max_position_embeddings=4096, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=151645)
# the 14B shape of its third (a shared prefix, a pool too small for all requests)
CONFIG_14B = dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8, vocab_size=152064, max_position_embeddings=8192, rms_norm_eps=1e-5,
                  rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=151645)
SHAPES = {"0.5b": CONFIG_05B, "7b": CONFIG_7B, "14b": CONFIG_14B}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
REFERENCE_UNAVAILABLE = ("the reference is a TypeScript program for Node >= 24 with a Node-API CUDA module; it has no "
                         "Python package to install (pip finds no setup.py or pyproject.toml) and node is not in this image")


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            found = {"source": "measured"}
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = raw.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                if isinstance(value, (int, float)):
                    found[key] = float(value)
            if "hbm_gbs" in found and "bf16_tflops" in found:
                return found
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                             "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        peak = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for s in self.samples for name, flag in zip(names, s[2:6]) if flag.lower().startswith("active")})
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(peak) if peak else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_folder(layers: int, shape: str = "0.5b", context: int = 0) -> Path:
    """The random-weights model folder of the benchmark shape (written once per temporary folder);
    ``context``: another context length than the shape's."""
    from sprout_lm_b200 import parse_config, write_random_model
    sizes = dict(SHAPES[shape], num_hidden_layers=layers)
    tag = "" if shape == "0.5b" else "_" + shape
    if context and context != sizes["max_position_embeddings"]:
        sizes["max_position_embeddings"] = context
        tag += f"_C{context}"
    folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}{tag}_L{layers}"
    config = parse_config({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", **sizes})
    marker = folder / "complete"
    if not marker.exists():
        print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
        write_random_model(folder, config, seed=0)
        marker.write_text("ok")
    return folder


def weight_bytes(model) -> int:
    """Bytes of every weight a decode step uses once (the tied head is the embedding matrix)."""
    seen, total = set(), 0

    def add(t):
        nonlocal total
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for block in model.blocks:
        for lin in (block.mixer.qkv, block.mixer.out, block.feed_forward.gate_up, block.feed_forward.down):
            add(lin.weight)
            add(lin.bias)
        for norm in block.norms:
            add(norm.gain)
    add(model.final_norm.gain)
    add(model.head.linear.weight)
    return total


def prefill_flops(cfg: dict, tokens: int) -> float:
    h, i, l = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    heads, kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = h // heads
    per_token = l * 2 * (h * (heads + 2 * kv) * hd + heads * hd * h + 2 * h * i + i * h)
    attention = l * 4 * heads * hd * tokens * (tokens + 1) / 2          # QK^T and PV over the causal half
    head = 2 * h * cfg["vocab_size"]                                     # logits at one place
    return per_token * tokens + attention + head


def timed_decode(runner, batch: int, prompt_len: int, steps: int, warmup: int, rng, sampler=None):
    """Prefill ``batch`` prompts, then time ``steps`` decode steps that run wholly on the device."""
    import torch
    from sprout_lm_b200.engine.batch import StepEntry
    vocab = runner.vocab_size
    seqs = []
    for _ in range(batch):
        seq = runner.new_sequence()
        assert runner.reserve(seq, prompt_len)
        seqs.append(seq)
    chunk = max(1, 4096 // prompt_len)
    first = []
    for at in range(0, batch, chunk):
        for begin in range(0, prompt_len, 4096):                 # long prompts in portions of 4,096 tokens
            n = min(4096, prompt_len - begin)
            last = begin + n == prompt_len
            entries = [StepEntry(s, [int(t) for t in rng.integers(0, vocab, n)], [n - 1] if last else [])
                       for s in seqs[at:at + chunk]]
            sampled = runner.step_and_sample(entries, [0.0] * len(entries) if last else [], [0.0] * len(entries) if last else [])
        first += sampled
    entries = [StepEntry(s, [t], [0]) for s, t in zip(seqs, first)]
    loop = runner.decode_loop(entries, [0.0] * batch, [0.0] * batch, max_steps=steps + warmup + 2)
    loop.run(max(warmup - 1, 0))                 # capture runs one more step
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    loop.run(steps)
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = begin.elapsed_time(end)
    mean_context = prompt_len + warmup + steps / 2
    tokens = loop.finish()
    runner.check_status()
    assert tokens.shape[0] == steps + warmup and int(tokens.min()) >= 0
    for s in seqs:
        runner.release(s)
    return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1000), "launches_per_step": loop.launches_per_step,
            "mean_context": mean_context, "clocks": clocks}


def ablation(model, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """Marginal cost of each kind of kernel in the decode step: the step is captured and timed
    with one kind replaced by a no-op (its outputs are then garbage; only the time is used).
    Shows where the step's time goes under the real launch pipeline, warm caches included."""
    import numpy as np
    import torch
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    real = {name: getattr(kernels, name) for name in ("attention_decode", "attention_decode_fused", "attention_decode_resident",
                                                      "rmsnorm", "rope_append", "gemm_bf16", "gemm_bf16_unscaled", "sample",
                                                      "ffn_decode", "linear_decode")}
    linear = real["linear_decode"]
    gemm = real["gemm_bf16"]
    hidden, inter = model.spec.hidden_size, model.blocks[0].feed_forward.intermediate_size
    qkv_rows = model.blocks[0].mixer.qkv.out_features

    def gemm_without(skip):
        def call(a, w, out, status, **kw):
            return None if skip(w, kw) else gemm(a, w, out, status, **kw)
        return call

    variants = {
        "baseline": {},
        "attention": {"attention_decode": lambda *a, **k: None, "attention_decode_fused": lambda *a, **k: None,
                      "attention_decode_resident": lambda *a, **k: None},
        "rmsnorm": {"rmsnorm": lambda *a, **k: None},
        "rope_append": {"rope_append": lambda *a, **k: None},
        # (from 17 tokens the q/k/v product may be the one that takes the norm's input as it is)
        "gemm_qkv": {"gemm_bf16": gemm_without(lambda w, kw: w.shape[0] == qkv_rows), "gemm_bf16_unscaled": lambda *a, **k: None},
        "gemm_o": {"gemm_bf16": gemm_without(lambda w, kw: tuple(w.shape) == (hidden, hidden))},
        "gemm_gate_up": {"gemm_bf16": gemm_without(lambda w, kw: bool(kw.get("swiglu")))},
        "gemm_down": {"gemm_bf16": gemm_without(lambda w, kw: tuple(w.shape) == (hidden, inter))},
        "gemm_lm_head": {"gemm_bf16": gemm_without(lambda w, kw: w.shape[0] == model.spec.vocab_size)},
        "sample": {"sample": lambda *a, **k: None},
        # the small-batch kernels (they take the place of the norms and of every product but the head at up to 8 tokens)
        "ffn_decode": {"ffn_decode": lambda *a, **k: None},
        "linear_norm_qkv": {"linear_decode": lambda w, out, st, a=None, norm=None: None if norm is not None else linear(w, out, st, a=a)},
        "linear_o": {"linear_decode": lambda w, out, st, a=None, norm=None: None if a is not None else linear(w, out, st, norm=norm)},
        "all_gemms": {"gemm_bf16": lambda *a, **k: None, "gemm_bf16_unscaled": lambda *a, **k: None},
    }
    out = {}
    for label, patches in variants.items():
        rng = np.random.default_rng(0)
        runner = ModelRunner(model, num_pages=batch * (-(-(prompt_len + steps + warmup + 16) // 16)) + 16, page_tokens=16,
                             max_requests=max(batch, 1), prefix_caching=False)
        seqs = []
        for _ in range(batch):
            seq = runner.new_sequence()
            assert runner.reserve(seq, prompt_len)
            seqs.append(seq)
        first = []
        for at in range(0, batch, 8):
            entries = [StepEntry(s, [int(t) for t in rng.integers(0, 1000, prompt_len)], [prompt_len - 1]) for s in seqs[at:at + 8]]
            first += runner.step_and_sample(entries, [0.0] * len(entries), [0.0] * len(entries))
        for name, fn in patches.items():
            setattr(kernels, name, fn)
        try:
            loop = runner.decode_loop([StepEntry(s, [t], [0]) for s, t in zip(seqs, first)], [0.0] * batch, [0.0] * batch,
                                      max_steps=steps + warmup + 2)
            loop.run(warmup)
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            loop.run(steps)
            end.record()
            torch.cuda.synchronize()
        finally:
            for name, fn in real.items():
                setattr(kernels, name, fn)
        runner.runtime.status.zero_()
        out[label] = round(begin.elapsed_time(end) / steps * 1000, 1)
    base = out["baseline"]
    return {"us_per_step": base, "saved_us_without": {k: round(base - v, 1) for k, v in out.items() if k != "baseline"}}


def timed_e2e(model, batch: int, prompt_len: int, steps: int, warmup: int, rng):
    """The same workload through Engine.step: host token ids in, host token ids out, every step."""
    import torch
    from sprout_lm_b200 import EngineOptions, make_engine
    pages = batch * (-(-(prompt_len + steps + warmup + 8) // 16)) + 8
    engine = make_engine(model, EngineOptions(block_size=16, num_blocks=pages, max_sequences=max(batch, 1),
                                              max_batch_tokens=8192, prefill_chunk_size=2048, prefix_caching=False,
                                              record_trace=False))
    for i in range(batch):
        engine.add(f"r{i}", [int(t) for t in rng.integers(0, model.spec.vocab_size, prompt_len)],
                   steps + warmup + 4, ignore_eos=True)
    while any(w["phase"] != "decode" for w in engine.step()["work"]):
        pass
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    before = dict(engine.runner.stats)
    start = time.perf_counter()
    produced, marks = 0, [start]
    for _ in range(steps):
        report = engine.step()
        produced += sum(1 for e in report["events"] if e["type"] == "token")
        marks.append(time.perf_counter())       # the step's tokens are on the host here
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start
    per_step = sorted((b - a) * 1000 for a, b in zip(marks, marks[1:]))
    engine.runner.check_status()
    assert produced == batch * steps
    h2d = (engine.runner.stats["h2d_bytes"] - before["h2d_bytes"]) // steps
    d2h = (engine.runner.stats["d2h_bytes"] - before["d2h_bytes"]) // steps
    return {"value": produced / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": seconds * 1000 / steps, "p50_ms": per_step[len(per_step) // 2],
            "p95_ms": per_step[min(len(per_step) - 1, int(len(per_step) * 0.95))]}


def timed_prefill(runner, tokens: int, rng, repeats: int = 5):
    """A prompt of ``tokens`` tokens in one step through ``ModelRunner.step`` (what the scheduler
    calls): token ids from the host, the last position's logits on the device.  The same sizes
    come every time, so from the fourth step on the runner replays its capture of the step."""
    import numpy as np
    import torch
    from sprout_lm_b200.engine.batch import StepEntry
    times = []
    for _ in range(repeats + 4):
        seq = runner.new_sequence()
        assert runner.reserve(seq, tokens)
        entry = StepEntry(seq, rng.integers(0, runner.vocab_size, tokens).astype(np.int32), [tokens - 1])
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        logits = runner.step([entry])
        end.record()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(logits).all())
        times.append(begin.elapsed_time(end))
        runner.release(seq)
    return statistics.median(times[4:])


def timed_serving(shape: str, layers: int, requests: int, workload: str = "mixed", seed: int = 0) -> dict:
    """Continuous batching through ``Engine.step``, host tokens in and out every step.

    ``mixed``: ``requests`` requests with uniform-random prompt lengths in [128, 2048] arrive at
    once, prompts are prefilled in portions beside the decoding of the others, every request
    generates 128 tokens.  ``shared-prefix``: prompts of 4,096 tokens whose first 1,024 are the
    same, 256 generated tokens each, prefix reuse on, and a pool that holds 60 % of what all
    requests need at their longest, so that requests wait or are preempted and recomputed
    (requests are admitted when the pool can take them; SPROUT_REFERENCE_ADMISSION=1 admits
    as the reference does, whenever a sequence slot is free)."""
    import numpy as np
    import torch
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    sizes = SHAPES[shape]
    layers = layers or sizes["num_hidden_layers"]
    model = load_model(model_folder(layers, shape), dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(seed)
    shared = workload == "shared-prefix"
    if shared:
        lengths, new_tokens = [4096] * requests, 256
        if 4096 + new_tokens - 1 > sizes["max_position_embeddings"]:
            raise SystemExit(f"bench.py: the shared-prefix workload needs a context of 4,351 positions; shape {shape} has "
                             f"{sizes['max_position_embeddings']}")
        pages = int(0.6 * requests * -(-(4096 + new_tokens) // 16))
    else:
        lengths, new_tokens = [int(n) for n in rng.integers(128, 2049, requests)], 128
        pages = sum(-(-(n + new_tokens) // 16) for n in lengths) + 64
    options = EngineOptions(block_size=16, num_blocks=pages, max_sequences=requests, max_batch_tokens=2048,
                            prefill_chunk_size=1024, prefix_caching=shared, record_trace=False,
                            admit_within_pool=shared and os.environ.get("SPROUT_REFERENCE_ADMISSION") != "1")
    engine = make_engine(model, options)                 # one engine for both rounds: the second finds the graphs captured

    def run_once(tag):
        prefix = [int(t) for t in rng.integers(0, model.spec.vocab_size, 1024)]     # a new one each round: no hits across rounds
        for i, n in enumerate(lengths):
            tokens = [int(t) for t in rng.integers(0, model.spec.vocab_size, n)]
            if shared:
                tokens[:1024] = prefix
            engine.add(f"{tag}{i}", tokens, new_tokens, ignore_eos=True)
        times, kinds, preempted = [], {"prefill": 0, "mixed": 0, "decode": 0}, 0
        # the prompts are millions of Python integers: a full collection walking them in the middle
        # of the run would cost hundreds of milliseconds; collect now and set them aside
        gc.collect()
        gc.freeze()
        torch.cuda.synchronize()
        begin = time.perf_counter()
        while engine.pending:
            t0 = time.perf_counter()
            report = engine.step()
            times.append((time.perf_counter() - t0) * 1000)
            phases = {w["phase"] for w in report["work"]}
            kinds["decode" if phases == {"decode"} else "prefill" if "decode" not in phases else "mixed"] += 1
            preempted += sum(1 for e in report["events"] if e["type"] == "preempted")
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        gc.unfreeze()
        engine.runner.check_status()
        results = [engine.result(f"{tag}{i}") for i in range(requests)]
        assert all(len(r["output"]) == new_tokens for r in results)
        return seconds, times, kinds, preempted, engine.runner.step_graphs.replays, sum(r["prefixHits"] for r in results)

    run_once("warm")                                     # first use: kernel set-up, graph captures
    seconds, times, kinds, preempted, replays, hits = run_once("r")
    times.sort()
    pick = lambda q: round(times[min(len(times) - 1, int(q * len(times)))], 3)
    return {"impl": "ours", "only": "serve", "workload": workload, "shape": shape, "layers": layers,
            "layers_of_model": sizes["num_hidden_layers"], "requests": requests, "pool_pages": pages, "prefix_hit_tokens": hits, "prompt_tokens": sum(lengths), "new_tokens": requests * new_tokens,
            "seconds": round(seconds, 4), "generated_tokens_per_s": round(requests * new_tokens / seconds, 1),
            "all_tokens_per_s": round((sum(lengths) + requests * new_tokens) / seconds, 1),
            "steps": len(times), "step_kinds": kinds, "step_ms": {"p50": pick(0.5), "p95": pick(0.95), "max": times[-1].__round__(3)},
            "preempted": preempted, "prefill_steps_replayed": replays,
            "decode_graphs": {"keys": engine.runner.graphs.keys_used, "held": len(engine.runner.graphs.graphs),
                              "dropped": engine.runner.graphs.evictions},
            "steps_launched_ahead": {"taken": engine.runner.ahead_used, "let_go": engine.runner.ahead_dropped}}


def timed_attention(tokens: int, shape: str = "0.5b", repeats: int = 20) -> dict:
    """The prefill attention kernels alone, at the model's head sizes, over a paged cache: one
    request of ``tokens`` tokens attending to itself (causal), both kernels."""
    import torch
    from sprout_lm_b200 import kernels
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    head_dim, page = SHAPES[shape]["hidden_size"] // heads, 16
    pages = -(-tokens // page)
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).reshape(1, pages)
    q = torch.randn(tokens, heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    q_start = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flops = 4.0 * heads * head_dim * tokens * (tokens + 1) / 2
    result = {"impl": "ours", "only": "attention", "shape": shape, "tokens": tokens, "heads": heads, "kv_heads": kv_heads,
              "head_dim": head_dim, "page_tokens": page}
    for variant in ("mma_sync", "tcgen05"):
        call = lambda: kernels.attention_prefill(q, k, v, table, q_start, positions, out, heads, kv_heads, head_dim,
                                                 status, variant=variant)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(repeats):
            call()
        end.record()
        torch.cuda.synchronize()
        us = begin.elapsed_time(end) * 1000 / repeats
        result[f"{variant}_us"] = round(us, 1)
        result[f"{variant}_tflops"] = round(flops / us / 1e6, 1)
    assert int(status.item()) == 0
    return result


def timed_decode_attention(shape: str, batch: int, context: int, repeats: int = 10) -> dict:
    """The decode attention kernel alone (one query token per request, ``context`` keys each, pages
    scattered over the pool, block tables as wide as a replayed decode graph's): with the split
    plan the engine would pick, and with other split sizes for comparison.  Bytes are the keys and
    values read."""
    import torch
    from sprout_lm_b200 import kernels
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    head_dim, page = SHAPES[shape]["hidden_size"] // heads, 16
    width = -(-(-(-context // page)) // 64) * 64
    total = batch * width
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(total, device="cuda", generator=g).to(torch.int32).reshape(batch, width)
    lens = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    planned = -(-context // 128) * 128

    def replayed(split_keys):
        if split_keys == "resident":
            room = min(kernels.resident_cap(heads, kv_heads, head_dim, page), -(-context // 256) * 256)
            call = lambda: kernels.attention_decode_resident(k, v, table, lens, out, heads, kv_heads, head_dim, status, room, q=q)
        else:
            call = lambda: kernels.attention_decode(q, k, v, table, lens, out, heads, kv_heads, head_dim, status,
                                                    split_keys=split_keys, live_keys=planned)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(repeats):
                    call()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1000 / repeats)
        return statistics.median(times)

    megabytes = 2.0 * batch * context * kv_heads * head_dim * 2 / 1e6
    plan = kernels.decode_split_plan(batch, kv_heads, width * page, head_dim, planned)
    us = replayed(None)
    result = {"impl": "ours", "only": "decode-attention", "shape": shape, "batch": batch, "context": context,
              "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "table_keys": width * page,
              "plan": {"split_keys": plan[0], "splits": plan[1], "through_memory": plan[2]},
              "us": round(us, 1), "gbs": round(megabytes / us * 1e3), "mb": round(megabytes, 1), "other_splits_us": {}}
    for passes in (1, 2, 4, 8, 16, 32, width * page // 128):
        if passes * 128 <= width * page and width * page // (passes * 128) <= 256:
            result["other_splits_us"][str(passes * 128)] = round(replayed(passes * 128), 1)
    if context <= kernels.resident_cap(heads, kv_heads, head_dim, page):
        # the whole context of a (request, key/value head) in one CTA's shared memory, pages by TMA
        us = replayed("resident")
        result["resident_us"], result["resident_gbs"] = round(us, 1), round(megabytes / us * 1e3)
        result["engine_takes"] = kernels.decode_attention_plan(batch, heads, kv_heads, head_dim, page, width * page, planned)[0]
    assert int(status.item()) == 0
    return result


def timed_long_prompt(shape: str, layers: int, total: int, portion: int) -> dict:
    """One request of ``total`` tokens through ``ModelRunner.step`` in portions of ``portion``: the
    time of every step (CUDA events; the second of two runs), so that the attention over the cached
    keys shows as the increase from portion to portion (the products cost the same in each)."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    base = SHAPES[shape]
    layers = layers or base["num_hidden_layers"]
    context = base["max_position_embeddings"]
    while context < total:
        context *= 2
    model = load_model(model_folder(layers, shape, context), dtype="bfloat16", device="cuda:0")
    runner = ModelRunner(model, num_pages=-(-total // 16) + 16, page_tokens=16, max_requests=2, prefix_caching=False)
    rng = np.random.default_rng(0)
    heads, head_dim = base["num_attention_heads"], base["hidden_size"] // base["num_attention_heads"]
    steps = []
    for run in range(2):
        seq = runner.new_sequence()
        assert runner.reserve(seq, total)
        steps = []
        for begin in range(0, total, portion):
            n = min(portion, total - begin)
            tokens = [int(t) for t in rng.integers(0, base["vocab_size"], n)]
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(seq, tokens, [n - 1])])
            end.record()
            torch.cuda.synchronize()
            steps.append({"context": begin, "tokens": n, "ms": round(start.elapsed_time(end), 3)})
        runner.check_status()
        runner.release(seq)
    whole = sum(s["ms"] for s in steps)
    out = {"impl": "ours", "only": "long-prompt", "shape": shape, "layers": layers, "tokens": total, "portion": portion,
           "context_limit": context, "ms": round(whole, 2), "tokens_per_s": round(total / whole * 1000, 1), "steps": steps}
    full = [s for s in steps if s["tokens"] == portion]
    if len(full) >= 3:
        # attention over one more portion's worth of cached keys: 4 * portion^2 * heads * head_dim flops a layer
        growth = (full[-1]["ms"] - full[1]["ms"]) / (len(full) - 2)
        out["ms_more_per_portion_of_context"] = round(growth, 3)
        out["attention_tflops_from_growth"] = round(4.0 * portion * portion * heads * head_dim * layers / (growth / 1000) / 1e12, 1)
    return out


def timed_gemms(tokens: int, shape: str = "0.5b", repeats: int = 20) -> dict:
    """The model's four projections at ``tokens`` tokens, each alone: 20 launches replayed from a
    CUDA graph (no host time between them), beside the library's plain bfloat16 product of the
    same shape for scale (it fuses nothing and is not on the engine's path).  Up to 256 tokens (the
    decode regime, where a product is a stream of weights) the launches cycle through copies of
    the weights that together exceed L2, as the layers of a model do, and the RMSNorm that
    precedes a product is timed the same way."""
    import torch
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.linear import small_batch_split_k
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    hidden, inter = SHAPES[shape]["hidden_size"], SHAPES[shape]["intermediate_size"]
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    qkv = (heads + 2 * kv_heads) * (hidden // heads)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    rand = lambda *shape: (torch.randn(*shape, device="cuda", generator=g) * 0.05).to(torch.bfloat16)

    def replayed(call):
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for i in range(repeats):
                    call(i)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1000 / repeats

    result = {"impl": "ours", "only": "gemm", "shape": shape, "tokens": tokens}
    # up to 256 tokens the engine sums q/k/v in float32 over a split K range (bias and rotation follow in attention)
    cases = [("qkv", qkv, hidden, "bias" if tokens > 256 else "residual"), ("o", hidden, hidden, "residual"),
             ("gate_up", 2 * inter, hidden, "swiglu"), ("down", hidden, inter, "residual")]
    if tokens <= 256:
        x, gain, normed = torch.randn(tokens, hidden, device="cuda", generator=g), torch.ones(hidden, device="cuda"), rand(tokens, hidden)
        result["rmsnorm"] = {"shape": [tokens, hidden], "us": round(replayed(lambda i: kernels.rmsnorm(x, gain, normed, 1e-6)), 2)}
    for name, n, k, kind in cases:
        a, w = rand(tokens, k), rand(n, k)
        copies = min(repeats, -(-160_000_000 // (2 * n * k))) if tokens <= 256 else 1
        kw = {}
        if kind == "bias":
            out, kw = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda"), {"bias": torch.zeros(n, device="cuda")}
        elif kind == "residual":
            out = torch.zeros(tokens, n, device="cuda")
            kw = {"residual": out, "split_k": small_batch_split_k(n, k, tokens, True, kernels.sm_count())}
        else:
            w = interleave_gate_up(w[:n // 2].contiguous(), w[n // 2:].contiguous())
            out, kw = torch.empty(tokens, n // 2, dtype=torch.bfloat16, device="cuda"), {"swiglu": True}
        ws = [w] + [w.clone() for _ in range(copies - 1)]
        us = replayed(lambda i: kernels.gemm_bf16(a, ws[i % copies], out, status, **kw))
        library = replayed(lambda i: torch.matmul(a, ws[i % copies].t()))
        result[name] = {"shape": [tokens, n, k], "epilogue": kind, "split_k": kw.get("split_k", 1), "weight_copies": copies, "us": round(us, 1),
                        "tflops": round(2.0 * tokens * n * k / us / 1e6), "weight_gbs": round(2.0 * n * k / us / 1e3),
                        "library_plain_us": round(library, 1)}
    assert int(status.item()) == 0
    return result


# Tulipel (latent attention) at sizes that resemble a real model's layers, and the Qwen2 configuration of equal
# width, heads, head size (dim + rot_dim), layers, vocabulary and feed-forward parameters beside it
LATENT_SHAPES = {
    "1b": dict(width=2048, heads=16, dim=64, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, ff=8192, vocab=32768,
               qwen=dict(intermediate_size=5464, num_key_value_heads=4)),
    "0.3b": dict(width=1024, heads=8, dim=64, rot_dim=64, vdim=128, kv_rank=256, q_rank=384, ff=4096, vocab=32768,
                 qwen=dict(intermediate_size=2736, num_key_value_heads=2)),
}


def latent_folders(shape: str, layers: int):
    """(Tulipel folder, Qwen2 folder of equal size), random weights, written once."""
    from sprout_lm_b200 import parse_config, write_random_model
    z = LATENT_SHAPES[shape]
    scale = (z["dim"] + z["rot_dim"]) ** -0.5

    def mixer(kind, **extra):
        rot = {"base": 10000.0, "dims": z["rot_dim"]}
        if kind == "latent_attention_2":
            rot["scaling"] = {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}
        return {"type": kind, "mlp": {"kind": "dense", "ff": z["ff"]},
                "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
                          "scale": scale, "rot": rot, **extra}}
    entries = []
    for i in range(layers):                       # the two kinds in turn; every fourth layer reads the rows of the one two before
        if i % 2 == 0:
            entries.append(mixer("latent_attention_2", **({"kv_from": i - 2} if i % 4 == 2 else {})))
        else:
            entries.append(mixer("latent_attention", q_rank=z["q_rank"]))
    raw = {"architecture": "Tulipel", "vocab": z["vocab"], "width": z["width"], "postln_alpha": 2.0, "logit_softcap": 30.0,
           "norm": {"eps": 1e-5}, "layers": entries, "max_positions": 16384}
    qwen = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "hidden_size": z["width"],
            "num_hidden_layers": layers, "num_attention_heads": z["width"] // (z["dim"] + z["rot_dim"]), "vocab_size": z["vocab"],
            "max_position_embeddings": 16384, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False,
            "eos_token_id": 0, **z["qwen"]}
    folders = []
    for tag, config in (("tulipel", raw), ("qwen2", qwen)):
        folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}_latent_{shape}_{tag}_L{layers}"
        if not (folder / "complete").exists():
            print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
            write_random_model(folder, parse_config(config), seed=0)
            (folder / "complete").write_text("ok")
        folders.append(folder)
    return folders[0], folders[1], raw, qwen


def _median_us(call, repeats: int = 10) -> float:
    import torch
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(repeats):
            call()
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end) * 1000 / repeats)
    return statistics.median(times)


def timed_latent_kernels(shape: str, tokens: int, batch: int, context: int, peak: dict) -> dict:
    """The new design's attention kernels alone beside the grouped-query kernels at equal heads and head size:
    one prompt of ``tokens`` tokens (FLOPs of the causal half against the measured bf16 rate) and ``batch`` decode
    tokens over ``context`` keys each (cache bytes read against the measured copy rate)."""
    import torch
    from types import SimpleNamespace
    from sprout_lm_b200 import kernels
    z = LATENT_SHAPES[shape]
    heads, rank, width, page = z["heads"], z["kv_rank"], z["kv_rank"] + z["rot_dim"], 16
    g = torch.Generator(device="cuda").manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sink = torch.zeros(heads, device="cuda")
    out = {}

    def ctx_for(requests, new, held):
        t = requests * new
        return SimpleNamespace(seq_of_token=torch.arange(requests, dtype=torch.int32, device="cuda").repeat_interleave(new),
                               positions=(torch.arange(new, dtype=torch.int32, device="cuda") + (held - new)).repeat(requests),
                               q_start=(torch.arange(requests + 1, dtype=torch.int32, device="cuda") * new),
                               context_lens=torch.full((requests,), held, dtype=torch.int32, device="cuda"), max_q_len=new,
                               max_context=held, planned_context=0, num_seqs=requests, num_tokens=t)
    for label, requests, new, held in (("prefill", 1, tokens, tokens), ("decode", batch, 1, context)):
        pages = -(-held // page)
        table_width = -(-pages // 64) * 64
        cache = (torch.randn(requests * pages + 1, 1, page, width, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
        table = torch.full((requests, table_width), -1, dtype=torch.int32, device="cuda")
        table[:, :pages] = torch.randperm(requests * pages, device="cuda", generator=g).to(torch.int32).reshape(requests, pages)
        q = (torch.randn(requests * new, heads * width, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
        o = torch.empty(requests * new, heads * rank, dtype=torch.bfloat16, device="cuda")
        view = SimpleNamespace(k=cache, v=None, block_table=table, page_tokens=page, write=False)
        ctx = ctx_for(requests, new, held)
        us = _median_us(lambda: kernels.latent_attention(q, view, ctx, sink, o, heads, rank, z["dim"] ** -0.5, status),
                        repeats=3 if label == "prefill" else 10)
        if label == "prefill":
            flops = 2.0 * heads * (width + rank) * tokens * (tokens + 1) / 2
            out["latent_prefill"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                                     "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
        else:
            mb = batch * context * width * 2 / 1e6
            out["latent_decode"] = {"us": round(us, 1), "gbs": round(mb / us * 1e3), "mb": round(mb, 1),
                                    "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    # the grouped-query kernels at equal heads and head size
    kv_heads, head_dim = z["qwen"]["num_key_value_heads"], z["dim"] + z["rot_dim"]
    q_heads = z["width"] // head_dim
    pages = -(-tokens // page)
    k = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).reshape(1, pages)
    q = torch.randn(tokens, q_heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    o = torch.empty_like(q)
    q_start = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    variant = "tcgen05" if head_dim in (64, 128) else "mma_sync"
    us = _median_us(lambda: kernels.attention_prefill(q, k, v, table, q_start, positions, o, q_heads, kv_heads, head_dim, status, variant=variant))
    flops = 4.0 * q_heads * head_dim * tokens * (tokens + 1) / 2
    out["gqa_prefill"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "variant": variant,
                          "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
    table_width = -(-(-(-context // page)) // 64) * 64
    total = batch * table_width
    k = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(total, device="cuda", generator=g).to(torch.int32).reshape(batch, table_width)
    lens = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, q_heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    o = torch.empty_like(q)
    us = _median_us(lambda: kernels.attention_decode(q, k, v, table, lens, o, q_heads, kv_heads, head_dim, status,
                                                     live_keys=-(-context // 128) * 128))
    mb = 2.0 * batch * context * kv_heads * head_dim * 2 / 1e6
    out["gqa_decode"] = {"us": round(us, 1), "gbs": round(mb / us * 1e3), "mb": round(mb, 1),
                         "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    assert int(status.item()) == 0
    return out


def timed_latent(args) -> dict:
    """``--only latent``: prefill and decode throughput of Tulipel at ``--shape 1b|0.3b`` (random weights,
    ``--layers`` layers, 4 if not given) beside Qwen2 at equal size, through the same runner, and the attention
    kernels of both alone."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    shape = args.shape if args.shape in LATENT_SHAPES else "1b"
    layers = args.layers or 4
    peak = peaks()
    tulipel_dir, qwen_dir, _, _ = latent_folders(shape, layers)
    prompt_len = args.prompt_len
    result = {"impl": "ours", "only": "latent", "shape": shape, "layers": layers, "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": args.tokens, "decode_batch": args.batch, "decode_prompt_len": prompt_len, "steps": args.steps,
              "peaks": {"bf16_tflops": peak["bf16_tflops"], "hbm_gbs": peak["hbm_gbs"], "source": peak.get("source", "measured")}}
    for tag, folder in (("tulipel", tulipel_dir), ("qwen2", qwen_dir)):
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        slots = max(64, args.batch)
        pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + args.tokens // 16 + 16
        runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)
        rng = np.random.default_rng(0)
        ms = timed_prefill(runner, args.tokens, rng)
        decode = timed_decode(runner, args.batch, prompt_len, args.steps, args.warmup, rng)
        result[tag] = {"prefill_ms": round(ms, 3), "prefill_tokens_per_s": round(args.tokens / ms * 1000),
                       "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tokens_per_s"]),
                       "decode_launches_per_step": decode["launches_per_step"]}
        del runner, model
        torch.cuda.empty_cache()
    result["kernels"] = timed_latent_kernels(shape, args.tokens, max(args.batch, 64), 2048, peak)
    return result


# Letanex (differential attention, linear attention with decay and state, routed experts) at sizes that resemble a real
# model's layers, and the Qwen2 configuration of equal width, heads, layers, vocabulary and active feed-forward
# parameters beside it (grouped-query attention with heads of 128, SwiGLU)
LETANEX_SHAPES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, state_heads=16, state_dim=128, ff=8192, experts=32,
               identity=4, top=4, expert_ff=1024, shared_ff=2048, vocab=32768, qwen=dict(intermediate_size=6144, num_key_value_heads=4)),
    "0.3b": dict(width=1024, heads=8, kv_heads=2, dim=64, vdim=128, state_heads=8, state_dim=128, ff=4096, experts=16,
                 identity=2, top=4, expert_ff=512, shared_ff=1024, vocab=32768, qwen=dict(intermediate_size=3072, num_key_value_heads=2)),
}


def letanex_folders(shape: str, layers: int):
    """(Letanex folder, Qwen2 folder of equal size), random weights, written once.  Layers in fours: attention with a dense
    feed-forward, attention over the first one's keys and values with routed experts, two layers of linear attention with
    routed experts."""
    from sprout_lm_b200 import parse_config, write_random_model
    z = LETANEX_SHAPES[shape]
    moe = {"kind": "moe", "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 1.0},
           "expert": {"ff": z["expert_ff"], "limit": 7.0}, "shared": {"ff": z["shared_ff"], "limit": 7.0}}
    entries = []
    for i in range(layers):
        if i % 4 < 2:
            mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                     "diff": 0.5, "rot": {"base": 10000.0, "dims": z["dim"], "scaling": {"factor": 8.0}}}
            if i % 4 == 1:
                mixer["kv_from"] = i - 1
            entries.append({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": z["ff"]} if i % 4 == 0 else moe})
        else:
            decay = [float(1.0 - 2.0 ** (-5 - 3 * h / max(1, z["state_heads"] - 1))) for h in range(z["state_heads"])]
            entries.append({"type": "lightning", "mlp": moe,
                            "mixer": {"heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["vdim"], "decay": decay}})
    raw = {"architecture": "Letanex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": entries,
           "max_positions": 16384}
    qwen = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "hidden_size": z["width"],
            "num_hidden_layers": layers, "num_attention_heads": z["heads"], "vocab_size": z["vocab"],
            "max_position_embeddings": 16384, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False,
            "eos_token_id": 0, **z["qwen"]}
    folders = []
    for tag, config in (("letanex", raw), ("qwen2", qwen)):
        folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}_letanex_{shape}_{tag}_L{layers}"
        if not (folder / "complete").exists():
            print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
            write_random_model(folder, parse_config(config), seed=0)
            (folder / "complete").write_text("ok")
        folders.append(folder)
    return folders[0], folders[1], raw, qwen


def timed_letanex_kernels(shape: str, tokens: int, batch: int, context: int, peak: dict) -> dict:
    """The new design's kernels alone beside the closest kernels of the grouped-query model at equal sizes: attention over
    one prompt of ``tokens`` tokens (executed FLOPs of the causal half against the measured bf16 rate) and ``batch`` single
    tokens over ``context`` keys each (cache bytes against the measured copy rate); the linear attention's prompt kernel
    (bytes it must move against the copy rate; its FLOPs are small); the routed experts' two products beside the dense
    SwiGLU products of as many FLOPs."""
    import torch
    from types import SimpleNamespace
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.linear import Linear
    z = LETANEX_SHAPES[shape]
    heads, kv, dim, vdim, page = z["heads"], z["kv_heads"], z["dim"], z["vdim"], 16
    g = torch.Generator(device="cuda").manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}

    def rand(*shape_, scale=1.0):
        return (torch.randn(*shape_, device="cuda", generator=g) * scale).to(torch.bfloat16)

    def ctx_for(requests, new, held):
        return SimpleNamespace(seq_of_token=torch.arange(requests, dtype=torch.int32, device="cuda").repeat_interleave(new),
                               positions=(torch.arange(new, dtype=torch.int32, device="cuda") + (held - new)).repeat(requests),
                               q_start=(torch.arange(requests + 1, dtype=torch.int32, device="cuda") * new),
                               context_lens=torch.full((requests,), held, dtype=torch.int32, device="cuda"), max_q_len=new,
                               max_context=held, planned_context=0, num_seqs=requests, num_tokens=requests * new)
    gqa_dim = 2 * dim                                   # the grouped-query model's head size: as many query/key elements per head
    for label, requests, new, held in (("prefill", 1, tokens, tokens), ("decode", batch, 1, context)):
        pages = -(-held // page)
        width_t = -(-pages // 64) * 64
        table = torch.full((requests, width_t), -1, dtype=torch.int32, device="cuda")
        table[:, :pages] = torch.randperm(requests * pages, device="cuda", generator=g).to(torch.int32).reshape(requests, pages)
        ctx = ctx_for(requests, new, held)
        k2, v2 = rand(requests * pages + 1, kv, page, 2 * dim), rand(requests * pages + 1, kv, page, vdim)
        q2 = rand(requests * new, heads * 2 * dim, scale=0.3)
        o2 = torch.empty(requests * new, heads * vdim, dtype=torch.bfloat16, device="cuda")
        view = SimpleNamespace(k=k2, v=v2, block_table=table, page_tokens=page, write=False)
        us = _median_us(lambda: kernels.multimap_attention(q2, view, ctx, o2, heads, kv, 2, dim, vdim, dim ** -0.5, 0.4, 1e-5, 0.5, status),
                        repeats=3 if label == "prefill" else 10)
        kg, vg = rand(requests * pages + 1, kv, page, gqa_dim), rand(requests * pages + 1, kv, page, gqa_dim)
        qg = rand(requests * new, heads * gqa_dim, scale=0.3)
        og = torch.empty_like(qg)
        if label == "prefill":
            flops = 4.0 * heads * (dim + vdim) * tokens * (tokens + 1) / 2
            out["two_map_prefill"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                                      "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
            variant = "tcgen05" if gqa_dim in (64, 128) else "mma_sync"
            for name, var in (("gqa_prefill", variant), ("gqa_prefill_mma_sync", "mma_sync")):
                us = _median_us(lambda: kernels.attention_prefill(qg, kg, vg, table, ctx.q_start, ctx.positions, og, heads, kv, gqa_dim,
                                                                  status, variant=var), repeats=3)
                flops = 4.0 * heads * gqa_dim * tokens * (tokens + 1) / 2
                out[name] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "variant": var,
                             "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
        else:
            mb = batch * context * kv * (2 * dim + vdim) * 2 / 1e6
            out["two_map_decode"] = {"us": round(us, 1), "gbs": round(mb / us * 1e3), "mb": round(mb, 1),
                                     "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
            us = _median_us(lambda: kernels.attention_decode(qg, kg, vg, table, ctx.context_lens, og, heads, kv, gqa_dim, status,
                                                             live_keys=-(-context // 128) * 128))
            mb = 2.0 * batch * context * kv * gqa_dim * 2 / 1e6
            out["gqa_decode"] = {"us": round(us, 1), "gbs": round(mb / us * 1e3), "mb": round(mb, 1),
                                 "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    # linear attention with decay: a prompt, and single tokens
    sh, sd = z["state_heads"], z["state_dim"]
    decay = torch.full((sh,), 0.99, device="cuda")
    for label, requests, new in (("prefill", 1, tokens), ("decode", batch, 1)):
        rows = rand(requests * new, sh * (2 * sd + 2 * vdim), scale=0.5)
        state = torch.zeros(requests, sh, sd, vdim, device="cuda")
        view = SimpleNamespace(buffer=state, slots=torch.arange(requests, dtype=torch.int32, device="cuda"))
        o = torch.empty(requests * new, sh * vdim, device="cuda")
        ctx = ctx_for(requests, new, new)
        us = _median_us(lambda: kernels.decay_attention(rows, ctx, view, decay, o, sh, sd, vdim, True, status), repeats=3 if new > 1 else 10)
        mb = (requests * new * sh * ((2 * sd + vdim) * 2 + vdim * 4) + 2 * requests * sh * sd * vdim * 4) / 1e6
        out[f"decay_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                 "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                 "tflops": round(4.0 * requests * new * sh * sd * vdim / us / 1e6, 2)}
    # routed experts beside dense products of as many FLOPs
    W, E, top, ff = z["width"], z["experts"], z["top"], z["expert_ff"]
    w_gu, w_d = rand(E, 2 * ff, W, scale=0.02), rand(E, W, ff, scale=0.02)
    dense_gu = Linear(rand(2 * top * ff, W, scale=0.02), None, status)
    dense_d = Linear(rand(W, top * ff, scale=0.02), None, status)
    for label, n in (("prefill", tokens), ("decode", batch)):
        h = rand(n, W)
        ids = torch.stack([torch.randperm(E, device="cuda", generator=g)[:top] for _ in range(n)]).to(torch.int32).contiguous()
        counts = torch.bincount(ids.flatten().long(), minlength=E).to(torch.int32)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
        order, place_of = torch.empty(n * top, dtype=torch.int32, device="cuda"), torch.empty(n * top, dtype=torch.int32, device="cuda")
        kernels.moe_arrange(ids, counts, offsets, order, place_of, E)
        act = torch.empty(n * top, ff, dtype=torch.bfloat16, device="cuda")
        rows_out = torch.empty(n * top, W, device="cuda")
        us = _median_us(lambda: kernels.moe_experts(h, order, offsets, w_gu, w_d, act, rows_out, E, top, 7.0, 1.702), repeats=3 if n > 256 else 10)
        flops = 6.0 * n * top * W * ff
        mb = (w_gu.numel() + w_d.numel()) * 2 / 1e6
        out[f"experts_{label}"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3),
                                   "weights_gbs": round(mb / us * 1e3), "weights_of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
        x = torch.zeros(n, W, device="cuda")

        def dense():
            dense_d.forward(dense_gu.forward_swiglu(h, 8), residual=x)
        us = _median_us(dense, repeats=3 if n > 256 else 10)
        mb = (dense_gu.weight.numel() + dense_d.weight.numel()) * 2 / 1e6
        out[f"dense_swiglu_{label}"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3),
                                        "weights_gbs": round(mb / us * 1e3), "weights_of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    assert int(status.item()) == 0
    return out


def timed_letanex(args) -> dict:
    """``--only letanex``: prefill and decode throughput of Letanex at ``--shape 1b|0.3b`` (random weights, ``--layers``
    layers, 4 if not given) beside Qwen2 at equal size, through the same runner, and the kernels of both alone."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    shape = args.shape if args.shape in LETANEX_SHAPES else "1b"
    layers = args.layers or 4
    peak = peaks()
    letanex_dir, qwen_dir, _, _ = letanex_folders(shape, layers)
    prompt_len = args.prompt_len
    result = {"impl": "ours", "only": "letanex", "shape": shape, "layers": layers, "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": args.tokens, "decode_batch": args.batch, "decode_prompt_len": prompt_len, "steps": args.steps,
              "peaks": {"bf16_tflops": peak["bf16_tflops"], "hbm_gbs": peak["hbm_gbs"], "source": peak.get("source", "measured")}}
    for tag, folder in (("letanex", letanex_dir), ("qwen2", qwen_dir)):
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        slots = max(64, args.batch)
        pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + args.tokens // 16 + 16
        runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)
        rng = np.random.default_rng(0)
        ms = timed_prefill(runner, args.tokens, rng)
        decode = timed_decode(runner, args.batch, prompt_len, args.steps, args.warmup, rng)
        result[tag] = {"prefill_ms": round(ms, 3), "prefill_tokens_per_s": round(args.tokens / ms * 1000),
                       "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tokens_per_s"]),
                       "decode_launches_per_step": decode["launches_per_step"]}
        del runner, model
        torch.cuda.empty_cache()
    result["kernels"] = timed_letanex_kernels(shape, args.tokens, max(args.batch, 64), 2048, peak)
    return result


RARUTAR_SHAPES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, left_dim=64, left_vdim=128, rotated=64, window=1024, chunk=2048,
               state_heads=16, state_dim=128, state_vdim=128, tau=16.0, rank=32, ssm_heads=64, ssm_vdim=64, ssm_state=128,
               ssm_groups=8, taps=4, norm_groups=8, ff=4096, vocab=32768),
    "0.3b": dict(width=1024, heads=8, kv_heads=2, dim=128, left_dim=64, left_vdim=128, rotated=64, window=512, chunk=1024,
                 state_heads=8, state_dim=128, state_vdim=128, tau=16.0, rank=16, ssm_heads=32, ssm_vdim=64, ssm_state=64,
                 ssm_groups=4, taps=4, norm_groups=4, ff=2048, vocab=32768),
}


def rarutar_folders(shape: str, layers: int):
    """(Rarutar folder, Letanex folder of equal size), random weights, written once.  Rarutar's layers in fours: chunked
    attention whose values are its keys, windowed attention beside gated linear attention, a selective state space, the
    pair again; all with the gated feed-forward.  Letanex beside it: two-map attention, linear attention with a fixed
    decay, twice, with a dense feed-forward of as many weights (two matrices of 1.5 ff against three of ff)."""
    from sprout_lm_b200 import parse_config, write_random_model
    z = RARUTAR_SHAPES[shape]
    mlp = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    attention = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                 "mask": {"size": z["chunk"]}, "rot": {"base": 500000.0, "dims": z["rotated"]}}
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["left_dim"], "vdim": z["left_vdim"], "scale": z["left_dim"] ** -0.5,
            "mask": {"size": z["window"]},
            "rot": {"base": 500000.0, "dims": z["left_dim"], "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    right = {"heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["state_vdim"], "tau": z["tau"], "rank": z["rank"]}
    pair = {"left": left, "right": right, "left_scale": 0.5, "right_scale": 0.5}
    ssm = {"heads": z["ssm_heads"], "vdim": z["ssm_vdim"], "state": z["ssm_state"], "groups": z["ssm_groups"], "conv": z["taps"],
           "norm_groups": z["norm_groups"]}
    kinds = [("attention", attention), ("parallel", pair), ("mamba2", ssm), ("parallel", pair)]
    raw = {"architecture": "Rarutar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": mlp} for i in range(layers)], "max_positions": 16384}
    entries = []
    for i in range(layers):
        if i % 2 == 0:
            mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["left_dim"], "vdim": z["left_vdim"], "scale": z["left_dim"] ** -0.5,
                     "diff": 0.5, "rot": {"base": 10000.0, "dims": z["left_dim"], "scaling": {"factor": 8.0}}}
            entries.append({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": z["ff"] * 3 // 2}})
        else:
            decay = [float(1.0 - 2.0 ** (-5 - 3 * h / max(1, z["state_heads"] - 1))) for h in range(z["state_heads"])]
            entries.append({"type": "lightning", "mlp": {"kind": "dense", "ff": z["ff"] * 3 // 2},
                            "mixer": {"heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["state_vdim"], "decay": decay}})
    letanex = {"architecture": "Letanex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": entries,
               "max_positions": 16384}
    folders = []
    for tag, config in (("rarutar", raw), ("letanex", letanex)):
        folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}_rarutar2_{shape}_{tag}_L{layers}"
        if not (folder / "complete").exists():
            print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
            write_random_model(folder, parse_config(config), seed=0)
            (folder / "complete").write_text("ok")
        folders.append(folder)
    return folders[0], folders[1]


def timed_rarutar_kernels(shape: str, tokens: int, batch: int, context: int, peak: dict) -> dict:
    """The new design's kernels alone beside the like kernels of Letanex at equal sizes: attention with one map under a
    window or in chunks (gate, sink, unit-norm vectors) beside the two-map kernel, over one prompt of ``tokens`` tokens
    (executed FLOPs of the visible keys against the measured bf16 rate) and over ``batch`` single tokens with ``context``
    keys held (bytes of the visible keys against the measured copy rate); the scan with a decay per key channel and the
    one with a decay per head beside the linear attention with a fixed decay (bytes that must move against the copy
    rate); the short convolution and the gated group norm (bytes against the copy rate)."""
    import torch
    from types import SimpleNamespace
    from sprout_lm_b200 import kernels
    z = RARUTAR_SHAPES[shape]
    page = 16
    g = torch.Generator(device="cuda").manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}

    def rand(*shape_, scale=1.0, dtype=torch.bfloat16):
        return (torch.randn(*shape_, device="cuda", generator=g) * scale).to(dtype)

    def ctx_for(requests, new, held):
        return SimpleNamespace(seq_of_token=torch.arange(requests, dtype=torch.int32, device="cuda").repeat_interleave(new),
                               positions=(torch.arange(new, dtype=torch.int32, device="cuda") + (held - new)).repeat(requests),
                               q_start=(torch.arange(requests + 1, dtype=torch.int32, device="cuda") * new),
                               context_lens=torch.full((requests,), held, dtype=torch.int32, device="cuda"), max_q_len=new,
                               max_context=held, planned_context=0, num_seqs=requests, num_tokens=requests * new)

    def visible(mask, position):
        kind, size = mask
        return min(position + 1, size) if kind == "window" else position % size + 1

    heads, kv = z["heads"], z["kv_heads"]
    variants = (("windowed", 1, z["left_dim"], z["left_vdim"], ("window", z["window"]), False),
                ("chunked_sink", 1, z["dim"], z["dim"], ("chunk", z["chunk"]), True),
                ("two_map", 2, z["left_dim"], z["left_vdim"], None, False))
    for label, requests, new, held in (("prefill", 1, tokens, tokens), ("decode", batch, 1, context)):
        pages = -(-held // page)
        table = torch.full((requests, -(-pages // 64) * 64), -1, dtype=torch.int32, device="cuda")
        table[:, :pages] = torch.randperm(requests * pages, device="cuda", generator=g).to(torch.int32).reshape(requests, pages)
        ctx = ctx_for(requests, new, held)
        for name, maps, dim, vdim, mask, extras in variants:
            k2, v2 = rand(requests * pages + 1, kv, page, maps * dim), rand(requests * pages + 1, kv, page, vdim)
            rows = rand(requests * new, heads * maps * dim + 8 * (-(-heads // 8)), scale=0.3)
            q2, gate = rows[:, :heads * maps * dim], rows[:, heads * maps * dim:heads * maps * dim + heads]
            o2 = torch.empty(requests * new, heads * vdim, dtype=torch.bfloat16, device="cuda")
            view = SimpleNamespace(k=k2, v=v2, block_table=table, page_tokens=page, write=False)
            sink = torch.zeros(heads, device="cuda") if extras else None
            lam, eps = (0.4, 1e-5) if maps == 2 else (0.0, 0.0)
            us = _median_us(lambda: kernels.multimap_attention(q2, view, ctx, o2, heads, kv, maps, dim, vdim, dim ** -0.5, lam, eps, 0.5, status,
                                                               mask=mask, sink=sink, gate=None if maps == 2 else gate),
                            repeats=3 if label == "prefill" else 10)
            if label == "prefill":
                seen = sum(visible(mask, p) for p in range(tokens)) if mask else tokens * (tokens + 1) // 2
                flops = 2.0 * heads * (maps * dim + vdim) * seen
                out[f"{name}_prefill"] = {"us": round(us, 1), "visible_pairs": seen, "tflops": round(flops / us / 1e6, 1),
                                          "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
            else:
                seen = visible(mask, context - 1) if mask else context
                mb = batch * seen * kv * (maps * dim + vdim) * 2 / 1e6
                out[f"{name}_decode"] = {"us": round(us, 1), "visible_keys": seen, "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                         "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    # recurrent mixers: a decay per key channel, a decay per head, and the fixed decay of the linear attention.  The
    # first two are 32-bit arithmetic on CUDA cores (the decays enter the recurrence in 32-bit), so beside the bytes
    # their entries carry the share of the cores' nominal rate: SMs x 128 lanes x 2 x the highest SM clock; a token
    # costs 3 operations per element of the state (a S + (c k) v, then q S), counted as 2 FLOPs each.
    try:
        top_mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits", "-i", "0"],
                                       capture_output=True, text=True, timeout=20).stdout.split()[0])
    except (OSError, ValueError, IndexError, subprocess.SubprocessError):
        top_mhz = 1965.0
    fp32_tflops = torch.cuda.get_device_properties(0).multi_processor_count * 128 * 2 * top_mhz / 1e6
    out["fp32_cuda_core_tflops_nominal"] = round(fp32_tflops, 1)

    def of_cores(elements_tokens, us):
        return round(3 * 2.0 * elements_tokens / us / 1e6 / fp32_tflops, 3)
    sh, sd, sv = z["state_heads"], z["state_dim"], z["state_vdim"]
    mh, mv, mn, mg = z["ssm_heads"], z["ssm_vdim"], z["ssm_state"], z["ssm_groups"]
    for label, requests, new in (("prefill", 1, tokens), ("decode", batch, 1)):
        ctx = ctx_for(requests, new, new)
        n = requests * new
        slots = torch.arange(requests, dtype=torch.int32, device="cuda")
        rows = rand(n, sh * (2 * sd + sv), scale=0.5)
        zed = rand(n, sh * sd, dtype=torch.float32)
        bias = torch.full((sh * sd,), 3.0, device="cuda")
        state = SimpleNamespace(buffer=torch.zeros(requests, sh, sd, sv, device="cuda"), slots=slots)
        o = torch.empty(n, sh * sv, device="cuda")
        us = _median_us(lambda: kernels.gated_scan(rows[:, :sh * sd], rows[:, sh * sd:2 * sh * sd], rows[:, 2 * sh * sd:], zed, bias, ctx, state, o,
                                                   sh, sh, sd, sv, status, tau=z["tau"], q_scale=sd ** -0.5), repeats=3 if new > 1 else 10)
        mb = (n * sh * ((2 * sd + sv) * 2 + sd * 4 + sv * 4) + 2 * requests * sh * sd * sv * 4) / 1e6
        out[f"channel_decay_scan_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                              "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                              "tflops": round(4.0 * n * sh * sd * sv / us / 1e6, 2),
                                              "of_nominal_fp32_cores": of_cores(n * sh * sd * sv, us)}
        rows_l = rand(n, sh * (2 * sd + 2 * sv), scale=0.5)
        decay = torch.full((sh,), 0.99, device="cuda")
        state_l = SimpleNamespace(buffer=torch.zeros(requests, sh, sd, sv, device="cuda"), slots=slots)
        us = _median_us(lambda: kernels.decay_attention(rows_l, ctx, state_l, decay, o, sh, sd, sv, True, status), repeats=3 if new > 1 else 10)
        mb = (n * sh * ((2 * sd + sv) * 2 + sv * 4) + 2 * requests * sh * sd * sv * 4) / 1e6
        out[f"fixed_decay_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                       "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                       "tflops": round(4.0 * n * sh * sd * sv / us / 1e6, 2)}
        inner, channels = mh * mv, mh * mv + 2 * mg * mn
        proj = rand(n, inner + channels + 8 * (-(-mh // 8)), scale=0.5)
        conv = torch.empty(n, channels, dtype=torch.bfloat16, device="cuda")
        taps = z["taps"]
        conv_state = SimpleNamespace(buffer=torch.zeros(requests, taps - 1, channels, device="cuda"), slots=slots)
        weight, cbias = rand(channels, taps, scale=0.5, dtype=torch.float32), rand(channels, scale=0.1, dtype=torch.float32)
        us = _median_us(lambda: kernels.causal_conv(proj[:, inner:inner + channels], weight, cbias, conv, ctx, conv_state, status, silu=True))
        mb = (2 * n * channels * 2 + 2 * requests * (taps - 1) * channels * 4) / 1e6
        out[f"short_conv_{label}"] = {"us": round(us, 1), "mb": round(mb, 2), "gbs": round(mb / us * 1e3),
                                      "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
        ssm_state = SimpleNamespace(buffer=torch.zeros(requests, mh, mn, mv, device="cuda"), slots=slots)
        y = torch.empty(n, inner, device="cuda")
        dt_bias, a_log, skip = torch.zeros(mh, device="cuda"), torch.full((mh,), -2.0, device="cuda"), torch.ones(mh, device="cuda")
        us = _median_us(lambda: kernels.gated_scan(conv[:, inner + mg * mn:], conv[:, inner:inner + mg * mn], conv[:, :inner],
                                                   proj[:, inner + channels:inner + channels + mh], dt_bias, ctx, ssm_state, y, mh, mg, mn, mv,
                                                   status, per_head=True, a_log=a_log, skip=skip), repeats=3 if new > 1 else 10)
        mb = (n * (channels * 2 + mh * 2 + inner * 4) + 2 * requests * mh * mn * mv * 4) / 1e6
        out[f"head_decay_scan_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                           "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                           "tflops": round(4.0 * n * mh * mn * mv / us / 1e6, 2),
                                           "of_nominal_fp32_cores": of_cores(n * mh * mn * mv, us)}
        gated = torch.empty(n, inner, dtype=torch.bfloat16, device="cuda")
        gain = torch.ones(inner, device="cuda")
        us = _median_us(lambda: kernels.gated_group_norm(y, proj[:, :inner], gain, gated, 1e-5, groups=z["norm_groups"], gate_first=True, silu=True))
        mb = n * inner * (4 + 2 + 2) / 1e6
        out[f"gated_group_norm_{label}"] = {"us": round(us, 1), "mb": round(mb, 2), "gbs": round(mb / us * 1e3),
                                            "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    assert int(status.item()) == 0
    return out


def timed_rarutar(args) -> dict:
    """``--only rarutar``: prefill and decode throughput of Rarutar at ``--shape 1b|0.3b`` (random weights, ``--layers``
    layers, 4 if not given) beside Letanex at equal size, through the same runner, and the kernels of both alone."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    shape = args.shape if args.shape in RARUTAR_SHAPES else "1b"
    layers = args.layers or 4
    peak = peaks()
    rarutar_dir, letanex_dir = rarutar_folders(shape, layers)
    prompt_len = args.prompt_len
    result = {"impl": "ours", "only": "rarutar", "shape": shape, "layers": layers, "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": args.tokens, "decode_batch": args.batch, "decode_prompt_len": prompt_len, "steps": args.steps,
              "peaks": {"bf16_tflops": peak["bf16_tflops"], "hbm_gbs": peak["hbm_gbs"], "source": peak.get("source", "measured")}}
    for tag, folder in (("rarutar", rarutar_dir), ("letanex", letanex_dir)):
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        slots = max(64, args.batch)
        pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + args.tokens // 16 + 16
        runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)
        rng = np.random.default_rng(0)
        ms = timed_prefill(runner, args.tokens, rng)
        decode = timed_decode(runner, args.batch, prompt_len, args.steps, args.warmup, rng)
        result[tag] = {"weights_mb": round((folder / "model.safetensors").stat().st_size / 1e6, 1), "prefill_ms": round(ms, 3),
                       "prefill_tokens_per_s": round(args.tokens / ms * 1000),
                       "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tokens_per_s"]),
                       "decode_launches_per_step": decode["launches_per_step"]}
        del runner, model
        torch.cuda.empty_cache()
    result["kernels"] = timed_rarutar_kernels(shape, args.tokens, max(args.batch, 64), 2048, peak)
    return result


VURIPEL_SHAPES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, softcap=30.0, win_dim=64, win_vdim=128, rotated=32, window=1024,
               keep_first=4, win_softcap=50.0, mem_heads=16, mem_dim=128, mem_vdim=128, gate_cap=15.0, ff=4096, experts=32, top=4,
               groups=(4, 2), expert_ff=1024, shared_ff=2048, side_dim=64, vocab=32768),
    "0.3b": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, softcap=30.0, win_dim=64, win_vdim=128, rotated=32, window=512,
                 keep_first=4, win_softcap=50.0, mem_heads=8, mem_dim=128, mem_vdim=128, gate_cap=15.0, ff=2048, experts=16, top=4,
                 groups=(4, 2), expert_ff=512, shared_ff=1024, side_dim=32, vocab=32768),
}


def vuripel_folders(shape: str, layers: int):
    """(Vuripel folder, Rarutar folder of equal size), random weights, written once.  Vuripel's layers in fours: a matrix
    memory with a dense feed-forward, attention over everything (sink, gate, capped scores) with routed experts, attention over
    a window that keeps the first positions with a dense feed-forward, the same with routed experts; the experts' active
    weights equal the dense feed-forward's (top x 2 matrices of expert_ff + 2 of shared_ff = 3 of ff); a per-layer token input
    everywhere; all layers form one pass of a loop, so the pass's vector is added.  Rarutar beside it is ``--only rarutar``'s
    model at the same shape (width, feed-forward, vocabulary, attention heads and window alike)."""
    from sprout_lm_b200 import parse_config, write_random_model
    z = VURIPEL_SHAPES[shape]
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    memory = {"heads": z["mem_heads"], "dim": z["mem_dim"], "vdim": z["mem_vdim"], "gate_cap": z["gate_cap"]}
    full = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5, "softcap": z["softcap"]}
    windowed = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["win_dim"], "vdim": z["win_vdim"], "scale": z["win_dim"] ** -0.5,
                "softcap": z["win_softcap"], "mask": {"size": z["window"], "keep_first": z["keep_first"]},
                "rot": {"base": 1000000.0, "dims": z["rotated"]}}
    kinds = [("mlstm", memory, dense), ("attention", full, moe), ("attention_2", windowed, dense), ("attention_2", windowed, moe)]
    raw = {"architecture": "Vuripel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "token_side": {"dim": z["side_dim"]},
           "loop": {"start": 0, "stop": layers, "times": 1}, "max_positions": 16384,
           "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": kinds[i % 4][2]} for i in range(layers)]}
    folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}_vuripel_{shape}_L{layers}"
    if not (folder / "complete").exists():
        print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
        write_random_model(folder, parse_config(raw), seed=0)
        (folder / "complete").write_text("ok")
    return folder, rarutar_folders(shape if shape in RARUTAR_SHAPES else "1b", layers)[0]


def timed_vuripel_kernels(shape: str, tokens: int, batch: int, context: int, peak: dict) -> dict:
    """Vuripel's kernels alone beside the like kernels of the closest models at equal sizes.  Attention over everything with
    capped scores, a sink and a gate beside Rarutar's attention with a sink and a gate (chunks as long as the prompt), and
    attention over a window that keeps the first positions beside Rarutar's windowed attention: one prompt of ``tokens`` tokens
    (executed FLOPs of the visible keys against the measured bf16 rate) and ``batch`` single tokens with ``context`` keys held
    (bytes of the visible keys against the measured copy rate).  The matrix memory's scan (decays ready-made, a column of ones)
    beside the scan with a decay per head at the same sizes (bytes against the copy rate, 32-bit operations against the CUDA
    cores' nominal rate), its gates and its output kernel beside the gated group norm.  The experts without gates beside the
    gated experts of Letanex at the same sizes, the router with groups beside the one without, the gated gelu beside the clamped
    gated activation, and the per-layer token input (one launch for few tokens; five for a prompt)."""
    import torch
    from types import SimpleNamespace
    from sprout_lm_b200 import kernels
    z = VURIPEL_SHAPES[shape]
    page = 16
    g = torch.Generator(device="cuda").manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}

    def rand(*shape_, scale=1.0, dtype=torch.bfloat16):
        return (torch.randn(*shape_, device="cuda", generator=g) * scale).to(dtype)

    def ctx_for(requests, new, held):
        return SimpleNamespace(seq_of_token=torch.arange(requests, dtype=torch.int32, device="cuda").repeat_interleave(new),
                               positions=(torch.arange(new, dtype=torch.int32, device="cuda") + (held - new)).repeat(requests),
                               q_start=(torch.arange(requests + 1, dtype=torch.int32, device="cuda") * new),
                               context_lens=torch.full((requests,), held, dtype=torch.int32, device="cuda"), max_q_len=new,
                               max_context=held, planned_context=0, num_seqs=requests, num_tokens=requests * new,
                               token_ids=torch.randint(0, z["vocab"], (requests * new,), dtype=torch.int32, device="cuda", generator=g))

    def visible(mask, position):
        if mask is None:
            return position + 1
        kind, size = mask[0], mask[1]
        keep = mask[2] if len(mask) > 2 else 0
        if kind == "chunk":
            return position % size + 1
        seen = min(position + 1, size)
        return seen + min(keep, max(0, position + 1 - size))

    heads, kv = z["heads"], z["kv_heads"]
    variants = (("capped_sink_gate", z["dim"], z["vdim"], None, True, z["softcap"]),
                ("rarutar_sink_gate", z["dim"], z["vdim"], ("chunk", max(tokens, context)), True, 0.0),
                ("capped_window_kept", z["win_dim"], z["win_vdim"], ("window", z["window"], z["keep_first"]), False, z["win_softcap"]),
                ("rarutar_window", z["win_dim"], z["win_vdim"], ("window", z["window"]), False, 0.0))
    for label, requests, new, held in (("prefill", 1, tokens, tokens), ("decode", batch, 1, context)):
        pages = -(-held // page)
        table = torch.full((requests, -(-pages // 64) * 64), -1, dtype=torch.int32, device="cuda")
        table[:, :pages] = torch.randperm(requests * pages, device="cuda", generator=g).to(torch.int32).reshape(requests, pages)
        ctx = ctx_for(requests, new, held)
        for name, dim, vdim, mask, extras, cap in variants:
            k2, v2 = rand(requests * pages + 1, kv, page, dim), rand(requests * pages + 1, kv, page, vdim)
            rows = rand(requests * new, heads * dim + 8 * (-(-heads // 8)), scale=0.3)
            q2, gate = rows[:, :heads * dim], rows[:, heads * dim:heads * dim + heads]
            o2 = torch.empty(requests * new, heads * vdim, dtype=torch.bfloat16, device="cuda")
            view = SimpleNamespace(k=k2, v=v2, block_table=table, page_tokens=page, write=False)
            sink = torch.zeros(heads, device="cuda") if extras else None
            us = _median_us(lambda: kernels.multimap_attention(q2, view, ctx, o2, heads, kv, 1, dim, vdim, dim ** -0.5, 0.0, 0.0, 1.0, status,
                                                               mask=mask, sink=sink, gate=gate if extras or mask else None, softcap=cap),
                            repeats=3 if label == "prefill" else 10)
            if label == "prefill":
                seen = sum(visible(mask, p) for p in range(tokens))
                flops = 2.0 * heads * (dim + vdim) * seen
                out[f"{name}_prefill"] = {"us": round(us, 1), "visible_pairs": seen, "tflops": round(flops / us / 1e6, 1),
                                          "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3)}
            else:
                seen = visible(mask, context - 1)
                mb = batch * seen * kv * (dim + vdim) * 2 / 1e6
                out[f"{name}_decode"] = {"us": round(us, 1), "visible_keys": seen, "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                         "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    try:
        top_mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits", "-i", "0"],
                                       capture_output=True, text=True, timeout=20).stdout.split()[0])
    except (OSError, ValueError, IndexError, subprocess.SubprocessError):
        top_mhz = 1965.0
    fp32_tflops = torch.cuda.get_device_properties(0).multi_processor_count * 128 * 2 * top_mhz / 1e6
    out["fp32_cuda_core_tflops_nominal"] = round(fp32_tflops, 1)
    mh, md, mv = z["mem_heads"], z["mem_dim"], z["mem_vdim"]
    cols = (mv + 1 + 3) // 4 * 4
    width = z["width"]
    for label, requests, new in (("prefill", 1, tokens), ("decode", batch, 1)):
        ctx = ctx_for(requests, new, new)
        n = requests * new
        slots = torch.arange(requests, dtype=torch.int32, device="cuda")
        rows = rand(n, mh * (2 * md + 2 * mv) + 2 * mh, scale=0.5, dtype=torch.float32)
        at = mh * (2 * md + 2 * mv)
        tops = torch.zeros(requests, mh, device="cuda")
        bias = torch.zeros(mh, device="cuda")
        us = _median_us(lambda: kernels.exp_gates(rows[:, at:at + mh], rows[:, at + mh:at + 2 * mh], bias, bias, z["gate_cap"], ctx, tops, slots, status))
        out[f"exp_gates_{label}"] = {"us": round(us, 1), "mb": round(n * mh * 5 * 4 / 1e6, 3)}
        a, c, m = kernels.exp_gates(rows[:, at:at + mh], rows[:, at + mh:at + 2 * mh], bias, bias, z["gate_cap"], ctx, tops, slots, status)
        state = SimpleNamespace(buffer=torch.zeros(requests, mh, md, cols, device="cuda"), slots=slots)
        o = torch.empty(n, mh * cols, device="cuda")
        us = _median_us(lambda: kernels.gated_scan(rows[:, :mh * md], rows[:, mh * md:2 * mh * md], rows[:, 2 * mh * md:2 * mh * md + mh * mv], None,
                                                   None, ctx, state, o, mh, mh, md, cols, status, q_scale=md ** -0.5, given=(a, c), ones_col=True),
                        repeats=3 if new > 1 else 10)
        mb = (n * mh * ((2 * md + mv) * 4 + 2 * 4 + cols * 4) + 2 * requests * mh * md * cols * 4) / 1e6
        out[f"memory_scan_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                       "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                       "of_nominal_fp32_cores": round(6.0 * n * mh * md * cols / us / 1e6 / fp32_tflops, 3)}
        # the scan with a decay per head that the kernel makes itself, at the same sizes (bfloat16 projections)
        proj = rand(n, mh * (2 * md + mv) + 8 * (-(-mh // 8)), scale=0.5)
        state_h = SimpleNamespace(buffer=torch.zeros(requests, mh, md, mv, device="cuda"), slots=slots)
        y = torch.empty(n, mh * mv, device="cuda")
        zero, a_log = torch.zeros(mh, device="cuda"), torch.full((mh,), -2.0, device="cuda")
        us = _median_us(lambda: kernels.gated_scan(proj[:, :mh * md], proj[:, mh * md:2 * mh * md], proj[:, 2 * mh * md:2 * mh * md + mh * mv],
                                                   proj[:, mh * (2 * md + mv):mh * (2 * md + mv) + mh], zero, ctx, state_h, y, mh, mh, md, mv, status,
                                                   per_head=True, a_log=a_log), repeats=3 if new > 1 else 10)
        mb = (n * mh * ((2 * md + mv) * 2 + 2 + mv * 4) + 2 * requests * mh * md * mv * 4) / 1e6
        out[f"head_decay_scan_{label}"] = {"us": round(us, 1), "mb": round(mb, 1), "gbs": round(mb / us * 1e3),
                                           "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3),
                                           "of_nominal_fp32_cores": round(6.0 * n * mh * md * mv / us / 1e6 / fp32_tflops, 3)}
        gated = torch.empty(n, mh * mv, dtype=torch.bfloat16, device="cuda")
        gain = torch.ones(mh * mv, device="cuda")
        us = _median_us(lambda: kernels.exp_memory_out(o, m, rows[:, mh * (2 * md + mv):at], gain, gated, mh, mv, 1e-5))
        mb = n * mh * (cols * 4 + mv * 4 + mv * 2) / 1e6
        out[f"memory_out_{label}"] = {"us": round(us, 1), "mb": round(mb, 2), "gbs": round(mb / us * 1e3),
                                      "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
        us = _median_us(lambda: kernels.gated_group_norm(y, proj[:, :mh * mv], gain, gated, 1e-5, groups=mh, gate_first=False, silu=True))
        mb = n * mh * mv * (4 + 2 + 2) / 1e6
        out[f"gated_group_norm_{label}"] = {"us": round(us, 1), "mb": round(mb, 2), "gbs": round(mb / us * 1e3),
                                            "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
        # routed experts: without gates (one matrix up) beside with gates (two), at the same sizes and routing
        experts, top, ff = z["experts"], z["top"], z["expert_ff"]
        h = rand(n, width, scale=0.5)
        router = rand(experts, width, scale=0.05, dtype=torch.float32)
        ids = torch.empty((n, top), dtype=torch.int32, device="cuda")
        weights = torch.empty((n, top), dtype=torch.float32, device="cuda")
        counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
        offsets = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
        order = torch.empty(n * top, dtype=torch.int32, device="cuda")
        place_of = torch.empty(n * top, dtype=torch.int32, device="cuda")
        for name, groups in (("grouped", z["groups"]), ("free", None)):
            def route():
                kernels.moe_route(h, router, None, ids, weights, counts, experts, top, 1.0, groups=groups, renormalize=False)
                kernels.moe_arrange(ids, counts, offsets, order, place_of, experts)
            out[f"route_{name}_{label}"] = {"us": round(_median_us(route), 1)}
        act = torch.empty((n * top, ff), dtype=torch.bfloat16, device="cuda")
        rows_out = torch.empty((n * top, width), dtype=torch.float32, device="cuda")
        w_down = rand(experts, width, ff, scale=0.02)
        for name, mats, limit in (("plain", 1, 0.0), ("gated", 2, 7.0)):
            w_up = rand(experts, mats * ff, width, scale=0.02)
            us = _median_us(lambda: kernels.moe_experts(h, order, offsets, w_up, w_down, act, rows_out, experts, top, limit, 1.702),
                            repeats=3 if new > 1 else 10)
            flops = 2.0 * n * top * width * ff * (mats + 1)
            touched = min(experts, n * top)
            mb = touched * (mats + 1) * ff * width * 2 / 1e6
            out[f"experts_{name}_{label}"] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                                              "of_measured_bf16": round(flops / us / 1e6 / peak["bf16_tflops"], 3), "weights_mb": round(mb, 1),
                                              "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
            del w_up
        # activations of the dense feed-forward
        gate_up = rand(n, 2 * z["ff"], scale=1.0)
        dense_act = torch.empty((n, z["ff"]), dtype=torch.bfloat16, device="cuda")
        mb = n * z["ff"] * 3 * 2 / 1e6
        for name, call in (("gated_gelu", lambda: kernels.unit_act(gate_up, dense_act, "gelu_tanh", gated=True)),
                           ("clamped_glu", lambda: kernels.glu_clamped(gate_up, dense_act, 7.0, 1.702))):
            us = _median_us(call)
            out[f"{name}_{label}"] = {"us": round(us, 1), "mb": round(mb, 2), "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
        # the per-layer token input
        from sprout_lm_b200.config.specs import PartSpec
        from sprout_lm_b200.parts import Runtime, WeightSource, build_part
        side = build_part("side_input", PartSpec("gated_token_row", {"hidden_size": width, "vocab_size": z["vocab"], "dim": z["side_dim"],
                                                                     "first": z["side_dim"], "columns": 4 * z["side_dim"], "eps": 1e-5,
                                                                     "declares_table": True}), "l1.")
        tensors = {"side.embed": rand(z["vocab"], 4 * z["side_dim"]).cpu(), "l1.side.gate": rand(z["side_dim"], width, scale=0.02).cpu(),
                   "l1.side.proj": rand(width, z["side_dim"], scale=0.02).cpu(), "l1.side.norm": torch.ones(width)}
        side.load(WeightSource(lambda key: tensors[key], Runtime("cuda:0", torch.bfloat16)))
        stream = rand(min(n, 32) if new == 1 else n, width, dtype=torch.float32)
        side_ctx = SimpleNamespace(token_ids=ctx.token_ids[:stream.shape[0]])
        us = _median_us(lambda: side.forward(stream, side_ctx))
        mb = (stream.shape[0] * width * 8 + 2 * z["side_dim"] * width * 2) / 1e6
        out[f"token_input_{label}"] = {"us": round(us, 1), "tokens": stream.shape[0], "mb": round(mb, 2),
                                       "of_measured_copy": round(mb / us * 1e3 / peak["hbm_gbs"], 3)}
    assert int(status.item()) == 0
    return out


def timed_vuripel(args) -> dict:
    """``--only vuripel``: prefill and decode throughput of Vuripel at ``--shape 1b|0.3b`` (random weights, ``--layers`` layers,
    4 if not given) beside Rarutar at equal size, through the same runner, and the kernels of both alone."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    shape = args.shape if args.shape in VURIPEL_SHAPES else "1b"
    layers = args.layers or 4
    peak = peaks()
    vuripel_dir, rarutar_dir = vuripel_folders(shape, layers)
    prompt_len = args.prompt_len
    result = {"impl": "ours", "only": "vuripel", "shape": shape, "layers": layers, "dtype": "bf16", "data": "synthetic",
              "prefill_tokens": args.tokens, "decode_batch": args.batch, "decode_prompt_len": prompt_len, "steps": args.steps,
              "peaks": {"bf16_tflops": peak["bf16_tflops"], "hbm_gbs": peak["hbm_gbs"], "source": peak.get("source", "measured")}}
    for tag, folder in (("vuripel", vuripel_dir), ("rarutar", rarutar_dir)):
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        slots = max(64, args.batch)
        pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + args.tokens // 16 + 16
        runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)
        rng = np.random.default_rng(0)
        ms = timed_prefill(runner, args.tokens, rng)
        decode = timed_decode(runner, args.batch, prompt_len, args.steps, args.warmup, rng)
        result[tag] = {"weights_mb": round((folder / "model.safetensors").stat().st_size / 1e6, 1), "prefill_ms": round(ms, 3),
                       "prefill_tokens_per_s": round(args.tokens / ms * 1000),
                       "decode_ms_per_step": round(decode["ms_per_step"], 4), "decode_tokens_per_s": round(decode["tokens_per_s"]),
                       "decode_launches_per_step": decode["launches_per_step"]}
        del runner, model
        torch.cuda.empty_cache()
    result["kernels"] = timed_vuripel_kernels(shape, args.tokens, max(args.batch, 64), 2048, peak)
    return result


def run(args) -> dict:
    import numpy as np
    import torch
    from sprout_lm_b200 import kernels, load_model
    from sprout_lm_b200.cache.storage import cache_bytes_per_token
    from sprout_lm_b200.engine.step import ModelRunner
    kernels.load_library(verbose=True)
    if args.only == "latent":
        return timed_latent(args)
    if args.only == "letanex":
        return timed_letanex(args)
    if args.only == "rarutar":
        return timed_rarutar(args)
    if args.only == "vuripel":
        return timed_vuripel(args)
    if args.only == "attention":
        return timed_attention(args.tokens, args.shape)
    if args.only == "gemm":
        return timed_gemms(args.tokens, args.shape)
    if args.only == "decode-attention":
        return timed_decode_attention(args.shape, args.batch, args.tokens)
    if args.only == "serve":
        return timed_serving(args.shape, args.layers, args.requests, args.workload)
    if args.only == "long-prompt":
        return timed_long_prompt(args.shape, args.layers, args.tokens, args.portion)
    if args.only == "all" and args.shape != "0.5b":
        raise SystemExit("bench.py: the full line is measured at the 0.5b shape; give --only with another --shape")
    base = SHAPES[args.shape]
    layers = args.layers or base["num_hidden_layers"]
    batch, prompt_len, context = args.batch, 512, base["max_position_embeddings"]
    if args.prompt_len != 512:
        if args.only != "decode":
            raise SystemExit("bench.py: --prompt-len goes with --only decode (the full line is measured at 512-token prompts)")
        prompt_len = args.prompt_len
        need = prompt_len + args.warmup + args.steps + 8
        while context < need:                     # a longer context than the shape names: said in the line
            context *= 2
    folder = model_folder(layers, args.shape, context)
    model = load_model(folder, dtype="bfloat16", device="cuda:0")
    cfg = dict(base, num_hidden_layers=layers)
    peak = peaks()
    rng = np.random.default_rng(0)
    if prompt_len + args.warmup + args.steps + 8 > context:
        raise SystemExit(f"bench.py: {prompt_len}-token prompts and {args.warmup} + {args.steps} decode steps do not fit the "
                         f"{context}-token context of the benchmark configuration; use at most {context - prompt_len - args.warmup - 8} steps")
    slots = max(64, batch)
    pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + 2048 // 16 + 16
    runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)

    if args.only == "ablate":
        return {"impl": "ours", "only": "ablate", "shape": args.shape, "layers": layers, "batch": batch,
                **ablation(model, batch, prompt_len, min(args.steps, 60), args.warmup)}
    if args.only == "prefill":
        prefill_ms = timed_prefill(runner, 2048, rng, repeats=1)
        return {"impl": "ours", "only": "prefill", "shape": args.shape, "layers": layers, "ms": round(prefill_ms, 4),
                "frac": round(prefill_flops(cfg, 2048) / (prefill_ms / 1000) / (peak["bf16_tflops"] * 1e12), 4)}
    # the clocks are sampled over all timed sections together (a single section of a few
    # milliseconds is shorter than nvidia-smi's sampling period)
    sampler = ClockSampler()
    sampler.start()
    main = timed_decode(runner, batch, prompt_len, args.steps, args.warmup, rng)
    if args.only == "decode":
        sampler.stop()
        step_bytes = weight_bytes(model) + batch * main["mean_context"] * cache_bytes_per_token(model, torch.bfloat16)
        out = {"impl": "ours", "only": "decode", "shape": args.shape, "layers": layers, "batch": batch,
               "ms_per_step": round(main["ms_per_step"], 4), "launches_per_step": main["launches_per_step"],
               "gbs": round(step_bytes / (main["ms_per_step"] / 1000) / 1e9, 1)}
        if prompt_len != 512:
            out.update({"prompt_len": prompt_len, "context": context, "mb_per_step": round(step_bytes / 1e6, 1),
                        "hbm_frac": round(step_bytes / (main["ms_per_step"] / 1000) / 1e9 / peak["hbm_gbs"], 3)})
        phases = kernels.ffn_decode_phase_stamps()       # from a build with SPROUT_BUILD_FLAGS=-DFFN_STAMPS
        if phases:
            out["ffn_decode_phases_us"] = {k: {n: round(v, 2) for n, v in d.items()} for k, d in phases.items()}
        phases = kernels.attention_decode_phase_stamps() # from a build with SPROUT_BUILD_FLAGS=-DATTN_STAMPS
        if phases:
            out["attention_decode_phases_us"] = {n: round(v, 2) for n, v in phases.items()}
        timeline = kernels.decode_timeline()             # from a build with SPROUT_BUILD_FLAGS=-DSPROUT_TIMELINE
        if timeline:
            out["last_layer_timeline_us"] = {k: {n: round(v, 2) for n, v in d.items()} for k, d in timeline.items()}
        return out
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(timed_decode(runner, b, prompt_len, args.steps, args.warmup, rng)["tokens_per_s"], 1)
    prefill_ms = timed_prefill(runner, 2048, rng)
    flops = prefill_flops(cfg, 2048)
    e2e = timed_e2e(model, batch, prompt_len, args.steps, args.warmup, rng)
    clocks = sampler.stop()

    step_bytes = weight_bytes(model) + batch * main["mean_context"] * cache_bytes_per_token(model, torch.bfloat16)
    achieved = step_bytes / (main["ms_per_step"] / 1000) / 1e9
    return {
        "metric": "decode tokens/s, Qwen2.5-0.5B shape, batch 8 (also batch 1/64 and prefill of 2,048 tokens)",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "impl": "ours",
        "config": {"model": "Qwen2.5-0.5B shape", "layers": layers, "layers_of_model": CONFIG_05B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": 64, "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied_head": True, "global_batch": batch, "prompt_len": prompt_len, "seq_len": context,
                   "page_tokens": 16, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 988 MB per step)"},
        "e2e": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main["launches_per_step"] * args.steps),
        "prefill": {"value": round(2048 / (prefill_ms / 1000), 1), "tokens": 2048, "ms": round(prefill_ms, 4),
                    "frac": round(flops / (prefill_ms / 1000) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points,
        "clocks": clocks,
    }


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--portion", type=int, default=4096, help="with --only long-prompt: tokens of a step (--tokens: of the whole prompt)")
    parser.add_argument("--prompt-len", type=int, default=512, help="with --only decode: tokens of every request's prompt (the context grows to hold it)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--only", choices=["all", "decode", "prefill", "ablate", "attention", "decode-attention", "gemm", "serve", "long-prompt", "latent", "letanex", "rarutar", "vuripel"], default="all",
                        help="measure one part only (for profiling captures); the JSON line then holds that part")
    parser.add_argument("--shape", choices=sorted(set(SHAPES) | set(LATENT_SHAPES) | set(LETANEX_SHAPES) | set(RARUTAR_SHAPES)), default="0.5b", help="with --only: the model's sizes")
    parser.add_argument("--requests", type=int, default=64, help="with --only serve: requests of the workload")
    parser.add_argument("--workload", choices=["mixed", "shared-prefix"], default="mixed",
                        help="with --only serve: mixed prompt lengths, or long prompts that share a prefix in a pool too small for all")
    parser.add_argument("--tokens", type=int, default=2048, help="with --only attention or gemm: tokens of the one request; with decode-attention: the context of each request")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    result = run(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
