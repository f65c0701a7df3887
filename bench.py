#!/usr/bin/env python3
"""Benchmark: decode throughput of GPT-2 small (random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests whose contexts end at the model's
context length (1024).  ``value`` is decoded tokens per second, timed on the device with CUDA
events around exactly K steps; ``e2e`` is the same metric through the Python entry point
(``LLM.generate``): token ids from the host in, sampled token ids to the host out, every
step.  The same line carries the prefill of 2,048 tokens (two prompts of 1024), the decode
step's memory roofline, and under ``points``: decode throughput at batch 1 and 64; the decode
workload as the target states it (512-token prompts, 256 greedy tokens, pages of 16, through
the scheduler) at batch 1, 8 and 64 with its fraction of the HBM roofline; a mixed serving
workload; the 32-bit path's decode and prompt steps.  ``reference_tokens`` says whether this
engine's 32-bit path and the reference's choose the same greedy tokens from the same weights.
``--model medium`` and ``--model xl`` run those sizes with their scheduler workloads (32 mixed
requests with prompts in portions of 512; 64 requests side by side at temperature 1.0).

The reference's counterparts are ``engine/bench/bench_batch.c:24-122`` (batched decode:
prefill untimed, one warm-up step, then timed steps) and ``engine/bench/bench.c`` (prefill).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The headline configuration: GPT-2 small.  Layers may be reduced with --layers where time or
# memory needs it; the line then names both numbers.
GPT2_SMALL = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12,
              "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024, "activation_function": "gelu_new",
              "layer_norm_epsilon": 1e-5, "tie_word_embeddings": True}
# The other GPT-2 sizes, for runs beside the headline one (--model).
SIZES = {"small": {}, "medium": {"n_layer": 24, "n_embd": 1024, "n_head": 16, "n_inner": 4096},
         "large": {"n_layer": 36, "n_embd": 1280, "n_head": 20, "n_inner": 5120},
         "xl": {"n_layer": 48, "n_embd": 1600, "n_head": 25, "n_inner": 6400}}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in the line)")
    parser.add_argument("--model", default="small", choices=sorted(SIZES), help="GPT-2 size; the headline run is small")
    parser.add_argument("--plain-kernels", action="store_true")
    parser.add_argument("--no-extras", action="store_true", help="skip prefill, batch 1/64 and the end-to-end run")
    parser.add_argument("--page-size", type=int, default=None, help="tokens per cache page (the engine's default if not given)")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run the 2,048-token prompt step alone and print its own line (for profiling)")
    parser.add_argument("--kernels", action="store_true",
                        help="time single kernels (matrix products at forced tile widths, prompt attention) back to "
                             "back in a replayed graph and print one line each: the tables of profiles/ come from this")
    parser.add_argument("--tokens-out", default=None,
                        help="(--impl reference) write the greedy tokens of the fixed check workload to this file "
                             "and print nothing else")
    return parser.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            out = dict(FALLBACK_PEAKS)
            for key in out:
                if isinstance(raw.get(key), (int, float)):
                    out[key] = float(raw[key])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.process = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.process = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                             "-i", "0", "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        self.process.wait()
        self.file.flush()
        self.file.seek(0)
        clocks, top, reasons = [], None, set()
        for line in self.file.read().splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 6:
                continue
            try:
                clocks.append(float(cells[0]))
                top = float(cells[1])
            except ValueError:
                continue
            for name, cell in zip(self.NAMES, cells[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": top,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(config: dict, dtype_bytes: int):
    e, i, v, layers = config["n_embd"], config["n_inner"], config["vocab_size"], config["n_layer"]
    matrix_params = layers * (e * 3 * e + e * e + 2 * e * i)
    vector_params = layers * (3 * e + e + i + e + 4 * e) + 2 * e
    weight_bytes = (matrix_params + v * e) * dtype_bytes + vector_params * 4      # every weight a decode step uses, once
    kv_bytes_per_token = layers * 2 * e * dtype_bytes
    return matrix_params, weight_bytes, kv_bytes_per_token


def prefill_flops(config: dict, n_prompts: int, length: int, wanted_rows: int) -> float:
    e, v, layers = config["n_embd"], config["vocab_size"], config["n_layer"]
    matrix_params, _, _ = model_numbers(config, 2)
    tokens = n_prompts * length
    gemm = 2.0 * tokens * matrix_params
    attention = layers * n_prompts * 2.0 * length * length * e          # causal half of QK^T and PV
    head = 2.0 * wanted_rows * v * e
    return gemm + attention + head


def make_model_folder(config: dict, folder: str) -> str:
    from mini_llm_b200.config import config_from_dict
    from mini_llm_b200.weights import write_random_model
    return write_random_model(config_from_dict(config), 0, folder, recipe="gpt2", store_dtype="float32")


def decode_run(engine, batch: int, steps: int, warmup: int, context: int, vocab: int):
    """Device-timed decode: ``batch`` requests prefilled so that the timed steps end at
    ``context`` tokens.  Token ids are fixed in advance (nothing is read back inside the timed
    region); every step samples greedily on the device.  Returns (ms per step, launches per
    step, mean cached tokens per request during the timed steps)."""
    import numpy as np
    import torch
    from mini_llm_b200.engine import SamplingParams, StepEntry

    rng = np.random.default_rng(1234)
    prompt_len = context - steps - warmup
    if prompt_len < 1:
        raise SystemExit(f"--steps + --warmup must stay below the context length {context}")
    slots = [engine.open_request() for _ in range(batch)]
    for slot in slots:                                   # untimed prefill, one request per step
        engine.step([StepEntry(slot, rng.integers(0, vocab, prompt_len).tolist(), [])])
    feed = rng.integers(0, vocab, (steps + warmup, batch))
    greedy = [SamplingParams() for _ in range(batch)]

    def one(index):
        engine.step([StepEntry(slot, [int(feed[index, b])], [0]) for b, slot in enumerate(slots)], greedy)

    for index in range(warmup):
        one(index)
    torch.cuda.synchronize()
    launches_before = engine.kernels.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for index in range(warmup, warmup + steps):
        one(index)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = (engine.kernels.launches - launches_before) / steps
    for slot in slots:
        engine.close_request(slot)
    mean_cached = prompt_len + warmup + (steps - 1) / 2.0
    return ms, launches, mean_cached


def prefill_run(engine, n_prompts: int, length: int, vocab: int, repeats: int = 5, from_idle: bool = False):
    """Milliseconds of one prompt step of ``n_prompts`` x ``length`` tokens.  The steps run one
    behind the other (a step's host work, the filling of its control block, then falls beside
    the step before it on the GPU, as in serving) between two events with a synchronise on
    both sides; the first five steps, which run eagerly and capture the graph, are not timed.
    ``from_idle``: each step alone instead, from an idle GPU, host work included (the median)."""
    import numpy as np
    import torch
    from mini_llm_b200.engine import StepEntry

    rng = np.random.default_rng(99)
    prompts = [rng.integers(0, vocab, length).tolist() for _ in range(n_prompts)]

    def one_step():
        slots = [engine.open_request() for _ in range(n_prompts)]
        engine.step([StepEntry(slot, prompt, [length - 1]) for slot, prompt in zip(slots, prompts)])
        for slot in slots:
            engine.close_request(slot)

    for _ in range(5):
        one_step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if from_idle:
        times = []
        for _ in range(repeats):
            torch.cuda.synchronize()
            start.record()
            one_step()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        return statistics.median(times)
    torch.cuda.synchronize()
    start.record()
    for _ in range(repeats):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeats


def e2e_run(folder, args, context: int, vocab: int):
    """The same decode metric through ``LLM.generate``: prompts go in as host token ids, every
    step uploads its control block from pinned host memory and reads the sampled ids back."""
    import numpy as np
    from mini_llm_b200.generate import LLM

    steps, warmup, batch = args.steps, args.warmup, args.batch
    rng = np.random.default_rng(4321)
    prompt_len = context - steps - warmup
    prompts = [rng.integers(0, vocab, prompt_len).tolist() for _ in range(batch)]
    # every prompt is admitted in the first step, so that all requests decode side by side to the end
    llm = LLM(folder, dtype=args.dtype, max_sessions=batch, cache_tokens=batch * context,
              max_tokens_per_step=batch * context, plain_kernels=args.plain_kernels)
    best = None
    for _ in range(2):                                     # the better of two runs (the host is a shared machine)
        stamps, uploads = [], []

        def on_token(index, token, reason):
            if index == batch - 1:
                stamps.append(time.perf_counter())
                uploads.append(llm.engine.control.last_upload_bytes)

        out = llm.generate(prompts, max_new_tokens=steps + warmup, temperature=0.0, on_token=on_token)
        assert all(len(tokens) == steps + warmup for tokens in out)
        seconds = stamps[-1] - stamps[warmup - 1]              # K steps after the warm-up steps
        if best is None or seconds < best[0]:
            best = (seconds, uploads[len(uploads) // 2])       # and the control block of a decode step, as copied
    seconds, control_bytes = best
    return {"value": batch * steps / seconds, "unit": "tokens/s", "h2d_bytes_per_step": control_bytes,
            "d2h_bytes_per_step": 4 * batch + 4, "ms_per_step": 1000.0 * seconds / steps, "runs": 2}


def serving_run(folder, args, vocab: int):
    """Tokens a second through the scheduler for a mixed workload: 64 requests, prompts of 16 to
    768 tokens, 32 to 256 new tokens each, temperature 0.8 and top-p 0.95, at most 32 live, a
    token budget of 512 per step (prompts in portions beside decoding requests)."""
    import numpy as np
    import torch
    from mini_llm_b200.engine.scheduler import Request
    from mini_llm_b200.generate import LLM

    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, vocab, int(rng.integers(16, 769))).tolist() for _ in range(64)]
    lengths = [int(rng.integers(32, 257)) for _ in range(64)]
    llm = LLM(folder, dtype=args.dtype, max_sessions=32, cache_tokens=24 * 1024, max_tokens_per_step=512,
              max_prefill_chunk=512, plain_kernels=args.plain_kernels)
    # The same 64 requests pass after pass: a step shape with prompt portions is captured as a
    # CUDA graph the second time it is seen, so the first passes run some steps eagerly and pay
    # for captures; the passes go on until one ran every step from a graph or the one kernel
    # (eight at most).  Returns the first pass's and the best pass's tokens a second and the
    # number of passes.
    first, best, passes = 0.0, 0.0, 0
    for _ in range(8):
        requests = [Request(p, n, None, 0.8, 0.95, 100 + i) for i, (p, n) in enumerate(zip(prompts, lengths))]
        before = dict(llm.engine.step_kinds)
        torch.cuda.synchronize()
        start = time.perf_counter()
        for request in requests:
            llm.scheduler.submit(request)
        llm.scheduler.run()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - start
        assert all(r.error is None and len(r.generated) == n for r, n in zip(requests, lengths))
        passes += 1
        rate = sum(lengths) / seconds
        first = first or rate
        best = max(best, rate)
        if all(llm.engine.step_kinds[kind] == before[kind] for kind in ("eager", "captured")):
            break
    return first, best, passes


def scheduled_decode_run(folder, args, batch: int, prompt_len: int, new_tokens: int, page_size: int, context: int,
                         vocab: int, weight_bytes: float, kv_per_token: float, hbm_gbs: float):
    """The decode workload as the target states it: ``batch`` requests, each a prompt of
    ``prompt_len`` uniform ids, ``new_tokens`` greedy tokens through the scheduler
    (``LLM.generate``), pages of ``page_size`` tokens.  The prompts are prefilled outside the
    timing: the clock runs from every request's first token to its last, host tokens out
    every step (the reference's bench_batch times its steps after untimed prefills too,
    engine/bench/bench_batch.c:74-114).  Returns tokens a second and the fraction of the HBM
    roofline at the mean context."""
    import numpy as np
    from mini_llm_b200.generate import LLM

    rng = np.random.default_rng(77 + batch)
    prompts = [rng.integers(0, vocab, prompt_len).tolist() for _ in range(batch)]
    llm = LLM(folder, dtype=args.dtype, page_size=page_size, max_sessions=batch, cache_tokens=batch * context,
              max_tokens_per_step=max(2048, batch * prompt_len), plain_kernels=args.plain_kernels)
    best = None
    for _ in range(2):                                  # the second pass finds its step shapes captured
        stamps = []

        def on_token(index, token, reason):
            if index == batch - 1:
                stamps.append(time.perf_counter())

        out = llm.generate(prompts, max_new_tokens=new_tokens, temperature=0.0, on_token=on_token)
        assert all(len(tokens) == new_tokens for tokens in out)
        seconds = stamps[-1] - stamps[0]                  # new_tokens - 1 decode steps
        best = seconds if best is None else min(best, seconds)
    steps = new_tokens - 1
    mean_context = prompt_len + new_tokens / 2.0
    step_bytes = weight_bytes + batch * mean_context * kv_per_token
    return batch * steps / best, step_bytes / (best / steps) / 1e9 / hbm_gbs


def workload_run(folder, args, vocab: int, context: int, n_requests: int, prompt_range, output_range, live: int,
                 budget: int, chunk: int, temperature: float, top_p: float, page_size: int):
    """A workload through the continuous-batching scheduler: ``n_requests`` requests with
    seeded prompt and output lengths, at most ``live`` at a time, a token budget per step and
    prompts in portions of at most ``chunk`` tokens beside decoding requests.  Returns
    generated tokens a second (wall clock, host tokens in and out) and the scheduler's
    counters."""
    import numpy as np
    import torch
    from mini_llm_b200.engine.scheduler import Request
    from mini_llm_b200.generate import LLM

    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, vocab, int(rng.integers(prompt_range[0], prompt_range[1] + 1))).tolist()
               for _ in range(n_requests)]
    lengths = [int(rng.integers(output_range[0], output_range[1] + 1)) for _ in range(n_requests)]
    llm = LLM(folder, dtype=args.dtype, page_size=page_size, max_sessions=live, cache_tokens=live * context,
              max_tokens_per_step=budget, max_prefill_chunk=chunk, plain_kernels=args.plain_kernels)
    best, stats = 0.0, {}
    for _ in range(2):                                   # the second pass finds its step shapes captured
        requests = [Request(p, n, None, temperature, top_p, 100 + i) for i, (p, n) in enumerate(zip(prompts, lengths))]
        before = dict(llm.scheduler.counters)
        torch.cuda.synchronize()
        start = time.perf_counter()
        for request in requests:
            llm.scheduler.submit(request)
        llm.scheduler.run()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - start
        assert all(r.error is None and len(r.generated) == n for r, n in zip(requests, lengths))
        if sum(lengths) / seconds > best:
            best = sum(lengths) / seconds
            after = llm.scheduler.counters
            steps = after["steps"] - before.get("steps", 0)
            tokens = (after["prefill_tokens"] + after["decode_tokens"] - before.get("prefill_tokens", 0)
                      - before.get("decode_tokens", 0))
            stats = {"steps": steps, "tokens_per_step": tokens / max(1, steps),
                     "preemptions": after["preemptions"] - before.get("preemptions", 0),
                     "pages": llm.engine.cache.groups[0].pool.n_pages}
    return best, stats


CHECK_PROMPT_SEED, CHECK_PROMPT_TOKENS, CHECK_NEW_TOKENS = 2024, 32, 16


def check_prompt(vocab: int):
    import numpy as np
    return np.random.default_rng(CHECK_PROMPT_SEED).integers(0, vocab, CHECK_PROMPT_TOKENS).tolist()


def compare_with_reference(folder, vocab: int) -> dict:
    """Whether the two arms choose the same greedy tokens: the 32-bit path of this engine and
    the reference's 32-bit GPU path, same seeded weights, a prompt of 32 ids and 16 new tokens.
    The reference runs in a process of its own (``--impl reference --tokens-out``)."""
    from mini_llm_b200.generate import generate
    if not os.path.isdir(os.path.join(REFERENCE, "mini_llm")):
        return {"unavailable": "the reference is not installed under baseline/_ref"}
    with tempfile.TemporaryDirectory() as scratch:
        path = os.path.join(scratch, "tokens.json")
        try:
            done = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--tokens-out", path],
                                  capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            return {"unavailable": "the reference did not finish in ten minutes"}
        if done.returncode != 0 or not os.path.isfile(path):
            return {"unavailable": (done.stdout.strip() or done.stderr.strip())[-200:]}
        with open(path) as handle:
            theirs = json.load(handle)["tokens"]
    (mine,) = generate(folder, [check_prompt(vocab)], max_new_tokens=CHECK_NEW_TOKENS, temperature=0.0, dtype="float32",
                       page_size=16, max_sessions=2, cache_tokens=1024)
    same = 0
    while same < len(mine) and mine[same] == theirs[same]:
        same += 1
    return {"agree": same, "of": len(mine)}


def run_ours(args):
    import torch
    from mini_llm_b200.engine import Engine

    config = dict(GPT2_SMALL, **SIZES[args.model])
    layers_of_model = config["n_layer"]
    if args.layers is not None:
        config["n_layer"] = args.layers
    context, vocab = config["n_positions"], config["vocab_size"]
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    peak = peaks()
    with tempfile.TemporaryDirectory() as folder:
        make_model_folder(config, folder)
        engine = Engine(folder, dtype=args.dtype, max_requests=64, cache_tokens=64 * context,
                        max_tokens_per_step=2048, plain_kernels=args.plain_kernels,
                        **({"page_size": args.page_size} if args.page_size else {}))
        _, weight_bytes, kv_per_token = model_numbers(config, dtype_bytes)

        if args.only_prefill:
            prefill_ms = prefill_run(engine, 2, 1024, vocab, repeats=max(1, args.steps))
            idle_ms = prefill_run(engine, 2, 1024, vocab, repeats=max(1, min(args.steps, 20)), from_idle=True)
            print(json.dumps({"metric": "prefill of 2,048 tokens", "ms": prefill_ms, "ms_from_idle": idle_ms,
                              "n_layer": config["n_layer"], "value": 2048 / (prefill_ms * 1e-3), "unit": "tokens/s"}))
            return 0
        sampler = ClockSampler()
        sampler.start()
        ms, launches, mean_cached = decode_run(engine, args.batch, args.steps, args.warmup, context, vocab)
        clocks = sampler.stop()
        step_bytes = weight_bytes + args.batch * mean_cached * kv_per_token
        achieved = step_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": f"decode tokens/s, GPT-2 {args.model}, batch {args.batch}, context {context}", "value": args.batch / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype_bytes == 2 else "fp32",
            "data": "synthetic: seeded random weights (N(0, 0.02)) and uniform random token ids", "impl": "ours",
            "config": {"model": f"gpt2-{args.model}", "n_layer": config["n_layer"], "n_layer_of_model": layers_of_model,
                       "n_embd": config["n_embd"], "n_head": config["n_head"], "n_inner": config["n_inner"],
                       "vocab_size": vocab, "n_positions": context, "global_batch": args.batch, "seq_len": context,
                       "prompt_tokens": context - args.steps - args.warmup, "page_size": engine.page_size,
                       "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + cache per step)",
                       "peaks": peak["source"]},
            "gpu_launches": int(round(launches * args.steps)),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
            "clocks": clocks,
        }
        if not args.no_extras:
            points = {}
            for batch in (1, 64):
                p_ms, _, _ = decode_run(engine, batch, min(args.steps, 64), max(3, min(args.warmup, 8)), context, vocab)
                points[f"decode_b{batch}"] = batch / (p_ms * 1e-3)
            line["points"] = points
            # K steps one behind the other between two events; and one step alone from an idle GPU,
            # which also holds the host's filling of the step's control block
            prefill_ms = prefill_run(engine, 2, 1024, vocab, repeats=32)
            idle_ms = prefill_run(engine, 2, 1024, vocab, repeats=7, from_idle=True)
            flops = prefill_flops(config, 2, 1024, 2)
            peak_flops = (peak["bf16_tflops"] if dtype_bytes == 2 else peak["bf16_tflops"]) * 1e12
            line["prefill"] = {"value": 2048 / (prefill_ms * 1e-3), "tokens": 2048, "ms": prefill_ms,
                               "frac": flops / (prefill_ms * 1e-3) / peak_flops, "flops": flops, "steps": 32,
                               "ms_from_idle": idle_ms}
            line["device"] = engine.device_info()
            del engine
            torch.cuda.empty_cache()
            line["e2e"] = e2e_run(folder, args, context, vocab)
            points = line["points"]
            if args.model == "small" and args.layers is None:
                # the decode workload as stated: 512-token prompts, 256 greedy tokens, pages of 16, through the scheduler
                for batch in (1, 8, 64):
                    value, frac = scheduled_decode_run(folder, args, batch, 512, 256, 16, context, vocab, weight_bytes,
                                                       kv_per_token, peak["hbm_gbs"])
                    points[f"sched_p16_b{batch}"] = value
                    points[f"sched_p16_b{batch}_hbm_frac"] = frac
                first, best, passes = serving_run(folder, args, vocab)
                points["serve_mixed_64"], points["serve_mixed_64_first_pass"], points["serve_mixed_64_passes"] = best, first, passes
                if args.dtype == "bfloat16":
                    # the true 32-bit path: the same decode step and prompt step through the plain kernels
                    plain = Engine(folder, dtype="float32", max_requests=8, cache_tokens=8 * context, max_tokens_per_step=2048)
                    f_ms, _, _ = decode_run(plain, 8, 16, 3, context, vocab)
                    points["decode_b8_float32"] = 8 / (f_ms * 1e-3)
                    points["prefill_2048_float32"] = 2048 / (prefill_run(plain, 2, 1024, vocab, repeats=2) * 1e-3)
                    del plain
                    torch.cuda.empty_cache()
                    line["reference_tokens"] = compare_with_reference(folder, vocab)
            elif args.model == "medium":
                # 32 requests, prompts of 16 to 768 tokens, 32 to 256 new tokens, prompts in portions of 512
                value, stats = workload_run(folder, args, vocab, context, 32, (16, 768), (32, 256), 32, 512, 512, 0.0, 1.0, 16)
                points["sched_medium_32"] = value
                points.update({f"sched_medium_32_{k}": v for k, v in stats.items()})
            elif args.model == "xl":
                # 64 requests side by side, 256-token prompts and 768 new tokens each, temperature 1.0, pages of 16
                value, stats = workload_run(folder, args, vocab, context, 64, (256, 256), (768, 768), 64, 2048, 2048, 1.0,
                                            1.0, 16)
                points["sched_xl_64"] = value
                points.update({f"sched_xl_64_{k}": v for k, v in stats.items()})
    print(json.dumps(line))
    return 0


REFERENCE = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def build_reference_library(target: str) -> str | None:
    """The reference's ``make gpu-lib`` (Makefile:165-180 of WillyBruhn/mini_llm) with its
    sources unchanged and only the target architecture replaced (it names sm_86 and sm_61)."""
    import glob
    import shutil
    engine = os.path.join(REFERENCE, "engine")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isdir(engine) or not os.path.isfile(nvcc):
        return "the reference's engine sources or nvcc are missing"
    pic = os.path.join(REFERENCE, "build", "pic")
    os.makedirs(pic, exist_ok=True)
    include = ["-I" + os.path.join(engine, "include"), "-I" + os.path.join(engine, "tests")]
    objects = []
    for source in sorted(glob.glob(os.path.join(engine, "src", "*.c"))):
        obj = os.path.join(pic, os.path.basename(source)[:-2] + ".o")
        done = subprocess.run(["gcc", "-O2", "-std=c11", *include, "-fPIC", "-c", "-o", obj, source], capture_output=True)
        if done.returncode != 0:
            return "gcc failed on the reference's sources"
        objects.append(obj)
    done = subprocess.run([nvcc, "-O2", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", *include, "-Xcompiler",
                           "-fPIC", "-shared", "-o", target, *sorted(glob.glob(os.path.join(engine, "src", "*.cu"))),
                           *objects, "-lm"], capture_output=True)
    return None if done.returncode == 0 else "nvcc failed on the reference's sources"


def export_reference_weights(config: dict, folder: str) -> None:
    """The same seeded random weights as our arm, in the reference's format: one raw
    little-endian fp32 file per tensor, named ``transformer.<name>.bin``
    (scripts/dump_weights.py:37-53, engine/src/gpt2.c:21-34,131-137)."""
    from mini_llm_b200.config import config_from_dict, describe_model
    from mini_llm_b200.weights import random_tensors
    for name, values in random_tensors(describe_model(config_from_dict(config)), 0, "gpt2").items():
        values.astype("<f4").tofile(os.path.join(folder, f"transformer.{name}.bin"))


def run_reference(args):
    """The unmodified reference through its own public API: ``NativeGPT2`` (ctypes binding),
    ``prefill_greedy`` per request, then ``decode_batch`` steps
    (pytorch/src/mini_llm/batch_api.py:44-70), fp16 decode weights as in its published runs."""
    if not os.path.isdir(os.path.join(REFERENCE, "mini_llm")):
        return unavailable("the reference is not installed under baseline/_ref")
    if args.batch > 16:
        return unavailable("the reference's batched decode takes at most 16 sequences")
    library = os.path.join(REFERENCE, "build", "libmini_llm_gpu.so")
    if not os.path.isfile(library):
        problem = build_reference_library(library)
        if problem:
            return unavailable(problem)
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    sys.path.insert(0, REFERENCE)
    try:
        from mini_llm.native import EngineOptions, NativeGPT2
    except Exception as error:
        return unavailable(f"the reference's binding does not import: {error}")
    config = dict(GPT2_SMALL)                # the reference's sizes are compile-time constants: GPT-2 small only
    context, vocab = config["n_positions"], config["vocab_size"]
    steps, warmup, batch = args.steps, args.warmup, args.batch
    prompt_len = context - steps - warmup
    rng = np.random.default_rng(1234)
    with tempfile.TemporaryDirectory() as folder:
        export_reference_weights(config, folder)
        engine = NativeGPT2(folder, library, backend="gpu",
                            options=EngineOptions(use_kv_cache=True, max_sessions=16, fp16_decode=not args.tokens_out))
    if args.tokens_out:
        # the fixed check workload, 32-bit weights: greedy tokens for the other arm to compare with
        cache = engine.try_take_cache()
        tokens = [engine.prefill_greedy(cache, check_prompt(vocab))]
        while len(tokens) < CHECK_NEW_TOKENS:
            tokens.append(engine.decode_batch([cache], [tokens[-1]])[0])
        engine.release_cache(cache)
        engine.close()
        with open(args.tokens_out, "w") as handle:
            json.dump({"tokens": [int(t) for t in tokens]}, handle)
        return 0
    sampler = ClockSampler()
    caches = [engine.try_take_cache() for _ in range(batch)]
    tokens = [engine.prefill_greedy(cache, rng.integers(0, vocab, prompt_len).tolist()) for cache in caches]
    for _ in range(warmup):
        tokens = engine.decode_batch(caches, tokens)
    torch.cuda.synchronize()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    start.record()
    for _ in range(steps):
        tokens = engine.decode_batch(caches, tokens)       # host tokens in and out, every step
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall
    clocks = sampler.stop()
    ms = start.elapsed_time(stop) / steps
    for cache in caches:
        engine.release_cache(cache)
    line = {"metric": f"decode tokens/s, GPT-2 {args.model}, batch {args.batch}, context {context}", "value": batch / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 weights, fp32 arithmetic",
            "data": "synthetic: seeded random weights (N(0, 0.02)) and uniform random token ids", "impl": "reference",
            "config": {"model": "gpt2-small", "n_layer": 12, "n_embd": 768, "n_head": 12, "n_inner": 3072,
                       "vocab_size": vocab, "n_positions": context, "global_batch": batch, "seq_len": context,
                       "prompt_tokens": prompt_len, "parallelism": "single GPU", "arch": "sources rebuilt for sm_100a"},
            "e2e": {"value": batch * steps / wall, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                    "d2h_bytes_per_step": 4 * batch},
            "clocks": clocks}
    if not args.no_extras:
        cache = engine.try_take_cache()
        token = engine.prefill_greedy(cache, rng.integers(0, vocab, prompt_len).tolist())
        torch.cuda.synchronize()
        begin = time.perf_counter()
        for _ in range(min(steps, 64)):
            token = engine.decode_batch([cache], [token])[0]
        torch.cuda.synchronize()
        line["points"] = {"decode_b1": min(steps, 64) / (time.perf_counter() - begin)}
        engine.release_cache(cache)
        cache = engine.try_take_cache()
        prompts = [rng.integers(0, vocab, 1024).tolist() for _ in range(2)]
        torch.cuda.synchronize()
        begin = time.perf_counter()
        for prompt in prompts:                               # a prompt is never batched: one after the other
            engine.prefill_greedy(cache, prompt)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        line["prefill"] = {"value": 2048 / seconds, "tokens": 2048, "ms": 1000.0 * seconds}
        engine.release_cache(cache)
    engine.close()
    print(json.dumps(line))
    return 0


def replayed_us(torch, launch, repeats=12):
    """Microseconds per call of ``launch(i)``, i = 0 .. repeats - 1 (each on operands of its own,
    so that nothing stays in L2 from call to call), captured once and replayed: the best of five."""
    launch(0)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(repeats):
            launch(i)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(5):
        first.record()
        graph.replay()
        last.record()
        torch.cuda.synchronize()
        best = min(best, first.elapsed_time(last) * 1000.0 / repeats)
    return best


def run_kernels():
    """Single kernels at the sizes the profiles quote: the residual-sum product at every tile
    code the launcher knows (0: its own choice), and the prompt attention with one and with two
    tiles per CTA.  One JSON line per measurement."""
    import math
    import torch
    from mini_llm_b200.kernels import ops
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    codes = (0, 2064, 2096, 2128, 192, 256, 7002, 7004, 7102, 7104)
    shapes = ((640, 768, 3072), (1024, 768, 3072), (1536, 768, 3072), (2048, 768, 3072), (4096, 768, 3072),
              (2048, 768, 768), (1024, 1024, 4096), (2048, 1024, 4096), (1024, 1600, 6400), (2048, 1600, 6400))
    for m, n, k in shapes:
        xs = [torch.randn(m, k, device="cuda").bfloat16() for _ in range(12)]
        ws = [(torch.randn(n, k, device="cuda") / math.sqrt(k)).bfloat16() for _ in range(12)]
        bias, out = torch.randn(n, device="cuda"), torch.zeros(m, n, device="cuda")
        for code in codes:
            def launch(i, code=code):
                if code == 0:
                    ops.gemm_bf16(out, xs[i], ws[i], bias, "add", status)
                else:
                    ops.gemm_bf16_tile(out, xs[i], ws[i], bias, "add", status, code)
            print(json.dumps({"kernel": "gemm, residual sum", "m": m, "n": n, "k": k, "tile_code": code,
                              "us": round(replayed_us(torch, launch), 2)}), flush=True)
    heads, head, page = 12, 64, 64
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    for name, lengths, new in (("2 x 1024", [1024, 1024], [1024, 1024]), ("1 x 1024", [1024], [1024]),
                               ("4 x 512", [512] * 4, [512] * 4), ("8 x 256 after 768", [1024] * 8, [256] * 8),
                               ("700 + 300 + 1000 + 48 after 976", [700, 300, 1000, 1024], [700, 300, 1000, 48])):
        blocks = [-(-length // page) for length in lengths]
        k_pages = torch.randn(sum(blocks) + 1, page, heads, head, device="cuda").bfloat16()
        v_pages = torch.randn(sum(blocks) + 1, page, heads, head, device="cuda").bfloat16()
        table = torch.zeros(len(lengths), max(blocks), dtype=torch.int32)
        at = 0
        for i, count in enumerate(blocks):
            table[i, :count] = torch.arange(at, at + count, dtype=torch.int32)
            at += count
        table = table.cuda()
        q = torch.randn(sum(new), heads * head, device="cuda").bfloat16()
        out = torch.empty_like(q)
        offsets = [sum(new[:i]) for i in range(len(new))]
        starts = [length - count for length, count in zip(lengths, new)]
        tiles, _, _ = ops.attention_tiles(offsets, new, starts, split=False)
        tiles_d = torch.tensor(tiles, dtype=torch.int32, device="cuda")
        units, n_split, most = ops.attention_units(offsets, new, starts, heads, torch.cuda.get_device_properties(0).multi_processor_count)
        units_d = torch.tensor(units, dtype=torch.int32, device="cuda")
        scratch = None
        if n_split:
            scratch = (torch.empty(n_split * heads * most * ops.ATTENTION_UNIT * (head + 4), device="cuda"),
                       torch.zeros(2 * n_split * heads, dtype=torch.int32, device="cuda"))
        one = replayed_us(torch, lambda i: ops.attention_prefill(out, q, k_pages, v_pages, table, tiles_d, len(tiles), heads, heads,
                                                                head, page, 0.125, 0, status, work))
        two = replayed_us(torch, lambda i: ops.attention_prefill_two_tiles(out, q, k_pages, v_pages, table, units_d, len(units), heads,
                                                                          heads, head, page, 0.125, 0, status, work, scratch, n_split,
                                                                          most))
        print(json.dumps({"kernel": "prompt attention, 12 heads of 64", "prompts": name, "one_tile_per_cta_us": round(one, 2),
                          "two_tiles_per_cta_us": round(two, 2)}), flush=True)
    if int(status.item()) != 0:
        print(json.dumps({"error": "a bounded wait inside a kernel ran out", "status": int(status.item())}))
        return 1
    return 0


def main():
    args = parse_args()
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.kernels:
        return run_kernels()
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
