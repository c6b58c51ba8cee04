#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200 (Llama 3.2 1B sizes, random weights).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 (device time, CUDA
events around K decode steps through the engine's step function and device sampler; the
window of K steps is timed five times and the median is reported, with the fastest and the
slowest beside it); ``e2e`` is the same through the scheduler that ``LLM.generate`` drives,
with host token lists in and out; ``prefill`` is one 2,048-token prompt in one step (median
of twenty) and also as four portions of 512; ``points`` holds decode at batch 1 and 64;
``roofline`` compares the bytes a decode step must read with the measured copy bandwidth.

``--workload 3b`` and ``--workload 8b`` run the two other workloads instead: continuous
batching of up to 64 requests with prompts of 512 to 4,096 tokens at the Llama 3.2 3B layer
sizes (through the scheduler), and steps of one 2,048-token portion beside 64 decode rows at
contexts up to 16,384 at the Llama 3.1 8B layer sizes; each prints its own JSON line.
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

METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Llama 3.2 1B)"

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "attention_bias": False, "mlp_bias": False, "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": [128001],
}
# Other layer sizes of the same architecture (--size), to see how the kernels hold up away from the headline model.
OTHER_SIZES = {
    "3b": dict(num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
               intermediate_size=8192),
    "8b": dict(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, tie_word_embeddings=False,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192}),
}
SIZE_NAMES = {"1b": "Llama-3.2-1B sizes", "3b": "Llama-3.2-3B sizes", "8b": "Llama-3.1-8B sizes"}
PROMPT_TOKENS = 2048
REPEATS_PREFILL = 20      # the prefill step is timed this often; the median counts
REPEATS_DECODE = 5        # so is the window of K decode steps
CONTEXT = 4096
PAGE_SIZE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, windows):
        if self.proc is not None:
            self.proc.terminate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.samples:
            if windows and not any(a <= stamp <= b for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def reference_arm():
    print(json.dumps({"impl": "reference",
                      "unavailable": "Leikoe/tesseract is a Rust crate (cargo/rustc are not in this image and cannot "
                                     "be fetched offline) whose kernels are compiled at run time for sm_80 by cuTile; "
                                     "it has no Python package to pip-install"}))
    return 0


def model_numbers(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = h * (nh + 2 * nkv) * d + nh * d * h + 3 * h * i
    matmul_params = layers * per_layer + v * h
    weight_bytes = 2 * (matmul_params + (2 * layers + 1) * h)       # bfloat16; embedding shared with the head
    kv_bytes_per_token = layers * 2 * nkv * d * 2
    return {"layer_params": per_layer, "matmul_params": matmul_params, "weight_bytes": weight_bytes,
            "kv_bytes_per_token": kv_bytes_per_token}


def prefill_flops(cfg, layers, tokens, wanted_rows=1):
    n = model_numbers(cfg, layers)
    gemm = 2 * tokens * layers * n["layer_params"] + 2 * wanted_rows * cfg["vocab_size"] * cfg["hidden_size"]
    attention = layers * 2 * tokens * tokens * cfg["head_dim"] * cfg["num_attention_heads"]    # causal: half of 4*T^2*d
    return gemm + attention


def run_ours(args):
    import numpy as np
    import torch

    from tesseract_b200 import LLM, SamplingParams, kernels
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.weights.random_init import write_random_model

    model = dict(LLAMA_1B, **OTHER_SIZES.get(args.size, {}))
    layers = args.layers or model["num_hidden_layers"]
    cfg = dict(model, num_hidden_layers=layers)
    pk = peaks()
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    windows = []
    scratch = tempfile.TemporaryDirectory(prefix="tesseract_bench_")
    write_random_model(scratch.name, cfg, seed=0)
    max_batch = max(args.batch, 64)
    # `--only decode --decode-context N`: the decode windows start behind prompts of N tokens instead of 2,048
    decode_prompt = args.decode_context if args.only == "decode" and args.decode_context else PROMPT_TOKENS
    context_limit = max(CONTEXT, decode_prompt + 512)
    if decode_prompt != PROMPT_TOKENS:
        max_batch = args.batch
    decode_capacity = args.repeats * max_batch * (decode_prompt + 320)     # every window's requests at once
    llm = LLM(scratch.name, dtype="bfloat16", max_running=args.repeats * max_batch, max_batch_tokens=4096,
              prefill_chunk_tokens=PROMPT_TOKENS, kv_capacity_tokens=max(decode_capacity, max_batch * CONTEXT),
              page_size=PAGE_SIZE,
              max_sequence_length=context_limit, cuda_graphs=not args.no_graphs)
    stepper, cache = llm.stepper, llm.stepper.cache
    numbers = model_numbers(cfg, layers)
    sampler.start()

    def prompt(tokens=PROMPT_TOKENS):
        return rng.integers(0, cfg["vocab_size"], tokens).tolist()

    # ---------------------------------------------------------------- prefill: one 2,048-token prompt, one step
    def prefill_once(rid):
        assert cache.admit(rid)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tokens = prompt()
        torch.cuda.synchronize()
        start.record()
        logits = stepper.step([StepEntry(rid, tokens, [PROMPT_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        cache.release(rid)
        return start.elapsed_time(stop), logits

    portion_graphs = None
    if not args.no_graphs:
        from tesseract_b200.engine.graph import ChunkGraphs

        portion_graphs = ChunkGraphs(stepper, 512, CONTEXT, max_batch, max_portions=1)

    def prefill_in_portions(rid, portion):
        """The same prompt as portions of ``portion`` tokens, one step each (the reference's default portion is 512)."""
        assert cache.admit(rid)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tokens = prompt()
        torch.cuda.synchronize()
        start.record()
        for at in range(0, PROMPT_TOKENS, portion):
            last = at + portion >= PROMPT_TOKENS
            entries = [StepEntry(rid, tokens[at:at + portion], [portion - 1] if last else [])]
            if portion_graphs is not None and portion_graphs.eligible(entries):
                portion_graphs.step(entries)       # as an engine configured with this portion size replays it
            else:
                stepper.step(entries)
        stop.record()
        torch.cuda.synchronize()
        cache.release(rid)
        return start.elapsed_time(stop)

    if args.only == "decode":
        prefill_times, portions_times = [float("nan")], [float("nan")]
    else:
        for k in range(3):
            prefill_once(f"warm{k}")
            prefill_in_portions(f"warmp{k}", 512)
        t0 = time.time()
        # (`--repeats N` below the default also shortens the prefill: a run under a profiler wants few launches)
        prefill_repeats = REPEATS_PREFILL if args.repeats >= REPEATS_DECODE else max(1, args.repeats)
        prefill_in_order = [prefill_once(f"pre{k}")[0] for k in range(prefill_repeats)]
        prefill_times = sorted(prefill_in_order)
        portions_times = sorted(prefill_in_portions(f"prp{k}", 512) for k in range(prefill_repeats))
        windows.append((t0, time.time()))
    prefill_ms = statistics.median(prefill_times)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "ms": prefill_ms, "tokens_per_s": PROMPT_TOKENS / (prefill_ms / 1e3),
                          "ms_min": prefill_times[0], "ms_max": prefill_times[-1],
                          "ms_in_order": [round(t, 3) for t in prefill_in_order],
                          "ms_4x512": statistics.median(portions_times)}))
        return 0
    flops = prefill_flops(cfg, layers, PROMPT_TOKENS)
    portions_ms = statistics.median(portions_times)
    prefill = {"value": PROMPT_TOKENS / (prefill_ms / 1e3), "tokens": PROMPT_TOKENS, "ms": prefill_ms,
               "frac": flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "peak": f"{pk['source']} bf16",
               # the peak is a best-of-ten burst; the median of twenty back-to-back steps runs under the power cap:
               # beside it the fastest step against the burst peak and the median against the sustained peak
               "frac_fastest": flops / (prefill_times[0] / 1e3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained": flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12),
               "repeats": len(prefill_times), "ms_min": prefill_times[0], "ms_max": prefill_times[-1],
               "ms_4x512": portions_ms, "value_4x512": PROMPT_TOKENS / (portions_ms / 1e3)}

    # ---------------------------------------------------------------- decode on the device clock
    def decode_device(batch, steps, warmup, repeats=None):
        repeats = repeats or args.repeats
        greedy, ones = [0.0] * batch, [1.0] * batch
        # Every window decodes the same stretch (positions 2,048 + warmup .. + steps) with `batch` requests of its
        # own; all their 2,048-token prompts are cached before the first window, so that no prefill runs between
        # two windows.
        sets = [[f"d{batch}_{w}_{k}" for k in range(batch)] for w in range(repeats)]
        for window_ids in sets:
            for rid in window_ids:
                assert cache.admit(rid)
                ids_of_prompt = prompt(decode_prompt)
                for at in range(0, decode_prompt, PROMPT_TOKENS):
                    stepper.step([StepEntry(rid, ids_of_prompt[at:at + PROMPT_TOKENS], [])])
        ids = list(sets[0])

        entries = [StepEntry(rid, [0], [0]) for rid in ids]
        all_fed = [True] * batch

        def launch(previous, tokens):
            # as the scheduler does while every request decodes: the step is launched before the tokens of the
            # step before have been read; they reach it on the device
            if previous is None:
                first = [StepEntry(rid, [t], [0]) for rid, t in zip(ids, tokens)]
                return stepper.launch_decode(first, greedy, greedy) if stepper.graphs else None
            return stepper.launch_decode(entries, greedy, greedy, previous, all_fed)

        def one_step(tokens):
            return stepper.step_and_sample([StepEntry(rid, [t], [0]) for rid, t in zip(ids, tokens)],
                                           greedy, ones, greedy)

        def launched():
            return kernels.launch_count + (stepper.graphs.kernels_replayed if stepper.graphs else 0)

        times = []
        for window_ids in sets:                           # the same window of `steps` steps, several times
            ids[:] = window_ids
            entries[:] = [StepEntry(rid, [0], [0]) for rid in ids]
            last = [int(rng.integers(0, cfg["vocab_size"])) for _ in ids]
            for _ in range(warmup):
                last = one_step(last)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            launches = launched()
            t0 = time.time()
            start.record()
            if stepper.graphs is not None:
                inflight = launch(None, last)
                for _ in range(steps - 1):
                    following = launch(inflight, None)
                    last = inflight.tokens()              # host tokens out, one step behind the launches
                    inflight = following
                last = inflight.tokens()
            else:
                for _ in range(steps):
                    last = one_step(last)
            stop.record()
            torch.cuda.synchronize()
            windows.append((t0, time.time()))
            launches = launched() - launches
            times.append(start.elapsed_time(stop) / steps)
        context = cache.length(ids[0])
        for window_ids in sets:
            for rid in window_ids:
                cache.release(rid)
        times.sort()
        return statistics.median(times), launches, context, times

    ms_step, launches, context, step_times = decode_device(args.batch, args.steps, args.warmup)
    if args.only == "decode":
        step_bytes = numbers["weight_bytes"] + args.batch * context * numbers["kv_bytes_per_token"]
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": ms_step,
                          "tokens_per_s": args.batch / (ms_step / 1e3), "context": context,
                          "gb_per_step": step_bytes / 1e9,
                          "frac_of_hbm_peak": step_bytes / (ms_step / 1e3) / 1e9 / pk["hbm_gbs"]}))
        return 0
    point_steps = max(8, min(args.steps, 64))
    ms_b1, _, context_b1, _ = decode_device(1, point_steps, args.warmup)
    ms_b64, _, context_b64, _ = decode_device(64, point_steps, args.warmup)
    step_bytes = numbers["weight_bytes"] + args.batch * context * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    def point_frac(batch, ms, ctx):
        return (numbers["weight_bytes"] + batch * ctx * numbers["kv_bytes_per_token"]) / (ms / 1e3) / 1e9 / pk["hbm_gbs"]

    # ---------------------------------------------------------------- end to end through the scheduler
    # (every request must still be decoding at the end of the timed steps: the first ones start decoding while the
    # last prompts are still being prefilled, two to a step)
    params = SamplingParams(max_tokens=args.steps + args.warmup + 4 + args.batch, temperature=0.0, ignore_eos=True)
    for _ in range(args.batch):
        llm.scheduler.add_request(prompt(), params)
    while any(r.computed_tokens < len(r.prompt) for r in llm.scheduler.requests.values()) or llm.scheduler.waiting:
        llm.scheduler.step()
    for _ in range(args.warmup):
        llm.scheduler.step()
    torch.cuda.synchronize()
    t0 = time.time()
    produced = 0
    for _ in range(args.steps):
        produced += llm.scheduler.step().token_count()
    torch.cuda.synchronize()
    e2e_seconds = time.time() - t0
    windows.append((t0, time.time()))
    for rid in list(llm.scheduler.requests):
        llm.scheduler.cancel(rid)
    pages = -(-context // PAGE_SIZE)
    h2d = 4 * (args.batch * 6 + 1 + args.batch * pages)
    e2e = {"value": produced / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * args.batch}

    clocks = sampler.stop(windows)
    value = args.batch / (ms_step / 1e3)
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "ms_per_step_min": step_times[0], "ms_per_step_max": step_times[-1],
        "repeats": args.repeats, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": SIZE_NAMES[args.size], "layers": layers, "layers_of_model": model["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS,
                   "decode_context": context, "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({numbers['weight_bytes'] / 1e9:.2f} GB of weights read every step)",
                   "decode_steps": "CUDA graph per step, launched one ahead of the token read-back",
                   "timing": "median of 5 windows of `steps` steps (decode) and of 20 steps (prefill)"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"]},
        "points": {"decode_b1": 1 / (ms_b1 / 1e3), "decode_b64": 64 / (ms_b64 / 1e3),
                   "decode_b1_frac": point_frac(1, ms_b1, context_b1), "decode_b64_frac": point_frac(64, ms_b64, context_b64)},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "impl": "ours",
    }
    print(json.dumps(line))
    scratch.cleanup()
    return 0


WORKLOAD_LAYERS = 8      # layers the workload runs build by default (of 28 and 32): memory and time; --layers says otherwise


def run_workload(args):
    """The two workloads beside the headline one (each prints its own JSON line):

    ``3b``  Llama 3.2 3B layer sizes, continuous batching through the scheduler: 128 requests with prompts of 512 to
            4,096 random tokens and 128 generated tokens each, at most 64 running, portions of 512, context 8,192.
    ``8b``  Llama 3.1 8B layer sizes, the mixed step of continuous batching under load: one 2,048-token portion of a
            16,384-token prompt beside 64 decode rows whose contexts spread from 2,048 to 16,000 tokens.
    """
    import numpy as np
    import torch

    from tesseract_b200 import LLM, SamplingParams, kernels
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.weights.random_init import write_random_model

    size = args.workload
    model = dict(LLAMA_1B, **OTHER_SIZES[size])
    layers = args.layers or WORKLOAD_LAYERS
    cfg = dict(model, num_hidden_layers=layers)
    pk = peaks()
    numbers = model_numbers(cfg, layers)
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    scratch = tempfile.TemporaryDirectory(prefix="tesseract_bench_")
    write_random_model(scratch.name, cfg, seed=0)
    vocab, d, nh = cfg["vocab_size"], cfg["head_dim"], cfg["num_attention_heads"]
    base = {"metric": METRIC, "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "higher_is_better": True,
            "data": "synthetic: seeded random weights N(0,0.02) and random token ids", "impl": "ours"}
    shape = {"model": SIZE_NAMES[size], "layers": layers, "layers_of_model": model["num_hidden_layers"],
             "hidden": cfg["hidden_size"], "heads": nh, "kv_heads": cfg["num_key_value_heads"], "head_dim": d,
             "intermediate": cfg["intermediate_size"], "vocab": vocab, "page_size": PAGE_SIZE}
    sampler.start()
    if size == "3b":
        context, running, requests, generated = 8192, 64, 128, 128
        llm = LLM(scratch.name, dtype="bfloat16", max_running=running, max_queue=requests, max_batch_tokens=4096,
                  prefill_chunk_tokens=512, kv_capacity_tokens=running * context, page_size=PAGE_SIZE,
                  max_sequence_length=context, cuda_graphs=not args.no_graphs)
        lengths = rng.integers(512, 4097, requests).tolist()
        prompts = [rng.integers(0, vocab, n).tolist() for n in lengths]
        params = SamplingParams(max_tokens=generated, temperature=0.0, ignore_eos=True)
        # warm-up: the workload itself, once (a serving process has captured the graphs of its step shapes long
        # before the stretch that counts; the first run's time is reported beside the second's)
        torch.cuda.synchronize()
        t_first = time.time()
        llm.generate(prompts, params)
        torch.cuda.synchronize()
        first_seconds = time.time() - t_first
        steps_before, t0 = llm.scheduler.steps, time.time()
        outs = llm.generate(prompts, params)
        torch.cuda.synchronize()
        seconds = time.time() - t0
        produced = sum(len(o.token_ids) for o in outs)
        assert produced == requests * generated, "every request must run to its length"
        prompt_tokens = sum(lengths)
        # what the model computed: every prompt and generated token once through the products, each attending to all before it
        flops = 2 * (prompt_tokens + produced) * layers * numbers["layer_params"] + 2 * produced * vocab * cfg["hidden_size"]
        flops += sum(layers * 2 * (n + generated) ** 2 * d * nh for n in lengths)
        line = dict(base, workload="continuous batching: 128 requests, prompts of 512-4,096 tokens, 128 generated each, "
                                   "at most 64 running, portions of 512, context 8,192, through the scheduler",
                    value=(prompt_tokens + produced) / seconds, generated_tokens_per_s=produced / seconds,
                    seconds=seconds, first_run_seconds=first_seconds,
                    scheduler_steps=llm.scheduler.steps - steps_before,
                    graphs={"decode": len(llm.stepper.graphs.graphs) if llm.stepper.graphs else 0,
                            "portions": len(llm.stepper.chunk_graphs.graphs) if llm.stepper.chunk_graphs else 0,
                            "portion_replays": llm.stepper.chunk_graphs.replays if llm.stepper.chunk_graphs else 0},
                    prompt_tokens=prompt_tokens, generated_tokens=produced,
                    frac_of_bf16_peak=flops / seconds / (pk["bf16_tflops"] * 1e12), peak=f"{pk['source']} bf16",
                    config=dict(shape, global_batch=running, seq_len=context, prefill_chunk_tokens=512))
        windows = [(t0, t0 + seconds)]
    else:
        context, decodes, portion = 16384, 64, PROMPT_TOKENS
        portions_per_prompt = context // portion
        steps = args.steps if args.steps != 128 else 2 * portions_per_prompt
        capacity = decodes * context + 2 * context
        llm = LLM(scratch.name, dtype="bfloat16", max_running=decodes + 2, max_batch_tokens=portion + decodes,
                  prefill_chunk_tokens=portion, kv_capacity_tokens=capacity, page_size=PAGE_SIZE,
                  max_sequence_length=context, cuda_graphs=not args.no_graphs)
        stepper, cache = llm.stepper, llm.stepper.cache
        contexts = np.linspace(2048, 16000, decodes).astype(int).tolist()
        ids = [f"d{k}" for k in range(decodes)]
        for rid, n in zip(ids, contexts):      # the decode rows' earlier tokens: pages held, contents whatever they are
            assert cache.admit(rid)
            cache.extend(rid, n)
            cache.commit(rid, n)
        state = {"prompt": 0, "at": 0}

        def mixed_step():
            if state["at"] == 0:
                assert cache.admit(("p", state["prompt"]))
            rid = ("p", state["prompt"])
            last = state["at"] + portion >= context - portion       # leave room: the prompt ends one portion early
            entries = [StepEntry(rid, rng.integers(0, vocab, portion).tolist(), [portion - 1] if last else [])]
            entries += [StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in ids]
            stepper.step(entries)
            state["at"] += portion
            if last:
                cache.release(rid)
                state["prompt"] += 1
                state["at"] = 0

        for _ in range(max(args.warmup, portions_per_prompt)):
            mixed_step()
        times, windows = [], []
        launches = 0
        for _ in range(REPEATS_DECODE):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            before = kernels.launch_count + (stepper.chunk_graphs.kernels_replayed if stepper.chunk_graphs else 0)
            t0 = time.time()
            start.record()
            for _ in range(steps):
                mixed_step()
            stop.record()
            torch.cuda.synchronize()
            windows.append((t0, time.time()))
            launches = kernels.launch_count + (stepper.chunk_graphs.kernels_replayed if stepper.chunk_graphs else 0) - before
            times.append(start.elapsed_time(stop) / steps)
        times.sort()
        ms = statistics.median(times)
        rows = portion + decodes
        mean_decode_context = float(np.mean([cache.length(r) for r in ids]))
        mean_prompt_context = (context - portion) / 2            # a portion sees, on average, half the prompt before it
        flops = 2 * rows * layers * numbers["layer_params"] + 2 * (decodes + 1) * vocab * cfg["hidden_size"]
        flops += layers * 4 * portion * (mean_prompt_context + portion / 2) * d * nh      # QK^T and PV of the portion
        embedding_bytes = 0 if cfg.get("tie_word_embeddings") else 2 * vocab * cfg["hidden_size"]
        step_bytes = numbers["weight_bytes"] + embedding_bytes * 0 + (decodes * mean_decode_context + mean_prompt_context) * numbers["kv_bytes_per_token"]
        t_compute = flops / (pk["bf16_tflops"] * 1e12)
        t_memory = step_bytes / (pk["hbm_gbs"] * 1e9)
        line = dict(base, workload="mixed step: one 2,048-token portion of a 16,384-token prompt beside 64 decode rows "
                                   "(contexts 2,048 to 16,000)",
                    value=rows / (ms / 1e3), ms_per_step=ms, ms_per_step_min=times[0], ms_per_step_max=times[-1],
                    steps=steps, repeats=REPEATS_DECODE, gpu_launches=launches,
                    bound={"compute_ms": t_compute * 1e3, "hbm_ms": t_memory * 1e3,
                           "frac": max(t_compute, t_memory) / (ms / 1e3), "of": pk["source"]},
                    config=dict(shape, global_batch=decodes + 1, seq_len=context, prompt_portion=portion,
                                mean_decode_context=mean_decode_context))
    line["clocks"] = sampler.stop(windows)
    line["tcgen05_wait_timeouts"] = kernels.tcgen05_error()
    print(json.dumps(line))
    scratch.cleanup()
    return 0


def run_kernels(args):
    """Each hot kernel alone at the 1B model's sizes: device time per launch, in a CUDA graph of 16 launches over 16
    distinct weight or cache buffers (so that nothing stays in L2 from one launch to the next)."""
    import math

    import torch

    from tesseract_b200 import kernels, plan

    torch.manual_seed(0)
    dev = "cuda"
    pk = peaks()
    out_lines = {}

    def timed(fns, reps=20):
        torch.cuda.synchronize()          # the inputs were made on the default stream: they must exist first
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for f in fns:
                f()
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000 / reps / len(fns)

    m = args.batch
    for name, n, k, fused in (("qkv", 3072, 2048, True), ("o", 2048, 2048, False), ("gate_up", 16384, 2048, True),
                              ("down", 2048, 8192, False)):
        ws = [(torch.randn(n, k, device=dev) / math.sqrt(k)).to(torch.bfloat16) for _ in range(16)]
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        upd = torch.randn(m, k, device=dev).to(torch.bfloat16)
        nw = torch.ones(k, device=dev)
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        res_out = torch.empty_like(x)
        mb = n * k * 2 / 1e6
        entry = {"weight_mb": mb, "hbm_floor_us": mb / pk["hbm_gbs"] * 1e3,
                 "library_us": timed([lambda w=w: torch.mm(x, w.t(), out=out) for w in ws]),
                 "decode_linear_us": timed([lambda w=w: kernels.decode_linear(w, out, x=x) for w in ws])}
        if fused:
            entry["decode_linear_add_norm_us"] = timed([lambda w=w: kernels.decode_linear(
                w, out, residual=x, update=upd, norm_weight=nw, eps=1e-5, residual_out=res_out) for w in ws])
        out_lines[f"decode_linear_m{m}_{name}"] = entry
        del ws

    # 17 to 128 rows: the swapped-operand tcgen05 product against the library GEMM, plain, with SwiGLU (against the
    # tcgen05 GEMM that carried it before) and as the product that does a norm's work (against product + norm kernel)
    for rows in (32, 64, 128):
        for name, n, k in (("qkv", 3072, 2048), ("o", 2048, 2048), ("gate_up", 16384, 2048), ("down", 2048, 8192)):
            ws = [(torch.randn(n, k, device=dev) / math.sqrt(k)).to(torch.bfloat16) for _ in range(16)]
            x = torch.randn(rows, k, device=dev).to(torch.bfloat16)
            out = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
            mb = n * k * 2 / 1e6
            entry = {"weight_mb": mb, "hbm_floor_us": mb / pk["hbm_gbs"] * 1e3,
                     "library_us": timed([lambda w=w: torch.mm(x, w.t(), out=out) for w in ws]),
                     "skinny_us": timed([lambda w=w: kernels.skinny_tcgen05(x, w, out) for w in ws])}
            if name == "gate_up":
                act = torch.empty(rows, n // 2, device=dev, dtype=torch.bfloat16)
                entry["gemm_tcgen05_swiglu_us"] = timed(
                    [lambda w=w: kernels.gemm_tcgen05(x, w, act, epilogue=kernels.EPI_SWIGLU) for w in ws])
                entry["skinny_swiglu_us"] = timed(
                    [lambda w=w: kernels.skinny_tcgen05(x, w, act, epilogue=kernels.EPI_SWIGLU) for w in ws])
            if name in ("o", "down"):
                res, nw = torch.randn(rows, n, device=dev).to(torch.bfloat16), torch.ones(n, device=dev)
                res_out, xw = torch.empty_like(res), torch.empty_like(res)
                sums = torch.empty(kernels.skinny_tcgen05_sums_shape(n), device=dev)
                entry["skinny_prepare_us"] = timed([lambda w=w: kernels.skinny_tcgen05(
                    x, w, None, prepare=(res, nw, res_out, xw, sums)) for w in ws])
                entry["library_then_add_norm_us"] = timed([lambda w=w: (
                    torch.mm(x, w.t(), out=out), kernels.add_rms_norm(res, out, nw, 1e-5, xw, res_out)) for w in ws])
            out_lines[f"skinny_m{rows}_{name}"] = entry
            del ws

    nh, nkv, d, ps, ctx = 32, 8, 64, PAGE_SIZE, 2100
    for batch in (1, 8, 64):
        pages = -(-ctx // ps)
        caches = [torch.randn(batch * pages + 1, 2, nkv, ps, d, device=dev).to(torch.bfloat16) for _ in range(16)]
        table = (torch.arange(batch * pages, device=dev, dtype=torch.int32).view(batch, pages) + 1).contiguous()
        q = torch.randn(batch, nh * d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        row_start = torch.arange(batch + 1, device=dev, dtype=torch.int32)
        seq_begin = torch.full((batch,), ctx - 1, device=dev, dtype=torch.int32)
        splits = plan.attention_splits(batch, nkv, ctx)
        us = timed([lambda c=c: kernels.attention_mma(q, out, c, row_start, seq_begin, table, batch, 1, nh, nkv, d, ps, 0,
                                                      0.125, False, True, splits) for c in caches])
        mb = batch * ctx * 2 * nkv * d * 2 / 1e6
        out_lines[f"attention_decode_b{batch}_ctx{ctx}"] = {"kv_mb": mb, "hbm_floor_us": mb / pk["hbm_gbs"] * 1e3,
                                                           "splits": splits, "us": us}
        del caches

    tokens = PROMPT_TOKENS
    pages = tokens // ps
    caches = [torch.randn(pages + 1, 2, nkv, ps, d, device=dev).to(torch.bfloat16) for _ in range(16)]
    table = (torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages) + 1).contiguous()
    q = torch.randn(tokens, nh * d, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    row_start = torch.tensor([0, tokens], device=dev, dtype=torch.int32)
    seq_begin = torch.zeros(1, device=dev, dtype=torch.int32)
    flops = 2 * tokens * tokens * d * nh
    t_mma = timed([lambda c=c: kernels.attention_mma(q, out, c, row_start, seq_begin, table, 1, tokens, nh, nkv, d, ps, 0,
                                                     0.125, True, False, 1) for c in caches])
    t_tc = timed([lambda c=c: kernels.attention_tcgen05(q, out, c, row_start, seq_begin, table, 1, tokens, nh, nkv, d,
                                                        ps, 0, 0.125) for c in caches])
    out_lines[f"attention_prefill_{tokens}"] = {"causal_gflop": flops / 1e9, "mma_sync_us": t_mma,
                                                "mma_sync_tflops": flops / t_mma / 1e6, "tcgen05_us": t_tc,
                                                "tcgen05_tflops": flops / t_tc / 1e6}
    del caches

    for name, n, k in (("qkv", 3072, 2048), ("o", 2048, 2048), ("gate_up", 16384, 2048), ("down", 2048, 8192)):
        ws = [(torch.randn(n, k, device=dev) / math.sqrt(k)).to(torch.bfloat16) for _ in range(8)]
        x = torch.randn(tokens, k, device=dev).to(torch.bfloat16)
        out = torch.empty(tokens, n, device=dev, dtype=torch.bfloat16)
        fl = 2 * tokens * n * k
        t_lib = timed([lambda w=w: torch.mm(x, w.t(), out=out) for w in ws], reps=5)
        t_own = timed([lambda w=w: kernels.gemm_tcgen05(x, w, out) for w in ws], reps=5)
        out_lines[f"gemm_m{tokens}_{name}"] = {"gflop": fl / 1e9, "library_us": t_lib, "library_tflops": fl / t_lib / 1e6,
                                               "tcgen05_us": t_own, "tcgen05_tflops": fl / t_own / 1e6}
        del ws
    out_lines["tcgen05_wait_timeouts"] = kernels.tcgen05_error()
    print(json.dumps({"only": "kernels", "peaks": pk, "kernels": out_lines}))
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--size", default="1b", choices=["1b", "3b", "8b"],
                        help="layer sizes: the headline model's (1b) or another Llama's, for a look at other sizes")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--only", default="all", choices=["all", "decode", "prefill", "kernels"],
                        help="measure one part only (for profiling small cases); the JSON line then lacks the rest")
    parser.add_argument("--no-graphs", action="store_true", help="decode without CUDA-graph replay")
    parser.add_argument("--decode-context", type=int, default=0,
                        help="with --only decode: decode behind prompts of this many tokens instead of 2,048")
    parser.add_argument("--repeats", type=int, default=REPEATS_DECODE,
                        help="how often the window of --steps decode steps is timed (the median counts); 1 keeps a "
                             "profiling run short")
    parser.add_argument("--workload", choices=["3b", "8b"], default=None,
                        help="run another workload instead of the headline one: continuous batching at the 3B sizes, "
                             "or a 2,048-token portion beside 64 decode rows at the 8B sizes")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.workload:
        return run_workload(args)
    if args.only == "kernels":
        return run_kernels(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
