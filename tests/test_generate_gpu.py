"""Generation through the Python entry point and the command line, against the plain model."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.helpers import GREEDY_MARGIN, TINY, random_tokens
from tests.plain import llama

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_next(config, tensors, tokens):
    return llama.forward(config, tensors, tokens)[-1].numpy()


def check_greedy(config, tensors, prompt, generated, margin_rel):
    tokens = list(prompt)
    for k, got in enumerate(generated):
        logits = plain_next(config, tensors, tokens)
        best = int(np.argmax(logits))
        if got != best:
            margin = float(logits[best] - logits[got])
            assert margin <= margin_rel * float(np.abs(logits).max()), \
                f"generated token {k} is {got}, the plain model says {best} (margin {margin:.3e})"
        tokens.append(got)


@pytest.mark.parametrize("dtype, margin", sorted(GREEDY_MARGIN.items()))
@pytest.mark.parametrize("name, lengths, steps", [("a", [5, 17, 33], 8), ("b", [1, 40, 63, 129], 12)])
def test_greedy_generation_matches_plain(model_folders, name, lengths, steps, dtype, margin):
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders(name)
    config, tensors = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, seed=n) for n in lengths]
    llm = LLM(folder, dtype=dtype, kv_capacity_tokens=1024, max_running=4, prefill_chunk_tokens=16,
              max_batch_tokens=48)
    outs = llm.generate(prompts, SamplingParams(max_tokens=steps, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == steps and out.finish_reason == "length", out.error
        check_greedy(config, tensors, prompt, out.token_ids, margin)
    assert llm.stepper.cache.used_pages() == 0
    llm.stepper.cache.check()


@pytest.mark.parametrize("name, count", [("a", 13), ("b", 16), ("b", 21)])
@pytest.mark.parametrize("graphs", [False, True])
def test_wider_decode_batches_match_plain(model_folders, name, count, graphs):
    """Thirteen and sixteen decode rows take the sixteen-row form of the weight-streaming products (norm and SwiGLU
    folded in), twenty-one the products for more rows: each against the plain model, request by request."""
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders(name)
    config, tensors = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], 3 + (5 * k) % 11, seed=100 + k) for k in range(count)]
    llm = LLM(folder, dtype="bfloat16", kv_capacity_tokens=2048, max_running=count, prefill_chunk_tokens=64,
              max_batch_tokens=256, cuda_graphs=graphs)
    outs = llm.generate(prompts, SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == 5 and out.finish_reason == "length", out.error
        check_greedy(config, tensors, prompt, out.token_ids, GREEDY_MARGIN["bfloat16"])
    assert llm.stepper.cache.used_pages() == 0


def test_temperature_sampling_is_reproducible_and_follows_the_draws(model_folders):
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("b")
    config, tensors = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, seed=50 + n) for n in (1, 40, 63, 129)]
    params = [SamplingParams(max_tokens=12, temperature=0.7, seed=1000 + i, ignore_eos=True) for i in range(4)]
    runs = []
    for chunk, running in ((16, 4), (512, 1)):           # mixed with others in portions of 16; then each alone
        llm = LLM(folder, dtype="float32", kv_capacity_tokens=1024, max_running=running, prefill_chunk_tokens=chunk)
        runs.append([o.token_ids for o in llm.generate(prompts, params)])
    assert runs[0] == runs[1], "sampled tokens depend on the batching"
    for prompt, p, generated in zip(prompts, params, runs[0]):
        rng = llama.SplitMix64(p.seed)
        tokens = list(prompt)
        for got in generated:
            draw = rng.unit_f64()
            logits = plain_next(config, tensors, tokens)
            want = llama.sample_in_token_order(logits, 0.7, draw)
            if got != want:     # only a draw that lands within rounding of a boundary may differ, by one neighbour
                scaled = logits.astype(np.float32) / np.float32(0.7)
                cdf = np.cumsum(np.exp((scaled - scaled.max()).astype(np.float64)))
                cdf /= cdf[-1]
                assert abs(cdf[min(got, want)] - draw) < 1e-5, f"sampled {got}, the plain model says {want}"
            tokens.append(got)


def test_top_p_and_mixed_sampling_modes(model_folders):
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("a")
    config, tensors = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, seed=n) for n in (9, 12, 20)]
    params = [SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True),
              SamplingParams(max_tokens=5, temperature=0.9, top_p=0.5, seed=3, ignore_eos=True),
              SamplingParams(max_tokens=5, temperature=1.3, seed=4, ignore_eos=True)]
    llm = LLM(folder, dtype="float32", kv_capacity_tokens=512, max_running=4)
    outs = llm.generate(prompts, params)
    check_greedy(config, tensors, prompts[0], outs[0].token_ids, 1e-5)
    rng = llama.SplitMix64(3)
    tokens = list(prompts[1])
    for got in outs[1].token_ids:
        want = llama.sample_host(plain_next(config, tensors, tokens), 0.9, 0.5, rng.unit_f64())
        assert got == want
        tokens.append(got)


def test_eos_stops_generation(model_folders):
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("a")
    config, tensors = llama.load_folder(folder)
    prompt = random_tokens(config["vocab_size"], 7, seed=1)
    llm = LLM(folder, dtype="float32", kv_capacity_tokens=256, max_running=2)
    free = llm.generate([prompt], SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))[0].token_ids
    stop = free[-1]
    stopped = llm.generate([prompt], SamplingParams(max_tokens=6, temperature=0.0, stop_token_ids=[stop]))[0]
    assert stopped.token_ids == free[:free.index(stop) + 1] and stopped.finish_reason == "stop"


def test_command_line_generates(model_folders):
    folder = model_folders("a")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "tesseract"), "--model-path", folder, "--prompt-ids", "5,6,7,8",
           "--random-prompt", "11", "--max-tokens", "4", "--temperature", "0", "--ignore-eos", "--json",
           "--kv-capacity-tokens", "256", "--max-running", "2", "--dtype", "float32", "--check-weights"]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    assert "weights checked: model.norm.weight" in done.stderr
    records = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert len(records) == 2 and all(len(r["token_ids"]) == 4 and r["finish_reason"] == "length" for r in records)
    config, tensors = llama.load_folder(folder)
    check_greedy(config, tensors, [5, 6, 7, 8], records[0]["token_ids"], GREEDY_MARGIN["float32"])


def test_command_line_prints_the_kernel_plan(model_folders):
    """``--print-plan`` says, for every distinct layer and the head, which kernel each operation takes at each row
    count: the one answer every part then follows (the reference prints its plan too,
    src/cuda/kernel_plan.rs:140-161)."""
    folder = model_folders("b")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "tesseract"), "--model-path", folder, "--print-plan",
           "--kv-capacity-tokens", "256", "--max-running", "2"]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    text = done.stdout
    assert "kernel plan for LlamaForCausalLM in bfloat16" in text and "layers 0..2 (3)" in text
    for word in ("qkv", "attend", "gate/up", "down", "head", "decode_linear", "attention_decode", "library"):
        assert word in text, word
    assert "does the following add+norm's work" in text          # the small-batch products prepare the next norm


@pytest.mark.parametrize("dtype, margin", sorted(GREEDY_MARGIN.items()))
def test_graph_replay_decodes_like_the_eager_path(model_folders, dtype, margin):
    """Pure decode steps replayed as CUDA graphs (batch padded to a bucket) give the eager path's tokens."""
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("b")
    config, tensors = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, seed=70 + n) for n in (3, 40, 66)]      # three rows: bucket of 4
    params = [SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True),
              SamplingParams(max_tokens=25, temperature=0.8, seed=5, ignore_eos=True),
              SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)]
    outs = {}
    for graphs in (True, False):
        llm = LLM(folder, dtype=dtype, kv_capacity_tokens=1024, max_running=4, cuda_graphs=graphs)
        outs[graphs] = [o.token_ids for o in llm.generate(prompts, params)]
        if graphs:
            assert llm.stepper.graphs.replays >= 30 and llm.stepper.graphs.captures >= 1
            # the table width grows past its first bucket while decoding (8 pages = 128 tokens)
            assert len(llm.stepper.graphs.graphs) >= 2
        assert llm.stepper.cache.used_pages() == 0
    if dtype == "float32":
        assert outs[True] == outs[False]
    for k in (0, 2):
        check_greedy(config, tensors, prompts[k], outs[True][k], margin)


def test_steps_launched_ahead_give_the_same_tokens_as_ordinary_steps(model_folders):
    """With CUDA graphs the scheduler launches decode steps before it has read the tokens of the step before
    (they reach the next step on the device); without graphs every step waits.  Same tokens, with requests that
    end at different times, stop tokens, temperature rows, and a request that arrives while others decode."""
    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("c")
    config, _ = llama.load_folder(folder)
    prompts = [random_tokens(config["vocab_size"], n, seed=90 + n) for n in (3, 30, 70, 12, 45)]
    first = LLM(folder, dtype="float32", kv_capacity_tokens=2048, max_running=3, prefill_chunk_tokens=32,
                cuda_graphs=False)
    greedy = first.generate(prompts[:1], SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))[0].token_ids
    params = [SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True, stop_token_ids=[greedy[6]]),
              SamplingParams(max_tokens=31, temperature=0.9, seed=7, ignore_eos=True),
              SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True),
              SamplingParams(max_tokens=40, temperature=0.4, seed=8, ignore_eos=True),
              SamplingParams(max_tokens=17, temperature=0.0, ignore_eos=True)]
    want = [(o.token_ids, o.finish_reason) for o in first.generate(prompts, params)]
    ahead = LLM(folder, dtype="float32", kv_capacity_tokens=2048, max_running=3, prefill_chunk_tokens=32)
    got = [(o.token_ids, o.finish_reason) for o in ahead.generate(prompts, params)]
    assert got == want
    assert want[0][1] == "stop" and want[0][0][-1] == greedy[6]
    assert ahead.stepper.graphs.replays > 20
    assert ahead.stepper.cache.used_pages() == 0
    ahead.stepper.cache.check()


def test_many_requests_under_load_get_the_same_tokens_with_and_without_graphs(model_folders):
    """Forty requests of random lengths and options through a small cache (requests wait for pages, portions
    replay as graphs, decode steps are launched ahead, batches change shape all the time) against the same
    requests with every step run launch by launch: the same tokens and finish reasons, and every page returned."""
    import random

    from tesseract_b200 import LLM, SamplingParams

    folder = model_folders("b")
    config, _ = llama.load_folder(folder)
    rng = random.Random(5)
    prompts, params = [], []
    for i in range(40):
        prompts.append([rng.randrange(config["vocab_size"]) for _ in range(rng.choice([1, 2, 7, 31, 32, 33, 64, 90, 120]))])
        greedy = rng.random() < 0.5
        params.append(SamplingParams(max_tokens=rng.choice([1, 2, 5, 17, 40]), temperature=0.0 if greedy else 0.8,
                                     seed=100 + i, ignore_eos=rng.random() < 0.7,
                                     stop_token_ids=[rng.randrange(config["vocab_size"])] if rng.random() < 0.3 else []))
    results = []
    for graphs in (False, True):
        llm = LLM(folder, dtype="float32", kv_capacity_tokens=640, max_running=6, max_queue=64,
                  prefill_chunk_tokens=32, max_batch_tokens=96, max_sequence_length=256, cuda_graphs=graphs)
        alone = [rng2.randrange(config["vocab_size"]) for rng2 in [random.Random(9)] for _ in range(100)]
        outs = llm.generate([alone], SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))   # portions replay
        outs += llm.generate(prompts, params)
        results.append([(o.token_ids, o.finish_reason) for o in outs])
        assert llm.stepper.cache.used_pages() == 0
        llm.stepper.cache.check()
        if graphs:
            counts = (llm.stepper.graphs.replays, llm.stepper.chunk_graphs.replays, llm.stepper.steps_run)
            assert counts[0] > 10 and counts[1] >= 1, counts
    assert results[0] == results[1]
    assert {reason for _, reason in results[0]} >= {"length"}
