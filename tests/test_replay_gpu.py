"""The engine against the plain implementation under every way of cutting the work.

Each case drives the engine's own step function (model, cache manager, kernels) through
a trace and compares every wanted logits row with the plain whole-sequence model.
"""

import numpy as np
import pytest
import torch

from tests.helpers import (TINY, compare, max_live_tokens, plain_logits, random_tokens, replay, trace_mixed,
                           trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

# |diff| <= REL * max(1, max|logit|).  float32: summation-order noise only.  bfloat16: the
# unit roundoff 2^-8 through a few dozen rounding points, on logits of order one.
REL = {"float32": 2e-5, "bfloat16": 3e-2}

LENGTHS = {"a": [5, 17, 33, 100], "b": [1, 40, 63, 129, 200], "c": [3, 64, 65, 130]}


def make_requests(name):
    vocab = TINY[name]["vocab_size"]
    return {f"{name}{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def engines(model_folders):
    from tesseract_b200.engine import load_model, make_stepper

    cache = {}

    def get(name, dtype, capacity_tokens=4096, store="bfloat16"):
        key = (name, dtype, store)
        if key not in cache:
            cache[key] = load_model(model_folders(name, store), dtype=dtype)
        return make_stepper(cache[key], capacity_tokens=capacity_tokens, max_requests=8)

    return get


@pytest.fixture(scope="module")
def plains(model_folders):
    cache = {}

    def get(name, store="bfloat16"):
        if (name, store) not in cache:
            cache[(name, store)] = plain_logits(model_folders(name, store), make_requests(name))
        return cache[(name, store)]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_cuts_match_plain(engines, plains, name, dtype, cut):
    requests = make_requests(name)
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    got = replay(stepper, steps)
    compare(got, plains(name), REL[dtype], f"{name}/{dtype}/{cut}")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_mixed_with_page_reuse(engines, plains, name, dtype):
    requests = make_requests(name)
    requests.update({f"{name}x{i}": random_tokens(TINY[name]["vocab_size"], n, seed=7 + i)
                     for i, n in enumerate([50, 21, 90, 34])})
    steps = trace_mixed(requests, seed=3)
    assert max(len(e) for e, _ in steps) >= 3, "the trace should batch several requests"
    capacity = max_live_tokens(steps, 64)
    stepper = engines(name, dtype, capacity_tokens=capacity)
    got = replay(stepper, steps)
    plain = dict(plains(name))
    plain.update(_plain_extra(name, {rid: toks for rid, toks in requests.items() if rid not in plain}))
    compare(got, plain, REL[dtype], f"{name}/{dtype}/mixed")
    assert stepper.cache.pages_reused > 0, "the pool was meant to be small enough for pages to be used again"
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


_extra_cache = {}


def _plain_extra(name, extra):
    key = (name, tuple(sorted(extra)))
    if key not in _extra_cache:
        _extra_cache[key] = plain_logits(_FOLDERS(name, "bfloat16"), extra)
    return _extra_cache[key]


@pytest.fixture(scope="module", autouse=True)
def _bind_folders(model_folders):
    global _FOLDERS
    _FOLDERS = model_folders
    yield


def test_float32_cuts_agree_bitwise(engines):
    """In 32-bit every reduction order depends only on the row itself: cuts agree bit for bit."""
    name = "b"
    requests = make_requests(name)
    whole = replay(engines(name, "float32"), trace_whole(requests))
    portions = replay(engines(name, "float32"), trace_portions(requests))
    mixed = replay(engines(name, "float32", capacity_tokens=max_live_tokens(trace_mixed(requests, seed=5))),
                   trace_mixed(requests, seed=5))
    for key, row in portions.items():
        assert np.array_equal(row, whole[key]), f"portions differ from whole at {key}"
    for key, row in mixed.items():
        assert np.array_equal(row, whole[key]), f"mixed differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_stored_weights(engines, model_folders, dtype):
    """A checkpoint stored in 32-bit: the float32 path keeps every bit of it."""
    name = "a"
    requests = make_requests(name)
    got = replay(engines(name, dtype, store="float32"), trace_portions(requests))
    plain = plain_logits(model_folders(name, "float32"), requests)
    compare(got, plain, REL[dtype], f"{name}/{dtype}/float32-stored")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, plains, dtype):
    name = "b"
    tokens = make_requests(name)["b4"]          # 200 tokens, decoded one by one from the third on
    steps = [([("long", tokens[:3], [0, 1, 2])], [])]
    steps += [([("long", tokens[i:i + 1], [0])], []) for i in range(3, len(tokens))]
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(engines(name, dtype), steps)
    plain = {"long": plains(name)["b4"]}
    compare(got, plain, REL[dtype], f"{name}/{dtype}/long-decode")
    assert len(got) == len(tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(engines, plains, dtype):
    for name in ("a", "b"):
        requests = make_requests(name)
        steps = []
        for rid, tokens in requests.items():
            steps.append(([(rid, tokens[:1], [0])], []))
            if len(tokens) > 1:
                steps.append(([(rid, tokens[1:3], list(range(len(tokens[1:3]))))], [rid]))
            else:
                steps[-1] = (steps[-1][0], [rid])
        got = replay(engines(name, dtype), steps)
        compare(got, plains(name), REL[dtype], f"{name}/{dtype}/first-tokens")


def test_one_layer_of_the_1b_sizes_in_bfloat16(tmp_path):
    """The kernels that only the full-size model reaches (tcgen05 attention at head size 64, the tcgen05 gate/up
    product, 32-feature decode tiles, the 128,256-wide head) inside the engine: a one-layer model with the layer
    sizes of Llama 3.2 1B, a prompt in one step, then decoded tokens, against the plain model."""
    from tests.helpers import make_model_folder
    from tests.plain import llama
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "num_hidden_layers": 1, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
        "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "max_position_embeddings": 131072,
        "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": [128001],
    }
    folder = make_model_folder(str(tmp_path / "one_layer_1b"), config, "bfloat16", 3)
    plain_config, tensors = llama.load_folder(folder)
    tokens = random_tokens(config["vocab_size"], 300, seed=17)
    want_rows = [270, 299, 300, 301, 302]                       # the prompt's last rows, then decoded positions
    prompt = 300
    tokens = tokens + random_tokens(config["vocab_size"], 3, seed=18)
    hidden = llama.forward(plain_config, tensors, tokens, head_rows=want_rows)
    model = load_model(folder, dtype="bfloat16")
    stepper = make_stepper(model, capacity_tokens=512, max_requests=2)
    assert stepper.cache.admit("r")
    got = [stepper.step([StepEntry("r", tokens[:prompt], [270, 299])]).float().cpu()]
    for t in range(prompt, prompt + 3):
        got.append(stepper.step([StepEntry("r", tokens[t:t + 1], [0])]).float().cpu())
    got = torch.cat(got)
    from tesseract_b200 import kernels
    assert kernels.tcgen05_error() == 0
    scale = float(hidden.abs().max())
    assert float((got.double() - hidden).abs().max()) <= 3e-2 * max(1.0, scale)
    assert (got.argmax(dim=1) == hidden.argmax(dim=1)).float().mean() >= 0.6   # random weights: many near ties


def test_long_context_with_wide_heads_in_bfloat16_against_float32(tmp_path):
    """Head size 128 at a context of six thousand tokens: prompt portions of 2,048 (tcgen05 attention in 64-key
    blocks over thousands of earlier keys) and decoded tokens (the split decode kernel's six-warp form, many
    splits), bfloat16 against the engine's own 32-bit path, which other tests hold against the plain model."""
    from tests.helpers import make_model_folder
    from tesseract_b200 import kernels
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 128, "intermediate_size": 1024, "vocab_size": 512, "max_position_embeddings": 16384,
        "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 2048},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": [2],
    }
    folder = make_model_folder(str(tmp_path / "wide_heads"), config, "bfloat16", 5)
    prompt, decoded = 6000, 6
    tokens = random_tokens(config["vocab_size"], prompt + decoded, seed=23)
    logits = {}
    for dtype in ("float32", "bfloat16"):
        stepper = make_stepper(load_model(folder, dtype=dtype), capacity_tokens=8192, max_requests=2)
        assert stepper.cache.admit("r")
        rows = []
        for start in range(0, prompt, 2048):
            stop = min(prompt, start + 2048)
            want = [0, stop - start - 1]
            rows.append(stepper.step([StepEntry("r", tokens[start:stop], want)]).float().cpu())
        for t in range(prompt, prompt + decoded):
            rows.append(stepper.step([StepEntry("r", tokens[t:t + 1], [0])]).float().cpu())
        logits[dtype] = torch.cat(rows)
    assert kernels.tcgen05_error() == 0
    scale = float(logits["float32"].abs().max())
    assert float((logits["bfloat16"] - logits["float32"]).abs().max()) <= 3e-2 * max(1.0, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_prompt_portions_equal_ordinary_steps(model_folders, dtype):
    """A prompt fed in portions of the configured size goes through a captured CUDA graph (only device metadata
    changes between such steps); the logits are those of the same portions run launch by launch, bit for bit,
    for two requests whose portions interleave (different pages, different positions, the same graph)."""
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder = model_folders("c")
    config, _ = llama.load_folder(folder) if False else (TINY["c"], None)
    model = load_model(folder, dtype=dtype)
    chunk = 24
    tokens = {"p": random_tokens(config["vocab_size"], 3 * chunk + 5, seed=31),
              "q": random_tokens(config["vocab_size"], 2 * chunk, seed=32)}

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=512, max_requests=2)
        if graphs:
            stepper.enable_graphs(2, chunk_rows=chunk, max_sequence_length=256)
        out = []
        for r in tokens:
            assert stepper.cache.admit(r)
        at = {"p": 0, "q": 0}
        for r in ("p", "q", "p", "q", "p", "p"):                 # portions of the two requests in turn
            n = min(chunk, len(tokens[r]) - at[r])
            want = [n - 1] if at[r] + n >= len(tokens[r]) or r == "q" else []
            logits = stepper.step([StepEntry(r, tokens[r][at[r]:at[r] + n], want)])
            at[r] += n
            if logits is not None:
                out.append(logits.clone())
        return torch.cat(out), stepper

    want, _ = run(False)
    got, stepper = run(True)
    assert stepper.chunk_graphs.replays == 5 and len(stepper.chunk_graphs.graphs) == 2   # the 5-token tail ran eagerly
    assert torch.equal(got, want)
    stepper.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_portions_beside_decoded_tokens_equal_ordinary_steps(model_folders, dtype):
    """A prompt portion beside one to three decoded tokens of other requests (the common step of continuous
    batching) replays as a graph too, padded to a power of two of decode rows; bit-equal to launch by launch."""
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder = model_folders("c")
    config = TINY["c"]
    model = load_model(folder, dtype=dtype)
    chunk = 24
    long_prompt = random_tokens(config["vocab_size"], 4 * chunk, seed=41)
    others = {name: random_tokens(config["vocab_size"], n, seed=50 + n) for name, n in (("x", 9), ("y", 40), ("z", 17))}
    feed = {name: random_tokens(config["vocab_size"], 8, seed=60 + len(name) + ord(name)) for name in others}

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=512, max_requests=4)
        if graphs:
            stepper.enable_graphs(4, chunk_rows=chunk, max_sequence_length=256)
        for name, prompt in others.items():
            assert stepper.cache.admit(name)
            stepper.step([StepEntry(name, prompt, [])])
        assert stepper.cache.admit("p")
        out = []
        live = ["x", "y", "z"]
        for k in range(4):                                      # portions of p beside 3, 3, 2, 1 decoded tokens
            entries = [StepEntry("p", long_prompt[k * chunk:(k + 1) * chunk], [chunk - 1] if k == 3 else [])]
            entries += [StepEntry(name, [feed[name][k]], [0]) for name in live]
            out.append(stepper.step(entries).clone())
            if k >= 1:
                stepper.cache.release(live.pop())
        return torch.cat(out), stepper

    want, _ = run(False)
    got, stepper = run(True)
    assert stepper.chunk_graphs.replays == 4
    assert sorted(stepper.chunk_graphs.graphs) == [(1, True), (2, False), (4, False)]
    assert torch.equal(got, want)
    stepper.cache.check()
