"""The engine against the plain implementation under every way of cutting the work.

Each case drives the engine's own step function (model, cache manager, kernels) through
a trace and compares every wanted logits row with the plain whole-sequence model.
"""

import numpy as np
import pytest
import torch

from tests.helpers import (REL, TINY, bf16_noise, compare, keep_wants, max_live_tokens, plain_logits, random_tokens, replay,
                           trace_mixed, trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

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

    def noise(name, dtype, store="bfloat16"):
        """Measured bfloat16 rounding noise per request for the bfloat16 engine; None (a relative bound) in 32-bit."""
        if dtype != "bfloat16":
            return None
        if (name, store, "noise") not in cache:
            cache[(name, store, "noise")] = bf16_noise(model_folders(name, store), make_requests(name), get(name, store))
        return cache[(name, store, "noise")]

    get.noise = noise
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_cuts_match_plain(engines, plains, name, dtype, cut):
    requests = make_requests(name)
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    got = replay(stepper, steps)
    compare(got, plains(name), REL[dtype], f"{name}/{dtype}/{cut}", noise=plains.noise(name, dtype))
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
    extra = {rid: toks for rid, toks in requests.items() if rid not in plain}
    plain.update(_plain_extra(name, extra))
    noise = None
    if dtype == "bfloat16":
        noise = dict(plains.noise(name, dtype))
        noise.update(bf16_noise(_FOLDERS(name, "bfloat16"), extra, plain))
    compare(got, plain, REL[dtype], f"{name}/{dtype}/mixed", noise=noise)
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


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_float32_cuts_agree_bitwise(engines, name):
    """In 32-bit every reduction order depends only on the row itself: cuts agree bit for bit."""
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
    compare(got, plain, REL[dtype], f"{name}/{dtype}/float32-stored",
            noise=bf16_noise(model_folders(name, "float32"), requests, plain) if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, plains, dtype):
    name = "b"
    tokens = make_requests(name)["b4"]          # 200 tokens, decoded one by one from the third on
    steps = [([("long", tokens[:3], [0, 1, 2])], [])]
    steps += [([("long", tokens[i:i + 1], [0])], []) for i in range(3, len(tokens))]
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(engines(name, dtype), steps)
    plain = {"long": plains(name)["b4"]}
    noise = {"long": plains.noise(name, dtype)["b4"]} if dtype == "bfloat16" else None
    compare(got, plain, REL[dtype], f"{name}/{dtype}/long-decode", noise=noise)
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
        compare(got, plains(name), REL[dtype], f"{name}/{dtype}/first-tokens", noise=plains.noise(name, dtype))


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
    assert float((logits["bfloat16"] - logits["float32"]).abs().max()) <= REL["bfloat16"] * scale


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
    # (the 5-token end of p replays too, in a graph of its own whose other rows are padding)
    assert stepper.chunk_graphs.replays == 6 and len(stepper.chunk_graphs.graphs) == 3
    if dtype == "float32":
        assert torch.equal(got, want)
    else:       # launched alone, five rows take the kernels of small batches; in their graph, those of 24 rows
        assert torch.equal(got[:-1], want[:-1])
        assert float((got[-1] - want[-1]).abs().max()) <= REL["bfloat16"] * float(want.abs().max())
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
        for name, prompt in others.items():
            assert stepper.cache.admit(name)
            stepper.step([StepEntry(name, prompt, [])])
        if graphs:      # (from here on: the short prompts above, replayed as ends of prompts, would take other kernels)
            stepper.enable_graphs(4, chunk_rows=chunk, max_sequence_length=256)
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
    assert sorted(stepper.chunk_graphs.graphs) == [(1, 0, 1, True, 8), (1, 0, 2, False, 8), (1, 0, 4, False, 8)]
    assert torch.equal(got, want)
    stepper.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_with_several_portions_equal_ordinary_steps(model_folders, dtype):
    """A burst of arrivals: three prompts' portions in one step beside decoded tokens of two other requests, then
    two portions, then one, as the scheduler builds them under its token budget.  Each shape replays as one graph
    (the last rows of all portions go through the head when one of them is wanted); bit-equal to launch by
    launch."""
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder = model_folders("c")
    config = TINY["c"]
    model = load_model(folder, dtype=dtype)
    chunk = 24
    prompts = {name: random_tokens(config["vocab_size"], n * chunk, seed=70 + n) for name, n in (("p", 4), ("q", 3), ("r", 2))}
    others = {name: random_tokens(config["vocab_size"], n, seed=80 + n) for name, n in (("x", 30), ("y", 7))}
    feed = {name: random_tokens(config["vocab_size"], 8, seed=90 + ord(name)) for name in others}

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=512, max_requests=5)
        for name, prompt in others.items():
            assert stepper.cache.admit(name)
            stepper.step([StepEntry(name, prompt, [])])
        if graphs:
            stepper.enable_graphs(4, chunk_rows=chunk, max_sequence_length=256, max_batch_tokens=4 * chunk)
        for name in prompts:
            assert stepper.cache.admit(name)
        out = []
        for k in range(4):
            entries = []
            for name, tokens in prompts.items():
                if (k + 1) * chunk <= len(tokens):
                    last = (k + 1) * chunk == len(tokens)
                    entries.append(StepEntry(name, tokens[k * chunk:(k + 1) * chunk], [chunk - 1] if last else []))
            entries += [StepEntry(name, [feed[name][k]], [0]) for name in (("x", "y") if k < 2 else ("x",))]
            out.append(stepper.step(entries).clone())
        return torch.cat(out), stepper

    want, _ = run(False)
    got, stepper = run(True)
    assert stepper.chunk_graphs.replays == 4
    assert sorted(stepper.chunk_graphs.graphs) == [(1, 0, 1, True, 8), (2, 0, 1, True, 8), (3, 0, 2, False, 8),
                                                   (3, 0, 2, True, 8)]
    assert got.shape == want.shape and torch.equal(got, want)
    stepper.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_with_the_end_of_a_prompt_equal_ordinary_steps(model_folders, dtype):
    """The end of a prompt (fewer tokens than a portion) beside full portions of other prompts and decoded tokens:
    such a step replays as a graph whose tail rows are padded with a sequence that lives on the scratch page.  The
    logits are those of the same steps launched one by one (bit for bit in 32-bit; in bfloat16 the product kernels
    depend on the step's row count, which the padding changes), for tails of 2 to 23 tokens through the same graph,
    and the requests decode on afterwards from an intact cache."""
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder = model_folders("c")
    config = TINY["c"]
    model = load_model(folder, dtype=dtype)
    chunk = 24
    lengths = {"a": chunk + 5, "b": 2 * chunk + 23, "c": 2, "d": 3 * chunk + 13}
    prompts = {name: random_tokens(config["vocab_size"], n, seed=300 + n) for name, n in lengths.items()}
    other = random_tokens(config["vocab_size"], 11, seed=17)
    feed = random_tokens(config["vocab_size"], 40, seed=18)

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=1024, max_requests=6)
        if graphs:
            stepper.enable_graphs(4, chunk_rows=chunk, max_sequence_length=256, max_batch_tokens=4 * chunk)
        assert stepper.cache.admit("x")
        stepper.step([StepEntry("x", other, [])])
        out, fed = [], iter(feed)
        at = {name: 0 for name in prompts}
        for name in prompts:
            assert stepper.cache.admit(name)
        live = []
        # full portions of the prompts that still have one, then the end of one prompt, then the decode rows
        while any(at[n] < lengths[n] for n in prompts):
            entries, tail = [], None
            for name, tokens in prompts.items():
                left = lengths[name] - at[name]
                if left >= chunk:
                    entries.append(StepEntry(name, tokens[at[name]:at[name] + chunk], [chunk - 1] if left == chunk else []))
                    at[name] += chunk
                    if left == chunk:
                        live.append(name)
                elif left > 0 and tail is None:
                    tail = StepEntry(name, tokens[at[name]:], [left - 1])
                    at[name] = lengths[name]
            entries += [tail] if tail is not None else []
            entries += [StepEntry(name, [next(fed)], [0]) for name in ["x"] + live]
            if tail is not None:
                live.append(tail.request)
            out.append(stepper.step(entries).clone())
        for _ in range(3):                                      # and on, from what the replayed steps left in the cache
            out.append(stepper.step([StepEntry(name, [next(fed)], [0]) for name in ["x"] + live]).clone())
        return out, stepper

    want, _ = run(False)
    got, stepper = run(True)
    tails = [key for key in stepper.chunk_graphs.graphs if key[1]]
    assert tails and all(key[1] == chunk for key in tails) and stepper.chunk_graphs.replays >= 4
    assert len(got) == len(want)
    scale = max(float(w.abs().max()) for w in want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert a.shape == b.shape
        if dtype == "float32":
            assert torch.equal(a, b), f"step {k} differs from launch by launch"
        else:
            assert float((a - b).abs().max()) <= REL["bfloat16"] * scale, f"step {k} is off"
    stepper.cache.check()


# ----------------------------------------------------------------------------- the layer sizes of Llama 3.2 1B

SIZES_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": [128001],
}
LENGTHS_1B = {"w0": 70, "w1": 333, "w2": 200, "w3": 45, "w4": 90}


@pytest.fixture(scope="module")
def two_layers_of_the_1b_sizes(tmp_path_factory):
    """A model of 2 layers (Llama 3.2 1B has 16) with every layer size of Llama 3.2 1B, its requests, the positions
    whose logits are compared (every 16th and the last 33 of each request: all rows of a 128,256-wide vocabulary
    would be gigabytes) and the plain float64 model's logits there."""
    from tests.helpers import make_model_folder
    from tests.plain import llama

    folder = make_model_folder(str(tmp_path_factory.mktemp("two_layers_1b")), SIZES_1B, "bfloat16", 11)
    requests = {rid: random_tokens(SIZES_1B["vocab_size"], n, seed=200 + n) for rid, n in LENGTHS_1B.items()}
    keep = {rid: sorted(set(range(0, len(t), 16)) | set(range(max(0, len(t) - 33), len(t)))) for rid, t in requests.items()}
    config, tensors = llama.load_folder(folder)
    plain = {rid: llama.forward(config, tensors, t, head_rows=keep[rid]).numpy() for rid, t in requests.items()}
    rows_of = {rid: {position: row for row, position in enumerate(keep[rid])} for rid in requests}
    noise = bf16_noise(folder, requests, plain, head_rows=keep)
    return folder, requests, {rid: set(k) for rid, k in keep.items()}, plain, rows_of, noise


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_four_cuts_at_the_1b_layer_sizes_with_2_of_16_layers(two_layers_of_the_1b_sizes, dtype):
    """Whole prompts, the last 32 tokens one by one, portions of changing size down to two tokens, and up to three
    live requests mixed with so few pages that they are used again: every compared row against the plain model, and
    in 32-bit bit for bit across the cuts.  These are the sizes at which the products run over K = 8,192 and
    N = 128,256, the attention over 32 heads of 64 in 8 groups, and (bfloat16) the tcgen05 kernels."""
    from tesseract_b200 import kernels
    from tesseract_b200.engine import load_model, make_stepper

    folder, requests, keep, plain, rows_of, noise = two_layers_of_the_1b_sizes
    model = load_model(folder, dtype=dtype)
    mixed = trace_mixed(requests, seed=9, live_max=3)
    cuts = {"whole": trace_whole(requests), "tail": trace_tail(requests), "portions": trace_portions(requests),
            "mixed": mixed}
    results = {}
    for cut, steps in cuts.items():
        capacity = max_live_tokens(steps, 64) if cut == "mixed" else 4096
        stepper = make_stepper(model, capacity_tokens=capacity, max_requests=4)
        results[cut] = replay(stepper, keep_wants(steps, keep))
        compare(results[cut], plain, REL[dtype], f"1B sizes/{dtype}/{cut}", rows_of,
                noise if dtype == "bfloat16" else None)
        stepper.cache.check()
        assert stepper.cache.used_pages() == 0
        if cut == "mixed":
            assert max(len(e) for e, _ in steps) >= 3 and stepper.cache.pages_reused > 0
    assert kernels.tcgen05_error() == 0
    assert len(results["whole"]) == sum(len(k) for k in keep.values())
    if dtype == "float32":
        for cut in ("tail", "portions", "mixed"):
            for key, row in results[cut].items():
                assert np.array_equal(row, results["whole"][key]), f"{cut} differs from whole at {key}"


def test_decode_graphs_at_the_1b_head_geometry_across_a_table_width(two_layers_of_the_1b_sizes):
    """Decode steps replayed as graphs at 32 heads of 64 in 8 groups, two requests, while the longer one's context
    crosses 128 tokens (its block table outgrows eight pages: another graph, captured with another split count):
    every step's logits equal the launch-by-launch step's bit for bit, before and after the crossing."""
    from tesseract_b200 import kernels
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder, requests, *_ = two_layers_of_the_1b_sizes
    model = load_model(folder, dtype="bfloat16")
    prompts = {"long": requests["w2"][:120], "short": requests["w3"][:30]}
    feed = {"long": requests["w1"][:20], "short": requests["w4"][:20]}

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=1024, max_requests=4)
        if graphs:
            stepper.enable_graphs(4)
        for name, prompt in prompts.items():
            assert stepper.cache.admit(name)
            stepper.step([StepEntry(name, prompt, [])])
        out = []
        for k in range(20):
            entries = [StepEntry(name, [feed[name][k]], [0]) for name in prompts]
            if graphs:
                out.append(stepper.graphs.step(entries, [0.0, 0.0], [0.0, 0.0])[1].clone())
            else:
                out.append(stepper.step(entries).clone())
        return torch.stack(out), stepper

    want, _ = run(False)
    got, stepper = run(True)
    assert sorted(stepper.graphs.graphs) == [(2, 8), (2, 16)] and stepper.graphs.replays == 20
    assert kernels.tcgen05_error() == 0
    for k in range(20):
        assert torch.equal(got[k], want[k]), f"decode step {k} (context {120 + k + 1}) differs"


# ----------------------------------------------------------------------------- scratch memory under captured graphs

LONG_CONTEXT = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 256, "vocab_size": 512, "max_position_embeddings": 65536,
    "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "bos_token_id": 1, "eos_token_id": [2],
}


def test_graphs_that_use_split_scratch_survive_later_larger_steps(tmp_path):
    """With more than eight key splits the decode attention parks its partial results in scratch memory whose
    address a captured graph keeps.  A graph captured early (a portion beside one decode row at a context of
    65,000 tokens; a decode graph of one row) must give the same bits when it is replayed after steps that need
    more of that memory (more sequences, more rows) and after other tensors have been allocated and filled:
    nothing the graph points at may have been given back meanwhile."""
    from tests.helpers import make_model_folder
    from tesseract_b200 import kernels, plan
    from tesseract_b200.engine import StepEntry, load_model, make_stepper

    folder = make_model_folder(str(tmp_path / "long_context"), LONG_CONTEXT, "bfloat16", 7)
    model = load_model(folder, dtype="bfloat16")
    vocab, chunk, context = LONG_CONTEXT["vocab_size"], 64, 65000
    long_prompt = random_tokens(vocab, context, seed=1)
    portion = random_tokens(vocab, 4 * chunk, seed=2)
    decoded = random_tokens(vocab, 16, seed=3)
    shorts = {f"s{i}": random_tokens(vocab, 40 + i, seed=10 + i) for i in range(3)}
    # the split counts the graphs are captured with (a table width of 4,096 pages) and the launch-by-launch steps
    # take (the true context) have to agree for the comparison to be bit for bit; all of them use the scratch
    for seqs in (1, 2):
        captured = plan.attention_splits(seqs, 2, 4096 * 16, 64)
        assert captured == plan.attention_splits(seqs, 2, context + 8, 64) and captured > 8

    def run(graphs):
        stepper = make_stepper(model, capacity_tokens=context + 2048, max_requests=8)
        if graphs:
            stepper.enable_graphs(4, chunk_rows=chunk, max_sequence_length=65536)
        out = []
        assert stepper.cache.admit("long")
        for start in range(0, context, 2000):                    # launch by launch either way (not the portion size)
            stepper.step([StepEntry("long", long_prompt[start:start + 2000], [])])
        assert stepper.cache.admit("p")
        d = iter(decoded)

        def portion_step(k):
            entries = [StepEntry("p", portion[k * chunk:(k + 1) * chunk], []), StepEntry("long", [next(d)], [0])]
            return stepper.step(entries).clone()

        def decode_step(names):
            entries = [StepEntry(r, [next(d)], [0]) for r in names]
            if graphs:
                return stepper.graphs.step(entries, [0.0] * len(names), [0.0] * len(names))[1].clone()
            return stepper.step(entries).clone()

        out.append(portion_step(0))                              # captures the portion graph: 32 splits, scratch
        out.append(decode_step(["long"]))                        # captures the one-row decode graph
        # steps that need more scratch than either graph did: three more sequences of two rows beside the long one
        for rid, tokens in shorts.items():
            assert stepper.cache.admit(rid)
            stepper.step([StepEntry(rid, tokens[:-2], [])])
        out.append(stepper.step([StepEntry(rid, tokens[-2:], [0, 1]) for rid, tokens in shorts.items()]
                                + [StepEntry("long", [next(d)], [0])]).clone())
        out.append(decode_step(["long", "s0"]))                  # a second, wider decode graph
        fillers = [torch.full((1 << 20,), float(k), device="cuda") for k in range(1, 9)]    # takes whatever was freed
        out.append(portion_step(1))                              # the first graph again
        out.append(decode_step(["long"]))                        # the one-row graph again
        out.append(portion_step(2))
        torch.cuda.synchronize()
        for k, filler in enumerate(fillers, start=1):
            assert bool((filler == float(k)).all()), "a replayed graph wrote into memory it no longer owned"
        if graphs:
            # (three portion steps, and the three short prompts, each the end of a prompt in a graph of 64 rows)
            assert stepper.chunk_graphs.replays == 6 and stepper.graphs.replays == 3
        stepper.cache.check()
        return out

    want = run(False)
    got = run(True)
    assert kernels.tcgen05_error() == 0
    for k, (a, b) in enumerate(zip(got, want)):
        assert torch.equal(a, b), f"step {k} of the replayed run differs from launch by launch"


def test_portions_late_in_a_long_prompt_share_their_tiles_between_ctas(tmp_path):
    """Beyond some 4,000 tokens of context a step with few attention tiles gives every tile to several CTAs, each
    over a run of the tile's key blocks (``plan.prompt_key_splits``).  A prompt of 4,700 tokens fed as one large
    portion and then portions of 300 down to 2 tokens: the rows of the late portions against the plain model.  (That
    one far key among hundreds is found whichever run it lies in is the kernel test's part:
    test_attention_tcgen05_and_wide_decode_find_one_far_key_among_hundreds.)"""
    from tests.helpers import make_model_folder
    from tests.plain import llama
    from tesseract_b200 import kernels, plan
    from tesseract_b200.engine import load_model, make_stepper

    folder = make_model_folder(str(tmp_path / "long_prompt"), LONG_CONTEXT, "bfloat16", 5)
    total = 4700
    requests = {"long": random_tokens(LONG_CONTEXT["vocab_size"], total, seed=77)}
    sizes = [4096, 300, 200, 64, 30, 8, 2]
    assert sum(sizes) == total
    for new in sizes[1:4]:
        shared = plan.attention(torch.bfloat16, num_heads=4, num_kv_heads=2, head_dim=64, page_size=16,
                                new_tokens=[new], max_context=4400)
        assert shared.prompt == "tcgen05" and shared.key_splits >= 2
    keep = {"long": sorted(set(range(4096, total, 7)) | set(range(total - 40, total)))}
    config, tensors = llama.load_folder(folder)
    plain = {"long": llama.forward(config, tensors, requests["long"], head_rows=keep["long"]).numpy()}
    rows_of = {"long": {position: row for row, position in enumerate(keep["long"])}}
    noise = bf16_noise(folder, requests, plain, head_rows=keep)
    steps, at = [], 0
    for size in sizes:
        steps.append(([("long", requests["long"][at:at + size], list(range(size)))], ["long"] if at + size == total else []))
        at += size
    model = load_model(folder, dtype="bfloat16")
    stepper = make_stepper(model, capacity_tokens=total + 64, max_requests=2)
    got = replay(stepper, keep_wants(steps, {"long": set(keep["long"])}))
    assert kernels.tcgen05_error() == 0
    assert len(got) == len(keep["long"])
    compare(got, plain, REL["bfloat16"], "long prompt, late portions", rows_of, noise)
    stepper.cache.check()
