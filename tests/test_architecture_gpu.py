"""Another architecture, added the way a user would: a module outside the package registers its parts, its typed
configuration and its model description (``tests/toy_architecture.py``); a folder is written for it with the
random-weights writer; it generates through ``LLM.generate`` and the command line and replays through ``LLM.replay``
and ``bin/trace_run``: scheduler, cache manager (a paged group whose pages are not keys and values, a state group,
an ordinary key/value group), step function and samplers as they are."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.helpers import GREEDY_MARGIN, random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from tests import toy_architecture as toy
    from tesseract_b200.weights.random_init import write_random_model

    return write_random_model(str(tmp_path_factory.mktemp("toy_architecture")), toy.CONFIG, seed=21)


def plain(folder):
    from tests import toy_architecture as toy
    from tests.plain import llama

    config, tensors = llama.load_folder(folder)
    return lambda tokens: toy.plain_forward(config, tensors, tokens)


def test_the_registry_learns_the_architecture_from_a_plugin_variable(toy_folder):
    """A fresh interpreter that has never imported the module resolves the architecture through $TESSERACT_PLUGINS,
    and without it reports the unknown name (no device needed)."""
    code = ("import tesseract_b200.models; from tesseract_b200.config import load_model_description; "
            f"a, c, s = load_model_description({toy_folder!r}); print(a.name, len(s.layers), s.head.weights)")
    env = dict(os.environ, TESSERACT_PLUGINS="tests.toy_architecture", PYTHONPATH=ROOT)
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)
    assert done.returncode == 0, done.stderr
    assert done.stdout.split()[:2] == ["ToyMixedForTests", "3"] and "tokens" in done.stdout
    env.pop("TESSERACT_PLUGINS")
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)
    assert done.returncode != 0 and "unsupported architecture" in done.stderr


def test_cache_groups_of_the_toy_architecture(toy_folder):
    """Three needs, three groups: key/value pages, latent pages of the need's own shape, fixed-size state."""
    from tests import toy_architecture as toy
    from tesseract_b200.cache import CacheManager
    from tesseract_b200.parts import PagedKVNeed, StateNeed

    needs = [PagedKVNeed(1, 16), toy.LatentNeed(width=6), StateNeed((40,), torch.float32)]
    cache = CacheManager(needs, [None] * 3, num_pages=8, page_size=16, max_requests=2, dtype=torch.bfloat16,
                         device="cpu", max_step_tokens=16)
    assert [tuple(g.storage.shape) for g in cache.groups] == [(1, 9, 2, 1, 16, 16), (1, 9, 16, 6), (1, 3, 40)]
    assert cache.groups[1].storage.dtype == torch.float32 and cache.groups[0].storage.dtype == torch.bfloat16
    assert cache.bytes_per_token() == 2 * 16 * 2 + 6 * 4
    assert cache.admit("r", reserve_tokens=40)
    cache.extend("r", 40)
    cache.commit("r", 40)
    assert cache.used_pages() == 6 and sorted(cache.pages_of("r", 1)) == [0, 1, 2]
    cache.release("r")
    cache.check()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_generates_and_replays_through_the_entry_point(toy_folder, dtype):
    from tests import toy_architecture as toy
    from tesseract_b200 import LLM, SamplingParams

    forward = plain(toy_folder)
    vocab = toy.CONFIG["vocabulary"]
    prompts = [random_tokens(vocab - 1, n, seed=300 + n) for n in (4, 23, 41)]
    llm = LLM(toy_folder, dtype=dtype, kv_capacity_tokens=512, max_running=3, prefill_chunk_tokens=16,
              max_batch_tokens=40)
    assert llm.model.head.proj.weight.data_ptr() == llm.model.embedding.table.data_ptr()      # tied by tensor name
    assert llm.stepper.graphs is None or not llm.stepper.graphs.safe      # toy parts never said they may be captured
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == 6 and out.finish_reason == "length", out.error
        tokens = list(prompt)
        for k, got in enumerate(out.token_ids):
            logits = forward(tokens)[-1].numpy()
            best = int(np.argmax(logits))
            assert logits[best] - logits[got] <= GREEDY_MARGIN[dtype] * np.abs(logits).max(), \
                f"token {k}: {got}, the plain model says {best}"
            tokens.append(got)
    assert llm.stepper.cache.used_pages() == 0
    llm.stepper.cache.check()
    # the same engine replays a trace: a prompt in portions of 16, 2 and the rest, logits at every place
    tokens = random_tokens(vocab - 1, 45, seed=77)
    trace = [{"step": 0, "entries": [{"id": "t", "tokens": tokens[:16], "want": list(range(16))}], "end": []},
             {"step": 1, "entries": [{"id": "t", "tokens": tokens[16:18], "want": [0, 1]}], "end": []},
             {"step": 2, "entries": [{"id": "t", "tokens": tokens[18:], "want": list(range(27))}], "end": ["t"]}]
    got = torch.cat(llm.replay(trace)).double()
    want = forward(tokens)
    limit = (2e-5 if dtype == "float32" else 3e-2) * float(want.abs().max())     # torch-made toy parts in bfloat16
    assert float((got - want).abs().max()) <= limit
    assert llm.stepper.cache.used_pages() == 0


@pytest.mark.gpu
def test_toy_architecture_through_the_command_line_and_the_replay_program(toy_folder, tmp_path):
    from tests import toy_architecture as toy

    forward = plain(toy_folder)
    env = dict(os.environ, PYTHONPATH=ROOT)
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text("# two prompts\n5, 6, 7, 8\n\n9 10 11\n")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "tesseract"), "--plugin", "tests.toy_architecture",
                           "--model-path", toy_folder, "--dtype", "float32", "--prompt-file", str(prompt_file),
                           "--max-tokens", "4", "--temperature", "0", "--ignore-eos", "--json",
                           "--kv-capacity-tokens", "256", "--max-running", "2"],
                          capture_output=True, text=True, env=env, cwd=ROOT)
    assert done.returncode == 0, done.stderr
    records = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(records) == 2
    for prompt, record in zip(([5, 6, 7, 8], [9, 10, 11]), records):
        tokens = list(prompt)
        for got in record["token_ids"]:
            logits = forward(tokens)[-1].numpy()
            assert logits[int(np.argmax(logits))] - logits[got] <= GREEDY_MARGIN["float32"] * np.abs(logits).max()
            tokens.append(got)
    tokens = random_tokens(toy.CONFIG["vocabulary"] - 1, 20, seed=5)
    out = tmp_path / "logits"
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens[:17], "want": [16]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": tokens[17:], "want": [0, 1, 2]}], "end": ["a"]})]
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--plugin", "tests.toy_architecture",
                           "--model", toy_folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, cwd=ROOT)
    assert done.returncode == 0 and done.stdout.split() == ["done", "0", "done", "1"], done.stderr
    want = forward(tokens).numpy()
    got = np.concatenate([np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(-1, want.shape[1]) for k in (0, 1)])
    assert np.abs(got - want[16:20]).max() <= 2e-5 * np.abs(want).max()
