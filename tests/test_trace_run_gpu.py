"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from files."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.helpers import REL, TINY, bf16_noise, compare, max_live_tokens, plain_logits, random_tokens, trace_mixed, trace_tail

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, steps, out_dir, max_tokens):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for number, (entries, end) in enumerate(steps):
        record = {"step": number, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries], "end": end}
        proc.stdin.write(json.dumps(record) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {number}"       # the next step only after this line
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    got, at = {}, {}
    for number, (entries, end) in enumerate(steps):
        wanted = sum(len(w) for _, _, w in entries)
        path = os.path.join(out_dir, f"{number}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            rows = None
        else:
            rows = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        k = 0
        for r, tokens, want in entries:
            for place in want:
                got[(r, at.get(r, 0) + place)] = rows[k]
                k += 1
            at[r] = at.get(r, 0) + len(tokens)
        for r in end:
            at.pop(r, None)
    return got


@pytest.mark.parametrize("dtype, rel", sorted(REL.items()))
def test_trace_run_mixed_and_tail(model_folders, tmp_path, dtype, rel):
    name = "b"
    folder = model_folders(name)
    vocab = TINY[name]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, seed=i) for i, n in enumerate([70, 33, 129, 2, 64, 90])}
    steps = trace_mixed(requests, seed=11) + trace_tail({"t": requests["r2"]})
    steps.insert(3, ([], []))                                             # a step that brings nothing
    got = run_trace(folder, dtype, steps, str(tmp_path / dtype), max_live_tokens(steps, 64))
    plain = plain_logits(folder, requests)
    plain["t"] = plain["r2"]
    noise = None
    if dtype == "bfloat16":
        noise = bf16_noise(folder, requests, plain)
        noise["t"] = noise["r2"]
    compare(got, plain, rel, f"trace_run/{dtype}", noise=noise)
