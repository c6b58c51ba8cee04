"""Tiny configurations, traces and comparison helpers shared by the tests."""

from __future__ import annotations

import random
from typing import Dict, Hashable, List, Sequence, Tuple

import numpy as np
import torch

# Two tiny Llama configurations that differ in every size and option.
TINY = {
    "a": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "attention_bias": False, "mlp_bias": False,
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "max_position_embeddings": 128,
        "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "bos_token_id": 1, "eos_token_id": [2],
    },
    "b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "attention_bias": False, "mlp_bias": False,
        "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
        "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "max_position_embeddings": 256,
        "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "bos_token_id": 0, "eos_token_id": 383,
    },
    # head_dim * heads != hidden, an odd vocabulary, 48-wide heads, 6 query heads on 3 kv heads
    "c": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
        "num_hidden_layers": 2, "hidden_size": 72, "num_attention_heads": 6, "num_key_value_heads": 3,
        "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "max_position_embeddings": 512,
        "rope_theta": 20000.0, "rope_scaling": None, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
        "bos_token_id": 5, "eos_token_id": [7, 9],
    },
}


def make_model_folder(folder: str, config: dict, store: str, seed: int) -> str:
    from tesseract_b200.weights.random_init import write_random_model

    cfg = dict(config)
    cfg["torch_dtype"] = store
    return write_random_model(folder, cfg, seed)


def random_tokens(vocab: int, length: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(length)]


# ------------------------------------------------------------------ traces
# A trace is a list of steps; a step is (entries, end) with entries = [(id, tokens, want)].

def trace_whole(requests: Dict[Hashable, List[int]]):
    steps = []
    for rid, tokens in requests.items():
        steps.append(([(rid, tokens, list(range(len(tokens))))], [rid]))
    return steps


def trace_tail(requests: Dict[Hashable, List[int]], tail: int = 32):
    steps = []
    for rid, tokens in requests.items():
        head = max(0, len(tokens) - tail)
        if head:
            steps.append(([(rid, tokens[:head], [head - 1])], []))
        for i in range(head, len(tokens)):
            steps.append(([(rid, tokens[i:i + 1], [0])], [rid] if i == len(tokens) - 1 else []))
    return steps


def trace_portions(requests: Dict[Hashable, List[int]], sizes=(16, 7, 2, 5, 33, 2, 3, 11, 2, 64, 4)):
    steps = []
    k = 0
    for rid, tokens in requests.items():
        at = 0
        while at < len(tokens):
            size = sizes[k % len(sizes)]
            k += 1
            if len(tokens) - at - size == 1:      # never leave a one-token rest after a portion
                size += 1
            part = tokens[at:at + size]
            at += len(part)
            steps.append(([(rid, part, list(range(len(part))))], [rid] if at >= len(tokens) else []))
    return steps


def trace_mixed(requests: Dict[Hashable, List[int]], seed: int = 0, live_max: int = 4, decode_tail: int = 12):
    """Up to ``live_max`` live requests; portions of some beside single tokens of others; some sit out."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: Dict[Hashable, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < live_max and (not live or rng.random() < 0.7):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            tokens = requests[rid]
            at = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                          # left out of this step, goes on later
            rest = len(tokens) - at
            if rest <= decode_tail:
                size = 1
            else:
                size = min(rest - decode_tail, rng.choice([2, 3, 5, 8, 16, 17, 31]))
                if size < 2:
                    size = rest - decode_tail + 1 if rest - decode_tail + 1 >= 2 else 1
            part = tokens[at:at + size]
            want = list(range(len(part))) if len(part) <= 4 or rng.random() < 0.5 else [len(part) - 1]
            entries.append((rid, part, want))
            live[rid] = at + len(part)
            if live[rid] >= len(tokens):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, end))
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The --max-tokens a trace needs: peak of the live requests' lengths, each rounded up."""
    held: Dict[Hashable, int] = {}
    peak = 0
    for entries, end in steps:
        for rid, tokens, _ in entries:
            held[rid] = held.get(rid, 0) + len(tokens)
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in end:
            held.pop(rid, None)
    return peak


def replay(stepper, steps) -> Dict[Tuple[Hashable, int], np.ndarray]:
    """Drive the engine's own step function through a trace; ``{(request, position): logits}``."""
    from tesseract_b200.engine import StepEntry

    out: Dict[Tuple[Hashable, int], np.ndarray] = {}
    at: Dict[Hashable, int] = {}
    for entries, end in steps:
        batch = []
        for rid, tokens, want in entries:
            if not stepper.cache.is_live(rid):
                assert stepper.cache.admit(rid)
            batch.append(StepEntry(rid, tokens, want))
        logits = stepper.step(batch)
        rows = logits.float().cpu().numpy() if logits is not None else None
        r = 0
        for rid, tokens, want in entries:
            base = at.get(rid, 0)
            for place in want:
                out[(rid, base + place)] = rows[r]
                r += 1
            at[rid] = base + len(tokens)
        for rid in end:
            stepper.cache.release(rid)
            at.pop(rid, None)
    return out


# Allowed |engine - plain|.  float32: summation-order noise only, 2e-5 of the request's largest |logit| (no
# absolute floor).  bfloat16: the bound is set from measured rounding noise, not chosen: the plain model has a
# mode that rounds every activation the serving path stores in bfloat16, and the largest deviation of that mode
# from float64 over the compared rows of a request (``bf16_noise``: 0.003 to 0.007 of the largest logit on the tiny
# models, 0.011 at a vocabulary of 128,256, where the maximum runs over many more entries) times NOISE_FACTOR is
# what the engine may deviate.  The engine rounds at the same places or fewer, so its deviation is a second draw
# from the same distribution; the factor covers the spread between two such maxima.  A wrongly merged split, a
# dropped key or a stale page moves a logit by many times that.  Where no noise is measured, REL["bfloat16"]
# of the largest |logit| stands (the tiny models' noise at its upper end, times the factor).
REL = {"float32": 2e-5, "bfloat16": 1e-2}
NOISE_FACTOR = 1.5
# A greedy token may differ from the plain model's only where its top two logits are closer than this fraction
# of the largest |logit| (each of the two may be off by REL).
GREEDY_MARGIN = {"float32": 1e-5, "bfloat16": 2e-2}


def plain_logits(folder: str, requests: Dict[Hashable, List[int]], round_to=None) -> Dict[Hashable, np.ndarray]:
    from tests.plain import llama

    config, tensors = llama.load_folder(folder)
    return {rid: llama.forward(config, tensors, tokens, round_to=round_to).numpy() for rid, tokens in requests.items()}


def bf16_noise(folder: str, requests: Dict[Hashable, List[int]], plain: Dict[Hashable, np.ndarray],
               head_rows=None) -> Dict[Hashable, float]:
    """Per request: the largest |plain model in its bfloat16-rounding mode - plain float64 model| (``plain``) over
    the rows compared."""
    from tests.plain import llama

    config, tensors = llama.load_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        rounded = llama.forward(config, tensors, tokens, dtype=torch.float32, round_to=torch.bfloat16,
                                head_rows=None if head_rows is None else head_rows[rid]).numpy()
        out[rid] = float(np.abs(rounded.astype(np.float64) - plain[rid]).max())
    return out


def keep_wants(steps, keep):
    """The same trace asking only for the positions in ``keep[request]`` (logits of a 128,256-wide vocabulary at
    every row would be hundreds of megabytes)."""
    at: Dict[Hashable, int] = {}
    out = []
    for entries, end in steps:
        filtered = []
        for rid, tokens, want in entries:
            base = at.get(rid, 0)
            filtered.append((rid, tokens, [p for p in want if base + p in keep[rid]]))
            at[rid] = base + len(tokens)
        out.append((filtered, end))
    return out


def compare(got: Dict[Tuple[Hashable, int], np.ndarray], plain: Dict[Hashable, np.ndarray], rel: float, what: str,
            rows_of=None, noise: Dict[Hashable, float] = None):
    """Every replayed row against the plain implementation: |d| <= rel * max|logit| of that row's request, or,
    with ``noise`` (see ``bf16_noise``), |d| <= NOISE_FACTOR * noise[request].
    ``rows_of[request]`` maps a position to its row of ``plain[request]`` when the plain model computed only some."""
    assert got, f"{what}: nothing was replayed"
    worst = 0.0
    for (rid, position), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        want = plain[rid][position if rows_of is None else rows_of[rid][position]]
        scale = float(np.abs(plain[rid]).max())
        err = float(np.abs(row.astype(np.float64) - want).max())
        assert np.isfinite(row).all(), f"{what}: request {rid} position {position} has non-finite logits"
        limit = rel * scale if noise is None else NOISE_FACTOR * noise[rid]
        assert err <= limit, (f"{what}: first wrong token is request {rid!r} position {position}: "
                              f"max |diff| {err:.3e} > {limit:.3e}")
        worst = max(worst, err / limit)
    return worst
