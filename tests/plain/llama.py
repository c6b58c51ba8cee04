"""Plain, slow Llama: whole sequences, no cache, one function per part.

Written from the reference's formulas only (each function cites the file and lines of
Leikoe/tesseract it restates).  The reference cannot be compiled or imported here (it
is Rust with run-time compiled GPU kernels and has no CPU forward pass), so this module
rests on those formulas, not on outputs of the reference.  It shares no code with
``tesseract_b200``: it reads ``config.json`` and ``model.safetensors`` itself (through
the ``safetensors`` wheel) and computes with torch on the CPU.

``dtype`` is the arithmetic precision (float64 by default: the "exact" answer that
both the float32 and the bfloat16 engine paths are compared with).  ``round_to`` =
``torch.bfloat16`` additionally rounds every activation that the reference stores in
bfloat16, to model the serving path's rounding points.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
from safetensors import safe_open


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name)
    return config, tensors


def _rnd(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


def embed(tokens: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """h[t] = E[token[t]] — a pure gather, no scale (src/cuda/kernels.rs:10-24)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, round_to=None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, rounded once (src/cuda/kernels.rs:26-57)."""
    inv = torch.rsqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return _rnd(x * inv * weight, round_to)


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> np.ndarray:
    """Llama-3 scaled inverse frequencies in float32 (src/cuda/dense_decoder.rs:1520-1544)."""
    f32 = np.float32
    out = []
    for index in range(head_dim // 2):
        exponent = f32(2 * index) / f32(head_dim)
        base = f32(1.0) / f32(np.power(f32(theta), exponent))
        freq = base
        if scaling is not None:
            orig = f32(scaling["original_max_position_embeddings"])
            low, high, factor = f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"]), f32(scaling["factor"])
            wavelength = f32(math.tau) / base
            if wavelength < orig / high:
                freq = base
            elif wavelength > orig / low:
                freq = base / factor
            else:
                smooth = (orig / wavelength - low) / (high - low)
                freq = (f32(1.0) - smooth) * base / factor + smooth * base
        out.append(f32(freq))
    return np.asarray(out, dtype=np.float32)


def rope_tables(positions: Sequence[int], inv_freq: np.ndarray):
    """cos/sin of float32(position) * frequency, in float32 (src/cuda/dense_decoder.rs:1549-1556)."""
    pos = np.asarray(list(positions), dtype=np.float32)[:, None]
    angle = (pos * inv_freq[None, :]).astype(np.float32)
    # float64 trigonometry of the float32 angle, rounded to float32: the correctly rounded table entry
    return (torch.from_numpy(np.cos(angle.astype(np.float64)).astype(np.float32)),
            torch.from_numpy(np.sin(angle.astype(np.float64)).astype(np.float32)))


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, round_to=None) -> torch.Tensor:
    """x: [T, heads, d]; lo*cos - hi*sin | hi*cos + lo*sin (src/cuda/kernels.rs:210-242)."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return _rnd(torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1), round_to)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None,
              round_to=None) -> torch.Tensor:
    """Causal grouped-query softmax attention of a whole sequence (src/cuda/kernels.rs:447-562).

    q: [T, nh, d], k and v: [T, nkv, d].  Row t sees keys 0..t (or the last ``window``);
    query head h reads kv head h // (nh / nkv); scores are scaled before masking; the
    probabilities that multiply V are rounded when ``round_to`` is given, the sum is not.
    """
    T, nh, d = q.shape
    group = nh // k.shape[1]
    out = torch.empty_like(q)
    idx = torch.arange(T)
    mask = idx[None, :] <= idx[:, None]
    if window:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh, vh = k[:, h // group], v[:, h // group]
        s = (q[:, h] @ kh.T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(-1, keepdim=True).values
        p = torch.exp(s - m)
        l = p.sum(-1, keepdim=True)
        out[:, h] = (_rnd(p, round_to) @ vh) / l.clamp_min(1e-8)
    return _rnd(out, round_to)


def swiglu(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, round_to=None) -> torch.Tensor:
    """down( silu(x Wg^T) * (x Wu^T) ) (src/cuda/dense_decoder.rs:737-774, src/cuda/kernels.rs:191-208)."""
    g = _rnd(x @ gate.T, round_to)
    u = _rnd(x @ up.T, round_to)
    a = _rnd(g * (1.0 / (1.0 + torch.exp(-g))) * u, round_to)
    return _rnd(a @ down.T, round_to)


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            round_to: Optional[torch.dtype] = None, head_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (layer order of src/cuda/dense_decoder.rs:644-831); with
    ``head_rows`` only those rows go through the final norm and the head (src/cuda/dense_decoder.rs:784-823)."""
    w = {name: t.to(dtype) for name, t in tensors.items()}
    nh, nkv = config["num_attention_heads"], config.get("num_key_value_heads") or config["num_attention_heads"]
    d = config.get("head_dim") or config["hidden_size"] // nh
    eps = config["rms_norm_eps"]
    T = len(tokens)
    inv_freq = rope_inverse_frequencies(d, config["rope_theta"], config.get("rope_scaling"))
    cos, sin = rope_tables(range(T), inv_freq)
    h = embed(tokens, w["model.embed_tokens.weight"])
    pending = None      # the feed-forward output that the next norm adds (src/cuda/dense_decoder.rs:668-672)
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        # statistics on the unrounded sum; the residual is rounded once per addition (src/cuda/kernels.rs:59-103)
        c = h if pending is None else h + pending
        x = rms_norm(c, w[f"{p}.input_layernorm.weight"], eps, round_to)
        h = _rnd(c, round_to)
        q = _rnd(x @ w[f"{p}.self_attn.q_proj.weight"].T, round_to).view(T, nh, d)
        k = _rnd(x @ w[f"{p}.self_attn.k_proj.weight"].T, round_to).view(T, nkv, d)
        v = _rnd(x @ w[f"{p}.self_attn.v_proj.weight"].T, round_to).view(T, nkv, d)
        q, k = rotate_half(q, cos, sin, round_to), rotate_half(k, cos, sin, round_to)
        a = attention(q, k, v, 1.0 / math.sqrt(d), None, round_to).reshape(T, nh * d)
        o = _rnd(a @ w[f"{p}.self_attn.o_proj.weight"].T, round_to)
        c = h + o
        m = rms_norm(c, w[f"{p}.post_attention_layernorm.weight"], eps, round_to)
        h = _rnd(c, round_to)
        pending = swiglu(m, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                         w[f"{p}.mlp.down_proj.weight"], round_to)
    h = h if pending is None else h + pending
    if head_rows is not None:
        h = h[list(head_rows)]
    final = rms_norm(h, w["model.norm.weight"], eps, round_to)
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    return final @ head.T


class SplitMix64:
    """The reference's per-request generator (src/engine/scheduler.rs:326-343)."""

    def __init__(self, seed: int):
        self.state = seed & 0xFFFFFFFFFFFFFFFF

    def unit_f64(self) -> float:
        mask = 0xFFFFFFFFFFFFFFFF
        self.state = (self.state + 0x9E3779B97F4A7C15) & mask
        v = self.state
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & mask
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & mask
        v ^= v >> 31
        return (v >> 11) * (1.0 / (1 << 53))


def sample_host(logits: Sequence[float], temperature: float, top_p: float, draw: float) -> int:
    """The reference's host sampler (src/engine/sampling.rs:23-75), greedy ties to the lowest id
    as its device argmax does (src/cuda/kernels.rs:803-873)."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature == 0.0:
        return int(np.argmax(logits))
    inv = np.float32(1.0) / np.float32(temperature)
    scaled = logits * inv
    weights = np.exp((scaled - scaled.max()).astype(np.float64))
    order = np.argsort(-weights, kind="stable")
    total = weights.sum()
    cutoff = total * top_p
    mass, kept = 0.0, 0
    for i in order:
        mass += weights[i]
        kept += 1
        if mass >= cutoff:
            break
    target = draw * mass
    cumulative = 0.0
    for i in order[:kept]:
        cumulative += weights[i]
        if target < cumulative:
            return int(i)
    return int(order[kept - 1])


def sample_in_token_order(logits: Sequence[float], temperature: float, draw: float) -> int:
    """Inverse CDF over token ids in ascending order (the engine's device sampler, top_p = 1)."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature <= 0.0:
        return int(np.argmax(logits))
    scaled = logits * (np.float32(1.0) / np.float32(temperature))
    weights = np.exp((scaled - scaled.max()).astype(np.float64))
    cumulative = np.cumsum(weights)
    return int(min(np.searchsorted(cumulative, draw * cumulative[-1], side="right"), len(logits) - 1))
