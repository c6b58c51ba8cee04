"""Choosing tokens from 32-bit logits.

Greedy and temperature rows are chosen on the device by the package's sampling kernel
(argmax with ties to the lowest id, src/cuda/kernels.rs:803-873; inverse-CDF sampling
with the step's uniform draw).  Rows with ``top_p < 1`` are read back and chosen on the
host by a restatement of the reference's host sampler (src/engine/sampling.rs:38-75):
weights ``exp(l/T - max)`` in 64-bit, sorted by weight, the shortest prefix holding
``top_p`` of the mass, then the draw scaled by the retained mass.
"""

from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import kernels


class InvalidLogits(ValueError):
    """Empty or non-finite logits reached the sampler (src/engine/sampling.rs:24-27)."""


def sample_top_p_host(logits: np.ndarray, temperature: float, top_p: float, draw: float) -> int:
    if logits.size == 0 or not np.isfinite(logits).all():
        raise InvalidLogits("sampler received empty or non-finite logits")
    if temperature == 0.0:
        return int(np.argmax(logits))
    scaled = logits.astype(np.float32) * (np.float32(1.0) / np.float32(temperature))
    weights = np.exp((scaled - scaled.max()).astype(np.float64))
    order = np.argsort(-weights, kind="stable")
    sorted_weights = weights[order]
    total = float(sorted_weights.sum())
    if not np.isfinite(total) or total <= 0.0:
        raise InvalidLogits("sampler probability mass is invalid")
    cumulative = np.cumsum(sorted_weights)
    kept = int(np.searchsorted(cumulative, total * top_p, side="left")) + 1
    kept = min(kept, logits.size)
    retained = float(cumulative[kept - 1])
    pick = int(np.searchsorted(cumulative[:kept], draw * retained, side="right"))
    return int(order[min(pick, kept - 1)])


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], top_ps: Sequence[float],
               draws: Sequence[float]) -> List[int]:
        """One token per logits row."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        if not (len(temperatures) == len(top_ps) == len(draws) == rows):
            raise ValueError("one temperature, top_p and draw per logits row")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(t == 0.0 for t in temperatures):
            kernels.argmax(logits, out)
            return out.cpu().tolist()
        temps = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
        uniform = torch.tensor(list(draws), dtype=torch.float64).to(self.device, non_blocking=True)
        kernels.sample(logits, temps, uniform, out)
        tokens = out.cpu().tolist()
        nucleus = [i for i in range(rows) if temperatures[i] > 0.0 and top_ps[i] < 1.0]
        if nucleus:
            index = torch.tensor(nucleus, dtype=torch.long, device=self.device)
            host = logits.index_select(0, index).cpu().numpy()
            for k, i in enumerate(nucleus):
                tokens[i] = sample_top_p_host(host[k], temperatures[i], top_ps[i], draws[i])
        return tokens
