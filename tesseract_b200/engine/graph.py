"""CUDA-graph replay of pure decode steps.

A decode step of B single-token rows launches well over a hundred small kernels; at small
batches the launches, not the memory traffic, bound the step.  As the reference does
(src/cuda/dense_decoder/graph.rs:108-537: one captured graph per batch bucket and context
bucket, metadata copied in before each launch), a step in which every request brings one
token and wants its logits is captured once per (batch bucket, block-table width bucket)
and replayed: one host-to-device copy of the step's metadata, one graph launch (model and
sampling kernel), one device-to-host read of the sampled tokens.

Unlike the reference, temperature rows replay too (sampling runs on the device inside the
graph), and all graphs share the cache pages; rows that pad a batch up to its bucket point
at the scratch page and the scratch state slot, so they disturb nothing.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from ..parts.base import GroupView, StepContext
from .step import StepEntry, Stepper


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


class _Graph:
    """Persistent buffers and the captured graph for one (batch bucket, table width)."""

    def __init__(self, stepper: Stepper, batch: int, columns: int):
        cache, device = stepper.cache, stepper.runtime.device
        self.batch, self.columns = batch, columns
        self.paged = [i for i, g in enumerate(cache.groups) if g.pool is not None]
        ints = 3 * batch + len(self.paged) * batch * columns
        ints = (ints + 1) // 2 * 2                                  # keep the float64 block 8-byte aligned
        self.nbytes = ints * 4 + batch * 4 + (batch % 2) * 4 + batch * 8
        self.host = torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=True)
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)

        def carve(buffer):
            at = 0
            out = {}
            for name, count, dtype, width in (("tokens", batch, torch.int32, 4), ("positions", batch, torch.int32, 4),
                                              ("slots", batch, torch.int32, 4)):
                out[name] = buffer[at:at + count * width].view(dtype)
                at += count * width
            out["tables"] = []
            for _ in self.paged:
                out["tables"].append(buffer[at:at + batch * columns * 4].view(torch.int32).view(batch, columns))
                at += batch * columns * 4
            at = ints * 4
            out["temps"] = buffer[at:at + batch * 4].view(torch.float32)
            at += batch * 4 + (batch % 2) * 4
            out["uniform"] = buffer[at:at + batch * 8].view(torch.float64)
            return out

        self.h = carve(self.host)
        self.d = carve(self.dev)
        self.h_np = {k: (v.numpy() if not isinstance(v, list) else [t.numpy() for t in v]) for k, v in self.h.items()}
        self.h_np["slots"][:] = cache.scratch_slot
        self.dev.copy_(self.host)
        arange = torch.arange(batch + 1, dtype=torch.int32, device=device)
        self.out_tokens = torch.zeros(batch, dtype=torch.int32, device=device)
        groups: List[GroupView] = []
        tables = dict(zip(self.paged, self.d["tables"]))
        for index, g in enumerate(cache.groups):
            groups.append(GroupView(tables.get(index), cache.page_size if g.pool is not None else 0))
        self.ctx = StepContext(
            num_rows=batch, num_seqs=batch, token_ids=self.d["tokens"], positions=self.d["positions"],
            seq_of_row=arange[:batch], row_start=arange, seq_begin=self.d["positions"], state_slots=self.d["slots"],
            groups=groups, host_new=[1] * batch, host_begin=(), host_slots=(), max_new=1,
            max_context=columns * cache.page_size)
        self.want_rows = arange[:batch]
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._capture(stepper)

    def _run(self, stepper: Stepper) -> torch.Tensor:
        logits = stepper.model.forward(self.ctx, stepper.cache.bindings, self.want_rows)
        kernels.sample(logits, self.d["temps"], self.d["uniform"], self.out_tokens)
        return logits

    def _capture(self, stepper: Stepper) -> None:
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                      # warm-up: library workspaces and scratch buffers settle
                self._run(stepper)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count
        with torch.cuda.graph(graph):
            self.logits = self._run(stepper)
        self.kernels_per_replay = kernels.launch_count - before     # this package's kernels inside the graph
        self.graph = graph
        torch.cuda.synchronize()


class DecodeGraphs:
    """Chooses, captures and replays decode graphs for a :class:`Stepper`."""

    def __init__(self, stepper: Stepper, max_batch: int):
        self.stepper = stepper
        self.max_batch = max_batch
        self.graphs: Dict[Tuple[int, int], _Graph] = {}
        self.replays = 0
        self.captures = 0
        self.kernels_replayed = 0
        self.safe = all(getattr(block.mixer, "graph_safe", False) for block in stepper.model.layers)

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (self.safe and len(entries) <= self.max_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def step(self, entries: Sequence[StepEntry], temperatures: Sequence[float], draws: Sequence[float]
             ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Run one pure-decode step; returns (tokens int32 [B] on the device, logits [B, vocab])."""
        stepper, cache = self.stepper, self.stepper.cache
        stepper._validate(entries)
        for entry in entries:
            cache.extend(entry.request, 1)
        count = len(entries)
        lengths = [cache.length(e.request) for e in entries]
        pages = -(-(max(lengths) + 1) // cache.page_size)
        key = (min(_next_pow2(count), max(self.max_batch, count)), max(8, _next_pow2(pages)))
        graph = self.graphs.get(key)
        if graph is None:
            graph = _Graph(stepper, *key)
            self.graphs[key] = graph
            self.captures += 1
        h = graph.h_np
        slots = [cache.slot(e.request) for e in entries]
        h["tokens"][:count] = [int(e.tokens[0]) for e in entries]
        h["positions"][:count] = lengths
        h["slots"][:count] = slots
        h["temps"][:count] = temperatures
        h["uniform"][:count] = draws
        if count < graph.batch:
            h["tokens"][count:] = 0
            h["positions"][count:] = 0
            h["slots"][count:] = cache.scratch_slot
            h["temps"][count:] = 0.0
        for table, group_index in zip(h["tables"], graph.paged):
            table[:count] = cache.block_table_rows(group_index, slots, graph.columns)
            if count < graph.batch:
                table[count:] = 0
        graph.dev.copy_(graph.host, non_blocking=True)
        graph.graph.replay()
        for entry in entries:
            cache.commit(entry.request, 1)
        stepper.steps_run += 1
        self.replays += 1
        self.kernels_replayed += graph.kernels_per_replay
        return graph.out_tokens[:count], graph.logits[:count]
