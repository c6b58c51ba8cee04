"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere
(the reference's ragged batch, src/engine/batch.rs:175-239 and its lowering into flat
arrays, src/cuda/batch.rs:29-105).  It runs only the tokens it is given, as one packed
batch, against the keys and values that earlier steps left in the cache, and returns
32-bit logits at the wanted places only.  Generation, the scheduler, trace replay and
the benchmark all go through this one function.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..parts.base import GroupView, Runtime, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    """A step that breaks an invariant of the batch (src/engine/batch.rs:186-239)."""


class _Staging:
    """A small ring of pinned host buffers, so that a step's metadata goes up in one copy."""

    def __init__(self, device, depth: int = 4):
        self.device = device
        self.depth = depth
        self.host: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.cursor = 0

    def upload(self, arrays: Sequence[np.ndarray]) -> List[torch.Tensor]:
        offsets = []
        total = 0
        for a in arrays:
            offsets.append(total)
            total += (a.size + 3) // 4 * 4          # keep every array 16-byte aligned
        total = max(total, 4)
        index = self.cursor
        self.cursor = (self.cursor + 1) % self.depth
        if self.events[index] is not None:
            self.events[index].synchronize()
        host = self.host[index]
        if host is None or host.numel() < total:
            host = torch.empty(max(total, 1024), dtype=torch.int32, pin_memory=True)
            self.host[index] = host
        view = host.numpy()
        for a, off in zip(arrays, offsets):
            view[off:off + a.size] = a.reshape(-1)
        device_buffer = torch.empty(total, dtype=torch.int32, device=self.device)
        device_buffer.copy_(host[:total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[index] = event
        return [device_buffer[off:off + a.size].view(a.shape) for a, off in zip(arrays, offsets)]


class Stepper:
    """Owns nothing but the wiring: model, cache manager and the staging of batch metadata."""

    def __init__(self, model: DecoderModel, cache: CacheManager):
        self.model = model
        self.cache = cache
        self.runtime: Runtime = model.runtime
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self._staging = _Staging(self.runtime.device)
        self.steps_run = 0
        self.graphs = None          # set by enable_graphs()
        self.chunk_graphs = None    # set by enable_graphs(chunk_rows=...)
        self._sampler = None

    # ------------------------------------------------------------------ validation
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for entry in entries:
            if entry.request in seen:
                raise StepError(f"request {entry.request!r} appears twice in one step")
            seen.add(entry.request)
            if not self.cache.is_live(entry.request):
                raise StepError(f"request {entry.request!r} is not live (admit it first)")
            count = len(entry.tokens)
            if count == 0:
                raise StepError(f"request {entry.request!r} brings no tokens")
            ids = np.asarray(entry.tokens)
            if ids.dtype.kind not in "iu" or ids.ndim != 1:
                raise StepError(f"the tokens of request {entry.request!r} are not a list of integers")
            low, high = int(ids.min()), int(ids.max())
            if low < 0 or high >= self.vocab_size:
                raise StepError(f"token id {low if low < 0 else high} of request {entry.request!r} is outside the "
                                f"vocabulary of {self.vocab_size}")
            for place in entry.want:
                if not 0 <= int(place) < count:
                    raise StepError(f"wanted place {place} of request {entry.request!r} is outside its "
                                    f"{count} tokens")
            if self.cache.length(entry.request) + count > self.max_positions:
                raise StepError(f"request {entry.request!r} would pass the model's {self.max_positions} positions")

    # ------------------------------------------------------------------ the step
    def build_context(self, entries: Sequence[StepEntry]) -> Tuple[StepContext, Optional[torch.Tensor], int]:
        """Lower the entries into packed device arrays (pages must already exist)."""
        cache = self.cache
        new = [len(e.tokens) for e in entries]
        begin = [cache.length(e.request) for e in entries]
        slots = [cache.slot(e.request) for e in entries]
        num_seqs = len(entries)
        num_rows = sum(new)
        row_start = np.zeros(num_seqs + 1, dtype=np.int32)
        np.cumsum(new, out=row_start[1:])
        token_ids = np.fromiter((int(t) for e in entries for t in e.tokens), dtype=np.int32, count=num_rows)
        seq_of_row = np.repeat(np.arange(num_seqs, dtype=np.int32), new)
        begin_arr = np.asarray(begin, dtype=np.int32)
        positions = (np.arange(num_rows, dtype=np.int32) - row_start[:-1][seq_of_row] + begin_arr[seq_of_row]).astype(np.int32)
        want_rows = np.asarray([int(row_start[i]) + int(p) for i, e in enumerate(entries) for p in e.want],
                               dtype=np.int32)
        max_context = max(b + n for b, n in zip(begin, new))
        columns = -(-max_context // cache.page_size)
        arrays = [token_ids, positions, seq_of_row, row_start, begin_arr, np.asarray(slots, dtype=np.int32), want_rows]
        paged = [i for i, g in enumerate(cache.groups) if g.pool is not None]
        for group_index in paged:
            arrays.append(cache.block_table_rows(group_index, slots, columns))
        device = self._staging.upload(arrays)
        groups: List[GroupView] = []
        tables = dict(zip(paged, device[7:]))
        for index, g in enumerate(cache.groups):
            groups.append(GroupView(block_table=tables.get(index), page_size=cache.page_size if g.pool else 0))
        ctx = StepContext(
            num_rows=num_rows, num_seqs=num_seqs, token_ids=device[0], positions=device[1], seq_of_row=device[2],
            row_start=device[3], seq_begin=device[4], state_slots=device[5], groups=groups,
            host_new=new, host_begin=begin, host_slots=slots, max_new=max(new), max_context=max_context)
        return ctx, (device[6] if want_rows.size else None), int(want_rows.size)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch; return float32 logits ``[wanted, vocab]`` on the device, or ``None``.  (A replayed
        prompt portion returns a buffer that the next such step overwrites: read it before that.)"""
        if self.chunk_graphs is not None and self.chunk_graphs.eligible(entries):
            return self.chunk_graphs.step(entries)
        self._validate(entries)
        for entry in entries:
            self.cache.extend(entry.request, len(entry.tokens))
        ctx, want_rows, _ = self.build_context(entries)
        # every place of every entry wanted, in order (a decode step): the model need not pick rows out, and takes
        # the same path as a replayed decode step, bit for bit
        every_row = all(list(e.want) == list(range(len(e.tokens))) for e in entries)
        logits = self.model.forward(ctx, self.cache.bindings, want_rows, want_every_row=every_row)
        for entry in entries:
            self.cache.commit(entry.request, len(entry.tokens))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ step + sampling
    def enable_graphs(self, max_batch: int, chunk_rows: Optional[int] = None,
                      max_sequence_length: Optional[int] = None, max_batch_tokens: Optional[int] = None) -> None:
        """Replay pure decode steps as CUDA graphs from now on (if every part of the model allows it), and, with
        ``chunk_rows``, steps in which one or more sequences (as many as fit ``max_batch_tokens``) bring exactly
        that many prompt tokens each, beside single decoded tokens of others."""
        from .graph import ChunkGraphs, DecodeGraphs

        self.graphs = DecodeGraphs(self, max_batch)
        if chunk_rows is not None and chunk_rows > 16:
            portions = max(1, (max_batch_tokens or chunk_rows) // chunk_rows)
            self.chunk_graphs = ChunkGraphs(self, chunk_rows, max_sequence_length or self.max_positions, max_batch,
                                            max_portions=portions)

    def step_and_sample(self, entries: Sequence[StepEntry], temperatures: Sequence[float], top_ps: Sequence[float],
                        draws: Sequence[float]) -> List[int]:
        """One step, then one token per wanted row (entries want at most their last place).

        ``temperatures``, ``top_ps`` and ``draws`` hold one value per wanted row, in order.
        """
        from ..sampling.sampler import Sampler, sample_top_p_host

        if self._sampler is None:
            self._sampler = Sampler(self.runtime.device)
        wanted = sum(len(e.want) for e in entries)
        if wanted == 0:
            self.step(entries)
            return []
        if self.graphs is not None and wanted == len(entries) and self.graphs.eligible(entries):
            out, logits = self.graphs.step(entries, temperatures, draws)
            for i, (t, p) in enumerate(zip(temperatures, top_ps)):
                if t > 0.0 and p < 1.0:
                    out[i] = sample_top_p_host(logits[i].cpu().numpy(), t, p, draws[i])
            return out
        logits = self.step(entries)
        return self._sampler.sample(logits, temperatures, top_ps, draws)

    def can_launch_decode(self, rows: int, top_ps: Sequence[float]) -> bool:
        """Whether :meth:`launch_decode` takes a batch of ``rows`` single-token rows with these top-p values: a
        graph-replayed decode step, sampled on the device."""
        return (self.graphs is not None and self.graphs.safe and 0 < rows <= self.graphs.max_batch
                and all(p >= 1.0 for p in top_ps))

    def launch_decode(self, entries: Sequence[StepEntry], temperatures: Sequence[float], draws: Sequence[float],
                      previous=None, fed: Optional[Sequence[bool]] = None):
        """Enqueue a decode step without waiting for it; ``launch.tokens()`` waits and returns its tokens.  Entries
        marked in ``fed`` take their token from ``previous`` (the launch before) on the device."""
        return self.graphs.launch(entries, temperatures, draws, previous, fed)
