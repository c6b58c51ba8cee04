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

import gc
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


def graph_safe(model) -> bool:
    """Whether a step of this model may be captured: every part that runs in it (each block's norms, mixer and
    feed-forward, the embedding, the final norm and the head) declares ``graph_safe``, i.e. that everything which
    varies between two steps of the same shape reaches it through device tensors, never through a host-side field
    of the step context."""
    parts = [model.embedding, model.final_norm, model.head]
    for block in model.layers:
        parts += [block.mixer, block.feed_forward, *block.norms.values()]
    return all(getattr(part, "graph_safe", False) for part in parts)


HOST_RING = 3          # pinned copies of a graph's metadata: a launch may be prepared while two are still in flight


class _Graph:
    """Persistent buffers and the captured graph for one (batch bucket, table width)."""

    def __init__(self, stepper: Stepper, batch: int, columns: int, sampled: torch.Tensor):
        cache, device = stepper.cache, stepper.runtime.device
        self.batch, self.columns = batch, columns
        self.paged = [i for i, g in enumerate(cache.groups) if g.pool is not None]
        ints = 4 * batch + len(self.paged) * batch * columns
        ints = (ints + 1) // 2 * 2                                  # keep the float64 block 8-byte aligned
        self.nbytes = ints * 4 + batch * 4 + (batch % 2) * 4 + batch * 8
        self.hosts = [torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=True) for _ in range(HOST_RING)]
        self.host_events: List[Optional[torch.cuda.Event]] = [None] * HOST_RING
        self.next_host = 0
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)

        def carve(buffer):
            at = 0
            out = {}
            for name in ("tokens", "feed", "positions", "slots"):
                out[name] = buffer[at:at + batch * 4].view(torch.int32)
                at += batch * 4
            out["tables"] = []
            for _ in self.paged:
                out["tables"].append(buffer[at:at + batch * columns * 4].view(torch.int32).view(batch, columns))
                at += batch * columns * 4
            at = ints * 4
            out["temps"] = buffer[at:at + batch * 4].view(torch.float32)
            at += batch * 4 + (batch % 2) * 4
            out["uniform"] = buffer[at:at + batch * 8].view(torch.float64)
            return out

        self.d = carve(self.dev)
        self.h_np = []
        for host in self.hosts:
            views = carve(host)
            arrays = {k: (v.numpy() if not isinstance(v, list) else [t.numpy() for t in v]) for k, v in views.items()}
            arrays["slots"][:] = cache.scratch_slot
            arrays["feed"][:] = -1
            self.h_np.append(arrays)
        self.dev.copy_(self.hosts[0])
        arange = torch.arange(batch + 1, dtype=torch.int32, device=device)
        self.sampled = sampled                       # shared by all graphs: row i holds the last token of row i
        self.tokens = torch.zeros(batch, dtype=torch.int32, device=device)   # this step's token ids, chosen on the device
        groups: List[GroupView] = []
        tables = dict(zip(self.paged, self.d["tables"]))
        for index, g in enumerate(cache.groups):
            groups.append(GroupView(tables.get(index), cache.page_size if g.pool is not None else 0))
        self.ctx = StepContext(
            num_rows=batch, num_seqs=batch, token_ids=self.tokens, positions=self.d["positions"],
            seq_of_row=arange[:batch], row_start=arange, seq_begin=self.d["positions"], state_slots=self.d["slots"],
            groups=groups, host_new=[1] * batch, host_begin=(), host_slots=(), max_new=1,
            max_context=columns * cache.page_size)
        self.want_rows = arange[:batch]
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._capture(stepper)

    def host_arrays(self) -> Tuple[int, dict]:
        """The next pinned metadata block of the ring, once the copy that last read it is done."""
        index = self.next_host
        self.next_host = (index + 1) % HOST_RING
        event = self.host_events[index]
        if event is not None:
            event.synchronize()
        return index, self.h_np[index]

    def _run(self, stepper: Stepper) -> torch.Tensor:
        # a row's token comes from the host or, for a sequence that decoded in the step before, from that step's
        # sampler output, which never leaves the device
        kernels.select_tokens(self.d["tokens"], self.d["feed"], self.sampled, self.tokens, stepper.vocab_size)
        logits = stepper.model.forward(self.ctx, stepper.cache.bindings, self.want_rows, want_every_row=True)
        # the head may have left each of its CTAs' best token per row: the sampler's second stage of the argmax
        partials = getattr(stepper.model.head, "argmax_partials", lambda: None)()
        kernels.sample(logits, self.d["temps"], self.d["uniform"], self.sampled[:self.batch], partials=partials)
        return logits

    def _capture(self, stepper: Stepper) -> None:
        torch.cuda.synchronize()
        kept = self.sampled.clone()                 # the step before may be feeding its tokens to this one
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                      # warm-up: library workspaces and scratch buffers settle
                self._run(stepper)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.sampled.copy_(kept)
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count
        # No destructor may run while the stream is capturing: a dead graph of an earlier engine that the cycle
        # collector happened to free right then would make a CUDA call that invalidates the capture.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                self.logits = self._run(stepper)
        finally:
            if collecting:
                gc.enable()
        self.kernels_per_replay = kernels.launch_count - before     # this package's kernels inside the graph
        self.graph = graph
        torch.cuda.synchronize()


class DecodeLaunch:
    """A decode step that has been launched: where each request's row is, and where its tokens will arrive."""

    def __init__(self, rows: Dict, count: int, host_tokens: torch.Tensor, done: torch.cuda.Event, graph: _Graph):
        self.rows = rows                  # request -> row of this step
        self.count = count
        self.host_tokens = host_tokens    # pinned int32, filled by an asynchronous copy
        self.done = done
        self.graph = graph

    def tokens(self) -> List[int]:
        """Wait for the step and return its sampled tokens, one per row, in row order."""
        self.done.synchronize()
        return self.host_tokens[:self.count].tolist()


class DecodeGraphs:
    """Chooses, captures and replays decode graphs for a :class:`Stepper`."""

    def __init__(self, stepper: Stepper, max_batch: int):
        self.stepper = stepper
        self.max_batch = max_batch
        self.graphs: Dict[Tuple[int, int], _Graph] = {}
        self.replays = 0
        self.captures = 0
        self.kernels_replayed = 0
        self.safe = graph_safe(stepper.model)
        widest = max(_next_pow2(max_batch), max_batch)
        self.sampled = torch.zeros(widest, dtype=torch.int32, device=stepper.runtime.device)
        self._token_ring = [torch.zeros(widest, dtype=torch.int32, pin_memory=True) for _ in range(HOST_RING)]
        self._token_events: List[Optional[torch.cuda.Event]] = [None] * HOST_RING
        self._next_tokens = 0

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (self.safe and len(entries) <= self.max_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def launch(self, entries: Sequence[StepEntry], temperatures: Sequence[float], draws: Sequence[float],
               previous: Optional[DecodeLaunch] = None, fed: Optional[Sequence[bool]] = None) -> DecodeLaunch:
        """Enqueue one pure-decode step and return at once.  ``fed[i]`` says that entry i's token is whatever
        ``previous`` sampled for the same request (the entry's own token is then ignored): the step can be
        launched before the host has seen that token."""
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
            graph = _Graph(stepper, *key, self.sampled)
            self.graphs[key] = graph
            self.captures += 1
        slot_index, h = graph.host_arrays()
        slots = [cache.slot(e.request) for e in entries]
        h["tokens"][:count] = [int(e.tokens[0]) for e in entries]
        feed = [-1] * count
        if previous is not None and fed is not None:
            for i, entry in enumerate(entries):
                if fed[i]:
                    feed[i] = previous.rows[entry.request]
        h["feed"][:count] = feed
        h["positions"][:count] = lengths
        h["slots"][:count] = slots
        h["temps"][:count] = temperatures
        h["uniform"][:count] = draws
        if count < graph.batch:
            h["tokens"][count:] = 0
            h["feed"][count:] = -1
            h["positions"][count:] = 0
            h["slots"][count:] = cache.scratch_slot
            h["temps"][count:] = 0.0
        for table, group_index in zip(h["tables"], graph.paged):
            table[:count] = cache.block_table_rows(group_index, slots, graph.columns)
            if count < graph.batch:
                table[count:] = 0
        graph.dev.copy_(graph.hosts[slot_index], non_blocking=True)
        copied = torch.cuda.Event()
        copied.record()
        graph.host_events[slot_index] = copied
        graph.graph.replay()
        # the sampled tokens go to pinned memory at once: the next launch may overwrite the sampler's rows
        ring = self._next_tokens
        self._next_tokens = (ring + 1) % HOST_RING
        if self._token_events[ring] is not None:
            self._token_events[ring].synchronize()
        self._token_ring[ring][:count].copy_(self.sampled[:count], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._token_events[ring] = done
        for entry in entries:
            cache.commit(entry.request, 1)
        stepper.steps_run += 1
        self.replays += 1
        self.kernels_replayed += graph.kernels_per_replay
        return DecodeLaunch({e.request: i for i, e in enumerate(entries)}, count, self._token_ring[ring], done, graph)

    def step(self, entries: Sequence[StepEntry], temperatures: Sequence[float], draws: Sequence[float]
             ) -> Tuple[List[int], torch.Tensor]:
        """Run one pure-decode step and wait for it; returns (tokens, logits [B, vocab] on the device)."""
        launch = self.launch(entries, temperatures, draws)
        return launch.tokens(), launch.graph.logits[:launch.count]


class _ChunkGraph:
    """Buffers and the captured graph for steps in which ``portions`` sequences bring ``rows`` prompt tokens each
    (rows ``k * rows`` .. ``(k + 1) * rows - 1``), then (``tail`` > 0) one sequence brings the end of its prompt,
    fewer than ``tail`` tokens, and up to ``decodes`` others one decoded token each (the rows after them, all
    wanted).  With ``wants_last`` the last row of every portion goes through the head as well (the caller picks the
    ones it asked for); without, no portion row does.

    A tail has ``tail`` rows in the graph whatever its length: the rows behind its last token belong to a padding
    sequence whose block table names the scratch page only and whose state slot is the scratch slot, so that they
    compute on garbage and touch nothing.  Which rows are the tail's and which the padding's is data (the row
    starts, the sequence of each row, the row that goes through the head), so one graph serves every tail length
    below ``tail``.  The tail's last row always goes through the head."""

    def __init__(self, stepper: Stepper, rows: int, portions: int, decodes: int, wants_last: bool, columns: int,
                 pool=None, tail: int = 0):
        cache, device = stepper.cache, stepper.runtime.device
        self.rows, self.portions, self.decodes, self.columns = rows, portions, decodes, columns
        self.wants_last, self.tail = wants_last, tail
        prompt_rows = portions * rows + tail
        extra = 2 if tail else 0                       # the tail's sequence and the padding's
        total, seqs = prompt_rows + decodes, portions + extra + decodes
        self.total, self.seqs, self.prompt_rows = total, seqs, prompt_rows
        self.paged = [i for i, g in enumerate(cache.groups) if g.pool is not None]
        wanted = ([(k + 1) * rows - 1 for k in range(portions)] if wants_last else [])
        self.tail_want = len(wanted) if tail else None           # where among the wanted rows the tail's stands
        if tail:
            wanted.append(prompt_rows - 2)
        wanted += list(range(prompt_rows, total))
        self.wanted = len(wanted)
        # int32 block: tokens[total] positions[total] begin[seqs] slot[seqs], and with a tail seq_of_row[total]
        # row_start[seqs + 1] want[wanted]; block tables apart (only the columns in use are copied)
        self.ints = 2 * total + 2 * seqs + ((total + seqs + 1 + len(wanted)) if tail else 0)
        self.hosts = [torch.zeros(self.ints, dtype=torch.int32, pin_memory=True) for _ in range(HOST_RING)]
        self.host_tables = [[torch.zeros((seqs, columns), dtype=torch.int32, pin_memory=True) for _ in self.paged]
                            for _ in range(HOST_RING)]
        self.host_events: List[Optional[torch.cuda.Event]] = [None] * HOST_RING
        self.next_host = 0
        self.dev = torch.zeros(self.ints, dtype=torch.int32, device=device)
        self.dev_tables = [torch.zeros((seqs, columns), dtype=torch.int32, device=device) for _ in self.paged]
        d = self.dev
        tables = dict(zip(self.paged, self.dev_tables))
        groups = [GroupView(tables.get(index), cache.page_size if g.pool is not None else 0)
                  for index, g in enumerate(cache.groups)]
        seq_of_row_host = torch.cat([torch.arange(portions, dtype=torch.int32).repeat_interleave(rows),
                                     torch.full((max(0, tail - 1),), portions, dtype=torch.int32),
                                     torch.full((1 if tail else 0,), portions + 1, dtype=torch.int32),
                                     torch.arange(portions + extra, seqs, dtype=torch.int32)])
        row_start_host = torch.cat([torch.arange(0, portions * rows, rows, dtype=torch.int32),
                                    torch.tensor([portions * rows, prompt_rows - 1] if tail else [], dtype=torch.int32),
                                    torch.arange(prompt_rows, total + 1, dtype=torch.int32)])
        self.at_seq_of_row = 2 * total + 2 * seqs
        self.at_row_start = self.at_seq_of_row + total
        self.at_want = self.at_row_start + seqs + 1
        if tail:
            seq_of_row = d[self.at_seq_of_row:self.at_row_start]
            row_start = d[self.at_row_start:self.at_want]
            self.want_rows = d[self.at_want:self.at_want + len(wanted)]
            # a portion as long as the graph's rows, then a row of one: the plan then launches both the prompt
            # kernel and the kernel of the short sequences, whatever the tail's and the padding's lengths will be
            host_new = [rows] * portions + [tail, 1] + [1] * decodes
        else:
            seq_of_row, row_start = seq_of_row_host.to(device), row_start_host.to(device)
            self.want_rows = torch.tensor(wanted, dtype=torch.int32, device=device) if wanted else None
            host_new = [rows] * portions + [1] * decodes
        self.ctx = StepContext(
            num_rows=total, num_seqs=seqs, token_ids=d[:total], positions=d[total:2 * total], seq_of_row=seq_of_row,
            row_start=row_start, seq_begin=d[2 * total:2 * total + seqs],
            state_slots=d[2 * total + seqs:2 * total + 2 * seqs], groups=groups,
            host_new=host_new, host_begin=(), host_slots=(), max_new=max(rows if portions else 0, tail),
            max_context=columns * cache.page_size)
        # capture on harmless metadata: positions 0.., the scratch slot, the scratch page; a tail of all rows but one
        host = self.hosts[0].numpy()
        host[total:total + portions * rows] = np.tile(np.arange(rows, dtype=np.int32), portions)
        if tail:
            host[total + portions * rows:total + prompt_rows - 1] = np.arange(tail - 1, dtype=np.int32)
            host[self.at_seq_of_row:self.at_row_start] = seq_of_row_host.numpy()
            host[self.at_row_start:self.at_want] = row_start_host.numpy()
            host[self.at_want:self.at_want + len(wanted)] = np.asarray(wanted, dtype=np.int32)
        host[2 * total + seqs:2 * total + 2 * seqs] = cache.scratch_slot
        for other in self.hosts[1:]:                 # (the parts that no step rewrites must stand in every copy)
            other.copy_(self.hosts[0])
        self.dev.copy_(self.hosts[0])
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                stepper.model.forward(self.ctx, cache.bindings, self.want_rows)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()                                 # see _Graph._capture
        try:
            with torch.cuda.graph(graph, pool=pool):
                self.logits = stepper.model.forward(self.ctx, cache.bindings, self.want_rows)
        finally:
            if collecting:
                gc.enable()
        self.kernels_per_replay = kernels.launch_count - before
        self.graph = graph
        torch.cuda.synchronize()


class ChunkGraphs:
    """CUDA-graph replay of steps with prompt portions: the first one to ``max_portions`` sequences bring exactly
    ``rows`` tokens each (the configured portion size) and want nothing or their last place; then at most one
    sequence brings the end of its prompt (2 to ``rows`` - 1 tokens, wanting nothing or its last place); every
    other sequence brings one decoded token and wants it.  Between two such steps only device metadata differs
    (token ids, positions, block tables, and where a tail ends), so the launches of the whole model are replayed
    instead of issued one by one; at 2,048 rows of the 1B sizes that takes the step from 4.6 to 3.9 ms, and a step
    of 100 rows, which the host needs 2.8 ms to issue, takes the 1.2 ms of its kernels.  One graph per (portions,
    tail rows rounded up to 64, 128, ... ``rows``, decode rows rounded up to a power of two, whether any portion
    wants its last place, block-table width rounded up to a power of two): the width bounds the context, and with
    it the split count that the decode rows' attention is captured with, as for the decode graphs.  Rows that pad
    the tail and the decode part point at the scratch page and the scratch state slot.  If one portion wants its
    last place the last rows of all portions go through the head and the caller gets the ones it asked for.  The
    graphs share one memory pool (they never run at the same time), so the returned logits are valid until the
    next replayed step; at most ``MAX_GRAPHS`` are captured, other shapes run launch by launch."""

    MAX_GRAPHS = 96

    def __init__(self, stepper: Stepper, rows: int, max_sequence_length: int, max_decodes: int, max_portions: int = 1):
        self.stepper = stepper
        self.rows = rows
        self.max_decodes = max_decodes
        self.max_portions = max(1, max_portions)
        page = stepper.cache.page_size
        self.columns = max(1, -(-min(max_sequence_length, stepper.max_positions) // page))
        self.graphs: Dict[Tuple[int, int, int, bool, int], _ChunkGraph] = {}
        self.pool = None
        self.replays = 0
        self.kernels_replayed = 0
        self.safe = graph_safe(stepper.model)

    def _portions(self, entries: Sequence[StepEntry]) -> int:
        """How many leading entries are full portions that want nothing or their last place."""
        count = 0
        for entry in entries:
            if len(entry.tokens) != self.rows or list(entry.want) not in ([], [self.rows - 1]):
                break
            count += 1
        return count

    def _tail(self, entries: Sequence[StepEntry], portions: int) -> int:
        """Tokens of the entry behind the full portions if it is the end of a prompt (0 if there is none)."""
        if portions >= len(entries):
            return 0
        entry = entries[portions]
        n = len(entry.tokens)
        if 1 < n < self.rows and list(entry.want) in ([], [n - 1]):
            return n
        return 0

    def _tail_rows(self, n: int) -> int:
        """Rows that a tail of ``n`` tokens takes in its graph: more than ``n`` (a padding row at least)."""
        if n == 0:
            return 0
        bucket = 64
        while bucket <= n and bucket < self.rows:
            bucket <<= 1
        return min(bucket, self.rows)

    def _key(self, entries: Sequence[StepEntry], portions: int, tail: int) -> Tuple[int, int, int, bool, int]:
        cache = self.stepper.cache
        decodes = len(entries) - portions - (1 if tail else 0)
        bucket = 0 if decodes == 0 else min(_next_pow2(decodes), max(self.max_decodes, decodes))
        tail_rows = self._tail_rows(tail)
        pages = -(-max([cache.length(e.request) + len(e.tokens) for e in entries] + [tail_rows]) // cache.page_size)
        columns = min(self.columns, max(8, _next_pow2(pages)))
        return portions, tail_rows, bucket, any(e.want for e in entries[:portions]), columns

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        if not self.safe or not entries:
            return False
        portions = self._portions(entries)
        tail = self._tail(entries, portions)
        first_decode = portions + (1 if tail else 0)
        if first_decode == 0 or portions > self.max_portions or len(entries) - first_decode > self.max_decodes:
            return False
        if not all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries[first_decode:]):
            return False
        cache = self.stepper.cache
        limit = self.columns * cache.page_size
        if not all(cache.is_live(e.request) and cache.length(e.request) + len(e.tokens) <= limit for e in entries):
            return False
        if self._tail_rows(tail) > limit:
            return False
        return len(self.graphs) < self.MAX_GRAPHS or self._key(entries, portions, tail) in self.graphs

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        stepper, cache = self.stepper, self.stepper.cache
        stepper._validate(entries)
        rows, portions = self.rows, self._portions(entries)
        tail = self._tail(entries, portions)
        first_decode = portions + (1 if tail else 0)
        decodes = len(entries) - first_decode
        key = self._key(entries, portions, tail)
        _, tail_rows, bucket, wants_last, columns = key
        graph = self.graphs.get(key)
        if graph is None:
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            graph = _ChunkGraph(stepper, rows, portions, bucket, wants_last, columns, self.pool, tail=tail_rows)
            self.graphs[key] = graph
        total, seqs, prompt_rows = graph.total, graph.seqs, graph.prompt_rows
        full_rows = portions * rows
        begins = [cache.length(e.request) for e in entries]
        for entry in entries:
            cache.extend(entry.request, len(entry.tokens))
        index = graph.next_host
        graph.next_host = (index + 1) % HOST_RING
        if graph.host_events[index] is not None:
            graph.host_events[index].synchronize()
        host = graph.hosts[index].numpy()
        slots = [cache.slot(e.request) for e in entries]
        # sequence slots of the graph: the portions, (the tail, its padding,) the decode rows; entries skip the padding
        seq_of_entry = list(range(first_decode)) + [first_decode + (1 if tail else 0) + j for j in range(decodes)]
        host[full_rows:total] = 0
        host[total + full_rows:2 * total] = 0
        host[2 * total:2 * total + seqs] = 0
        host[2 * total + seqs:2 * total + 2 * seqs] = cache.scratch_slot
        for k in range(portions):
            host[k * rows:(k + 1) * rows] = np.asarray(entries[k].tokens, dtype=np.int32)
            host[total + k * rows:total + (k + 1) * rows] = np.arange(begins[k], begins[k] + rows, dtype=np.int32)
        if tail:
            host[full_rows:full_rows + tail] = np.asarray(entries[portions].tokens, dtype=np.int32)
            host[total + full_rows:total + full_rows + tail] = np.arange(begins[portions], begins[portions] + tail,
                                                                         dtype=np.int32)
            host[total + full_rows + tail:total + prompt_rows] = np.arange(tail_rows - tail, dtype=np.int32)   # padding
            seq_of_row = host[graph.at_seq_of_row:graph.at_row_start]
            seq_of_row[full_rows:full_rows + tail] = portions
            seq_of_row[full_rows + tail:prompt_rows] = portions + 1
            row_start = host[graph.at_row_start:graph.at_want]
            row_start[portions] = full_rows
            row_start[portions + 1] = full_rows + tail
            host[graph.at_want + graph.tail_want] = full_rows + tail - 1
        if decodes:
            host[prompt_rows:prompt_rows + decodes] = [int(e.tokens[0]) for e in entries[first_decode:]]
            host[total + prompt_rows:total + prompt_rows + decodes] = begins[first_decode:]
        for k, seq in enumerate(seq_of_entry):
            host[2 * total + seq] = begins[k]
            host[2 * total + seqs + seq] = slots[k]
        used = min(graph.columns, -(-max([b + len(e.tokens) for b, e in zip(begins, entries)] + [tail_rows])
                                    // cache.page_size))
        graph.dev.copy_(graph.hosts[index], non_blocking=True)
        for k, group_index in enumerate(graph.paged):
            table = graph.host_tables[index][k].numpy()
            table[:, :used] = 0
            table[seq_of_entry, :used] = cache.block_table_rows(group_index, slots, used)
            graph.dev_tables[k][:, :used].copy_(graph.host_tables[index][k][:, :used], non_blocking=True)
        copied = torch.cuda.Event()
        copied.record()
        graph.host_events[index] = copied
        graph.graph.replay()
        for entry in entries:
            cache.commit(entry.request, len(entry.tokens))
        stepper.steps_run += 1
        self.replays += 1
        self.kernels_replayed += graph.kernels_per_replay
        if graph.logits is None:
            return None
        # the head's rows: the portions' last places (if any portion wants one), the tail's, the decode rows'
        head_portions = portions if wants_last else 0
        picked = [k for k in range(head_portions) if entries[k].want]
        if tail and entries[portions].want:
            picked.append(head_portions)
        behind = head_portions + (1 if tail else 0)
        picked += list(range(behind, behind + decodes))
        if not picked:
            return None
        if picked == list(range(picked[0], picked[0] + len(picked))):
            return graph.logits[picked[0]:picked[0] + len(picked)]
        return graph.logits[torch.tensor(picked, dtype=torch.long, device=graph.logits.device)]
