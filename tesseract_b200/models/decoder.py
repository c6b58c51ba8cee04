"""A decoder-only model assembled from a :class:`ModelSpec`.

The builder looks every part kind up in the registries, asks the parts which checkpoint
tensors they expect, and wires them in the order the spec's ``run_order`` gives.  The
forward pass walks that list: embedding, then for each run entry the named layer with
the entry's cache binding, then the final norm and the head on the wanted rows only
(intermediate prompt portions that want no logits skip both, as in
src/cuda/dense_decoder.rs:784-787).
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

import torch

from .. import kernels
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, Block, CacheBinding, DeferredNorm,
                     ResidualStream, Runtime, StepContext)
from ..weights.loader import ExpectedTensor


def _part_specs(spec: ModelSpec):
    """Yield ``(registry, PartSpec)`` for every weight-bearing part of the model."""
    yield EMBEDDINGS, spec.embedding
    for layer in spec.layers:
        block_cls = BLOCKS.get(layer.block)
        norms = layer.norms
        for role in block_cls.norm_roles():
            if role not in norms:
                raise ValueError(f"block '{layer.block}' needs a norm for role '{role}'")
        for role in sorted(norms):
            yield NORMS, norms[role]
        yield MIXERS, layer.mixer
        yield FEED_FORWARDS, layer.feed_forward
    yield NORMS, spec.final_norm
    yield HEADS, spec.head


def expected_tensors(spec: ModelSpec) -> Dict[str, ExpectedTensor]:
    """Every checkpoint tensor the model reads, by name."""
    out: Dict[str, ExpectedTensor] = {}
    for registry, part in _part_specs(spec):
        for name, want in registry.get(part.kind).expected_tensors(part).items():
            if name in out and out[name] != want:
                raise ValueError(f"tensor '{name}' is expected with two shapes: {out[name]} and {want}")
            out[name] = want
    return out


def tensor_roles(spec: ModelSpec):
    """Yield ``(part class, PartSpec, role, checkpoint name, ExpectedTensor)`` once per distinct tensor."""
    seen = set()
    for registry, part in _part_specs(spec):
        cls = registry.get(part.kind)
        expected = cls.expected_tensors(part)
        for role, name in part.weights.items():
            if name in seen or name not in expected:
                continue
            seen.add(name)
            yield cls, part, role, name, expected[name]


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime

        def build(registry, part: PartSpec, **extra):
            cls = registry.get(part.kind)
            mine = {role: tensors[name] for role, name in part.weights.items()}
            return cls(part, mine, runtime, **extra)

        self.embedding = build(EMBEDDINGS, spec.embedding)
        self.layers: List[Block] = []
        for layer in spec.layers:
            block_cls = BLOCKS.get(layer.block)
            norms = {role: build(NORMS, part) for role, part in layer.norms.items()}
            mixer = build(MIXERS, layer.mixer)
            feed_forward = build(FEED_FORWARDS, layer.feed_forward)
            self.layers.append(block_cls(norms, mixer, feed_forward))
        self.final_norm = build(NORMS, spec.final_norm)
        # A head that names the embedding's checkpoint tensor (tied embeddings) gets the same host tensor, and the
        # runtime hands it the device copy that the embedding made: tying is a matter of tensor names alone.
        self.head = build(HEADS, spec.head)
        runtime.forget_uploads()

    # ------------------------------------------------------------------ cache description
    def cache_needs(self) -> List[Optional[object]]:
        """For each run entry: its mixer's cache need, or ``None`` if it keeps no cache of its own."""
        needs: List[Optional[object]] = []
        for index, entry in enumerate(self.spec.run_order):
            need = self.layers[entry.layer].mixer.cache_need()
            if entry.cache_of is not None:
                other = self.layers[self.spec.run_order[entry.cache_of].layer].mixer.cache_need()
                if other != need:
                    raise ValueError(f"run entry {index} reads the cache of entry {entry.cache_of}, "
                                     f"whose geometry {other} differs from its own {need}")
                needs.append(None)
            else:
                needs.append(need)
        return needs

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, bindings: Sequence[Optional[CacheBinding]],
                want_rows: Optional[torch.Tensor], want_every_row: bool = False) -> Optional[torch.Tensor]:
        """Run the step's rows; return float32 logits ``[len(want_rows), vocab]`` or ``None``.
        ``want_every_row``: the caller knows that ``want_rows`` is ``0 .. num_rows - 1`` (a decode step), so the
        rows need not be gathered before the head."""
        hidden = self.embedding.forward(ctx.token_ids[:ctx.num_rows])
        stream = ResidualStream(hidden, None)
        order = self.spec.run_order
        wants_logits = want_rows is not None and want_rows.numel() > 0
        every_row = wants_logits and want_every_row and want_rows.numel() == ctx.num_rows
        for index, entry in enumerate(order):
            block = self.layers[entry.layer]
            if not block.accepts_next_norm:
                stream = block.forward(stream, ctx, bindings[index])
                continue
            # the norm that will consume what this block returns: the next block's first one, or the final norm if
            # it runs on every row (on a few wanted rows it runs after they have been picked out)
            if index + 1 < len(order):
                next_norm = self.layers[order[index + 1].layer].entry_norm()
            else:
                next_norm = self.final_norm if every_row else None
            stream = block.forward(stream, ctx, bindings[index], next_norm=next_norm)
        if not wants_logits:
            return None
        return self.logits_at(stream, want_rows, every_row)

    def logits_at(self, stream: ResidualStream, want_rows: torch.Tensor, every_row: bool = False) -> torch.Tensor:
        count = want_rows.numel()
        width = stream.residual.shape[1]
        if every_row and stream.prepared is not None and stream.prepared.norm is self.final_norm:
            return self.head.forward(stream.prepared if self.head.accepts_deferred_norm else stream.prepared.materialize())
        if every_row:
            residual, update = stream.residual[:count], None if stream.update is None else stream.update[:count]
        else:
            residual = torch.empty((count, width), dtype=stream.residual.dtype, device=stream.residual.device)
            kernels.gather_rows(want_rows, stream.residual, residual)
            update = None
            if stream.update is not None:
                update = torch.empty_like(residual)
                kernels.gather_rows(want_rows, stream.update, update)
        final = DeferredNorm(self.final_norm, residual, update)
        return self.head.forward(final if self.head.accepts_deferred_norm else final.materialize())
