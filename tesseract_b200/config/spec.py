"""Architecture-neutral description of a decoder: which parts, with which numbers.

An architecture module turns its typed configuration into a :class:`ModelSpec`;
the model builder turns a ``ModelSpec`` into parts by looking every ``kind`` up
in the part registries.  Nothing below this line knows an architecture's name.

* A :class:`PartSpec` names a part kind (for example ``"attention"``), its
  parameters (sizes and constants) and the checkpoint tensor behind each of the
  part's weight roles.
* A :class:`LayerSpec` is one block: its arrangement kind, mixer, feed-forward
  and norms.  Layers may differ from one another freely.
* ``run_order`` is the list of :class:`RunEntry` that the step function walks.
  An entry names a layer (so a layer may run twice) and, optionally, an earlier
  entry whose cache it reads instead of keeping its own.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


def _freeze(mapping: Optional[Mapping[str, Any]]) -> Tuple[Tuple[str, Any], ...]:
    return tuple(sorted((mapping or {}).items()))


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params_items: Tuple[Tuple[str, Any], ...] = ()
    weight_items: Tuple[Tuple[str, str], ...] = ()
    children_items: Tuple[Tuple[str, "PartSpec"], ...] = ()

    @classmethod
    def make(cls, kind: str, params: Optional[Mapping[str, Any]] = None,
             weights: Optional[Mapping[str, str]] = None,
             children: Optional[Mapping[str, "PartSpec"]] = None) -> "PartSpec":
        return cls(kind, _freeze(params), _freeze(weights), _freeze(children))

    @property
    def params(self) -> Dict[str, Any]:
        return dict(self.params_items)

    @property
    def weights(self) -> Dict[str, str]:
        return dict(self.weight_items)

    @property
    def children(self) -> Dict[str, "PartSpec"]:
        return dict(self.children_items)


@dataclass(frozen=True)
class LayerSpec:
    """One block: ``block`` arranges ``norms``, ``mixer`` and ``feed_forward``."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms_items: Tuple[Tuple[str, PartSpec], ...]

    @classmethod
    def make(cls, block: str, mixer: PartSpec, feed_forward: PartSpec,
             norms: Mapping[str, PartSpec]) -> "LayerSpec":
        return cls(block, mixer, feed_forward, tuple(sorted(norms.items())))

    @property
    def norms(self) -> Dict[str, PartSpec]:
        return dict(self.norms_items)


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    ``layer`` indexes ``ModelSpec.layers``.  ``cache_of`` is ``None`` when the
    entry keeps a cache of its own, or the index (into ``run_order``) of an
    earlier entry whose cache this entry reads without writing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    bos_token_id: int = 0
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.run_order:
            raise ValueError("run_order is empty")
        for index, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"run_order[{index}] names layer {entry.layer}, model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ValueError(f"run_order[{index}].cache_of must name an earlier entry")
                if self.run_order[entry.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{index}].cache_of names an entry that keeps no cache")
