"""Interfaces of the parts a decoder is assembled from, and their registries.

A part is built from a :class:`~tesseract_b200.config.spec.PartSpec` (its kind, its numbers,
the checkpoint names of its tensors), the tensors themselves and a :class:`Runtime`
(dtype and device).  It never learns which model it is in.

Kinds and what each must provide:

``Norm``
    ``forward(x, out=None)`` and ``forward_add(residual, update, out=None)`` which sets
    ``residual += update`` and returns the normalised sum.
``PositionEncoding``
    ``apply(q, k, positions)`` rotating (or otherwise marking) the ``[T, heads, head_dim]``
    views in place; optionally ``rotary_inv_freq`` (a float32 ``[head_dim/2]`` device tensor)
    with which an attention mixer may fuse rotation into its cache write.
``Mixer``
    ``cache_need()`` -> ``None`` | :class:`PagedKVNeed` | :class:`StateNeed`;
    ``forward(x, ctx, cache)`` -> ``[T, hidden]``.  ``ctx`` is the step's
    :class:`StepContext`; ``cache`` the :class:`CacheBinding` of this run entry.
``FeedForward``
    ``forward(x, ctx)`` -> ``[T, hidden]``.
``Block``
    arranges norms, mixer and feed-forward: ``forward(stream, ctx, cache)`` on a
    :class:`ResidualStream`.
``Embedding`` / ``Head``
    ``forward(token_ids)`` -> ``[T, hidden]`` / ``forward(x)`` -> float32 ``[S, vocab]``.

Every class also has ``expected_tensors(spec)`` -> ``{checkpoint name: ExpectedTensor}``
so that the loader can check a checkpoint, and the random-weights writer can make one,
without building anything.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, List, Mapping, Optional, Sequence, Tuple, Type, TypeVar

import torch

from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor

T = TypeVar("T")


class Registry(Generic[T]):
    """Name -> class, for one family of parts."""

    def __init__(self, family: str):
        self.family = family
        self._classes: Dict[str, Type[T]] = {}

    def register(self, kind: str) -> Callable[[Type[T]], Type[T]]:
        def wrap(cls: Type[T]) -> Type[T]:
            if kind in self._classes and self._classes[kind] is not cls:
                raise ValueError(f"{self.family} kind '{kind}' is already registered")
            self._classes[kind] = cls
            cls.kind = kind
            return cls

        return wrap

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def get(self, kind: str) -> Type[T]:
        try:
            return self._classes[kind]
        except KeyError:
            raise KeyError(f"no {self.family} of kind '{kind}' is registered "
                           f"(known: {sorted(self._classes)})") from None

    def kinds(self) -> List[str]:
        return sorted(self._classes)


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs.

    While a model is being built, a checkpoint tensor that two parts name (an output head tied to the embedding
    table, say) is uploaded once: ``matrix`` and ``vector_f32`` hand the second part the first part's device copy.
    The builder calls :meth:`forget_uploads` when it is done."""

    dtype: torch.dtype
    device: torch.device
    _uploads: Dict[Tuple[int, torch.dtype], Tuple[torch.Tensor, torch.Tensor]] = field(
        default_factory=dict, compare=False, repr=False)

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32

    def _upload(self, tensor: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        key = (id(tensor), dtype)
        known = self._uploads.get(key)
        if known is not None and known[0] is tensor:
            return known[1]
        uploaded = tensor.to(device=self.device, dtype=dtype).contiguous()
        self._uploads[key] = (tensor, uploaded)
        return uploaded

    def matrix(self, tensor: torch.Tensor) -> torch.Tensor:
        """A weight matrix in the run dtype on the run device (bfloat16 widens exactly)."""
        return self._upload(tensor, self.dtype)

    def vector_f32(self, tensor: torch.Tensor) -> torch.Tensor:
        """A scale vector kept in (or widened exactly to) 32-bit."""
        return self._upload(tensor, torch.float32)

    def forget_uploads(self) -> None:
        self._uploads.clear()


# ----------------------------------------------------------------------------- cache needs


class PagedNeed:
    """What a mixer keeps per token, in pages.  A subclass (a frozen dataclass, so that equal needs share a group)
    gives the shape of one page of one run entry, ``page_shape(page_size)``, and optionally ``window`` (only the
    last ``window`` tokens are read; older pages go back to the pool) and ``dtype`` (``None``: the model's).  The
    cache manager allocates ``[entries, pages + 1, *page_shape]`` and hands each entry its ``[pages + 1, ...]``."""

    window: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        raise NotImplementedError


@dataclass(frozen=True)
class PagedKVNeed(PagedNeed):
    """Keys and values of every token (``window`` None) or of the last ``window`` tokens:
    a page is ``[2 (K, V), kv_heads, page_size, head_dim]``."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (2, self.num_kv_heads, page_size, self.head_dim)


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per live request, addressed by the request's state slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheBinding:
    """What one run entry sees of the cache.

    ``group`` indexes the step context's per-group views; ``storage`` is this entry's
    tensor: ``[pages, 2, kv_heads, page_size, head_dim]`` for paged keys and values, or
    ``[slots, *shape]`` for fixed-size state.  ``writes`` is False when the entry reads
    another entry's cache.
    """

    group: int
    storage: Optional[torch.Tensor]
    writes: bool = True
    page_size: int = 0


@dataclass
class GroupView:
    """Per-step view of one cache group: a block table row per sequence of the batch."""

    block_table: Optional[torch.Tensor]  # int32 [R, max_pages] on device; None for state groups
    page_size: int = 0


@dataclass
class StepContext:
    """Everything a part may know about the batch of one step.

    Rows are the step's tokens, packed sequence after sequence.  ``seq_*`` lists are host
    copies for decisions (kernel choice); the tensors are on the device.
    """

    num_rows: int
    num_seqs: int
    token_ids: torch.Tensor      # int32 [T]
    positions: torch.Tensor      # int32 [T] absolute position of each row
    seq_of_row: torch.Tensor     # int32 [T] index of the row's sequence within the batch
    row_start: torch.Tensor      # int32 [R+1] first row of each sequence
    seq_begin: torch.Tensor      # int32 [R] position of the sequence's first new token
    state_slots: torch.Tensor    # int32 [R] state slot of each sequence
    groups: List[GroupView]
    host_new: Sequence[int] = ()     # new tokens per sequence
    host_begin: Sequence[int] = ()   # tokens already cached per sequence
    host_slots: Sequence[int] = ()
    max_new: int = 1
    max_context: int = 1

    @property
    def decode_only(self) -> bool:
        return self.max_new == 1


@dataclass
class ResidualStream:
    """The hidden state between blocks: ``residual + update`` (``update`` may be absent).

    Keeping the pending update apart lets the next norm fuse the addition
    (src/cuda/dense_decoder.rs:668-672, 775).  ``prepared``: the block in front has already added its update and
    done the work of the norm that consumes this stream (a :class:`PreparedNorm`; ``residual`` is then the new
    residual and ``update`` is None).
    """

    residual: torch.Tensor
    update: Optional[torch.Tensor] = None
    prepared: Optional["PreparedNorm"] = None


class DeferredNorm:
    """``norm(residual [+ update])`` that has not been computed yet.

    A block hands this to a mixer or feed-forward that sets ``accepts_deferred_norm``; such a part may
    fold the addition and the normalisation into its first kernel and then calls :meth:`fused` with the
    new residual.  Any other consumer calls :meth:`materialize`, which runs the norm's own kernel.
    Either way ``residual`` afterwards is the updated residual stream.
    """

    def __init__(self, norm: "Norm", residual: torch.Tensor, update: Optional[torch.Tensor]):
        self.norm = norm
        self.residual = residual
        self.update = update
        self._value: Optional[torch.Tensor] = None
        self.done = False

    @property
    def rows(self) -> int:
        return self.residual.shape[0]

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            if self.update is None:
                self._value = self.norm.forward(self.residual)
            else:
                self._value = self.norm.forward_add(self.residual, self.update)   # residual += update, in place
            self.done = True
        return self._value

    def fused(self, new_residual: Optional[torch.Tensor]) -> None:
        """A consumer computed the norm inside its own kernel; ``new_residual`` holds ``residual + update``."""
        if new_residual is not None:
            self.residual = new_residual
        self.done = True


class FollowNorm:
    """What a part is told about the norm BEHIND it, so that its last product may do that norm's work on the way
    out: ``norm`` follows the part's output, which is added to the residual stream as it stands once ``before``
    (the deferred norm in front of the part) has been consumed (``before.residual``)."""

    def __init__(self, norm: "Norm", before: DeferredNorm):
        self.norm = norm
        self.before = before


class PreparedNorm(DeferredNorm):
    """``norm(residual)`` whose work the product in front has already done: ``residual`` holds the new residual
    (the update is added), ``rows`` holds ``round(residual_unrounded * weight)`` and ``sums`` the sums of squares of
    the unrounded rows per tile of features.  A product that can apply the scale to its own sums takes ``rows``
    and ``sums`` (``Linear.forward_normed``); any other consumer calls :meth:`materialize`, which runs the norm's
    own kernel on the new residual."""

    def __init__(self, norm: "Norm", residual: torch.Tensor, rows: torch.Tensor, sums: torch.Tensor,
                 made_by: str = "decode_linear"):
        super().__init__(norm, residual, None)
        self.scaled_rows = rows
        self.sums = sums
        self.made_by = made_by      # the kernel that left ``sums`` (their layout is that kernel's own)


# ----------------------------------------------------------------------------- part bases


class Part:
    kind: str = ""
    # True if everything that varies between two steps of the same shape reaches ``forward`` through device
    # tensors (never through a host-side field of the step context): only then may a step be captured in a CUDA
    # graph.  Every part of a model is asked (norms, mixers, feed-forwards, embedding, head); the parts of this
    # package set it, a new part has to say so itself.
    graph_safe = False

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.runtime = runtime

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        return {}

    @classmethod
    def random_tensor(cls, spec: PartSpec, role: str, shape: Tuple[int, ...], generator: torch.Generator) -> torch.Tensor:
        """A seeded random value for one of this part's tensors (32-bit; the writer casts)."""
        return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02


class Norm(Part):
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, residual: torch.Tensor, update: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    rotary_inv_freq: Optional[torch.Tensor] = None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    # True if ``forward`` also takes a :class:`DeferredNorm` in place of ``x``.
    accepts_deferred_norm = False
    # True if ``forward`` takes ``follow=FollowNorm(...)`` and may then return a :class:`PreparedNorm` instead of
    # its output rows (its last product did the following norm's work).
    accepts_follow_norm = False
    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[CacheBinding]) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    accepts_deferred_norm = False     # True if ``forward`` also takes a :class:`DeferredNorm` in place of ``x``
    accepts_follow_norm = False       # True if ``forward`` takes ``follow=FollowNorm(...)`` (see :class:`Mixer`)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    accepts_deferred_norm = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    kind: str = ""
    # True if ``forward`` takes ``next_norm`` (the norm that will consume the stream this block returns) and may
    # return a stream whose ``prepared`` is set for it.
    accepts_next_norm = False

    def __init__(self, norms: Mapping[str, Norm], mixer: Mixer, feed_forward: FeedForward):
        self.norms = dict(norms)
        self.mixer = mixer
        self.feed_forward = feed_forward

    def entry_norm(self) -> Optional[Norm]:
        """The norm that consumes the incoming stream first (None: the block does not say)."""
        return None

    @classmethod
    def norm_roles(cls) -> Tuple[str, ...]:
        return ()

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding]) -> ResidualStream:
        raise NotImplementedError


NORMS: Registry[Norm] = Registry("norm")
POSITION_ENCODINGS: Registry[PositionEncoding] = Registry("position encoding")
MIXERS: Registry[Mixer] = Registry("mixer")
FEED_FORWARDS: Registry[FeedForward] = Registry("feed-forward")
BLOCKS: Registry[Block] = Registry("block")
EMBEDDINGS: Registry[Embedding] = Registry("embedding")
HEADS: Registry[Head] = Registry("head")
