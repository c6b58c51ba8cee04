"""The kernel plan: which kernel, in which form, every operation of a step takes.

One place decides, for a data type, a row count and the sizes of an operation, which of this package's kernels
runs it (the reference resolves one plan per model and prints it: src/cuda/kernel_plan.rs:140-161, 168-239).
The parts ask these functions and do what the answer says; ``describe`` prints the answers for a whole model
(``tesseract --print-plan``); ``tests/test_kernel_choices.py`` pins them.  There is no other backend to dispatch
to: a size no kernel takes is an error where the part is built or called.

Thresholds, with the measurement behind each:

* ``DECODE_LINEAR_MAX_ROWS`` (16): up to this many rows a product streams its weights once through the skinny
  ``decode_linear`` kernel (mma.sync, 16 warps splitting K), with the residual addition and the RMSNorm in front
  and SwiGLU or a 32-bit store behind folded in.  Against the library product with norm and activation kernels
  of their own a decode step of 16 rows of the 1B sizes takes 0.94 instead of 1.33 ms.
* ``SKINNY_MAX_ROWS`` (128): from 17 rows up to here a product streams its weights through ``skinny_tcgen05``
  (tcgen05 with the weights as the 128-row operand, K splits as a thread-block cluster), with SwiGLU or a 32-bit
  store behind it, and with the same division of a norm's work between the product in front of it and the product
  behind it as ``decode_linear`` has.
* ``FUSED_GATE_UP_MIN_ROWS`` (17): above ``SKINNY_MAX_ROWS`` gate/up + SwiGLU is one tcgen05 GEMM (100 against
  114 us per product at 2,048 rows).
* Plain bfloat16 products over more than 128 rows (QKV, O, down, the head) call the library GEMM, where the
  reference calls one (src/cuda/cublas.rs:49-92).
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import List, Optional, Sequence

import torch

from . import kernels

DECODE_LINEAR_MAX_ROWS = 16
SKINNY_MAX_ROWS = kernels.SKINNY_MAX_ROWS
FUSED_GATE_UP_MIN_ROWS = 17
MAX_ATTENTION_SPLITS = kernels.MAX_ATTENTION_SPLITS
CLUSTER_SPLITS = 8            # up to this many splits merge inside a thread-block cluster; more go through scratch

BF16, F32, SWIGLU = "bf16", "f32", "swiglu"
_EPILOGUE_CODE = {BF16: kernels.EPI_BF16, F32: kernels.EPI_F32, SWIGLU: kernels.EPI_SWIGLU}


@lru_cache(maxsize=None)
def _decode_linear_takes(rows: int, out_features: int, in_features: int, prologue: int) -> bool:
    return kernels.decode_linear_supported(rows, out_features, in_features, prologue)


@lru_cache(maxsize=None)
def _skinny_takes(rows: int, out_features: int, in_features: int, epilogue: int) -> bool:
    return kernels.skinny_tcgen05_supported(rows, out_features, in_features, epilogue)


@lru_cache(maxsize=None)
def _gemm_tcgen05_takes(rows: int, out_features: int, in_features: int, epilogue: int) -> bool:
    return kernels.gemm_tcgen05_supported(rows, out_features, in_features, epilogue)


@lru_cache(maxsize=None)
def _attention_tcgen05_takes(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return kernels.attention_tcgen05_supported(num_heads, num_kv_heads, head_dim, page_size)


@dataclass(frozen=True)
class ProductPlan:
    """``kernel``: ``gemm_f32`` (true 32-bit FFMA), ``decode_linear`` (weight streaming, at most 16 rows),
    ``skinny_tcgen05`` (weight streaming on the tensor-memory cores, at most 128 rows), ``gemm_tcgen05`` (this
    package's tensor-memory GEMM: CTA pairs on 256-row tiles above 128 rows) or ``library``.
    ``norm_folded``: the RMSNorm (and the residual addition) in front runs inside the product's kernel.  ``epilogue``: what the kernel stores;
    ``activation_apart``: SwiGLU was asked for but runs as a kernel of its own behind the product.
    ``prepares_norm``: the product also does the work of the norm BEHIND it (new residual, rows times the norm's
    weights, sums of squares); the product behind that then runs with ``norm="prepared"`` (``takes_prepared``): it
    takes those rows as they are and applies the scale to its 32-bit sums."""

    kernel: str
    norm_folded: bool = False
    epilogue: str = BF16
    activation_apart: bool = False
    prepares_norm: bool = False
    takes_prepared: bool = False

    @property
    def epilogue_code(self) -> int:
        return _EPILOGUE_CODE[self.epilogue]

    def __str__(self) -> str:
        extras = [f"{self.epilogue} store"]
        if self.takes_prepared:
            extras.insert(0, "rows prepared by the product in front, the norm's scale on the sums")
        elif self.norm_folded:
            extras.insert(0, "add+norm folded in front")
        if self.activation_apart:
            extras.append("SwiGLU as a kernel of its own")
        if self.prepares_norm:
            extras.append("does the following add+norm's work")
        return f"{self.kernel} ({', '.join(extras)})"


def product(dtype: torch.dtype, rows: int, out_features: int, in_features: int, *, epilogue: str = BF16,
            norm: Optional[str] = None, contiguous_rows: bool = True, follow: bool = False) -> ProductPlan:
    """The kernel for ``[rows, in] @ [out, in]^T``.  ``norm``: ``"norm"`` or ``"add_norm"`` if an RMSNorm (with the
    residual addition) stands in front and may be folded in, ``"prepared"`` if the product in front has done that
    norm's work; ``epilogue``: ``bf16``, ``f32`` (logits) or ``swiglu`` (the weight's rows interleave eight gates
    and eight up projections); ``follow``: an addition and an RMSNorm of the product's own width follow it."""
    if dtype == torch.float32:
        return ProductPlan("gemm_f32", False, F32, activation_apart=epilogue == SWIGLU)
    if rows <= DECODE_LINEAR_MAX_ROWS and contiguous_rows:
        if norm == "prepared":
            if _decode_linear_takes(rows, out_features, in_features, kernels.PRO_NONE):
                return ProductPlan("decode_linear", True, epilogue, takes_prepared=True)
            return ProductPlan("library", False, BF16 if epilogue == SWIGLU else epilogue, activation_apart=epilogue == SWIGLU)
        if follow and norm is None and epilogue == BF16 and _decode_linear_takes(rows, out_features, in_features,
                                                                                kernels.PRO_NONE):
            return ProductPlan("decode_linear", False, BF16, prepares_norm=True)
        if norm is not None:
            prologue = kernels.PRO_NORM if norm == "norm" else kernels.PRO_ADD_NORM
            if _decode_linear_takes(rows, out_features, in_features, prologue):
                return ProductPlan("decode_linear", True, epilogue)
        if _decode_linear_takes(rows, out_features, in_features, kernels.PRO_NONE):
            return ProductPlan("decode_linear", False, epilogue)
    if DECODE_LINEAR_MAX_ROWS < rows <= SKINNY_MAX_ROWS and in_features % 8 == 0:
        # (rows whose stride is no multiple of 8 elements are refused by the kernel's caller, which then copies)
        if norm == "prepared" and _skinny_takes(rows, out_features, in_features, _EPILOGUE_CODE[epilogue]):
            return ProductPlan("skinny_tcgen05", True, epilogue, takes_prepared=True)
        if (follow and norm is None and epilogue == BF16
                and _skinny_takes(rows, out_features, in_features, kernels.EPI_ADD_NORM)):
            return ProductPlan("skinny_tcgen05", False, BF16, prepares_norm=True)
        if norm != "prepared" and _skinny_takes(rows, out_features, in_features, _EPILOGUE_CODE[epilogue]):
            return ProductPlan("skinny_tcgen05", False, epilogue)
    if (epilogue == SWIGLU and rows >= FUSED_GATE_UP_MIN_ROWS
            and _gemm_tcgen05_takes(rows, out_features, in_features, kernels.EPI_SWIGLU)):
        return ProductPlan("gemm_tcgen05", False, SWIGLU)
    if epilogue == SWIGLU:
        return ProductPlan("library", False, BF16, activation_apart=True)
    return ProductPlan("library", False, epilogue)


def attention_splits(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 64,
                     sms: Optional[int] = None) -> int:
    """How many key splits the decode kernel uses.

    A CTA's warps (eight up to a head size of 64, six up to 128, four above) each stream their share of the tiles
    of 16 keys at about 0.65 microseconds a tile of 64-wide heads (wider heads in proportion); merging splits
    costs about 2.5 microseconds inside a thread-block cluster (up to 8 splits) and 5 through scratch memory; two
    CTAs fit an SM up to a head size of 128, one above.  The choice minimises that estimate over the split counts
    that keep all CTAs resident at once (at most 32: one sequence of 131,072 tokens reads its keys at 5.2 TB/s
    with 32 splits, 4.5 with 16)."""
    tiles = -(-max_context // 16)
    warps = 8 if head_dim <= 64 else 6 if head_dim <= 128 else 4
    ctas = max(1, num_seqs * num_kv_heads)
    per_sm = 2 if head_dim <= 128 else 1
    tile_cost = 0.65 * max(1.0, head_dim / 64.0)
    limit = max(1, min(MAX_ATTENTION_SPLITS, per_sm * (sms or kernels.sm_count()) // ctas))
    best, best_cost = 1, float("inf")
    for splits in range(1, limit + 1):
        per_warp = -(-(-(-tiles // splits)) // warps)
        merge = 0.0 if splits == 1 else 2.5 if splits <= CLUSTER_SPLITS else 5.0
        cost = tile_cost * per_warp + merge + 0.15 * splits
        if cost < best_cost:
            best, best_cost = splits, cost
    return best


def prompt_key_splits(tile_ctas: int, max_context: int, head_dim: int = 64, sms: Optional[int] = None) -> int:
    """CTAs per tile of the tcgen05 prompt kernel.  A tile of 128 folded rows walks over its key blocks (128 keys
    up to head size 64, else 64) one after the other, and two CTAs fit an SM: a step with fewer tiles than that (a
    512-token portion of one prompt is 128 tiles of the 1B sizes) leaves SMs idle while every tile walks its whole
    context.  Such a step gives each tile to several CTAs, each over a run of at least 2,048 keys, as many as are
    resident at once (at most 8); the last one to finish adds the runs.  Leaving and adding the partial rows costs
    about 10 microseconds (a round of stores, a fence, a counter, three rounds of loads from L2), and two CTAs on an
    SM share its exponential unit, so short contexts lose, at either head size: a 512-token portion at context
    2,048 takes 27.3 us alone and 32.6 shared by two (head size 128: 42.9 and 53.5), at 3,072 38.6 and 39.0 (61.0
    and 62.8), at 4,096 50.3 and 45.0 (78.6 and 72.3), at 8,192 94.4 and 68.5 (150 and 110); ``head_dim`` is taken for
    the callers' sake and does not enter."""
    resident = 2 * (sms or kernels.sm_count())
    return max(1, min(8, resident // max(1, tile_ctas), max_context // 2048))


@dataclass(frozen=True)
class AttentionPlan:
    """``fused_decode``: one kernel rotates q and the new key, writes the cache page and attends (a pure decode
    step).  Otherwise a rotation + cache-write kernel runs first and ``prompt`` (``tcgen05``, ``mma_tiles`` or
    None) takes the sequences with more than 16 folded rows (new tokens x query heads per kv head), ``split``
    (True/False) the others through the split decode kernel.  ``rows``: the 32-bit path's one kernel.
    ``splits``/``merge``: key splits of the split kernel and how they meet (``none``, ``cluster``, ``scratch``).
    ``key_splits``: CTAs per tile of the tcgen05 prompt kernel (``prompt_key_splits``)."""

    fused_decode: bool = False
    prompt: Optional[str] = None
    split: bool = False
    rows: bool = False
    splits: int = 1
    key_splits: int = 1

    @property
    def merge(self) -> str:
        return "none" if self.splits == 1 else "cluster" if self.splits <= CLUSTER_SPLITS else "scratch"

    def __str__(self) -> str:
        if self.rows:
            return "attention_rows (one warp per row and head, fixed order)"
        if self.fused_decode:
            return f"attention_decode (rotation and cache write folded in; {self.splits} split(s), merge: {self.merge})"
        parts = ["rope_kv_write"]
        if self.prompt:
            shared = f", {self.key_splits} CTAs a tile" if self.key_splits > 1 else ""
            parts.append(f"attention_{self.prompt} for prompt portions{shared}")
        if self.split:
            parts.append(f"attention_decode for short sequences ({self.splits} split(s), merge: {self.merge})")
        return " + ".join(parts)


def attention(dtype: torch.dtype, *, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
              new_tokens: Sequence[int], max_context: int, rotary_in_kernel: bool = True,
              prompt_kernel: str = "tcgen05", sms: Optional[int] = None) -> AttentionPlan:
    """The attention kernels of a step whose sequences bring ``new_tokens`` tokens each."""
    if dtype == torch.float32:
        return AttentionPlan(rows=True)
    fold = num_heads // num_kv_heads
    seqs = len(new_tokens)
    if rotary_in_kernel and fold <= 16 and all(n == 1 for n in new_tokens):
        return AttentionPlan(fused_decode=True, splits=attention_splits(seqs, num_kv_heads, max_context, head_dim, sms))
    long_seqs = any(n * fold > 16 for n in new_tokens)
    short_seqs = any(n * fold <= 16 for n in new_tokens)
    prompt = None
    if long_seqs:
        prompt = "mma_tiles"
        if prompt_kernel == "tcgen05" and _attention_tcgen05_takes(num_heads, num_kv_heads, head_dim, page_size):
            prompt = "tcgen05"
    splits = attention_splits(seqs, num_kv_heads, max_context, head_dim, sms) if short_seqs else 1
    key_splits = 1
    if prompt == "tcgen05":
        tile_ctas = -(-(max(new_tokens) * fold) // 128) * num_kv_heads * seqs      # the kernel's grid, per key split
        key_splits = prompt_key_splits(tile_ctas, max_context, head_dim, sms)
    return AttentionPlan(prompt=prompt, split=short_seqs, splits=splits, key_splits=key_splits)


def describe(model, row_counts: Sequence[int] = (1, 8, 16, 17, 64, 512, 2048), context: int = 4096,
             page_size: int = 16, sms: Optional[int] = None) -> str:
    """The plan of a built model as text: for every distinct layer and the head, the kernel of each operation at
    each of ``row_counts`` (a decode step of that many sequences; from 17 rows on also one prompt portion of
    that many rows)."""
    from .parts.attention import Attention
    from .parts.mlp import SwiGLU

    dtype = model.runtime.dtype
    lines: List[str] = [f"kernel plan for {model.spec.architecture} in {str(dtype).replace('torch.', '')} "
                        f"(context {context}, pages of {page_size})"]
    seen = {}
    for index, block in enumerate(model.layers):
        key = (repr(model.spec.layers[index].mixer.params), repr(model.spec.layers[index].feed_forward.params))
        if key in seen:
            seen[key].append(index)
            continue
        seen[key] = [index]
    for key, layers in seen.items():
        block = model.layers[layers[0]]
        lines.append(f"layers {layers[0]}..{layers[-1]} ({len(layers)}): mixer '{block.mixer.kind}', "
                     f"feed-forward '{block.feed_forward.kind}'")
        for rows in row_counts:
            lines.append(f"  {rows} rows")
            mixer, ffn = block.mixer, block.feed_forward
            down_prepares = False
            if isinstance(ffn, SwiGLU):
                down_prepares = product(dtype, rows, ffn.down_proj.out_features, ffn.down_proj.in_features,
                                        follow=True).prepares_norm
            if isinstance(mixer, Attention):
                qkv = mixer.qkv_proj
                lines.append(f"    qkv      {product(dtype, rows, qkv.out_features, qkv.in_features, norm='add_norm')}")
                if down_prepares:
                    behind = product(dtype, rows, qkv.out_features, qkv.in_features, norm='prepared')
                    lines.append(f"             behind a layer whose down product prepared the norm: {behind}")
                decode = attention(dtype, num_heads=mixer.num_heads, num_kv_heads=mixer.num_kv_heads,
                                   head_dim=mixer.head_dim, page_size=page_size, new_tokens=[1] * rows,
                                   max_context=context, prompt_kernel=mixer.prompt_kernel, sms=sms)
                lines.append(f"    attend   decode step: {decode}")
                if rows >= 17:
                    portion = attention(dtype, num_heads=mixer.num_heads, num_kv_heads=mixer.num_kv_heads,
                                        head_dim=mixer.head_dim, page_size=page_size, new_tokens=[rows],
                                        max_context=context, prompt_kernel=mixer.prompt_kernel, sms=sms)
                    lines.append(f"             one portion: {portion}")
                o = mixer.o_proj
                o_plan = product(dtype, rows, o.out_features, o.in_features, follow=True)
                lines.append(f"    o        {o_plan}")
            else:
                lines.append(f"    mixer    '{mixer.kind}' (its own code)")
            if isinstance(ffn, SwiGLU):
                gu, down = ffn.gate_up_proj, ffn.down_proj
                epilogue = SWIGLU if ffn.interleaved else BF16
                prepared = isinstance(mixer, Attention) and o_plan.prepares_norm
                lines.append(f"    gate/up  {product(dtype, rows, gu.out_features, gu.in_features, epilogue=epilogue, norm='prepared' if prepared else 'add_norm')}")
                lines.append(f"    down     {product(dtype, rows, down.out_features, down.in_features, follow=True)}")
            else:
                lines.append(f"    feed-forward '{ffn.kind}' (its own code)")
    proj = getattr(model.head, "proj", None)
    if proj is not None:
        lines.append("head (wanted rows only)")
        for rows in row_counts:
            text = f"  {rows} rows  {product(dtype, rows, proj.out_features, proj.in_features, epilogue=F32, norm='add_norm')}"
            behind = product(dtype, rows, proj.out_features, proj.in_features, epilogue=F32, norm='prepared')
            if behind.takes_prepared:
                text += f"; on every row of a step: {behind}"
            lines.append(text)
    return "\n".join(lines)
