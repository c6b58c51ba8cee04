"""Grouped-query attention over paged keys and values.

Per row: ``q, k, v`` projections (one fused product over the concatenated weights, each
output column identical to the separate products of src/cuda/dense_decoder.rs:675-707),
position encoding on q and k, new k and v stored in the request's pages (k after
rotation), softmax attention of every row over the request's keys up to and including
its own position (src/cuda/kernels.rs:447-562), optional sliding window, then the output
projection (src/cuda/dense_decoder.rs:722-734).  Query head ``h`` reads kv head
``h // (num_heads / num_kv_heads)``; the score scale is ``1/sqrt(head_dim)`` unless the
spec gives another (src/cuda/dense_decoder/flat_kv.rs:165).
"""

from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import (MIXERS, POSITION_ENCODINGS, CacheBinding, DeferredNorm, Mixer, PagedKVNeed, Runtime,
                   StepContext)
from .linear import Linear


@MIXERS.register("attention")
class Attention(Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, head_dim``, optional ``window``, ``scale``, ``prompt_kernel``.
    weights: ``q, k, v, o``.  children: ``position`` (a position encoding spec)."""

    accepts_deferred_norm = True
    accepts_follow_norm = True
    graph_safe = True      # reads only device-side metadata of the step, so a decode step can be captured

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p["window"]) if p.get("window") else 0
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention kernels take head_dim in steps of 16 up to 256, got {self.head_dim}")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        fused = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0)
        self.qkv_proj = Linear(fused, runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        # Which kernel runs prompt portions in bfloat16: "tcgen05" (tensor-memory accumulators, TMA-fed; head_dim 64
        # or 128, other sizes fall back) or "mma" (mma.sync tiles, every head size).
        self.prompt_kernel = str(p.get("prompt_kernel") or "tcgen05")
        if self.prompt_kernel not in ("mma", "tcgen05"):
            raise ValueError(f"prompt_kernel must be 'mma' or 'tcgen05', got '{self.prompt_kernel}'")
        position_spec = spec.children.get("position")
        if position_spec is None:
            position_spec = PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if not runtime.is_float32:
            kernels.attention_workspace(runtime.device)     # permanent: captured graphs keep its addresses

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, d = int(p["hidden_size"]), int(p["head_dim"])
        q_width, kv_width = int(p["num_heads"]) * d, int(p["num_kv_heads"]) * d
        return {
            w["q"]: ExpectedTensor((q_width, hidden)),
            w["k"]: ExpectedTensor((kv_width, hidden)),
            w["v"]: ExpectedTensor((kv_width, hidden)),
            w["o"]: ExpectedTensor((hidden, q_width)),
        }

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window or None)

    def forward(self, x, ctx: StepContext, cache: Optional[CacheBinding], follow=None):
        if cache is None or cache.storage is None:
            raise RuntimeError("attention needs a paged key/value cache binding")
        group = ctx.groups[cache.group]
        qkv = None
        if isinstance(x, DeferredNorm):
            qkv = self.qkv_proj.forward_normed(x)       # the norm folded into the projection, if possible
            if qkv is None:
                x = x.materialize()
        if qkv is None:
            qkv = self.qkv_proj.forward(x)
        inv_freq = self.position.rotary_inv_freq
        rows = qkv.shape[0]
        attended = torch.empty((rows, self.q_width), dtype=qkv.dtype, device=qkv.device)
        new_tokens = ctx.host_new if len(ctx.host_new) == ctx.num_seqs else [ctx.max_new] * ctx.num_seqs
        choice = plan.attention(self.runtime.dtype, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                                head_dim=self.head_dim, page_size=cache.page_size, new_tokens=new_tokens,
                                max_context=ctx.max_context, prompt_kernel=self.prompt_kernel,
                                rotary_in_kernel=inv_freq is not None or self.position.kind == "none")
        if choice.fused_decode:
            # a pure decode step: rotation, cache write and attention in one kernel
            kernels.attention_decode_rope(qkv, attended, cache.storage, ctx.row_start, ctx.seq_begin,
                                          group.block_table, ctx.num_seqs, self.num_heads, self.num_kv_heads,
                                          self.head_dim, cache.page_size, self.window, self.scale, inv_freq,
                                          cache.writes, choice.splits)
            return self.o_proj.forward(attended, follow=follow)
        if inv_freq is None and self.position.kind != "none":
            q_view = qkv[:, :self.q_width].view(rows, self.num_heads, self.head_dim)
            k_view = qkv[:, self.q_width:self.q_width + self.kv_width].view(rows, self.num_kv_heads, self.head_dim)
            self.position.apply(q_view, k_view, ctx.positions)
        kernels.rope_kv_write(qkv, ctx.positions, ctx.seq_of_row, group.block_table, inv_freq, cache.storage,
                              self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size,
                              write_kv=cache.writes)
        q = qkv[:, :self.q_width]
        if choice.rows:
            # the 32-bit path: one warp per (row, head), a fixed order of every reduction
            kernels.attention_rows(q, attended, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                   self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                                   self.scale)
            return self.o_proj.forward(attended, follow=follow)
        tiles = choice.prompt == "mma_tiles"
        if choice.prompt == "tcgen05":
            # prompt portions on the fifth-generation tensor cores; decode rows (if any) by the split kernel
            kernels.attention_tcgen05(q, attended, cache.storage, ctx.row_start, ctx.seq_begin, group.block_table,
                                      ctx.num_seqs, ctx.max_new, self.num_heads, self.num_kv_heads, self.head_dim,
                                      cache.page_size, self.window, self.scale, key_splits=choice.key_splits)
        if tiles or choice.split:
            kernels.attention_mma(q, attended, cache.storage, ctx.row_start, ctx.seq_begin, group.block_table,
                                  ctx.num_seqs, ctx.max_new, self.num_heads, self.num_kv_heads, self.head_dim,
                                  cache.page_size, self.window, self.scale, tiles, choice.split, choice.splits)
        return self.o_proj.forward(attended, follow=follow)
