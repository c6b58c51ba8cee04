"""Token embedding (a row gather, src/cuda/kernels.rs:10-24) and the output head.

The head multiplies the normalised hidden rows by the ``[vocab, hidden]`` matrix
(src/cuda/dense_decoder.rs:824-831) and returns 32-bit logits.  With tied embeddings the
model description names one checkpoint tensor for both parts, and both keep one device copy.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import EMBEDDINGS, HEADS, Embedding, Head, Runtime
from .linear import BestOfRows, Linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size, hidden_size``; weights: ``table``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.table = runtime.matrix(tensors["table"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p = spec.params
        return {spec.weights["table"]: ExpectedTensor((int(p["vocab_size"]), int(p["hidden_size"])))}

    def forward(self, token_ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((token_ids.numel(), self.hidden_size), dtype=self.table.dtype, device=self.table.device)
        return kernels.embedding(token_ids, self.table, out)


@HEADS.register("lm_head")
class LMHead(Head):
    """params: ``vocab_size, hidden_size``; weights: ``weight``.  Returns float32 logits."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.proj = Linear(tensors["weight"], runtime)     # the embedding's device copy if both name one tensor
        # per-CTA best logit of each row, left by the product when it is the weight-streaming kernel (at most 16
        # rows): the sampler then need not read the logits again to find a row's best token
        self.best = BestOfRows(runtime.device) if not runtime.is_float32 else None

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p = spec.params
        return {spec.weights["weight"]: ExpectedTensor((int(p["vocab_size"]), int(p["hidden_size"])))}

    accepts_deferred_norm = True

    def forward(self, x, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .base import DeferredNorm

        if self.best is not None:
            self.best.valid = False
        if isinstance(x, DeferredNorm):
            logits = self.proj.forward_normed(x, float32_out=True, best=self.best)
            if logits is not None:
                return logits
            x = x.materialize()
        return self.proj.forward(x, out=out, float32_out=True, best=self.best)

    def argmax_partials(self):
        """``(values, indices)`` that the last ``forward`` left for the sampler, or None if it left none."""
        return self.best.buffers if self.best is not None and self.best.valid else None
