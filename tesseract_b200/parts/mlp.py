"""Gated feed-forward with the SiLU activation (SwiGLU).

``down( silu(x Wg^T) * (x Wu^T) )`` (src/cuda/dense_decoder.rs:737-774,
src/cuda/kernels.rs:191-208).  Gate and up weights are merged at load so that one product
feeds the activation; each output column equals the separate product's.  When the
intermediate size is a multiple of eight the merged rows alternate in blocks of eight
(eight gate rows, the eight matching up rows, ...), which lets the decode kernel apply
the activation to its own accumulators; otherwise the gate rows come first.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import FEED_FORWARDS, DeferredNorm, FeedForward, Runtime, StepContext
from .linear import Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``hidden_size, intermediate_size``; weights: ``gate, up, down``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.interleaved = self.intermediate_size % 8 == 0
        if self.interleaved:
            blocks = self.intermediate_size // 8
            merged = torch.stack([tensors["gate"].view(blocks, 8, self.hidden_size),
                                  tensors["up"].view(blocks, 8, self.hidden_size)], dim=1)
            merged = merged.reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            merged = torch.cat([tensors["gate"], tensors["up"]], dim=0)
        self.gate_up_proj = Linear(merged, runtime)
        self.down_proj = Linear(tensors["down"], runtime)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        return {
            w["gate"]: ExpectedTensor((inter, hidden)),
            w["up"]: ExpectedTensor((inter, hidden)),
            w["down"]: ExpectedTensor((hidden, inter)),
        }

    accepts_deferred_norm = True
    accepts_follow_norm = True

    def forward(self, x, ctx: StepContext, follow=None):
        activated = None
        epilogue = plan.SWIGLU if self.interleaved else plan.BF16
        if isinstance(x, DeferredNorm):
            if self.interleaved:      # norm, both projections and the activation in one kernel, if the plan has one
                activated = self.gate_up_proj.forward_normed(x, epilogue=epilogue)
            if activated is None:
                x = x.materialize()
        if activated is None and self.interleaved:
            activated = self.gate_up_proj.forward(x, epilogue=epilogue)     # both projections + SwiGLU, if planned
        if activated is None:
            gate_up = self.gate_up_proj.forward(x)
            activated = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.silu_mul(gate_up, activated, interleaved=self.interleaved)
        return self.down_proj.forward(activated, follow=follow)
