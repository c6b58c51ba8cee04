"""Gated feed-forward with the SiLU activation (SwiGLU).

``down( silu(x Wg^T) * (x Wu^T) )`` (src/cuda/dense_decoder.rs:737-774,
src/cuda/kernels.rs:191-208).  Gate and up weights are concatenated at load so that one
product feeds the activation kernel; each output column equals the separate product's.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext
from .linear import Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``hidden_size, intermediate_size``; weights: ``gate, up, down``."""

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.gate_up_proj = Linear(torch.cat([tensors["gate"], tensors["up"]], dim=0), runtime)
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

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gate_up = self.gate_up_proj.forward(x)
        activated = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.silu_mul(gate_up, activated)
        return self.down_proj.forward(activated)
