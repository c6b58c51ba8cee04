"""Root-mean-square normalisation, alone and fused with the residual addition.

``y = round(x * rsqrt(mean(x^2) + eps) * w)`` with 32-bit statistics and the weight
multiplied before the single rounding (src/cuda/kernels.rs:26-57); the fused form
adds first and takes the statistics of the unrounded sum (src/cuda/kernels.rs:59-103).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import NORMS, Norm, Runtime


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``; weights: ``weight`` ``[size]``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = runtime.vector_f32(tensors["weight"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        return {spec.weights["weight"]: ExpectedTensor((int(spec.params["size"]),))}

    @classmethod
    def random_tensor(cls, spec, role, shape: Tuple[int, ...], generator) -> torch.Tensor:
        return 1.0 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02

    def rms_parameters(self) -> Tuple[torch.Tensor, float]:
        """``(weight, eps)``: what a product kernel needs to compute this norm in its own first phase.  A norm that
        has this method may be folded into the product behind it; one that has not runs its own kernel."""
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(x)
        return kernels.rms_norm(x, self.weight, self.eps, out)

    def forward_add(self, residual: torch.Tensor, update: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(residual)
        kernels.add_rms_norm(residual, update, self.weight, self.eps, out, residual)
        return out
