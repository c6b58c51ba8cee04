"""Rotary position encoding (rotate-half) with optional Llama-3 frequency scaling.

Inverse frequencies are computed on the host in 32-bit exactly as the reference does
(src/cuda/dense_decoder.rs:1516-1544): ``f = 1 / theta^(2i/d)``; wavelength ``2*pi/f``;
unchanged above the high-frequency cut, divided by ``factor`` below the low-frequency
cut, interpolated between.  The angle of position ``p`` is ``float32(p) * f'_i``
(src/cuda/dense_decoder.rs:1549-1556); the kernels take cos and sin of it in 32-bit
instead of reading a ``[max_position, d/2]`` table.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional

import numpy as np
import torch

from .. import kernels
from ..config.spec import PartSpec
from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


def rotary_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping[str, float]]) -> np.ndarray:
    """float32 ``[head_dim/2]`` inverse frequencies, Llama-3 scaled when ``scaling`` is given."""
    f32 = np.float32
    half = head_dim // 2
    out = np.empty(half, dtype=np.float32)
    theta32 = f32(theta)
    for index in range(half):
        exponent = f32(2 * index) / f32(head_dim)
        base = f32(1.0) / np.power(theta32, exponent, dtype=np.float32)
        frequency = base
        if scaling is not None:
            original = f32(scaling["original_max_position_embeddings"])
            low_ff = f32(scaling["low_freq_factor"])
            high_ff = f32(scaling["high_freq_factor"])
            factor = f32(scaling["factor"])
            wavelength = f32(2.0 * math.pi) / base
            low_wavelength = original / low_ff
            high_wavelength = original / high_ff
            if wavelength < high_wavelength:
                frequency = base
            elif wavelength > low_wavelength:
                frequency = base / factor
            else:
                smooth = (original / wavelength - low_ff) / (high_ff - low_ff)
                frequency = (f32(1.0) - smooth) * base / factor + smooth * base
        out[index] = frequency
    return out


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``scaling`` (mapping or None)."""

    def __init__(self, spec: PartSpec, tensors, runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.head_dim = int(params["head_dim"])
        scaling = params.get("scaling")
        self.inv_freq_host = rotary_inverse_frequencies(self.head_dim, float(params["theta"]),
                                                        dict(scaling) if scaling else None)
        self.rotary_inv_freq = torch.from_numpy(self.inv_freq_host).to(runtime.device)

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError("rotary encoding is applied by the attention mixer's fused rotate-and-store kernel")


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def apply(self, q, k, positions) -> None:
        return None
