"""Matrix product ``y = x @ W^T`` with a weight kept as ``[out, in]``.

Which kernel runs a product is the kernel plan's decision (``tesseract_b200.plan.product``); this class carries
the decision out.  In float32: the package's own 32-bit kernel (a fixed K-ordered chain per output element).  In
bfloat16: the weight-streaming kernels up to 16 rows (``decode_linear``, optionally with the norm in front and
SwiGLU behind folded in) and up to 128 rows (``skinny_tcgen05``), the tcgen05 GEMM where the plan says so, else
the library GEMM with 32-bit accumulation, where the reference
also calls a library (src/cuda/cublas.rs:49-92: bfloat16 in and out, 32-bit compute, the weight transposed).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels, plan
from .base import Runtime


class BestOfRows:
    """Where a 32-bit product leaves, per CTA, its best output value of each row and that value's lowest column (the
    first stage of a two-stage argmax; the sampler is the second).  The buffers are made once and kept (a captured
    graph holds their addresses); ``valid`` says whether the product that ran last filled them."""

    def __init__(self, device):
        self.device = device
        self.buffers = None
        self.valid = False

    def take(self, out_features: int) -> None:
        shape = (kernels.decode_linear_ctas(out_features), kernels.SS_STRIDE)
        if self.buffers is None or tuple(self.buffers[0].shape) != shape:
            self.buffers = (torch.empty(shape, dtype=torch.float32, device=self.device),
                            torch.empty(shape, dtype=torch.int32, device=self.device))
        self.valid = True


def _tma_rows(x: torch.Tensor) -> torch.Tensor:
    """Rows as a bulk tensor copy can fetch them: a 16-byte aligned base, a row stride of a multiple of 8 elements."""
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        return x.contiguous()
    return x


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        self.runtime = runtime
        self.weight = runtime.matrix(weight)
        self.out_features, self.in_features = self.weight.shape

    def plan(self, rows: int, epilogue: str = plan.BF16, norm: Optional[str] = None,
             contiguous_rows: bool = True, follow: bool = False) -> plan.ProductPlan:
        return plan.product(self.runtime.dtype, rows, self.out_features, self.in_features, epilogue=epilogue,
                            norm=norm, contiguous_rows=contiguous_rows, follow=follow)

    def _out(self, rows: int, choice: plan.ProductPlan, device) -> torch.Tensor:
        width = self.out_features // 2 if choice.epilogue == plan.SWIGLU else self.out_features
        dtype = torch.float32 if choice.epilogue == plan.F32 else self.runtime.dtype
        return torch.empty((rows, width), dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, float32_out: bool = False,
                epilogue: Optional[str] = None, follow=None, best=None):
        """``x @ W^T``; with ``epilogue="swiglu"`` the activated product ``[rows, out / 2]`` if the plan has a kernel
        that folds the activation in, else ``None`` (the caller then activates the plain product itself).  With
        ``follow`` (a :class:`FollowNorm`) the product may do the work of the norm behind it and return a
        :class:`PreparedNorm` instead of its rows, if the plan has a kernel for that."""
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear expects width {self.in_features}, got {x.shape[-1]}")
        if not x.is_cuda:
            raise RuntimeError("tesseract_b200 has no CPU path; tensors must be on a CUDA device")
        rows = x.shape[0]
        wanted = epilogue or (plan.F32 if float32_out or self.runtime.is_float32 else plan.BF16)
        choice = self.plan(rows, wanted, contiguous_rows=x.stride(1) == 1)
        if wanted == plan.SWIGLU and choice.activation_apart:
            return None
        if follow is not None and out is None and wanted == plan.BF16:
            prepared = self._prepare(x, follow)
            if prepared is not None:
                return prepared
        if choice.kernel == "library":
            if choice.epilogue == plan.F32:
                result = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
                return result if out is None else out.copy_(result)
            return torch.mm(x, self.weight.t()) if out is None else torch.mm(x, self.weight.t(), out=out)
        if out is None:
            out = self._out(rows, choice, x.device)
        if choice.kernel == "gemm_f32":
            return kernels.gemm_f32_nt(x, self.weight, out)
        if choice.kernel == "decode_linear":
            if best is not None and choice.epilogue == plan.F32:
                best.take(self.out_features)
            return kernels.decode_linear(self.weight, out, x=x, epilogue=choice.epilogue_code,
                                         best=best.buffers if best is not None and best.valid else None)
        if choice.kernel == "skinny_tcgen05":
            return kernels.skinny_tcgen05(_tma_rows(x), self.weight, out, epilogue=choice.epilogue_code)
        return kernels.gemm_tcgen05(x, self.weight, out, epilogue=choice.epilogue_code)

    def _prepare(self, x: torch.Tensor, follow):
        """The product with the following norm's work folded behind it, or None if that cannot be."""
        from .base import PreparedNorm

        parameters = getattr(follow.norm, "rms_parameters", None)
        residual = follow.before.residual
        rows = x.shape[0]
        if (parameters is None or not follow.before.done or residual.shape != (rows, self.out_features)
                or residual.dtype != self.runtime.dtype or not residual.is_contiguous() or x.stride(1) != 1):
            return None
        choice = self.plan(rows, plan.BF16, follow=True)
        if not choice.prepares_norm:
            return None
        weight, _ = parameters()
        if weight.numel() != self.out_features:
            return None
        new_residual = torch.empty_like(residual)
        scaled_rows = torch.empty_like(residual)
        if choice.kernel == "skinny_tcgen05":
            sums = torch.empty(kernels.skinny_tcgen05_sums_shape(self.out_features), dtype=torch.float32,
                               device=residual.device)
            kernels.skinny_tcgen05(_tma_rows(x), self.weight, None,
                                   prepare=(residual, weight, new_residual, scaled_rows, sums))
        else:
            tiles = self.out_features // kernels.decode_linear_tile_features(self.out_features)
            sums = torch.empty((tiles, kernels.SS_STRIDE), dtype=torch.float32, device=residual.device)
            kernels.decode_linear(self.weight, None, x=x, prepare=(residual, weight, new_residual, scaled_rows, sums))
        return PreparedNorm(follow.norm, new_residual, scaled_rows, sums, made_by=choice.kernel)

    def forward_normed(self, deferred, float32_out: bool = False, epilogue: Optional[str] = None,
                       best=None) -> torch.Tensor:
        """``norm(residual [+ update]) @ W^T`` with the norm folded into the product's kernel, or ``None`` when the
        plan has no such kernel for these sizes or the norm does not offer its parameters for folding
        (``rms_parameters()``): the caller then lets the norm run on its own."""
        from .base import PreparedNorm

        parameters = getattr(deferred.norm, "rms_parameters", None)
        if parameters is None or deferred.done or not deferred.residual.is_contiguous():
            return None
        wanted = epilogue or (plan.F32 if float32_out else plan.BF16)
        if isinstance(deferred, PreparedNorm):
            # the product in front left the rows times the norm's weights and their sums of squares: this product
            # takes them as they are and applies the scale to its 32-bit sums
            choice = self.plan(deferred.rows, wanted, norm="prepared")
            if not choice.norm_folded or choice.kernel != deferred.made_by:     # the sums' layout is the kernel's own
                return None
            _, eps = parameters()
            out = self._out(deferred.rows, choice, deferred.residual.device)
            if choice.kernel == "skinny_tcgen05":
                kernels.skinny_tcgen05(deferred.scaled_rows, self.weight, out, epilogue=choice.epilogue_code,
                                       scaled_by=deferred.sums, eps=eps)
                deferred.fused(None)
                return out
            if best is not None and choice.epilogue == plan.F32:
                best.take(self.out_features)
            kernels.decode_linear(self.weight, out, x=deferred.scaled_rows, scaled_by=deferred.sums, eps=eps,
                                  epilogue=choice.epilogue_code,
                                  best=best.buffers if best is not None and best.valid else None)
            deferred.fused(None)
            return out
        choice = self.plan(deferred.rows, wanted, norm="norm" if deferred.update is None else "add_norm")
        if not choice.norm_folded:
            return None
        weight, eps = parameters()
        out = self._out(deferred.rows, choice, deferred.residual.device)
        new_residual = torch.empty_like(deferred.residual) if deferred.update is not None else None
        if best is not None and choice.epilogue == plan.F32:
            best.take(self.out_features)
        kernels.decode_linear(self.weight, out, residual=deferred.residual, update=deferred.update,
                              norm_weight=weight, eps=eps, residual_out=new_residual, epilogue=choice.epilogue_code,
                              best=best.buffers if best is not None and best.valid else None)
        deferred.fused(new_residual)
        return out
