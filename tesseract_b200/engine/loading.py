"""From a model folder to a model on the device, its cache and its step function."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_model_description
from ..models.decoder import DecoderModel, expected_tensors
from ..parts.base import Runtime
from ..weights.loader import check_and_load
from .step import Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name: str) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{name}'") from None


def require_cuda(device_index: int = 0) -> torch.device:
    """The CUDA device, or a loud failure: this package has no CPU path."""
    if not torch.cuda.is_available():
        raise RuntimeError("tesseract_b200 needs a CUDA device (sm_100a); none is visible and there is no CPU path")
    major, minor = torch.cuda.get_device_capability(device_index)
    if major != 10:
        raise RuntimeError(f"tesseract_b200 kernels are built for sm_100a; device {device_index} is sm_{major}{minor}")
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return torch.device("cuda", device_index)


def load_model(model_dir: str, dtype: str = "bfloat16", device_index: int = 0) -> DecoderModel:
    """Read ``config.json``, pick the architecture, check and load the checkpoint, build the parts."""
    import tesseract_b200.models  # noqa: F401  (registers architectures and parts)

    from .. import kernels

    device = require_cuda(device_index)
    kernels.prepare(parse_dtype(dtype))
    architecture, config, spec = load_model_description(model_dir)
    tensors = check_and_load(model_dir, expected_tensors(spec), architecture.ignorable_tensors(config))
    return DecoderModel(spec, tensors, Runtime(parse_dtype(dtype), device))


def check_upload(model: DecoderModel, model_dir: str) -> str:
    """Read the final norm's weight back from the device and compare it bit by bit with the checkpoint, as the
    reference's checkpoint report does with ``model.norm.weight`` (src/cuda/dense_decoder.rs:1429-1463).
    Returns the tensor's name; raises ``RuntimeError`` on a difference."""
    from ..weights.safetensors_io import SafetensorsSource

    name = model.spec.final_norm.weights.get("weight")
    on_device = getattr(model.final_norm, "weight", None)
    if name is None or on_device is None:
        raise RuntimeError("the model's final norm holds no weight to check")
    stored = SafetensorsSource(model_dir).tensor(name)
    same = torch.equal(stored.to(torch.float32).view(torch.int32), on_device.cpu().to(torch.float32).view(torch.int32))
    if not same:
        raise RuntimeError(f"{name} read back from the device differs from {model_dir}")
    return name


def make_stepper(model: DecoderModel, *, capacity_tokens: int, page_size: int = 16, max_requests: int = 32,
                 max_step_tokens: int = 4096) -> Stepper:
    """A cache sized for ``capacity_tokens`` and the step function over it."""
    needs = model.cache_needs()
    cache_of = [entry.cache_of for entry in model.spec.run_order]
    num_pages = max(1, -(-capacity_tokens // page_size))
    cache = CacheManager(needs, cache_of, num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                         dtype=model.runtime.dtype, device=model.runtime.device, max_step_tokens=max_step_tokens)
    return Stepper(model, cache)
