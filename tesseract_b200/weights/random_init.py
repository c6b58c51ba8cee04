"""Random-weights mode: writes a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with exactly the tensors the
architecture's parts expect, so it loads through the same path as a real checkpoint.
Each tensor has its own generator seeded from ``(seed, tensor name)``: matrices are
N(0, 0.02), norm scales 1 + N(0, 0.02) (each part class decides, see
``Part.random_tensor``), drawn in 32-bit and stored in the configuration's
``torch_dtype``.  The reference has no such mode (its weight trait only allows for
synthesised test tensors, src/model/weights.rs:83-86).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(config: Mapping[str, Any], seed: int) -> Dict[str, torch.Tensor]:
    """``{checkpoint name: tensor}`` for the architecture that ``config`` names."""
    from ..models.decoder import tensor_roles  # parts register on import

    architecture = resolve_architecture(config)
    typed = architecture.read_config(config)
    spec = architecture.build_spec(typed)
    store = _STORE[str(config.get("torch_dtype") or config.get("dtype") or "bfloat16")]
    out: Dict[str, torch.Tensor] = {}
    for cls, part, role, name, want in tensor_roles(spec):
        generator = torch.Generator(device="cpu")
        generator.manual_seed(tensor_seed(seed, name))
        value = cls.random_tensor(part, role, tuple(want.shape), generator)
        out[name] = value.to(torch.int32) if want.kind == "int" else value.to(store)
    return out


def write_random_model(model_dir: str, config: Mapping[str, Any], seed: int) -> str:
    """Create ``model_dir`` with ``config.json`` and seeded ``model.safetensors``; return the folder."""
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(config, seed)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(dict(config), handle, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
