"""Loading a checkpoint by tensor name, with one error that says everything wrong.

The model builder asks its parts which tensors they expect (name, shape, kind);
this module fetches exactly those from the safetensors source and checks them
before anything is sent to the GPU, as the reference validates names, dtypes and
shapes ahead of any device allocation (src/model/llama_3_2.rs:332-382).  Unlike
the reference, which stops at the first fault, every missing tensor, unexpected
tensor, wrong shape and wrong dtype is collected into a single
:class:`WeightError`.

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit
floating point stays 32-bit, and integer tables become int32.  The run dtype is
applied later, by the part that owns the tensor.
"""

from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsSource


@dataclass(frozen=True)
class ExpectedTensor:
    """What a part expects behind one checkpoint name."""

    shape: Tuple[int, ...]
    kind: str = "float"  # "float": bfloat16/float32 (float16 widened); "int": integer table


class WeightError(ValueError):
    """A checkpoint does not match the model; lists every mismatch at once."""

    def __init__(self, model_dir: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str, str]]):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"checkpoint in {model_dir} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name} is {list(actual)}, expected {list(expected)}" for name, expected, actual in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{name} is {actual}, expected {expected}" for name, expected, actual in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT_OK = (torch.bfloat16, torch.float32, torch.float16)
_INT_OK = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_and_load(model_dir: str, expected: Mapping[str, ExpectedTensor],
                   ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Return ``{name: CPU tensor}`` for every expected name, or raise :class:`WeightError`.

    ``ignorable`` holds shell-style patterns of tensor names that a checkpoint of
    this architecture may carry without the model using them.
    """
    source = SafetensorsSource(model_dir)
    patterns = list(ignorable)
    missing: List[str] = []
    wrong_shape = []
    wrong_dtype = []
    for name in sorted(expected):
        want = expected[name]
        if name not in source:
            missing.append(name)
            continue
        entry = source.entry(name)
        if tuple(entry.shape) != tuple(want.shape):
            wrong_shape.append((name, tuple(want.shape), tuple(entry.shape)))
        allowed = _FLOAT_OK if want.kind == "float" else _INT_OK
        if entry.dtype not in allowed:
            wrong_dtype.append((name, "bfloat16 or float32" if want.kind == "float" else "an integer type",
                                str(entry.dtype).replace("torch.", "")))
    unexpected = [name for name in source.names()
                  if name not in expected and not any(fnmatch.fnmatchcase(name, p) for p in patterns)]
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    out: Dict[str, torch.Tensor] = {}
    for name, want in expected.items():
        tensor = source.tensor(name)
        if want.kind == "int":
            tensor = tensor.to(torch.int32)
        elif tensor.dtype == torch.float16:
            tensor = tensor.to(torch.float32)
        out[name] = tensor
    return out
