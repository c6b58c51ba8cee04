"""Trace replay over the engine's own step function.

A trace is a sequence of steps ``{"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}``: each step's
entries run as one batch through :meth:`Stepper.step` (the function generation uses), the logits at the wanted
places come back, and the requests named in ``end`` give back what they hold.  Nothing is sampled.  The replay
program ``bin/trace_run`` and :meth:`LLM.replay` are both this class; it has no model, cache or kernel of its own.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from .. import kernels
from .step import StepEntry, Stepper


class TraceRunner:
    def __init__(self, stepper: Stepper):
        self.stepper = stepper

    def step(self, record: Mapping[str, Any]) -> Optional[torch.Tensor]:
        """Run one step of a trace; float32 logits ``[wanted, vocab]`` on the device, or ``None``."""
        stepper, cache = self.stepper, self.stepper.cache
        step = record.get("step")
        entries = []
        for item in record.get("entries", []):
            request = item["id"]
            if not cache.is_live(request) and not cache.admit(request):
                raise RuntimeError(f"step {step}: no state slot left for request {request!r} "
                                   f"({cache.max_requests} live at most)")
            entries.append(StepEntry(request, item["tokens"], item.get("want", [])))
        logits = None
        if entries:
            logits = stepper.step(entries)
            if logits is not None:
                logits = logits.to(torch.float32)
            torch.cuda.synchronize(stepper.runtime.device)
            code = kernels.tcgen05_error()
            if code:        # a bounded wait inside a kernel ran out: what this step wrote is not to be trusted
                raise RuntimeError(f"step {step}: a bounded wait inside a tcgen05 kernel ran out (code {code})")
        for request in record.get("end", []):
            cache.release(request)
        return logits
