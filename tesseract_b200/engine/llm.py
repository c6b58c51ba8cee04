"""The Python entry point: ``LLM(model_path).generate(prompts, sampling_params)``.

The reference is a server and has no Python interface; this class gives the same engine
(scheduler, step function, samplers) to a caller in process.  Engine options carry the
reference's names (src/config.rs:139-186): ``max_queue``, ``max_running``,
``max_batch_tokens``, ``prefill_chunk_tokens``, ``max_sequence_length``,
``kv_capacity_tokens``.  Prompts are lists of token ids; text is accepted and returned
only when the model folder has a ``tokenizer.json`` and the ``tokenizers`` package is
importable (tokenisation is outside the engine, as in src/model/tokenizer.rs).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, make_stepper
from .scheduler import FINISH_STOP, Request, Scheduler


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    text: Optional[str] = None
    error: Optional[str] = None

    @property
    def usage(self) -> Dict[str, int]:
        p, c = len(self.prompt_token_ids), len(self.token_ids)
        return {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c}


class LLM:
    def __init__(self, model_path: str, dtype: str = "bfloat16", device: int = 0, *, max_queue: int = 256,
                 max_running: int = 32, max_batch_tokens: int = 4096, prefill_chunk_tokens: int = 512,
                 max_sequence_length: int = 131072, kv_capacity_tokens: int = 32768, page_size: int = 16,
                 cuda_graphs: bool = True):
        self.config = EngineConfig(max_queue=max_queue, max_running=max_running, max_batch_tokens=max_batch_tokens,
                                   prefill_chunk_tokens=prefill_chunk_tokens, max_sequence_length=max_sequence_length,
                                   kv_capacity_tokens=kv_capacity_tokens, page_size=page_size, dtype=dtype,
                                   device=device, cuda_graphs=cuda_graphs)
        self.config.validate()
        self.model_path = model_path
        self.model = load_model(model_path, dtype=dtype, device_index=device)
        self.stepper = make_stepper(self.model, capacity_tokens=kv_capacity_tokens, page_size=page_size,
                                    max_requests=max_running, max_step_tokens=prefill_chunk_tokens)
        self.sampler = Sampler(self.model.runtime.device)
        if cuda_graphs:
            self.stepper.enable_graphs(max_running, chunk_rows=prefill_chunk_tokens,
                                       max_sequence_length=max_sequence_length, max_batch_tokens=max_batch_tokens)
        self.scheduler = Scheduler(self.config, self.stepper.cache, self.stepper.step, self.sampler.sample,
                                   eos_token_ids=self.model.spec.eos_token_ids,
                                   max_positions=self.model.spec.max_positions,
                                   capacity_tokens=self.stepper.cache.num_pages * page_size,
                                   run_and_sample=self.stepper.step_and_sample,
                                   launch_decode=self.stepper.launch_decode if cuda_graphs else None,
                                   can_launch_decode=self.stepper.can_launch_decode if cuda_graphs else None)
        self.tokenizer = self._load_tokenizer(model_path)

    @staticmethod
    def _load_tokenizer(model_path: str):
        path = os.path.join(model_path, "tokenizer.json")
        if not os.path.exists(path):
            return None
        try:
            from tokenizers import Tokenizer
        except ImportError:
            return None
        return Tokenizer.from_file(path)

    def _encode(self, prompt: Union[str, Sequence[int]]) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer.json in the model folder; pass token ids instead")
            return list(self.tokenizer.encode(prompt).ids)
        return [int(t) for t in prompt]

    @staticmethod
    def _check_device_waits() -> None:
        """Every wait inside the tcgen05 kernels is bounded; one that ran out leaves a code on the device and the
        results of that launch are not to be trusted.  Fail loudly rather than return them."""
        from .. import kernels

        code = kernels.tcgen05_error()
        if code:
            raise RuntimeError(f"a bounded wait inside a tcgen05 kernel ran out (code {code}); the generated "
                               f"tokens of this call are unreliable")

    def replay(self, trace) -> List[Optional["torch.Tensor"]]:
        """Feed given token ids step by step and return the logits at the wanted places: for each step of ``trace``
        (``{"step", "entries": [{"id", "tokens", "want"}], "end"}``, the replay program's records) float32
        ``[wanted, vocab]`` on the host, or ``None``.  It drives this engine's own step function and cache and
        samples nothing; use it while no generation is in flight."""
        from .replay import TraceRunner

        if self.scheduler.has_work():
            raise RuntimeError("replay needs an idle engine: generation is in flight")
        runner = TraceRunner(self.stepper)
        out = []
        for record in trace:
            logits = runner.step(record)
            out.append(None if logits is None else logits.cpu())
        return out

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[RequestOutput]:
        """Generate for every prompt under continuous batching; outputs in the order of the prompts."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or one for all)")
        encoded = [self._encode(p) for p in prompts]
        pending = list(zip(range(len(prompts)), encoded, sampling_params))
        room = self.config.max_pending + self.config.max_running
        done: Dict[int, Request] = {}
        ids: Dict[Hashable, int] = {}
        while pending or self.scheduler.has_work():
            while pending and len(self.scheduler.requests) < room:
                index, tokens, params = pending.pop(0)
                ids[self.scheduler.add_request(tokens, params)] = index
            result = self.scheduler.step()
            for request in result.finished:
                done[ids.pop(request.id)] = request
        self._check_device_waits()
        outputs = []
        for index in range(len(prompts)):
            request = done[index]
            tokens = list(request.generated)
            text = None
            if self.tokenizer is not None:
                text = self.tokenizer.decode(tokens)
                for stop in request.params.stop:
                    cut = text.find(stop)
                    if cut >= 0:
                        text = text[:cut]
            outputs.append(RequestOutput(index, request.prompt, tokens, request.finish_reason, text, request.error))
        return outputs
