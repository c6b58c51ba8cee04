"""The scheduler above the step function: admit, cut prompts into portions, decode, finish, free.

Behaviour follows the reference's engine thread (src/engine/scheduler.rs):

* ``add_request`` (:531-603) bounds the number of known requests by
  ``max_queue + max_running`` (overload is an error to the caller), validates the
  options, rejects an empty prompt and a request whose ``prompt + max_tokens`` exceeds
  the sequence limit, the model's positions or the whole cache.
* ``admit_waiting`` (:605-633) scans the waiting queue once, first come first served;
  a request is admitted only if the cache manager can give it a state slot **and**
  reserve pages for ``prompt + max_tokens`` tokens in every group.  One that does not
  fit goes to the back of the queue, so a smaller one may pass it.  This is what
  happens when pages run out: nothing running is ever preempted, swapped or
  recomputed, and a running request cannot run out, because its peak need was set
  aside at admission.
* ``build_batch`` (:635-722) spends ``max_batch_tokens`` on decode rows first (one token
  each), then on prompt portions of at most ``prefill_chunk_tokens``; only a portion that
  ends the known tokens samples; one uniform is drawn per sampled non-greedy row; the
  running queue rotates by one after every batch.
* ``apply`` (:724-833) appends sampled tokens and finishes on a stop token, an
  end-of-sequence id or ``max_tokens``; a failed step fails the requests of its batch,
  frees what they held and leaves the engine serving (:495-505).

Not in the reference: while every running request is decoding, steps are launched one ahead
of the read-back of their tokens.  The step function takes a sequence's token from the
previous step's sampler output on the device, so the host builds and launches step k + 1
while step k runs and only then looks at step k's tokens (stop tokens, end of sequence).
A request that turns out to have ended at step k has one row of step k + 1 computed in
vain; its token is dropped.  The tokens each request receives are the same either way.
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.rng import SplitMix64
from .step import StepEntry

FINISH_STOP = "stop"
FINISH_LENGTH = "length"
FINISH_CANCELLED = "cancelled"
FINISH_ERROR = "error"


class EngineOverloaded(RuntimeError):
    """More requests than ``max_queue + max_running`` are known to the engine."""


class RequestRejected(ValueError):
    """A request that can never be served (empty, too long, bad options)."""


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    rng: SplitMix64
    generated: List[int] = field(default_factory=list)
    computed_tokens: int = 0
    finish_reason: Optional[str] = None
    error: Optional[str] = None

    @property
    def target_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def reservation_tokens(self) -> int:
        return len(self.prompt) + self.params.max_tokens

    def token_range(self, begin: int, end: int) -> List[int]:
        n = len(self.prompt)
        if end <= n:
            return self.prompt[begin:end]
        if begin >= n:
            return self.generated[begin - n:end - n]
        return self.prompt[begin:] + self.generated[:end - n]


@dataclass
class ScheduledSequence:
    request: Request
    begin: int
    tokens: List[int]
    samples: bool
    draw: float = 0.0
    slot: int = -1          # launched ahead: index in ``request.generated`` that this step's token will fill

    @property
    def is_decode(self) -> bool:
        return self.begin >= len(self.request.prompt)


@dataclass
class StepResult:
    """What one scheduler iteration did.  ``new_tokens`` holds, per request, the tokens it received in this
    iteration, oldest first (two when a step launched ahead was read back and an ordinary step followed)."""

    batch: List[ScheduledSequence]
    new_tokens: Dict[Hashable, List[int]]
    finished: List[Request]

    def token_count(self) -> int:
        return sum(len(tokens) for tokens in self.new_tokens.values())

    def absorb_earlier(self, earlier: "StepResult") -> None:
        """Put the tokens and endings of a step that was read back before this one in front of this one's."""
        merged = {request: list(tokens) for request, tokens in earlier.new_tokens.items()}
        for request, tokens in self.new_tokens.items():
            merged.setdefault(request, []).extend(tokens)
        self.new_tokens = merged
        self.finished[:0] = earlier.finished


class Scheduler:
    """``run_step(entries)`` runs the model and returns logits rows for the wanted places;
    ``sample(logits, temperatures, top_ps, draws)`` returns one token per row.  Both are
    injected, so the scheduler's decisions can be tested without a device."""

    def __init__(self, config: EngineConfig, cache, run_step: Callable, sample: Callable, *, eos_token_ids=(),
                 max_positions: Optional[int] = None, capacity_tokens: Optional[int] = None,
                 run_and_sample: Optional[Callable] = None, launch_decode: Optional[Callable] = None,
                 can_launch_decode: Optional[Callable] = None):
        config.validate()
        self.config = config
        self.cache = cache
        self.run_step = run_step
        self.sample = sample
        self.run_and_sample = run_and_sample    # (entries, temperatures, top_ps, draws) -> tokens, in one call
        # launch_decode(entries, temperatures, draws, previous, fed) -> launch with .tokens(); can_launch_decode(
        # number of rows, top_ps) says whether a pure decode batch may go that way.  Both or neither.
        self.launch_decode = launch_decode
        self.can_launch_decode = can_launch_decode
        self._inflight: Optional[Tuple[List[ScheduledSequence], object]] = None   # launched, tokens not read yet
        self.eos_token_ids = frozenset(int(t) for t in eos_token_ids)
        self.max_positions = max_positions
        self.capacity_tokens = capacity_tokens if capacity_tokens is not None else config.kv_capacity_tokens
        self.requests: Dict[Hashable, Request] = {}
        self.waiting: Deque[Hashable] = deque()
        self.running: Deque[Hashable] = deque()
        self._ids = itertools.count()
        self.steps = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: SamplingParams, request_id: Hashable = None) -> Hashable:
        if len(self.requests) >= self.config.max_pending + self.config.max_running:
            raise EngineOverloaded("the inference engine is overloaded")
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRejected("the prompt is empty")
        total = len(prompt) + params.max_tokens
        limit = min(self.config.max_sequence_length, self.capacity_tokens)
        if self.max_positions is not None:
            limit = min(limit, self.max_positions)
        if total > limit:
            raise RequestRejected(f"prompt plus max_tokens ({total}) exceeds the configured capacity ({limit})")
        if request_id is None:
            request_id = next(self._ids)
        if request_id in self.requests:
            raise RequestRejected(f"request id {request_id!r} is already in use")
        seed = params.seed if params.seed is not None else hash(request_id) & ((1 << 64) - 1)
        self.requests[request_id] = Request(request_id, prompt, params, SplitMix64(seed))
        self.waiting.append(request_id)
        return request_id

    def cancel(self, request_id: Hashable) -> None:
        self._finish(request_id, FINISH_CANCELLED)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one iteration
    def admit_waiting(self) -> None:
        for _ in range(len(self.waiting)):
            if len(self.running) >= self.config.max_running:
                break
            request_id = self.waiting.popleft()
            request = self.requests.get(request_id)
            if request is None:
                continue
            if self.cache.admit(request_id, reserve_tokens=request.reservation_tokens):
                self.running.append(request_id)
            else:
                self.waiting.append(request_id)

    def build_batch(self) -> List[ScheduledSequence]:
        budget = self.config.max_batch_tokens
        batch: List[ScheduledSequence] = []
        ids = list(self.running)
        for decode_phase in (True, False):
            for request_id in ids:
                if budget == 0:
                    break
                request = self.requests.get(request_id)
                if request is None:
                    continue
                is_decode = request.computed_tokens >= len(request.prompt)
                if is_decode != decode_phase:
                    continue
                remaining = request.target_tokens - request.computed_tokens
                if remaining <= 0:
                    continue
                if is_decode and len(request.generated) >= request.params.max_tokens:
                    continue    # its last token is in flight (steps launched ahead): nothing more to compute
                limit = 1 if is_decode else self.config.prefill_chunk_tokens
                count = min(remaining, limit, budget)
                begin = request.computed_tokens
                samples = begin + count == request.target_tokens
                draw = 0.0
                if samples and request.params.temperature != 0.0:
                    draw = request.rng.unit_f64()
                batch.append(ScheduledSequence(request, begin, request.token_range(begin, begin + count), samples, draw))
                budget -= count
        if len(self.running) > 1:
            self.running.rotate(-1)
        # prompt portions first, then decode rows (src/engine/batch.rs:355-428); among the portions the full ones
        # first (a step of full portions, one shorter one and decode rows is a shape that replays as a graph); order
        # otherwise kept
        full = self.config.prefill_chunk_tokens
        batch.sort(key=lambda s: (s.is_decode, len(s.tokens) != full))
        return batch

    def step(self) -> StepResult:
        """Admit, build one batch, run it, sample, apply.  Returns what happened."""
        self.admit_waiting()
        if self._may_launch_ahead():
            return self._step_launched_ahead()
        drained = self._drain()
        batch = self.build_batch()
        if not batch:
            return drained or StepResult([], {}, [])
        self.steps += 1
        entries = [StepEntry(s.request.id, s.tokens, [len(s.tokens) - 1] if s.samples else []) for s in batch]
        sampled = [s for s in batch if s.samples]
        try:
            temperatures = [s.request.params.temperature for s in sampled]
            top_ps = [s.request.params.top_p for s in sampled]
            draws = [s.draw for s in sampled]
            if self.run_and_sample is not None:
                tokens = self.run_and_sample(entries, temperatures, top_ps, draws)
            else:
                logits = self.run_step(entries)
                tokens = self.sample(logits, temperatures, top_ps, draws) if sampled else []
            if len(tokens) != len(sampled):
                raise RuntimeError("the sampler returned a wrong number of tokens")
        except Exception as exc:  # noqa: BLE001 - a failed step fails its batch, the engine keeps serving
            result = self._fail(batch, exc)
        else:
            result = self._apply(batch, sampled, tokens)
        if drained is not None:
            result.absorb_earlier(drained)
        return result

    def _fail(self, batch, exc) -> StepResult:
        finished = []
        for s in batch:
            if s.request.finish_reason is None:
                s.request.error = f"{type(exc).__name__}: {exc}"
                finished.append(self._finish(s.request.id, FINISH_ERROR))
        return StepResult(batch, {}, [r for r in finished if r is not None])

    # ------------------------------------------------------------------ steps launched ahead of their read-back
    def _may_launch_ahead(self) -> bool:
        if self.launch_decode is None or not self.running:
            return False
        requests = [self.requests[i] for i in self.running]
        if any(r.computed_tokens < len(r.prompt) for r in requests):
            return False                                  # prompt portions: those steps run the ordinary way
        return bool(self.can_launch_decode(len(requests), [r.params.top_p for r in requests]))

    def _step_launched_ahead(self) -> StepResult:
        previous = self._inflight
        batch = self.build_batch()
        if not batch:                                     # every running request waits for a token in flight
            return self._drain() or StepResult([], {}, [])
        self.steps += 1
        fed = [s.tokens[0] is None for s in batch]        # the token is still on the device: feed it from there
        entries = [StepEntry(s.request.id, [0 if f else s.tokens[0]], [0]) for s, f in zip(batch, fed)]
        try:
            launch = self.launch_decode(entries, [s.request.params.temperature for s in batch],
                                        [s.draw for s in batch], previous[1] if previous else None, fed)
        except Exception as exc:  # noqa: BLE001
            self._inflight = None
            result = self._fail(batch, exc)
            if previous is not None:
                result.absorb_earlier(self._collect(previous))
            return result
        for s in batch:
            s.request.computed_tokens += 1
            s.slot = len(s.request.generated)
            s.request.generated.append(None)              # filled when the launch is read back
        self._inflight = (batch, launch)
        if previous is None:
            return StepResult(batch, {}, [])
        result = self._collect(previous)
        return StepResult(batch, result.new_tokens, result.finished)

    def _drain(self) -> Optional[StepResult]:
        """Read back the step that is in flight, if any."""
        if self._inflight is None:
            return None
        inflight, self._inflight = self._inflight, None
        return self._collect(inflight)

    def _collect(self, inflight) -> StepResult:
        batch, launch = inflight
        try:
            tokens = launch.tokens()
            if len(tokens) != len(batch):
                raise RuntimeError("the sampler returned a wrong number of tokens")
        except Exception as exc:  # noqa: BLE001
            return self._fail(batch, exc)
        new_tokens: Dict[Hashable, List[int]] = {}
        finished: List[Request] = []
        for s, token in zip(batch, tokens):
            request = s.request
            if request.finish_reason is not None:
                continue                                  # ended meanwhile: this row was computed in vain
            token = int(token)
            request.generated[s.slot] = token
            new_tokens.setdefault(request.id, []).append(token)
            reason = self._stop_reason(request, token, s.slot + 1)
            if reason is not None:
                del request.generated[s.slot + 1:]        # a token launched after the last one is dropped
                request.computed_tokens = min(request.computed_tokens, len(request.prompt) + s.slot)
                done = self._finish(request.id, reason)
                if done is not None:
                    finished.append(done)
        return StepResult(batch, new_tokens, finished)

    def _stop_reason(self, request: Request, token: int, generated: int) -> Optional[str]:
        if token in request.params.stop_token_ids:
            return FINISH_STOP
        if token in self.eos_token_ids and not request.params.ignore_eos:
            return FINISH_STOP
        if generated >= request.params.max_tokens:
            return FINISH_LENGTH
        return None

    def _apply(self, batch, sampled, tokens) -> StepResult:
        new_tokens: Dict[Hashable, List[int]] = {}
        finished: List[Request] = []
        for s in batch:
            s.request.computed_tokens += len(s.tokens)
        for s, token in zip(sampled, tokens):
            request = s.request
            token = int(token)
            request.generated.append(token)
            new_tokens.setdefault(request.id, []).append(token)
            reason = self._stop_reason(request, token, len(request.generated))
            if reason is not None:
                done = self._finish(request.id, reason)
                if done is not None:
                    finished.append(done)
        return StepResult(batch, new_tokens, finished)

    def _finish(self, request_id: Hashable, reason: str) -> Optional[Request]:
        request = self.requests.pop(request_id, None)
        if request is None:
            return None
        request.finish_reason = reason
        request.generated = [t for t in request.generated if t is not None]   # a token still in flight is dropped
        try:
            self.waiting.remove(request_id)
        except ValueError:
            pass
        try:
            self.running.remove(request_id)
        except ValueError:
            pass
        self.cache.release(request_id)
        return request
