from .llm import LLM, RequestOutput
from .loading import load_model, make_stepper, parse_dtype, require_cuda
from .replay import TraceRunner
from .scheduler import (EngineOverloaded, Request, RequestRejected, ScheduledSequence, Scheduler, StepResult)
from .step import StepEntry, StepError, Stepper
