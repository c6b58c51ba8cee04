from .loading import load_model, make_stepper, parse_dtype, require_cuda
from .step import StepEntry, StepError, Stepper
