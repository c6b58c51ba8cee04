"""Architectures; importing this package registers them."""

from . import llama  # noqa: F401  (registration)
from .decoder import DecoderModel, expected_tensors, tensor_roles
from .llama_config import LlamaConfig, RopeScaling
