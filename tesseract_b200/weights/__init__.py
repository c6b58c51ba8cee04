from .loader import ExpectedTensor, WeightError, check_and_load
from .safetensors_io import SafetensorsError, SafetensorsFile, SafetensorsSource, write_safetensors
