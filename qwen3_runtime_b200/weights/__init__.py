from .loader import DictSource, SafetensorsDir, WeightError, check_tensors, load_into, place
from .random_init import RandomDeviceSource, expected_tensors_for, random_state, write_random_model

__all__ = [
    "DictSource",
    "RandomDeviceSource",
    "SafetensorsDir",
    "WeightError",
    "check_tensors",
    "expected_tensors_for",
    "load_into",
    "place",
    "random_state",
    "write_random_model",
]
