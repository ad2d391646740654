"""Weights: the safetensors container, model folders, the one-error check, random weights."""

from .checkpoint import Checkpoint
from .loader import (ROLE_EMBEDDING, ROLE_LINEAR, ROLE_NORM, RandomWeights, WeightDecl, WeightStore, check_store,
                     device_dtype, load_weights, random_tensor, tensor_seed)
from .random_model import write_random_model
from .safetensors_io import SafetensorsFile, TensorRecord, save_safetensors

__all__ = [
    "Checkpoint", "ROLE_EMBEDDING", "ROLE_LINEAR", "ROLE_NORM", "RandomWeights", "SafetensorsFile",
    "TensorRecord", "WeightDecl", "WeightStore", "check_store", "device_dtype", "load_weights", "random_tensor",
    "save_safetensors", "tensor_seed", "write_random_model",
]
