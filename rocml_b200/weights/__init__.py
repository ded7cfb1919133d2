"""Weights: safetensors reading and writing, loading by name, random models."""
from .decl import TensorDecl
from .safetensors_io import ModelFiles, NativeReader, SafetensorsFile, save_state_dict, write_safetensors
from .loader import UnexpectedTensors, check_against, load_tensors, storage_dtype
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = [
    "TensorDecl", "ModelFiles", "NativeReader", "SafetensorsFile", "save_state_dict", "write_safetensors",
    "UnexpectedTensors", "check_against", "load_tensors", "storage_dtype", "random_tensor", "random_tensors",
    "write_random_model",
]
