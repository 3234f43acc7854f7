from .loader import (WeightError, build_model, check_tensors, load_model, parse_dtype, random_tensors,
                     read_safetensors, write_random_model)

__all__ = ["WeightError", "build_model", "check_tensors", "load_model", "parse_dtype", "random_tensors",
           "read_safetensors", "write_random_model"]
