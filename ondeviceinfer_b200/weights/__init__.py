from .loader import Fetcher, WeightsError, check
from .random_init import write_random_model
from .tensors import RandomSource, SafetensorsSource, StoredTensor, TensorDecl

__all__ = ["Fetcher", "WeightsError", "check", "write_random_model", "RandomSource",
           "SafetensorsSource", "StoredTensor", "TensorDecl"]
