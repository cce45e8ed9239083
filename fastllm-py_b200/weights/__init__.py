from .loader import WeightError, check_store, load_tensors, write_model_folder
from .store import RandomStore, SafetensorsStore, kept_dtype

__all__ = ["WeightError", "check_store", "load_tensors", "write_model_folder", "RandomStore",
           "SafetensorsStore", "kept_dtype"]
