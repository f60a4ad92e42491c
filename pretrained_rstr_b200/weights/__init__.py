from .loader import (TensorExpectation, WeightError, WeightStore, load_weights,
                     make_random_model, normal, tensor_generator, write_model_folder)
from .safetensors_io import SafetensorsError, SafetensorsFile, load_file, save_file

__all__ = ["TensorExpectation", "WeightError", "WeightStore", "load_weights",
           "make_random_model", "normal", "tensor_generator", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "load_file", "save_file"]
