"""Weights by tensor name: safetensors files, checks, seeded random filling."""
from .loader import (DictSource, WeightError, WeightSpec, check_source, load_tensors, open_model_folder,
                     random_tensors, write_model_folder)
from .safetensors_io import SafetensorsError, SafetensorsFile, SafetensorsFolder, write_safetensors
