from .loader import Checkpoint, TensorSource, WeightError, storage_dtype
from .random_init import draw_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
