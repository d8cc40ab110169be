from .loader import WeightsError, check_tensors, load_tensors
from .random_init import make_tensor, write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, save_file
