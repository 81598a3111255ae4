from .loader import WeightsError, load_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_folder, save_file
