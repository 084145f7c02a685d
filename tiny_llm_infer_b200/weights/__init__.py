from .loader import WeightsError, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files, save_file, save_sharded
