from .loader import WeightError, check_names, clean_name, load_tensors
from .random_init import write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, model_files, read_header, write_safetensors
