from .loader import WeightsError, check, load
from .random_init import write_random_model
from .safetensors_io import CheckpointReader, SafetensorsError, SafetensorsFile, SafetensorsWriter, save_file
