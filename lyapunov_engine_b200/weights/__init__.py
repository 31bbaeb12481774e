from .loader import FolderWeights, RandomWeights, WeightsError, write_random_model
from .safetensors_io import SafetensorsError, open_folder, save_file

__all__ = ["FolderWeights", "RandomWeights", "WeightsError", "write_random_model", "SafetensorsError",
           "open_folder", "save_file"]
