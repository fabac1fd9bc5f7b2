from .checkpoint_reader import CheckpointReader
from .convert_v1_to_v2 import convert_v1_to_v2
from .loader import Loader
from .saver import Saver

__all__ = ["Saver", "Loader", "CheckpointReader", "convert_v1_to_v2"]
