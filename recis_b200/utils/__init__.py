from .data_utils import copy_data_to_device
from .logger import Logger
from .parser import ArgumentParser

__all__ = ["Logger", "copy_data_to_device", "ArgumentParser"]
