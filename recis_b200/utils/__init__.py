from .async_scalar import AsyncScalarReader
from .data_utils import copy_data_to_device
from .launch import finish_distributed, init_distributed
from .logger import Logger
from .parser import ArgumentParser

__all__ = ["Logger", "AsyncScalarReader", "copy_data_to_device", "ArgumentParser", "init_distributed", "finish_distributed"]
