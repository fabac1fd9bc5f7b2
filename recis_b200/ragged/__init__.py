from .tensor import RaggedPadInfo, RaggedTensor

__all__ = ["RaggedTensor", "RaggedPadInfo"]
