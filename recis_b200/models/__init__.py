from .deepfm import DeepFM
from .dlrm import DLRM
from .seq_model import SequenceModel

__all__ = ["DLRM", "DeepFM", "SequenceModel"]
