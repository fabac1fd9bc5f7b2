from .feature import Feature
from .feature_engine import FeatureEngine
from .op import Bucketize, FeatureCross, Hash, IDMultiHash, Mod, SelectField, SelectFields, SequenceTruncate

__all__ = ["Feature", "FeatureEngine", "SelectField", "SelectFields", "Hash", "Mod", "Bucketize", "FeatureCross",
           "SequenceTruncate", "IDMultiHash"]
