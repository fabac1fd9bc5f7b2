"""Feature engine: op chains per feature, compiled step-wise so that same-type ops of a step run as one fused kernel call.

Public names (the reference's ``recis.features`` plus ``Feature``): see ``__all__``."""
from . import feature as _feature_mod
from . import feature_engine as _engine_mod
from . import op as _op_mod

_OP_NAMES = ("SelectField", "SelectFields", "Hash", "Mod", "Bucketize", "IDMultiHash", "SequenceTruncate", "FeatureCross")

Feature = _feature_mod.Feature
FeatureEngine = _engine_mod.FeatureEngine
globals().update({_n: getattr(_op_mod, _n) for _n in _OP_NAMES})

__all__ = ["Feature", "FeatureEngine", *_OP_NAMES]
