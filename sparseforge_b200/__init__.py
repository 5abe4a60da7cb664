"""B200-native (sm_100a) implementation of the SparseForge SparseLinear hot path.

Python host code mirroring the reference's ``legacy/sparse_modeling.py``, ``legacy/utils.py`` and
``legacy/adamw.py`` interfaces over a C-ABI CUDA library (``include/sparseforge_b200.h``).
"""
from . import _lib  # noqa: F401
from .adamw import AdamW  # noqa: F401
from .sparse_modeling import (  # noqa: F401
    STE,
    SRSTE,
    Distill_Model,
    FusedMaskedLinearSTE,
    SparseLinear,
    SparseLinearConfig,
)

__all__ = ["AdamW", "STE", "SRSTE", "Distill_Model", "FusedMaskedLinearSTE", "SparseLinear", "SparseLinearConfig"]
