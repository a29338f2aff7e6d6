"""B200-native MemSolve layer (forward + backward of the token mixer on sm_100a).

Public names mirror the reference package ``memsolve`` (memsolve/__init__.py:1-7):
``MemSolve``, ``MemSolveConfig``, ``CoreMode``.  The CUDA path is the only
evaluation path shipped here; there is no CPU fallback.
"""
from .ball import CoreMode, MemSolve, MemSolveConfig

__version__ = "0.1.0"

__all__ = ["CoreMode", "MemSolve", "MemSolveConfig", "__version__"]
