"""B200-native MemSolve layer (forward + backward of the token mixer on sm_100a).

Public names mirror the reference package ``memsolve`` (memsolve/__init__.py:1-7):
``MemSolve``, ``MemSolveConfig``, ``CoreMode``.  The CUDA path is the only
evaluation path shipped here; there is no CPU fallback.
"""
from memsolve_b200 import ball as _ball

__version__ = "0.2.0"

MemSolve = _ball.MemSolve
MemSolveConfig = _ball.MemSolveConfig
CoreMode = _ball.CoreMode

__all__ = ("MemSolve", "MemSolveConfig", "CoreMode", "__version__")
