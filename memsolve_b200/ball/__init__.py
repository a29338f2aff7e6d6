"""The layer, its configuration and the CUDA operator module (``memsolve_b200.ball.cuda``).

The three public names are those of the reference's ``memsolve.ball`` package.
"""
from . import config as _config
from . import model as _model

CoreMode = _config.CoreMode
MemSolveConfig = _config.MemSolveConfig
MemSolve = _model.MemSolve

__all__ = ("MemSolve", "MemSolveConfig", "CoreMode")
