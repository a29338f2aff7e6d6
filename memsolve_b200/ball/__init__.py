from .config import CoreMode, MemSolveConfig
from .model import MemSolve

__all__ = ["CoreMode", "MemSolve", "MemSolveConfig"]
