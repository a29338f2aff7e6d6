from .distributed import SequenceParallel

__all__ = ["SequenceParallel"]
