"""Layer configuration, mirroring the reference's ``MemSolveConfig``.

Field names, defaults, validation order and error types follow
memsolve/ball/config.py:9-106 of the reference so that code constructing the
reference configuration constructs this one unchanged.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Literal

RecomputePolicy = Literal["auto"] | bool


def _validate_recompute_readout(value: object) -> RecomputePolicy:
    """True / False / "auto" (memsolve/ball/config.py:9-20)."""
    if isinstance(value, bool):
        return value
    if isinstance(value, str):
        if value != "auto":
            raise ValueError(f"recompute_readout must be True, False, or 'auto', got {value!r}")
        return "auto"
    raise TypeError(f"recompute_readout must be a bool or 'auto', got {type(value).__name__}")


class CoreMode(str, Enum):
    """``equilibrium`` learns the per-head core; ``complement`` fixes F = 0."""

    EQUILIBRIUM = "equilibrium"
    COMPLEMENT = "complement"


def _is_plain_int(value: object) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


@dataclass(frozen=True, slots=True)
class MemSolveConfig:
    dim: int
    num_heads: int
    rank: int = 16
    core_mode: CoreMode = CoreMode.EQUILIBRIUM
    bias: bool = False
    skew_coupling: bool = True
    scalar_complement: bool = True
    rotary: bool = False
    rotary_base: float = 10000.0
    rotary_train_length: int = 128
    rotary_scaling: str = "yarn"
    recompute_readout: RecomputePolicy = "auto"

    def __post_init__(self) -> None:
        for field in ("dim", "num_heads", "rank", "rotary_train_length"):
            value = getattr(self, field)
            if not _is_plain_int(value):
                raise TypeError(f"{field} must be an integer, got {type(value).__name__}")
        try:
            mode = CoreMode(self.core_mode)
        except (TypeError, ValueError) as error:
            names = ", ".join(m.value for m in CoreMode)
            raise ValueError(f"core_mode must be one of {{{names}}}, got {self.core_mode!r}") from error
        object.__setattr__(self, "core_mode", mode)
        if not isinstance(self.bias, bool):
            raise TypeError(f"bias must be a bool, got {type(self.bias).__name__}")
        for field in ("skew_coupling", "scalar_complement", "rotary"):
            if not isinstance(getattr(self, field), bool):
                raise TypeError(f"{field} must be a bool")
        if min(self.dim, self.num_heads, self.rank) <= 0:
            raise ValueError("dim, num_heads, and rank must be positive")
        if self.dim % self.num_heads:
            raise ValueError(f"dim={self.dim} must be divisible by num_heads={self.num_heads}")
        if self.rotary_train_length <= 0:
            raise ValueError("rotary_train_length must be positive")
        if not isinstance(self.rotary_base, (int, float)) or isinstance(self.rotary_base, bool):
            raise TypeError("rotary_base must be a real number")
        if not math.isfinite(self.rotary_base) or self.rotary_base <= 1:
            raise ValueError("rotary_base must be finite and greater than one")
        if self.rotary_scaling not in ("none", "yarn"):
            raise ValueError("rotary_scaling must be 'none' or 'yarn'")
        if self.rotary and self.head_dim % 2:
            raise ValueError("rotary requires an even head_dim")
        object.__setattr__(self, "recompute_readout", _validate_recompute_readout(self.recompute_readout))

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads


__all__ = ["CoreMode", "MemSolveConfig"]
