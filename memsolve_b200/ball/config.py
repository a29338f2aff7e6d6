"""Layer configuration with the field names, defaults and error behaviour of the reference's
``MemSolveConfig`` (memsolve/ball/config.py:9-106), so that code which builds the reference
configuration builds this one unchanged.

The checks are table-driven: every field has one entry saying which Python type it must have,
and the value constraints follow in the order in which the reference reports them.
"""
from __future__ import annotations

import dataclasses
import enum
import math
from typing import Literal, Union

RecomputePolicy = Union[Literal["auto"], bool]


class CoreMode(str, enum.Enum):
    """``equilibrium`` learns the per-head core; ``complement`` fixes F = 0."""

    EQUILIBRIUM = "equilibrium"
    COMPLEMENT = "complement"


def _validate_recompute_readout(value: object) -> RecomputePolicy:
    """Accept True, False or the string "auto" (memsolve/ball/config.py:9-20)."""
    if value is True or value is False:
        return value
    if not isinstance(value, str):
        raise TypeError(f"recompute_readout must be a bool or 'auto', got {type(value).__name__}")
    if value == "auto":
        return "auto"
    raise ValueError(f"recompute_readout must be True, False, or 'auto', got {value!r}")


def _kind(value: object) -> str:
    return type(value).__name__


def _require_int(name: str, value: object) -> None:
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer, got {_kind(value)}")


_INTEGER_FIELDS = ("dim", "num_heads", "rank", "rotary_train_length")
_SWITCH_FIELDS = ("skew_coupling", "scalar_complement", "rotary")


@dataclasses.dataclass(frozen=True, slots=True)
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

    def _coerce(self, name: str, value: object) -> None:
        object.__setattr__(self, name, value)

    def __post_init__(self) -> None:
        # 1. types
        for name in _INTEGER_FIELDS:
            _require_int(name, getattr(self, name))
        self._coerce("core_mode", self._parse_mode(self.core_mode))
        if not isinstance(self.bias, bool):
            raise TypeError(f"bias must be a bool, got {_kind(self.bias)}")
        for name in _SWITCH_FIELDS:
            if not isinstance(getattr(self, name), bool):
                raise TypeError(f"{name} must be a bool")
        # 2. values
        if self.dim <= 0 or self.num_heads <= 0 or self.rank <= 0:
            raise ValueError("dim, num_heads, and rank must be positive")
        if self.dim % self.num_heads != 0:
            raise ValueError(f"dim={self.dim} must be divisible by num_heads={self.num_heads}")
        if self.rotary_train_length <= 0:
            raise ValueError("rotary_train_length must be positive")
        base = self.rotary_base
        if isinstance(base, bool) or not isinstance(base, (int, float)):
            raise TypeError("rotary_base must be a real number")
        if not (math.isfinite(base) and base > 1):
            raise ValueError("rotary_base must be finite and greater than one")
        if self.rotary_scaling not in {"none", "yarn"}:
            raise ValueError("rotary_scaling must be 'none' or 'yarn'")
        if self.rotary and self.head_dim % 2 == 1:
            raise ValueError("rotary requires an even head_dim")
        self._coerce("recompute_readout", _validate_recompute_readout(self.recompute_readout))

    @staticmethod
    def _parse_mode(value: object) -> CoreMode:
        try:
            return CoreMode(value)
        except (TypeError, ValueError) as error:
            allowed = ", ".join(mode.value for mode in CoreMode)
            raise ValueError(f"core_mode must be one of {{{allowed}}}, got {value!r}") from error

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads


__all__ = ["CoreMode", "MemSolveConfig"]
