"""``MemSolve`` layer module: host-side mirror of the reference's ``memsolve.ball.model``.

Parameters, their initialisation order, the checkpoint contract and the
``forward`` signature follow memsolve/ball/model.py:33-635 so that weights and
state dicts move between the two packages unchanged.  Only
``implementation="cuda"`` is evaluated here: projection (BF16 GEMM) -> mixer
kernels (``cuda.fast_mix``) -> projection.  The reference's CPU formulation is
not shipped; asking for it raises.
"""
from __future__ import annotations

import math
from typing import Literal

import torch
import torch.nn as nn

from . import cuda as cuda_backend
from .config import CoreMode, MemSolveConfig, _validate_recompute_readout
from .rotary import rotary_position_factors

_CONTRACT_VERSION = 26
_ETA_INIT = 0.9
_ETA_INIT_RAW = math.atanh(_ETA_INIT)
_SUPPORTED_ACTIVATION_DTYPES = frozenset((torch.float16, torch.bfloat16, torch.float32, torch.float64))
_INTEGER_DTYPES = (torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64)


class MemSolve(nn.Module):
    """Low-rank accretive-equilibrium token mixer (B200 CUDA path only)."""

    def __init__(self, config: MemSolveConfig) -> None:
        super().__init__()
        self.config = config
        self._recompute_readout: Literal["auto"] | bool = _validate_recompute_readout(config.recompute_readout)
        self._rotary_cache: dict = {}
        # creation order fixes the RNG stream and therefore the default weights (model.py:50-71)
        self.w_bc = nn.Linear(config.dim, config.num_heads * config.rank + config.dim, bias=config.bias)
        self.w_o = nn.Linear(config.dim, config.dim, bias=config.bias)
        if config.core_mode is CoreMode.EQUILIBRIUM:
            self.core_base_raw = nn.Parameter(torch.zeros(config.num_heads, config.rank, config.rank))
        else:
            self.register_parameter("core_base_raw", None)
        self.eta_raw = nn.Parameter(
            torch.full((config.num_heads,), _ETA_INIT_RAW if config.scalar_complement else 0.0,
                       dtype=torch.float32),
            requires_grad=config.scalar_complement,
        )

    # ---- runtime policy -------------------------------------------------------------
    @property
    def recompute_readout(self) -> Literal["auto"] | bool:
        """Readout recomputation policy ('auto' recomputes when N > 512)."""
        return self._recompute_readout

    @recompute_readout.setter
    def recompute_readout(self, value: Literal["auto"] | bool) -> None:
        self._recompute_readout = _validate_recompute_readout(value)

    def complement(self) -> torch.Tensor:
        """Per-head eta = (1 - eps) tanh(eta_raw) (zeros when scalar_complement is off)."""
        if not self.config.scalar_complement:
            return torch.zeros_like(self.eta_raw)
        raw = self.eta_raw.float()
        return (1.0 - torch.finfo(torch.float32).eps) * torch.tanh(raw)

    # ---- checkpoint contract (model.py:90-162) ----------------------------------------
    def _contract_state(self) -> dict[str, object]:
        c = self.config
        state: dict[str, object] = {
            "version": _CONTRACT_VERSION,
            "operator": "accretive_equilibrium",
            "dim": c.dim,
            "num_heads": c.num_heads,
            "rank": c.rank,
            "core_mode": c.core_mode.value,
            "eta_parameterization": "per_head_interior_tanh",
            "numerics": "tf32-wbc-ieee-fgram-tc16-v6",
            "bias": c.bias,
        }
        if not c.skew_coupling:
            state["skew_coupling"] = False
        if not c.scalar_complement:
            state["scalar_complement"] = False
        if c.rotary:
            state["rotary"] = {
                "type": "value_transport",
                "layout": "full_head_adjacent_pairs",
                "base": c.rotary_base,
                "train_length": c.rotary_train_length,
                "scaling": c.rotary_scaling,
                "yarn_beta": [32, 1],
                "amplitude": 1.0,
            }
        return state

    def get_extra_state(self) -> dict[str, object]:
        return self._contract_state()

    def set_extra_state(self, state: object) -> None:
        expected = self._contract_state()
        if not isinstance(state, dict):
            raise RuntimeError("MemSolve checkpoint is missing its configuration contract")
        if state != expected:
            diff = ", ".join(
                f"{key}: checkpoint={state.get(key)!r}, model={expected.get(key)!r}"
                for key in sorted(set(state) | set(expected))
                if state.get(key) != expected.get(key)
            )
            raise RuntimeError(f"incompatible MemSolve checkpoint contract ({diff})")

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs) -> None:
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)
        key = f"{prefix}_extra_state"
        if key not in state_dict:
            error_msgs.append(f"MemSolve checkpoint is missing its configuration contract ({key!r})")

    # ---- validation -------------------------------------------------------------------
    @staticmethod
    def _validate_mask(valid_mask, *, batch: int, length: int, device: torch.device) -> torch.Tensor:
        if valid_mask is None:
            return torch.ones(batch, length, dtype=torch.bool, device=device)
        if valid_mask.shape != (batch, length):
            raise ValueError(f"valid_mask must have shape {(batch, length)}, got {tuple(valid_mask.shape)}")
        if valid_mask.dtype != torch.bool:
            raise TypeError(f"valid_mask must have dtype torch.bool, got {valid_mask.dtype}")
        return valid_mask.to(device=device)

    def _validate_input(self, x: torch.Tensor) -> None:
        if x.ndim != 3 or x.shape[-1] != self.config.dim:
            raise ValueError(f"x must have shape [B, N, {self.config.dim}], got {tuple(x.shape)}")
        if x.dtype not in _SUPPORTED_ACTIVATION_DTYPES:
            raise TypeError(
                f"MemSolve does not support x with dtype {x.dtype}; use a floating-point tensor in "
                "torch.float16, torch.bfloat16, torch.float32, or torch.float64"
            )
        if x.shape[0] == 0:
            raise ValueError("batch size must be positive")
        if x.shape[1] == 0:
            raise ValueError("sequence length must be positive")

    # ---- rotary tables (model.py:498-560) ----------------------------------------------
    def _rotary_factors(self, x, valid_mask, position_ids, context_length, *, sequence_parallel=None):
        config = self.config
        if not config.rotary:
            if position_ids is not None or context_length is not None:
                raise ValueError("position_ids and rotary_context_length require rotary=True")
            return None, None
        batch, length, _ = x.shape
        default_positions = position_ids is None
        offset = 0
        if default_positions:
            offset = 0 if sequence_parallel is None else sequence_parallel.offset
        else:
            if not isinstance(position_ids, torch.Tensor) or position_ids.dtype not in _INTEGER_DTYPES:
                raise TypeError("position_ids must be an integer tensor")
            if position_ids.ndim == 1:
                position_ids = position_ids[None]
            if (position_ids.ndim != 2 or position_ids.shape[1] != length
                    or position_ids.shape[0] not in (1, batch)):
                raise ValueError("position_ids must have shape [N], [1,N], or [B,N]")
            position_ids = position_ids.to(device=x.device)
        if context_length is None:
            physical = length if sequence_parallel is None else sequence_parallel.global_length
            if valid_mask is None or config.rotary_scaling == "none" or physical <= config.rotary_train_length:
                context_length = physical
            elif sequence_parallel is not None:
                raise ValueError("masked sequence parallel rotary requires explicit global rotary_context_length")
            else:
                mask = self._validate_mask(valid_mask, batch=batch, length=length, device=x.device)
                index = torch.arange(length, device=x.device)[None]
                first = torch.where(mask, index, length).amin(dim=-1)
                last = torch.where(mask, index, -1).amax(dim=-1)
                context_length = (last - first + 1).clamp_min(1)
        if isinstance(context_length, torch.Tensor):
            if context_length.dtype not in _INTEGER_DTYPES or context_length.requires_grad:
                raise TypeError("rotary_context_length must be a non-differentiable integer tensor")
            if context_length.shape != (batch,):
                raise ValueError("rotary_context_length tensor must have shape [B]")
            context_length = context_length.to(device=x.device)
        elif not isinstance(context_length, int) or isinstance(context_length, bool):
            raise TypeError("rotary_context_length must be an integer or integer tensor [B]")
        elif context_length <= 0:
            raise ValueError("rotary_context_length must be positive")
        # default positions with an integer context give the same table on every call: keep the
        # most recent ones instead of rebuilding them with a dozen small launches per forward
        key = None
        if default_positions and isinstance(context_length, int) and x.dtype != torch.float64:
            key = (x.device, length, offset, context_length)
            cached = self._rotary_cache.get(key)
            if cached is not None:
                return cached
        if default_positions:
            position_ids = torch.arange(offset, offset + length, device=x.device)[None]
        tables = rotary_position_factors(
            position_ids, head_dim=config.head_dim, base=config.rotary_base,
            train_length=config.rotary_train_length, context_length=context_length,
            scaling=config.rotary_scaling, dtype=x.dtype,
        )
        if key is not None and not torch.cuda.is_current_stream_capturing():
            if len(self._rotary_cache) >= 8:
                self._rotary_cache.pop(next(iter(self._rotary_cache)))
            self._rotary_cache[key] = tables
        return tables

    # ---- CUDA forward (model.py:185-356) -----------------------------------------------
    def _forward_cuda(self, x, valid_mask, *, sequence_parallel=None, valid_counts=None, position_ids=None,
                      rotary_context_length=None, rotary_factors=None) -> torch.Tensor:
        config = self.config
        if not config.skew_coupling or not config.scalar_complement or config.rank not in (16, 32, 48, 64):
            raise ValueError(
                "implementation='cuda' requires skew_coupling=True, scalar_complement=True, "
                "and rank in {16, 32, 48, 64}"
            )
        if x.device.type != "cuda":
            raise ValueError("implementation='cuda' requires x to be a CUDA tensor")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError(
                "implementation='cuda' supports x with dtype torch.float16 or torch.bfloat16; "
                f"got {x.dtype}"
            )
        for name, parameter in (
            ("core_base_raw", self.core_base_raw), ("eta_raw", self.eta_raw),
            ("w_bc.weight", self.w_bc.weight), ("w_bc.bias", self.w_bc.bias),
            ("w_o.weight", self.w_o.weight), ("w_o.bias", self.w_o.bias),
        ):
            if parameter is None:
                continue
            if parameter.device != x.device:
                raise RuntimeError(f"implementation='cuda' requires {name} on {x.device}, got {parameter.device}")
            if parameter.dtype != torch.float32:
                raise TypeError(f"implementation='cuda' requires {name} to use torch.float32, got {parameter.dtype}")
            if not parameter.is_contiguous():
                raise RuntimeError(f"implementation='cuda' requires contiguous {name}")

        batch, length, _ = x.shape
        mask = None if valid_mask is None else self._validate_mask(valid_mask, batch=batch, length=length,
                                                                   device=x.device)
        if sequence_parallel is not None:
            sequence_parallel.validate(length, config.rank)
        if rotary_factors is not None:
            rotary_cos, rotary_sin = rotary_factors
        else:
            rotary_cos, rotary_sin = self._rotary_factors(x, mask, position_ids, rotary_context_length,
                                                          sequence_parallel=sequence_parallel)
        if valid_counts is None:
            if sequence_parallel is not None:
                valid_counts = sequence_parallel.valid_counts(mask, batch_size=batch, device=x.device)
            elif mask is not None:
                valid_counts = mask.sum(dim=-1, dtype=torch.float32).clamp_min(1.0)
        elif (valid_counts.shape != (batch,) or valid_counts.device != x.device
              or valid_counts.dtype != torch.float32 or valid_counts.requires_grad
              or not valid_counts.is_contiguous()):
            raise ValueError("valid_counts must be non-differentiable contiguous FP32 [batch] on the input device")

        # packed BF16 coordinates; masked rows are zeroed in the projection epilogue
        projected = cuda_backend.tensor_core_linear(
            x, self.w_bc.weight, self.w_bc.bias, output_dtype=torch.bfloat16,
            fuse_weight_bias_grad=True, output_mask=mask, input_mask=mask,
        )
        core_base = (self.core_base_raw if self.core_base_raw is not None
                     else self.eta_raw.new_empty((config.num_heads, config.rank, 0)))
        policy: Literal["auto"] | bool = (
            self._recompute_readout if torch.is_grad_enabled() and self.w_o.weight.requires_grad else False
        )
        if policy == "auto":
            policy = length > 512
        if torch.compiler.is_compiling() and policy is not False:
            if sequence_parallel is None:
                # traced: mixer + output projection as one registered operator that keeps the compact tape
                return cuda_backend._traced_mix_output_linear(
                    projected, core_base, self.eta_raw, valid_counts, rotary_cos, rotary_sin, self.w_o.weight,
                    self.w_o.bias, x.dtype, mask)
            policy = False
        mix_kwargs = dict(sequence_parallel=sequence_parallel, rotary_cos=rotary_cos, rotary_sin=rotary_sin)
        if policy is False:
            mixed = cuda_backend.fast_mix(projected, core_base, self.eta_raw, valid_counts, **mix_kwargs)
            del projected
            return cuda_backend.tensor_core_linear(
                mixed, self.w_o.weight, self.w_o.bias, output_dtype=x.dtype,
                fuse_weight_bias_grad=True, output_mask=mask)
        with cuda_backend._recompute_scope(policy) as recompute:
            mixed = cuda_backend.fast_mix(projected, core_base, self.eta_raw, valid_counts, **mix_kwargs)
        del projected
        if recompute.spec is not None:
            return cuda_backend._recompute_output_linear(
                mixed, recompute.spec, self.w_o.weight, self.w_o.bias,
                output_dtype=x.dtype, fuse_weight_bias_grad=True, output_mask=mask)
        return cuda_backend.tensor_core_linear(
            mixed, self.w_o.weight, self.w_o.bias, output_dtype=x.dtype,
            fuse_weight_bias_grad=True, output_mask=mask)

    def forward(
        self,
        x: torch.Tensor,
        valid_mask: torch.Tensor | None = None,
        *,
        implementation: str = "reference",
        sequence_parallel=None,
        valid_counts: torch.Tensor | None = None,
        position_ids: torch.Tensor | None = None,
        rotary_context_length: int | torch.Tensor | None = None,
        rotary_factors: tuple[torch.Tensor, torch.Tensor] | None = None,
    ) -> torch.Tensor:
        """Same signature as the reference (model.py:562-573).

        ``implementation="reference"`` remains the default argument value for call
        compatibility, but this package evaluates only ``implementation="cuda"``.
        """
        self._validate_input(x)
        config = self.config
        if rotary_factors is not None and (not config.rotary or position_ids is not None
                                           or rotary_context_length is not None):
            raise ValueError("precomputed rotary_factors require rotary=True and replace position/context inputs")
        if implementation == "cuda":
            return self._forward_cuda(
                x, valid_mask, sequence_parallel=sequence_parallel, valid_counts=valid_counts,
                position_ids=position_ids, rotary_context_length=rotary_context_length,
                rotary_factors=rotary_factors,
            )
        if implementation != "reference":
            raise ValueError(f"implementation must be 'reference' or 'cuda', got {implementation!r}")
        raise RuntimeError(
            "memsolve_b200 ships only the sm_100a CUDA path: call layer(x, implementation='cuda') with a "
            "CUDA tensor. The pure-PyTorch reference formulation is not part of this package."
        )

    def extra_repr(self) -> str:
        c = self.config
        return (f"dim={c.dim}, num_heads={c.num_heads}, rank={c.rank}, core_mode={c.core_mode.value}, "
                f"eta=per-head-interior-tanh, rotary={c.rotary}")


__all__ = ["MemSolve"]
