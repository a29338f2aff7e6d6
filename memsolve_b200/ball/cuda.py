"""Loader and autograd boundary of the B200 MemSolve mixer kernels.

Mirrors the public surface of the reference's ``memsolve.ball.cuda``
(memsolve/ball/cuda.py): ``load``, ``is_available``, ``require_available``,
``fast_mix`` and the private hooks the layer module uses (``_recompute_scope``,
``_recompute_output_linear``, ``_is_default_fast_mix``, ``_TensorCoreLinear``).

Instead of a ``torch.ops`` namespace the native code is a C-ABI shared library
(``memsolve_equilibrium_sm100.so``, declared in ``include/memsolve_b200.h``) opened
with :mod:`ctypes`; tensors cross the boundary as raw device pointers plus the
current CUDA stream.  There is no CPU or PyTorch fallback for the mixer: when
the library is missing every entry point raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from contextlib import contextmanager
from pathlib import Path
from threading import Lock, local
from typing import List, Literal, NamedTuple, Optional

import torch
from torch.autograd.function import once_differentiable

from .config import _validate_recompute_readout

_LOAD_LOCK = Lock()
_RECOMPUTE_LOCAL = local()
_SUPPORTED_ARCHITECTURES = frozenset((100,))
_NATIVE_CONTRACT_VERSION = 1
_LIBRARY_ENV = "MEMSOLVE_CUDA_LIBRARY"
_LIBRARY_PATTERN = re.compile(r"^memsolve_equilibrium(_sm(\d+))?\.so$")

_LIB: ctypes.CDLL | None = None
_LIB_PATH: str | None = None
_LOADED_ARCHITECTURE: frozenset[int] | None = None


# --------------------------------------------------------------------------------------
# C structures (include/memsolve_b200.h)
# --------------------------------------------------------------------------------------
class _Shape(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        "batch", "tokens", "heads", "rank", "head_dim", "complement", "rotary_rows", "reserved")]


class _Tape(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in (
        "eta", "eta_slope", "core_map", "core_info", "inverse", "state", "coeff")]


_P = ctypes.c_void_p
_SIGNATURES = {
    "ms_abi_version": (ctypes.c_int, []),
    "ms_supported_architectures": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int32), ctypes.c_int]),
    "ms_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ms_padded_head_dim": (ctypes.c_int, [ctypes.c_int]),
    "ms_device_error": (ctypes.c_int, []),
    "ms_set_peer_wait_ms": (ctypes.c_int, [ctypes.c_int]),
    "ms_linear_forward": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _P, _P, _P, _P, _P, _P, _P]),
    "ms_linear_input_grad": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _P, _P, _P, _P, _P, _P]),
    "ms_linear_weight_grad_workspace": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]),
    "ms_linear_weight_grad": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _P, _P, _P, _P, _P,
                                             ctypes.c_size_t, _P]),
    "ms_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(_Shape)]),
    "ms_packed_stats_floats": (ctypes.c_size_t, [ctypes.POINTER(_Shape), ctypes.c_int]),
    "ms_core_forward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, ctypes.POINTER(_Tape), _P]),
    "ms_stats_forward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, ctypes.c_size_t, _P, _P]),
    "ms_stats_forward_static": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, _P]),
    "ms_compact_forward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, ctypes.c_size_t, _P,
                                          ctypes.POINTER(_Tape), _P]),
    "ms_readout": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, ctypes.POINTER(_Tape), _P, _P]),
    "ms_readout_short": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, ctypes.POINTER(_Tape), _P, _P]),
    "ms_mix_forward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t,
                                      ctypes.POINTER(_Tape), _P, _P]),
    "ms_stats_backward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, _P, ctypes.c_size_t, _P, _P]),
    "ms_compact_backward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, ctypes.c_size_t, _P,
                                           ctypes.POINTER(_Tape), _P, _P, ctypes.c_float, _P, _P, _P, _P, _P]),
    "ms_token_backward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, ctypes.POINTER(_Tape),
                                         _P, _P, _P, _P]),
    "ms_readout_debug": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, ctypes.POINTER(_Tape), _P, _P, _P]),
    "ms_token_backward_debug": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, ctypes.POINTER(_Tape),
                                               _P, _P, _P, _P, _P]),
    "ms_stats_forward_core": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t,
                                             _P, ctypes.POINTER(_Tape), _P]),
    "ms_token_backward_core": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, ctypes.POINTER(_Tape),
                                              _P, _P, _P, _P, _P, ctypes.c_size_t, ctypes.c_float, _P, _P, _P]),
    "ms_mix_backward": (ctypes.c_int, [ctypes.POINTER(_Shape), _P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_size_t,
                                       ctypes.POINTER(_Tape), _P, _P, _P, _P, _P, _P]),
    "ms_peer_sum_area_bytes": (ctypes.c_size_t, [ctypes.c_size_t]),
    "ms_peer_sum": (ctypes.c_int, [_P, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t,
                                   ctypes.c_int, ctypes.c_int, _P]),
    "ms_exchange_area_bytes": (ctypes.c_size_t, [ctypes.POINTER(_Shape)]),
    "ms_stats_exchange": (ctypes.c_int, [ctypes.POINTER(_Shape), ctypes.c_int, _P, ctypes.c_size_t, _P,
                                         ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_int,
                                         ctypes.c_int, _P, _P]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)


# --------------------------------------------------------------------------------------
# loading
# --------------------------------------------------------------------------------------
def default_library_path() -> Path:
    """In-tree build product (``python -m memsolve_b200.csrc.build``)."""
    return Path(__file__).resolve().parent.parent / "lib" / "memsolve_equilibrium_sm100.so"


def _open_library(path: str | os.PathLike) -> ctypes.CDLL:
    """dlopen + bind every symbol of the header; needs no GPU."""
    lib = ctypes.CDLL(os.fspath(path))
    for name, (restype, argtypes) in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as error:
            raise RuntimeError(
                f"{path} does not export {name}; it is not a MemSolve sm_100 library"
            ) from error
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def _check_native_contract(lib: ctypes.CDLL) -> None:
    version = lib.ms_abi_version()
    if version != _NATIVE_CONTRACT_VERSION:
        raise RuntimeError(
            "the loaded MemSolve CUDA extension has native contract version "
            f"{version}, but this package requires {_NATIVE_CONTRACT_VERSION}; "
            "rebuild it with `python -m memsolve_b200.csrc.build` and restart the process"
        )


def _library_architectures(lib: ctypes.CDLL) -> frozenset[int]:
    buf = (ctypes.c_int32 * 8)()
    count = lib.ms_supported_architectures(buf, 8)
    return frozenset(int(buf[i]) for i in range(min(count, 8)))


def _device_architecture(device: torch.device | int | None = None) -> int:
    """SM number of ``device`` normalised the way the reference does
    (memsolve/ball/cuda.py:183-211): 10.3 and 11.0 count as 100."""
    if not torch.cuda.is_available():
        raise RuntimeError("the MemSolve CUDA fast path requires an available CUDA device")
    if device is None:
        resolved = torch.device("cuda", torch.cuda.current_device())
    elif isinstance(device, int):
        resolved = torch.device("cuda", device)
    else:
        resolved = torch.device(device)
    if resolved.type != "cuda":
        raise ValueError(f"the MemSolve CUDA fast path requires a CUDA device, got {resolved}")
    if resolved.index is None:
        resolved = torch.device("cuda", torch.cuda.current_device())
    major, minor = torch.cuda.get_device_capability(resolved)
    architecture = major * 10 + minor
    if architecture in (103, 110):
        architecture = 100
    if architecture not in _SUPPORTED_ARCHITECTURES:
        raise RuntimeError(
            f"this build of the MemSolve CUDA fast path supports SM100 (B200) only; got SM{major}{minor}"
        )
    return architecture


def _resolve_library_path(path: str | os.PathLike | None) -> Path:
    if path is None:
        env = os.environ.get(_LIBRARY_ENV)
        path = env if env else default_library_path()
    resolved = Path(path)
    if not _LIBRARY_PATTERN.match(resolved.name):
        raise RuntimeError(
            "the MemSolve CUDA library must be named memsolve_equilibrium.so or "
            f"memsolve_equilibrium_sm<arch>.so, got {resolved.name!r}"
        )
    if not resolved.exists():
        raise RuntimeError(
            f"the MemSolve CUDA extension is not built: {resolved} does not exist; "
            "run `python -m memsolve_b200.csrc.build`"
        )
    return resolved


def load(path: str | os.PathLike | None = None, *, device: torch.device | int | None = None) -> None:
    """Open the native library and check it against ``device``.

    Same call shape as the reference loader (memsolve/ball/cuda.py:334-339).
    Idempotent and serialised by a lock; a later call for a device whose SM is
    not in the loaded library raises ``"targets SM..., not requested SM..."``.
    """
    global _LIB, _LIB_PATH, _LOADED_ARCHITECTURE
    requested = _device_architecture(device)
    with _LOAD_LOCK:
        if _LIB is not None:
            if requested not in _LOADED_ARCHITECTURE:
                built = ", ".join(f"SM{a}" for a in sorted(_LOADED_ARCHITECTURE))
                raise RuntimeError(
                    f"the loaded MemSolve CUDA extension targets {built}, not requested SM{requested}"
                )
            return
        resolved = _resolve_library_path(path)
        lib = _open_library(resolved)
        _check_native_contract(lib)
        architectures = _library_architectures(lib)
        if requested not in architectures:
            built = ", ".join(f"SM{a}" for a in sorted(architectures))
            raise RuntimeError(f"{resolved} targets {built}, not requested SM{requested}")
        _LIB, _LIB_PATH, _LOADED_ARCHITECTURE = lib, str(resolved), architectures


def is_available() -> bool:
    """Whether the native library has been loaded and verified."""
    return _LIB is not None


def require_available() -> None:
    """Reject a CUDA request until the extension is loaded (memsolve/ball/cuda.py:164-180)."""
    if _LIB is None:
        raise RuntimeError(
            "the MemSolve accretive-equilibrium CUDA extension is not loaded; build it with "
            "`python -m memsolve_b200.csrc.build`, then call memsolve_b200.ball.cuda.load(); "
            f"native contract version {_NATIVE_CONTRACT_VERSION} is required"
        )


def loaded_library_path() -> str | None:
    return _LIB_PATH


def _check(status: int, what: str) -> None:
    if status != 0:
        text = _LIB.ms_status_string(status).decode() if _LIB is not None else str(status)
        raise RuntimeError(f"MemSolve CUDA {what} failed: {text} (status {status})")


# --------------------------------------------------------------------------------------
# recompute-readout scope (memsolve/ball/cuda.py:26-59)
# --------------------------------------------------------------------------------------
class _RecomputeSpec(NamedTuple):
    projected: torch.Tensor
    tape: "_TapeTensors"
    counts: torch.Tensor | None
    rotary_cos: torch.Tensor | None
    rotary_sin: torch.Tensor | None
    shape: tuple
    short: bool = False   # single-rank forward over no more tokens than the rank (token-space eta term)


class _RecomputeScopeState:
    __slots__ = ("policy", "spec")

    def __init__(self, policy: Literal["auto"] | bool) -> None:
        self.policy = _validate_recompute_readout(policy)
        self.spec: _RecomputeSpec | None = None

    @property
    def enabled(self) -> bool:
        return self.policy is not False


@contextmanager
def _recompute_scope(policy: Literal["auto"] | bool = "auto"):
    previous = getattr(_RECOMPUTE_LOCAL, "active", None)
    state = _RecomputeScopeState(policy)
    _RECOMPUTE_LOCAL.active = state
    try:
        yield state
    finally:
        _RECOMPUTE_LOCAL.active = previous


# --------------------------------------------------------------------------------------
# native call helpers
# --------------------------------------------------------------------------------------
def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


class _TapeTensors(NamedTuple):
    eta: torch.Tensor
    eta_slope: torch.Tensor
    core_map: torch.Tensor
    core_info: torch.Tensor
    inverse: torch.Tensor
    state: torch.Tensor
    coeff: torch.Tensor

    def as_struct(self) -> _Tape:
        return _Tape(*(t.data_ptr() for t in self))


def _make_shape(projected, base, cos) -> tuple[_Shape, tuple]:
    batch, length, width = projected.shape
    heads, rank, columns = base.shape
    head_dim = (width - heads * rank) // heads
    rows = 0 if cos is None else int(cos.shape[0])
    dims = (batch, length, heads, rank, head_dim, int(columns == 0), rows)
    return _Shape(*dims, 0), dims


def _alloc_tape(dims, device) -> _TapeTensors:
    batch, _length, heads, rank, head_dim, _comp, _rows = dims
    f32 = dict(device=device, dtype=torch.float32)
    dpad = _LIB.ms_padded_head_dim(head_dim)
    return _TapeTensors(
        eta=torch.empty(heads, **f32),
        eta_slope=torch.empty(heads, **f32),
        core_map=torch.empty(heads, rank, rank, **f32),
        core_info=torch.empty(heads, device=device, dtype=torch.int32),
        inverse=torch.empty(batch, heads, rank, rank, **f32),
        state=torch.empty(batch, heads, rank, head_dim, **f32),
        coeff=torch.empty(batch, heads, 2, rank, dpad, device=device, dtype=torch.bfloat16),
    )


def _workspace(shape: _Shape, device) -> torch.Tensor:
    nbytes = _LIB.ms_workspace_bytes(ctypes.byref(shape))
    return torch.empty(max(int(nbytes), 16), device=device, dtype=torch.uint8)


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _sp_active(sequence_parallel) -> bool:
    return sequence_parallel is not None and getattr(sequence_parallel, "world_size", 2) > 1


def _sum_statistics(sequence_parallel, shape, backward: int, ws, counts, device, stream) -> torch.Tensor:
    """SUM over the ranks of the statistics whose per-chunk partials are in `ws`, by one kernel through
    the peer-memory exchange areas of the layout (`SequenceParallel.use_peer_exchange`)."""
    packed = torch.empty(_LIB.ms_packed_stats_floats(ctypes.byref(shape), backward), device=device,
                         dtype=torch.float32)
    exchange = sequence_parallel.peer_exchange
    areas, area_bytes = exchange.areas(int(_LIB.ms_exchange_area_bytes(ctypes.byref(shape))), device)
    _check(_LIB.ms_stats_exchange(ctypes.byref(shape), backward, ws.data_ptr(), ws.numel(), _ptr(counts), areas,
                                  area_bytes, sequence_parallel.world_size, sequence_parallel.rank,
                                  packed.data_ptr(), stream), "statistics exchange")
    return packed


def _mix_forward(projected, base, raw, counts, sequence_parallel, cos, sin):
    """Launch the forward kernels; returns (mixed, tape, dims)."""
    shape, dims = _make_shape(projected, base, cos)
    device = projected.device
    batch, length, heads, rank, head_dim = dims[:5]
    with torch.cuda.device(device):
        tape = _alloc_tape(dims, device)
        tape_c = tape.as_struct()
        ws = _workspace(shape, device)
        mixed = torch.empty(batch, length, heads * head_dim, device=device, dtype=torch.bfloat16)
        stream = _stream(device)
        base_ptr = None if dims[5] else base.data_ptr()
        if not _sp_active(sequence_parallel):
            _check(_LIB.ms_mix_forward(
                ctypes.byref(shape), projected.data_ptr(), base_ptr, raw.data_ptr(), _ptr(cos), _ptr(sin),
                _ptr(counts), ws.data_ptr(), ws.numel(), ctypes.byref(tape_c), mixed.data_ptr(), stream),
                "forward")
        else:
            peer = getattr(sequence_parallel, "peer_exchange", None) is not None
            packed = None if peer else torch.empty(_LIB.ms_packed_stats_floats(ctypes.byref(shape), 0),
                                                   device=device, dtype=torch.float32)
            _check(_LIB.ms_stats_forward_core(ctypes.byref(shape), projected.data_ptr(), base_ptr, raw.data_ptr(),
                                              _ptr(cos), _ptr(sin), _ptr(counts), ws.data_ptr(), ws.numel(),
                                              _ptr(packed), ctypes.byref(tape_c), stream),
                   "statistics")
            # the only cross-GPU step of the forward: SUM of the packed (G, Q) statistics
            if peer:
                packed = _sum_statistics(sequence_parallel, shape, 0, ws, counts, device, stream)
            else:
                (packed,) = sequence_parallel.sum_tensors(packed)
            _check(_LIB.ms_compact_forward(ctypes.byref(shape), _ptr(counts), None, 0, packed.data_ptr(),
                                           ctypes.byref(tape_c), stream), "compact forward")
            _check(_LIB.ms_readout(ctypes.byref(shape), projected.data_ptr(), _ptr(cos), _ptr(sin),
                                   _ptr(counts), ctypes.byref(tape_c), mixed.data_ptr(), stream), "readout")
    return mixed, tape, dims


def _readout(projected, tape: _TapeTensors, dims, counts, cos, sin, short: bool = False) -> torch.Tensor:
    """Rebuild ``mixed`` from the compact tape.  ``short``: the tape comes from a single-rank forward over no more
    tokens than the rank, whose coefficient tensor holds the core part only (``ms_readout_short``)."""
    batch, length, heads, rank, head_dim, comp, rows = dims
    shape = _Shape(*dims, 0)
    device = projected.device
    with torch.cuda.device(device):
        mixed = torch.empty(batch, length, heads * head_dim, device=device, dtype=torch.bfloat16)
        tape_c = tape.as_struct()
        entry = _LIB.ms_readout_short if short else _LIB.ms_readout
        _check(entry(ctypes.byref(shape), projected.data_ptr(), _ptr(cos), _ptr(sin), _ptr(counts),
                               ctypes.byref(tape_c), mixed.data_ptr(), _stream(device)), "readout")
    return mixed


def _mix_backward(projected, gradient, base, raw, counts, sequence_parallel, cos, sin, tape, dims):
    batch, length, heads, rank, head_dim, comp, rows = dims
    shape = _Shape(*dims, 0)
    device = projected.device
    with torch.cuda.device(device):
        tape_c = tape.as_struct()
        ws = _workspace(shape, device)
        dpad = _LIB.ms_padded_head_dim(head_dim)
        gram_grad = torch.empty(batch, heads, 2, rank, rank, device=device, dtype=torch.bfloat16)
        cross_grad = torch.empty(batch, heads, 2, rank, dpad, device=device, dtype=torch.bfloat16)
        d_projected = torch.empty_like(projected)
        d_base = None if comp else torch.empty(heads, rank, rank, device=device, dtype=torch.float32)
        d_raw = torch.empty(heads, device=device, dtype=torch.float32)
        stream = _stream(device)
        base_ptr = None if comp else base.data_ptr()
        if not _sp_active(sequence_parallel):
            _check(_LIB.ms_mix_backward(
                ctypes.byref(shape), projected.data_ptr(), gradient.data_ptr(), base_ptr, raw.data_ptr(),
                _ptr(cos), _ptr(sin), _ptr(counts), ws.data_ptr(), ws.numel(), ctypes.byref(tape_c),
                gram_grad.data_ptr(), cross_grad.data_ptr(), d_projected.data_ptr(), _ptr(d_base),
                d_raw.data_ptr(), stream), "backward")
        else:
            peer = getattr(sequence_parallel, "peer_exchange", None) is not None
            packed = None if peer else torch.empty(_LIB.ms_packed_stats_floats(ctypes.byref(shape), 1),
                                                   device=device, dtype=torch.float32)
            _check(_LIB.ms_stats_backward(ctypes.byref(shape), projected.data_ptr(), gradient.data_ptr(),
                                          _ptr(cos), _ptr(sin), _ptr(counts), ws.data_ptr(), ws.numel(),
                                          _ptr(packed), stream), "adjoint statistics")
            if peer:
                packed = _sum_statistics(sequence_parallel, shape, 1, ws, counts, device, stream)
            else:
                (packed,) = sequence_parallel.sum_tensors(packed)
            # replicated parameters: every rank holds the full adjoint, a later SUM must count it once
            scale = 1.0 / float(sequence_parallel.world_size)
            _check(_LIB.ms_compact_backward(
                ctypes.byref(shape), _ptr(counts), ws.data_ptr(), ws.numel(), packed.data_ptr(),
                ctypes.byref(tape_c), base_ptr, raw.data_ptr(), scale, gram_grad.data_ptr(),
                cross_grad.data_ptr(), None, None, stream), "compact backward")
            # the per-head parameter gradients ride along with the token pass
            _check(_LIB.ms_token_backward_core(
                ctypes.byref(shape), projected.data_ptr(), gradient.data_ptr(), _ptr(cos), _ptr(sin),
                _ptr(counts), ctypes.byref(tape_c), gram_grad.data_ptr(), cross_grad.data_ptr(),
                d_projected.data_ptr(), base_ptr, ws.data_ptr(), ws.numel(), scale, _ptr(d_base),
                d_raw.data_ptr(), stream), "token backward")
    return d_projected, d_base, d_raw


# --------------------------------------------------------------------------------------
# autograd boundary (memsolve/ball/cuda.py:3146-3227)
# --------------------------------------------------------------------------------------
class _NoFrameMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, projected, base, raw, counts, sequence_parallel, rotary_cos, rotary_sin):
        mixed, tape, dims = _mix_forward(projected, base, raw, counts, sequence_parallel, rotary_cos, rotary_sin)
        ctx.sequence_parallel = sequence_parallel
        ctx.dims = dims
        ctx.has_counts = counts is not None
        ctx.has_rotary = rotary_cos is not None
        saved = [projected, base, raw, *tape]
        if counts is not None:
            saved.append(counts)
        if rotary_cos is not None:
            saved += [rotary_cos, rotary_sin]
        ctx.save_for_backward(*saved)
        scope = getattr(_RECOMPUTE_LOCAL, "active", None)
        if scope is not None and (scope.policy is True or (scope.policy == "auto" and projected.shape[1] > 512)):
            scope.spec = _RecomputeSpec(
                projected.detach(), _TapeTensors(*(t.detach() for t in tape)), counts, rotary_cos, rotary_sin, dims,
                not _sp_active(sequence_parallel) and dims[1] <= dims[3])
        return mixed

    @staticmethod
    @once_differentiable
    def backward(ctx, gradient):
        saved = list(ctx.saved_tensors)
        projected, base, raw = saved[:3]
        tape = _TapeTensors(*saved[3:10])
        rest = saved[10:]
        counts = rest.pop(0) if ctx.has_counts else None
        cos, sin = (rest[0], rest[1]) if ctx.has_rotary else (None, None)
        gradient = gradient.contiguous()
        if gradient.dtype != torch.bfloat16:
            gradient = gradient.to(torch.bfloat16)
        d_projected, d_base, d_raw = _mix_backward(
            projected, gradient, base, raw, counts, ctx.sequence_parallel, cos, sin, tape, ctx.dims)
        if d_base is None:
            d_base = torch.zeros_like(base)
        return d_projected, d_base, d_raw, None, None, None, None


# --------------------------------------------------------------------------------------
# operator registration (memsolve/ball/cuda.py:4164-5003 of the reference): the mixer as
# torch.library operators with fake (shape-only) kernels and an autograd formula, so that
# torch.compile(fullgraph=True) and other tracers see one opaque call per direction
# --------------------------------------------------------------------------------------
def _dims_of(projected, base, cos) -> tuple:
    batch, length, width = projected.shape
    heads, rank, columns = base.shape
    head_dim = (width - heads * rank) // heads
    return (batch, length, heads, rank, head_dim, int(columns == 0), 0 if cos is None else int(cos.shape[0]))


@torch.library.custom_op("memsolve_b200::fast_mix_fwd", mutates_args=(), device_types="cuda")
def _fast_mix_fwd_op(projected: torch.Tensor, core_base_raw: torch.Tensor, eta_raw: torch.Tensor,
                     valid_counts: Optional[torch.Tensor], rotary_cos: Optional[torch.Tensor],
                     rotary_sin: Optional[torch.Tensor]) -> List[torch.Tensor]:
    """mixed plus the compact tape (eta, eta_slope, core_map, core_info, inverse, state, coeff)."""
    require_available()
    _validate_no_frame_inputs(projected, core_base_raw, eta_raw, valid_counts)
    mixed, tape, _ = _mix_forward(projected, core_base_raw, eta_raw, valid_counts, None, rotary_cos, rotary_sin)
    return [mixed, *tape]


@_fast_mix_fwd_op.register_fake
def _fast_mix_fwd_fake(projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin):
    batch, length, heads, rank, head_dim, _comp, _rows = _dims_of(projected, core_base_raw, rotary_cos)
    dpad = (head_dim + 7) // 8 * 8
    f32 = eta_raw.new_empty
    return [projected.new_empty((batch, length, heads * head_dim)), f32((heads,)), f32((heads,)),
            f32((heads, rank, rank)), eta_raw.new_empty((heads,), dtype=torch.int32),
            f32((batch, heads, rank, rank)), f32((batch, heads, rank, head_dim)),
            projected.new_empty((batch, heads, 2, rank, dpad))]


@torch.library.custom_op("memsolve_b200::fast_mix_infer", mutates_args=(), device_types="cuda")
def _fast_mix_infer_op(projected: torch.Tensor, core_base_raw: torch.Tensor, eta_raw: torch.Tensor,
                       valid_counts: Optional[torch.Tensor], rotary_cos: Optional[torch.Tensor],
                       rotary_sin: Optional[torch.Tensor]) -> torch.Tensor:
    """mixed alone, for graphs traced without gradients (memsolve/ball/cuda.py:4164-4201): the tape is dropped."""
    require_available()
    _validate_no_frame_inputs(projected, core_base_raw, eta_raw, valid_counts)
    return _mix_forward(projected, core_base_raw, eta_raw, valid_counts, None, rotary_cos, rotary_sin)[0]


@_fast_mix_infer_op.register_fake
def _fast_mix_infer_fake(projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin):
    batch, length, heads, _rank, head_dim, _comp, _rows = _dims_of(projected, core_base_raw, rotary_cos)
    return projected.new_empty((batch, length, heads * head_dim))


@torch.library.custom_op("memsolve_b200::fast_mix_bwd", mutates_args=(), device_types="cuda")
def _fast_mix_bwd_op(projected: torch.Tensor, gradient: torch.Tensor, core_base_raw: torch.Tensor,
                     eta_raw: torch.Tensor, valid_counts: Optional[torch.Tensor],
                     rotary_cos: Optional[torch.Tensor], rotary_sin: Optional[torch.Tensor],
                     tape: List[torch.Tensor]) -> List[torch.Tensor]:
    """Gradients of projected, core_base_raw and eta_raw."""
    dims = _dims_of(projected, core_base_raw, rotary_cos)
    gradient = gradient.contiguous()
    if gradient.dtype != torch.bfloat16:
        gradient = gradient.to(torch.bfloat16)
    d_projected, d_base, d_raw = _mix_backward(projected, gradient, core_base_raw, eta_raw, valid_counts, None,
                                               rotary_cos, rotary_sin, _TapeTensors(*tape), dims)
    if d_base is None:
        d_base = torch.zeros_like(core_base_raw)
    return [d_projected, d_base, d_raw]


@_fast_mix_bwd_op.register_fake
def _fast_mix_bwd_fake(projected, gradient, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin, tape):
    return [torch.empty_like(projected), torch.empty_like(core_base_raw), torch.empty_like(eta_raw)]


def _fast_mix_setup_context(ctx, inputs, output):
    projected, base, raw, counts, cos, sin = inputs
    ctx.has_counts, ctx.has_rotary = counts is not None, cos is not None
    extra = ([counts] if counts is not None else []) + ([cos, sin] if cos is not None else [])
    ctx.save_for_backward(projected, base, raw, *output[1:], *extra)


def _fast_mix_autograd(ctx, grads):
    saved = list(ctx.saved_tensors)
    projected, base, raw = saved[:3]
    tape, rest = saved[3:10], saved[10:]
    counts = rest.pop(0) if ctx.has_counts else None
    cos, sin = (rest[0], rest[1]) if ctx.has_rotary else (None, None)
    d_projected, d_base, d_raw = torch.ops.memsolve_b200.fast_mix_bwd(
        projected, grads[0], base, raw, counts, cos, sin, tape)
    return d_projected, d_base, d_raw, None, None, None


torch.library.register_autograd("memsolve_b200::fast_mix_fwd", _fast_mix_autograd,
                                setup_context=_fast_mix_setup_context)


# --------------------------------------------------------------------------------------
# public mixer entry (memsolve/ball/cuda.py:5175-5278)
# --------------------------------------------------------------------------------------
def _validate_no_frame_inputs(projected, base, raw, counts) -> None:
    def require(condition, message):
        if not condition:
            raise RuntimeError(message)

    require(projected.is_cuda, "projected must be a CUDA tensor")
    require(projected.ndim == 3 and projected.is_contiguous(), "projected must be contiguous [B, N, H*R + D]")
    require(projected.dtype == torch.bfloat16,
            "projected must use bfloat16 under the mixed precision CUDA contract")
    for name, value in (("core_base_raw", base), ("eta_raw", raw)):
        require(value.device == projected.device and value.is_contiguous(),
                f"{name} must be contiguous on the same CUDA device")
        require(value.dtype == torch.float32, f"{name} must use float32")
    require(base.ndim == 3, "core_base_raw must have shape [H,R,R] or [H,R,0]")
    batch, length, width = projected.shape
    heads, rank, columns = base.shape
    require(batch > 0 and length > 0 and heads > 0, "B, N, and H must be positive")
    require(rank in (16, 32, 48, 64), "the CUDA fast path supports rank in {16,32,48,64}")
    require(columns in (0, rank), "core_base_raw must have shape [H,R,R] or [H,R,0]")
    content = width - heads * rank
    require(content > 0 and content % heads == 0, "projected content width must be positive and divisible by H")
    require(raw.ndim == 1 and raw.shape[0] == heads, "eta_raw must have shape [H]")
    if counts is not None:
        require(counts.device == projected.device and counts.dtype == torch.float32 and counts.is_contiguous(),
                "valid_counts must be contiguous float32 on the same CUDA device")
        require(counts.ndim == 1 and counts.shape[0] == batch, "valid_counts must have shape [B]")


def fast_mix(
    projected: torch.Tensor,
    core_base_raw: torch.Tensor,
    eta_raw: torch.Tensor,
    valid_counts: torch.Tensor | None = None,
    *, sequence_parallel=None, rotary_cos=None, rotary_sin=None,
) -> torch.Tensor:
    """Mix pre-projected BF16 tokens ``[B, N, H*r + D]`` -> ``[B, N, D]`` (BF16).

    Same arguments, checks and messages as the reference entry point
    (memsolve/ball/cuda.py:5222-5278).  ``core_base_raw`` with a zero last
    dimension selects complement mode.  All sequence lengths, including
    ``N <= r``, take the rank-space kernels.
    """
    if valid_counts is not None and valid_counts.requires_grad:
        raise ValueError("the MemSolve CUDA fast path does not support gradients for valid_counts")
    if torch.compiler.is_compiling() and sequence_parallel is None:
        # traced: one registered operator (its kernel repeats the checks below when it runs)
        if not (torch.is_grad_enabled() and any(t.requires_grad for t in (projected, core_base_raw, eta_raw))):
            return torch.ops.memsolve_b200.fast_mix_infer(projected, core_base_raw, eta_raw, valid_counts,
                                                          rotary_cos, rotary_sin)
        return torch.ops.memsolve_b200.fast_mix_fwd(projected, core_base_raw, eta_raw, valid_counts,
                                                    rotary_cos, rotary_sin)[0]
    require_available()
    _validate_no_frame_inputs(projected, core_base_raw, eta_raw, valid_counts)
    if (rotary_cos is None) != (rotary_sin is None):
        raise ValueError("rotary_cos and rotary_sin must be supplied together")
    if rotary_cos is not None:
        batch, length, width = projected.shape
        heads, rank = core_base_raw.shape[:2]
        head_dim = (width - heads * rank) // heads
        if head_dim % 2:
            raise ValueError("rotary content requires an even head dimension")
        for name, table in (("rotary_cos", rotary_cos), ("rotary_sin", rotary_sin)):
            if (table.device != projected.device or table.dtype != torch.float32
                    or not table.is_contiguous() or table.requires_grad):
                raise ValueError(f"{name} must be non-differentiable contiguous FP32 on the input device")
            if (table.ndim != 3 or table.shape[1] != length or table.shape[2] != head_dim // 2
                    or table.shape[0] not in (1, batch)):
                raise ValueError(f"{name} must have shape [1 or B,N,Dhead/2]")
        if rotary_cos.shape != rotary_sin.shape:
            raise ValueError("rotary_cos and rotary_sin must share their shape")
    record = torch.is_grad_enabled() and any(
        value.requires_grad for value in (projected, core_base_raw, eta_raw))
    if sequence_parallel is not None:
        sequence_parallel.validate(projected.shape[1], core_base_raw.shape[1])
        if valid_counts is None:
            raise ValueError("sequence parallelism requires global valid_counts")
    if record:
        return _NoFrameMix.apply(projected, core_base_raw, eta_raw, valid_counts, sequence_parallel,
                                 rotary_cos, rotary_sin)
    with torch.no_grad():
        return _mix_forward(projected, core_base_raw, eta_raw, valid_counts, sequence_parallel,
                            rotary_cos, rotary_sin)[0]


_ORIGINAL_FAST_MIX = fast_mix


def _is_default_fast_mix() -> bool:
    return fast_mix is _ORIGINAL_FAST_MIX


# --------------------------------------------------------------------------------------
# projections around the mixer (memsolve/ball/cuda.py:933-1041, 1307-1342)
# --------------------------------------------------------------------------------------
_MM_OUT_DTYPE = True


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """BF16 x BF16 GEMM whose FP32 accumulator is returned without a BF16 rounding."""
    global _MM_OUT_DTYPE
    if _MM_OUT_DTYPE:
        try:
            return torch.mm(a, b, out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    return torch.mm(a.float(), b.float())


def _masked_rows(value: torch.Tensor, mask: torch.Tensor | None) -> torch.Tensor:
    if mask is None:
        return value
    return torch.where(mask.reshape(-1, 1), value, torch.zeros((), dtype=value.dtype, device=value.device))


# Projections with a BF16 result: the library's tcgen05 GEMM (ms_linear_forward) has the row masks, the FP32 bias and
# the single BF16 rounding fused into its epilogue.  It runs within 3-15 % of cuBLAS on the bare product
# ([32768 x 768] x [768 x 768]: 37.1 against 36.0 us; x [768 x 1152]: 57.6 against 49.4 us on one B200), so by default it
# is taken when there is an epilogue to fuse (bias or masks: each would otherwise be another pass over the output) and
# cuBLAS when there is none.  MEMSOLVE_TCGEN05_LINEAR=1 takes it always, =0 never.
_OWN_LINEAR = os.environ.get("MEMSOLVE_TCGEN05_LINEAR", "auto")


def _fused_linear_forward(flat, weight_bf16, bias, output_mask, input_mask):
    """out = mask_out * (mask_in * flat @ weight^T + bias) as one tcgen05 kernel, or None when the shape is not one
    the kernel takes."""
    rows, in_features = flat.shape
    out_features = weight_bf16.shape[0]
    if (_LIB is None or not flat.is_cuda or flat.dtype != torch.bfloat16 or not flat.is_contiguous()
            or not weight_bf16.is_contiguous() or in_features % 64 or out_features % 128 or rows == 0):
        return None
    bias32 = None if bias is None else bias.detach().to(torch.float32).contiguous()
    masks = []
    for mask in (input_mask, output_mask):
        masks.append(None if mask is None else mask.reshape(-1).to(torch.bool).contiguous())
    out = torch.empty(rows, out_features, device=flat.device, dtype=torch.bfloat16)
    with torch.cuda.device(flat.device):
        status = _LIB.ms_linear_forward(rows, in_features, out_features, flat.data_ptr(), weight_bf16.data_ptr(),
                                        _ptr(bias32), _ptr(masks[0]), _ptr(masks[1]), out.data_ptr(),
                                        _stream(flat.device))
    if status == 9:      # MS_ERR_LINEAR_SHAPE
        return None
    _check(status, "linear forward")
    return out


def _fused_linear_input_grad(flat_g, weight_bf16, output_mask, input_mask):
    """dx = masks * (flat_g @ weight) as one tcgen05 kernel (the weight is read in place as an N-major operand), or
    None when the shape is not one the kernel takes."""
    rows, out_features = flat_g.shape
    in_features = weight_bf16.shape[1]
    if (_LIB is None or not flat_g.is_cuda or flat_g.dtype != torch.bfloat16 or not flat_g.is_contiguous()
            or not weight_bf16.is_contiguous() or out_features % 64 or in_features % 128 or rows == 0):
        return None
    masks = []
    for mask in (input_mask, output_mask):
        masks.append(None if mask is None else mask.reshape(-1).to(torch.bool).contiguous())
    dx = torch.empty(rows, in_features, device=flat_g.device, dtype=torch.bfloat16)
    with torch.cuda.device(flat_g.device):
        status = _LIB.ms_linear_input_grad(rows, in_features, out_features, flat_g.data_ptr(), weight_bf16.data_ptr(),
                                           _ptr(masks[0]), _ptr(masks[1]), dx.data_ptr(), _stream(flat_g.device))
    if status == 9:      # MS_ERR_LINEAR_SHAPE
        return None
    _check(status, "linear input gradient")
    return dx


def _fused_linear_weight_grad(flat_g, flat_v, need_db):
    """(dW, db) = (flat_g^T @ flat_v, column sums of flat_g) in FP32 by one tcgen05 kernel with a fixed summation
    order, or None when the shape is not one the kernel takes.  No row masks."""
    rows, out_features = flat_g.shape
    in_features = flat_v.shape[1]
    if (_LIB is None or not flat_g.is_cuda or flat_g.dtype != torch.bfloat16 or flat_v.dtype != torch.bfloat16
            or not flat_g.is_contiguous() or not flat_v.is_contiguous() or out_features % 128 or in_features % 128
            or rows == 0):
        return None
    nbytes = int(_LIB.ms_linear_weight_grad_workspace(rows, in_features, out_features))
    if nbytes == 0:
        return None
    device = flat_g.device
    ws = torch.empty(nbytes, device=device, dtype=torch.uint8)
    dw = torch.empty(out_features, in_features, device=device, dtype=torch.float32)
    db = torch.empty(out_features, device=device, dtype=torch.float32) if need_db else None
    with torch.cuda.device(device):
        status = _LIB.ms_linear_weight_grad(rows, in_features, out_features, flat_v.data_ptr(), flat_g.data_ptr(),
                                            dw.data_ptr(), _ptr(db), ws.data_ptr(), nbytes, _stream(device))
    if status == 9:
        return None
    _check(status, "linear weight gradient")
    return dw, db


def _linear_forward(value, weight_bf16, bias, output_dtype, output_mask, input_mask):
    """BF16 x BF16 with FP32 accumulation, FP32 bias, row masks, one rounding."""
    wanted = _OWN_LINEAR == "1" or (_OWN_LINEAR != "0" and (bias is not None or output_mask is not None
                                                          or input_mask is not None))
    if wanted and output_dtype == torch.bfloat16 and value.dtype == torch.bfloat16:
        fused = _fused_linear_forward(value.reshape(-1, value.shape[-1]), weight_bf16, bias, output_mask, input_mask)
        if fused is not None:
            return fused.reshape(value.shape[:-1] + (weight_bf16.shape[0],))
    flat = value.reshape(-1, value.shape[-1])
    flat = _masked_rows(flat, None if input_mask is None else input_mask.reshape(-1))
    flat = flat.to(torch.bfloat16)
    target = output_dtype if output_dtype is not None else torch.float32
    if bias is None and output_mask is None and target == torch.bfloat16:
        out = flat @ weight_bf16.mT
    else:
        out = _mm_f32(flat, weight_bf16.mT)
        if bias is not None:
            out = out + bias.to(torch.float32)
        out = _masked_rows(out, None if output_mask is None else output_mask.reshape(-1))
        out = out.to(target)
    return out.reshape(value.shape[:-1] + (weight_bf16.shape[0],))


def _linear_backward(grad_output, value, weight_bf16, output_mask, input_mask, needs, value_dtype,
                     weight_dtype, bias, out_features=None):
    """Gradients of the projection.  The library's tcgen05 kernels are taken where they fuse passes that would
    otherwise run separately (measured at 32768 rows on one B200, L2 flushed): the input gradient when row masks are
    present (57 against 50 us of cuBLAS for the bare product, but the masks are then free), and dW + db in one pass
    when a bias gradient is wanted and there are no masks (80 / 104 us against 91 / 110 us of cuBLAS plus the column
    sums; without a bias cuBLAS' bare dW is faster at 48 / 69 us).  MEMSOLVE_TCGEN05_LINEAR=1 takes them whenever the
    shape allows, =0 never."""
    need_dx, need_dw, need_db = needs
    if out_features is None:
        out_features = weight_bf16.shape[0]
    flat_g = grad_output.reshape(-1, out_features)
    grad_value = grad_weight = grad_bias = None
    masked = output_mask is not None or input_mask is not None
    own = _OWN_LINEAR != "0" and flat_g.dtype == torch.bfloat16
    if need_dx and own and value_dtype == torch.bfloat16 and (masked or _OWN_LINEAR == "1"):
        dx = _fused_linear_input_grad(flat_g.contiguous(), weight_bf16, output_mask, input_mask)
        if dx is not None:
            grad_value = dx.reshape(grad_output.shape[:-1] + (weight_bf16.shape[1],))
            need_dx = False
    if (need_dw or need_db) and own and not masked and (need_db or _OWN_LINEAR == "1") and value is not None \
            and value.dtype == torch.bfloat16:
        fused = _fused_linear_weight_grad(flat_g.contiguous(), value.reshape(-1, value.shape[-1]).contiguous(), need_db)
        if fused is not None:
            if need_dw:
                grad_weight = fused[0].to(weight_dtype)
            if need_db:
                grad_bias = fused[1].to(device=bias.device, dtype=bias.dtype)
            need_dw = need_db = False
    if not (need_dx or need_dw or need_db):
        return grad_value, grad_weight, grad_bias
    flat_g = _masked_rows(flat_g, None if output_mask is None else output_mask.reshape(-1))
    g_bf16 = flat_g if flat_g.dtype == torch.bfloat16 else flat_g.to(torch.bfloat16)
    if need_dw:
        flat_v = value.reshape(-1, value.shape[-1])
        flat_v = _masked_rows(flat_v, None if input_mask is None else input_mask.reshape(-1)).to(torch.bfloat16)
        grad_weight = _mm_f32(g_bf16.mT, flat_v).to(weight_dtype)
    if need_db:
        grad_bias = flat_g.sum(dim=0, dtype=torch.float32).to(device=bias.device, dtype=bias.dtype)
    if need_dx:
        if value_dtype == torch.bfloat16:
            dx = g_bf16 @ weight_bf16
        else:
            dx = _mm_f32(g_bf16, weight_bf16)
        dx = _masked_rows(dx, None if input_mask is None else input_mask.reshape(-1))
        grad_value = dx.reshape(grad_output.shape[:-1] + (weight_bf16.shape[1],)).to(value_dtype)
    return grad_value, grad_weight, grad_bias


class _TensorCoreLinear(torch.autograd.Function):
    """Projection with BF16 multiplicands, FP32 accumulation and dtype-aware stores.

    This node owns the data path only (forward GEMM, input gradient); the gradients of weight
    and bias come from `_ParameterGradients`, a node of its own that autograd runs first, so a
    hook on the weight (a sequence-parallel gradient SUM, say) starts while the input-gradient
    GEMM still runs.
    """

    @staticmethod
    def forward(ctx, value, weight, bias, output_dtype, output_mask, input_mask):
        weight_bf16 = weight.to(torch.bfloat16)
        ctx.save_for_backward(weight_bf16, output_mask, input_mask)
        ctx.value_dtype = value.dtype
        return _linear_forward(value, weight_bf16, bias, output_dtype, output_mask, input_mask)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        weight_bf16, output_mask, input_mask = ctx.saved_tensors
        gv = None
        if ctx.needs_input_grad[0]:
            gv = _linear_backward(grad_output, None, weight_bf16, output_mask, input_mask, (True, False, False),
                                  ctx.value_dtype, None, None)[0]
        return gv, None, None, None, None, None


class _ParameterGradients(torch.autograd.Function):
    """Identity on a projection's output; its backward forms dW = dY^T X and db = sum dY."""

    @staticmethod
    def forward(ctx, out, value, weight, bias, output_mask, input_mask):
        ctx.save_for_backward(value, output_mask, input_mask, bias)
        ctx.weight_dtype = weight.dtype
        ctx.out_features = weight.shape[0]
        return out.view_as(out)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, output_mask, input_mask, bias = ctx.saved_tensors
        needs = (False, ctx.needs_input_grad[2], bias is not None and ctx.needs_input_grad[3])
        _, gw, gb = _linear_backward(grad_output, value, None, output_mask, input_mask, needs, None,
                                     ctx.weight_dtype, bias, out_features=ctx.out_features)
        return grad_output, None, gw, gb, None, None


def tensor_core_linear(value, weight, bias=None, *, output_dtype=None, fuse_weight_bias_grad=False,
                       output_mask=None, input_mask=None):
    """CUDA branch of the reference's ``tensor_core_linear`` (memsolve/ball/reference.py:191-269)."""
    if value.shape[-1] != weight.shape[-1]:
        raise ValueError(
            f"tensor_core_linear input and weight features must agree, got {value.shape[-1]} and {weight.shape[-1]}")
    if torch.compiler.is_compiling():
        # traced: one registered operator per direction (the kernels are reached through ctypes, which a tracer
        # cannot follow)
        flat = torch.ops.memsolve_b200.tensor_core_linear(
            value.reshape(-1, value.shape[-1]), weight, bias, None if output_mask is None else output_mask.reshape(-1),
            None if input_mask is None else input_mask.reshape(-1), _DTYPE_CODES[output_dtype])
        return flat.reshape(value.shape[:-1] + (weight.shape[0],))
    out = _TensorCoreLinear.apply(value, weight.detach(), None if bias is None else bias.detach(), output_dtype,
                                  output_mask, input_mask)
    if torch.is_grad_enabled() and (weight.requires_grad or (bias is not None and bias.requires_grad)):
        out = _ParameterGradients.apply(out, value.detach(), weight, bias, output_mask, input_mask)
    return out


# --------------------------------------------------------------------------------------
# registered operators of the projections and of the output projection with readout recompute
# (memsolve/ball/cuda.py:1104-1304 `memsolve::tensor_core_linear[_backward]`, :4422-4882
# `memsolve::fast_mix_output_linear_fwd/_bwd`): what a traced layer calls, one opaque node per direction
# --------------------------------------------------------------------------------------
_DTYPE_CODES = {None: 0, torch.float32: 1, torch.bfloat16: 2, torch.float16: 3}
_CODE_DTYPES = {code: dtype for dtype, code in _DTYPE_CODES.items()}


@torch.library.custom_op("memsolve_b200::tensor_core_linear", mutates_args=(), device_types="cuda")
def _tensor_core_linear_op(flat_value: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                           output_mask: Optional[torch.Tensor], input_mask: Optional[torch.Tensor],
                           out_dtype_code: int) -> torch.Tensor:
    """out = output_mask * (input_mask * flat_value @ weight^T + bias): BF16 multiplicands, FP32 sums, one rounding."""
    weight_bf16 = weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)
    return _linear_forward(flat_value, weight_bf16, bias, _CODE_DTYPES[out_dtype_code], output_mask,
                           input_mask).contiguous()


@_tensor_core_linear_op.register_fake
def _tensor_core_linear_fake(flat_value, weight, bias, output_mask, input_mask, out_dtype_code):
    dtype = _CODE_DTYPES[out_dtype_code] or torch.float32
    return flat_value.new_empty((flat_value.shape[0], weight.shape[0]), dtype=dtype)


@torch.library.custom_op("memsolve_b200::tensor_core_linear_backward", mutates_args=(), device_types="cuda")
def _tensor_core_linear_bwd_op(grad_output: torch.Tensor, flat_value: torch.Tensor, weight: torch.Tensor,
                               bias: Optional[torch.Tensor], output_mask: Optional[torch.Tensor],
                               input_mask: Optional[torch.Tensor], need_dx: bool, need_dw: bool,
                               need_db: bool) -> List[torch.Tensor]:
    """[d flat_value, d weight, d bias]; a gradient that is not needed comes back as an empty tensor."""
    weight_bf16 = weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)
    gv, gw, gb = _linear_backward(grad_output.contiguous(), flat_value, weight_bf16, output_mask, input_mask,
                                  (need_dx, need_dw, need_db and bias is not None), flat_value.dtype, weight.dtype,
                                  bias)
    empty = lambda: grad_output.new_empty((0,))   # noqa: E731  (outputs of an operator may not alias each other)
    return [empty() if gv is None else gv.contiguous(), empty() if gw is None else gw.contiguous(),
            empty() if gb is None else gb.contiguous()]


@_tensor_core_linear_bwd_op.register_fake
def _tensor_core_linear_bwd_fake(grad_output, flat_value, weight, bias, output_mask, input_mask, need_dx, need_dw,
                                 need_db):
    empty = lambda: grad_output.new_empty((0,))   # noqa: E731
    return [torch.empty_like(flat_value) if need_dx else empty(),
            torch.empty_like(weight) if need_dw else empty(),
            torch.empty_like(bias) if need_db and bias is not None else empty()]


def _tensor_core_linear_setup(ctx, inputs, output):
    flat_value, weight, bias, output_mask, input_mask, _code = inputs
    ctx.save_for_backward(flat_value, weight, bias, output_mask, input_mask)


def _tensor_core_linear_autograd(ctx, grad_output):
    flat_value, weight, bias, output_mask, input_mask = ctx.saved_tensors
    needs = ctx.needs_input_grad
    gv, gw, gb = torch.ops.memsolve_b200.tensor_core_linear_backward(
        grad_output, flat_value, weight, bias, output_mask, input_mask, needs[0], needs[1],
        bias is not None and needs[2])
    return (gv if needs[0] else None, gw if needs[1] else None, gb if bias is not None and needs[2] else None,
            None, None, None)


torch.library.register_autograd("memsolve_b200::tensor_core_linear", _tensor_core_linear_autograd,
                                setup_context=_tensor_core_linear_setup)


@torch.library.custom_op("memsolve_b200::fast_mix_output_linear_fwd", mutates_args=(), device_types="cuda")
def _fast_mix_out_linear_fwd_op(projected: torch.Tensor, core_base_raw: torch.Tensor, eta_raw: torch.Tensor,
                                valid_counts: Optional[torch.Tensor], rotary_cos: Optional[torch.Tensor],
                                rotary_sin: Optional[torch.Tensor], weight: torch.Tensor,
                                bias: Optional[torch.Tensor], output_mask: Optional[torch.Tensor],
                                out_dtype_code: int) -> List[torch.Tensor]:
    """Mixer and output projection as one node that keeps the compact tape instead of `mixed`: returns the
    projected output and the tape (eta, eta_slope, core_map, core_info, inverse, state, coeff)."""
    require_available()
    _validate_no_frame_inputs(projected, core_base_raw, eta_raw, valid_counts)
    mixed, tape, _ = _mix_forward(projected, core_base_raw, eta_raw, valid_counts, None, rotary_cos, rotary_sin)
    weight_bf16 = weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)
    out = _linear_forward(mixed, weight_bf16, bias, _CODE_DTYPES[out_dtype_code], output_mask, None)
    return [out.contiguous(), *tape]


@_fast_mix_out_linear_fwd_op.register_fake
def _fast_mix_out_linear_fwd_fake(projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin, weight,
                                  bias, output_mask, out_dtype_code):
    fake = _fast_mix_fwd_fake(projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin)
    dtype = _CODE_DTYPES[out_dtype_code] or torch.float32
    out = projected.new_empty((projected.shape[0], projected.shape[1], weight.shape[0]), dtype=dtype)
    return [out, *fake[1:]]


@torch.library.custom_op("memsolve_b200::fast_mix_output_linear_bwd", mutates_args=(), device_types="cuda")
def _fast_mix_out_linear_bwd_op(grad_output: torch.Tensor, projected: torch.Tensor, core_base_raw: torch.Tensor,
                                eta_raw: torch.Tensor, valid_counts: Optional[torch.Tensor],
                                rotary_cos: Optional[torch.Tensor], rotary_sin: Optional[torch.Tensor],
                                weight: torch.Tensor, bias: Optional[torch.Tensor],
                                output_mask: Optional[torch.Tensor], tape: List[torch.Tensor], need_dw: bool,
                                need_db: bool) -> List[torch.Tensor]:
    """[d projected, d core_base_raw, d eta_raw, d weight, d bias]: the readout is rebuilt from the tape for the
    weight gradient, then the mixer's backward runs on d mixed = grad_output @ weight."""
    dims = _dims_of(projected, core_base_raw, rotary_cos)
    tape_t = _TapeTensors(*tape)
    weight_bf16 = weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)
    short = dims[1] <= dims[3]
    mixed = _readout(projected, tape_t, dims, valid_counts, rotary_cos, rotary_sin, short) if need_dw else None
    d_mixed, gw, gb = _linear_backward(grad_output.contiguous(), mixed, weight_bf16, output_mask, None,
                                       (True, need_dw, need_db and bias is not None), torch.bfloat16, weight.dtype,
                                       bias)
    del mixed
    d_mixed = d_mixed.contiguous()
    d_projected, d_base, d_raw = _mix_backward(projected, d_mixed, core_base_raw, eta_raw, valid_counts, None,
                                               rotary_cos, rotary_sin, tape_t, dims)
    if d_base is None:
        d_base = torch.zeros_like(core_base_raw)
    empty = lambda: grad_output.new_empty((0,))   # noqa: E731
    return [d_projected, d_base, d_raw, empty() if gw is None else gw.contiguous(),
            empty() if gb is None else gb.contiguous()]


@_fast_mix_out_linear_bwd_op.register_fake
def _fast_mix_out_linear_bwd_fake(grad_output, projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin,
                                  weight, bias, output_mask, tape, need_dw, need_db):
    empty = lambda: grad_output.new_empty((0,))   # noqa: E731
    return [torch.empty_like(projected), torch.empty_like(core_base_raw), torch.empty_like(eta_raw),
            torch.empty_like(weight) if need_dw else empty(),
            torch.empty_like(bias) if need_db and bias is not None else empty()]


def _fast_mix_out_linear_setup(ctx, inputs, output):
    projected, base, raw, counts, cos, sin, weight, bias, output_mask, _code = inputs
    ctx.flags = (counts is not None, cos is not None, bias is not None, output_mask is not None)
    extra = [t for t in (counts, cos, sin, bias, output_mask) if t is not None]
    ctx.save_for_backward(projected, base, raw, weight, *output[1:], *extra)


def _fast_mix_out_linear_autograd(ctx, grads):
    saved = list(ctx.saved_tensors)
    projected, base, raw, weight = saved[:4]
    tape, rest = saved[4:11], saved[11:]
    has_counts, has_rotary, has_bias, has_mask = ctx.flags
    counts = rest.pop(0) if has_counts else None
    cos, sin = (rest.pop(0), rest.pop(0)) if has_rotary else (None, None)
    bias = rest.pop(0) if has_bias else None
    output_mask = rest.pop(0) if has_mask else None
    needs = ctx.needs_input_grad
    d_projected, d_base, d_raw, gw, gb = torch.ops.memsolve_b200.fast_mix_output_linear_bwd(
        grads[0], projected, base, raw, counts, cos, sin, weight, bias, output_mask, tape, needs[6],
        has_bias and needs[7])
    return (d_projected, d_base, d_raw, None, None, None, gw if needs[6] else None,
            gb if has_bias and needs[7] else None, None, None)


torch.library.register_autograd("memsolve_b200::fast_mix_output_linear_fwd", _fast_mix_out_linear_autograd,
                                setup_context=_fast_mix_out_linear_setup)


def _traced_mix_output_linear(projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin, weight, bias,
                              output_dtype, output_mask):
    """The mixer followed by the output projection for a traced layer that recomputes the readout in backward."""
    mask = None if output_mask is None else output_mask.reshape(-1)
    return torch.ops.memsolve_b200.fast_mix_output_linear_fwd(
        projected, core_base_raw, eta_raw, valid_counts, rotary_cos, rotary_sin, weight, bias, mask,
        _DTYPE_CODES[output_dtype])[0]



class _RecomputeOutputLinear(torch.autograd.Function):
    """Output projection that rebuilds its ``mixed`` operand in backward from the compact tape
    (memsolve/ball/cuda.py:1345-1457) instead of keeping the [B,N,D] readout alive."""

    @staticmethod
    def forward(ctx, mixed, weight, bias, spec, output_dtype, output_mask):
        weight_bf16 = weight.to(torch.bfloat16)
        extra = [t for t in (spec.counts, spec.rotary_cos, spec.rotary_sin) if t is not None]
        ctx.save_for_backward(weight_bf16, output_mask, bias, spec.projected, *spec.tape, *extra)
        ctx.flags = (spec.counts is not None, spec.rotary_cos is not None)
        ctx.dims = spec.shape
        ctx.short = spec.short
        ctx.value_dtype, ctx.weight_dtype = mixed.dtype, weight.dtype
        return _linear_forward(mixed, weight_bf16, bias, output_dtype, output_mask, None)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        saved = list(ctx.saved_tensors)
        weight_bf16, output_mask, bias, projected = saved[:4]
        tape = _TapeTensors(*saved[4:11])
        rest = saved[11:]
        counts = rest.pop(0) if ctx.flags[0] else None
        cos, sin = (rest[0], rest[1]) if ctx.flags[1] else (None, None)
        need_dw = ctx.needs_input_grad[1]
        mixed = _readout(projected, tape, ctx.dims, counts, cos, sin, ctx.short) if need_dw else None
        needs = (ctx.needs_input_grad[0], need_dw, bias is not None and ctx.needs_input_grad[2])
        gv, gw, gb = _linear_backward(grad_output, mixed, weight_bf16, output_mask, None, needs,
                                      ctx.value_dtype, ctx.weight_dtype, bias)
        return gv, gw, gb, None, None, None


def _recompute_output_linear(mixed, spec, weight, bias, *, output_dtype, fuse_weight_bias_grad=True,
                             output_mask=None):
    return _RecomputeOutputLinear.apply(mixed, weight, bias, spec, output_dtype, output_mask)


__all__ = ["fast_mix", "is_available", "load", "require_available", "tensor_core_linear"]
