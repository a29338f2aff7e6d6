"""Sequence parallelism for the MemSolve layer: the token axis is split over the ranks of a
process group, every rank keeps a full copy of the weights.

Why it is exact: the Gram/moment statistics ``(G, Q)`` of the forward pass and the adjoint
statistics ``(E, de)`` of the backward pass are plain sums over tokens.  One SUM all-reduce of
``O(B*H*(r*r + r*d))`` floats per direction therefore gives every rank the statistics of the
whole sequence, the r x r solves that follow are identical on all ranks, and nothing of size N
ever crosses NVLink.

The public surface is the one of the reference's ``integrations.distributed.SequenceParallel``
(integrations/distributed.py:14-99): the constructor fields ``group``, ``shard_lengths``,
``rank``; ``create``, ``world_size``, ``global_length``, ``offset``, ``validate``, ``sum_``,
``sum_tensors``, ``valid_counts`` and ``reduce_gradients_`` with the same arguments, results and
exceptions.  Added here: ``overlap_gradient_sum``, which starts the SUM of each parameter
gradient from an autograd hook, on NCCL's own stream, while the rest of the backward pass still
runs, and ``use_peer_exchange``, which replaces the all-reduce of the statistics by one kernel
that reads the peers' values over NVLink.  Collectives are ``torch.distributed`` calls (NCCL over
NVLink on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import itertools
import os
from typing import Iterable, Sequence

import torch
import torch.distributed as dist

_SUM = dist.ReduceOp.SUM


class _GradientOverlap:
    """Hooks of one module that launch asynchronous gradient SUMs; returned by
    ``SequenceParallel.overlap_gradient_sum``.  ``remove()`` detaches the hooks."""

    def __init__(self, owner: "SequenceParallel", module: torch.nn.Module):
        self._owner = owner
        self._works: dict[int, object] = {}
        self._handles = [p.register_post_accumulate_grad_hook(self._launch)
                         for p in module.parameters() if p.requires_grad]

    def _launch(self, parameter: torch.Tensor) -> None:
        gradient = parameter.grad
        exchange = self._owner.peer_exchange
        if exchange is not None and exchange.can_sum(gradient):
            self._works[id(parameter)] = exchange.sum_async(gradient)
        else:
            self._works[id(parameter)] = dist.all_reduce(gradient, op=_SUM, group=self._owner.group, async_op=True)

    def finish(self, parameters: Sequence[torch.Tensor]) -> None:
        """Sum what no hook has started (a gradient written without autograd), then wait for all."""
        for parameter in parameters:
            if id(parameter) not in self._works:
                self._launch(parameter)
        works, self._works = self._works, {}
        for work in works.values():
            work.wait()

    def remove(self) -> None:
        for handle in self._handles:
            handle.remove()
        self._handles = []
        self._works = {}


class _PeerExchange:
    """Exchange areas in symmetric memory (one allocation per rank that every peer can address) for
    the kernel that sums the token statistics over the ranks without a collective library call."""

    MINIMUM_BYTES = 1 << 20

    def __init__(self, owner: "SequenceParallel"):
        self._owner = owner
        self._areas: dict[int, tuple] = {}       # per device: areas of the statistics exchange
        self._sum_areas: dict[int, tuple] = {}   # per device: areas of the gradient SUM (other layout)
        self._streams: dict[int, torch.cuda.Stream] = {}

    def _allocate(self, nbytes: int, device: torch.device) -> tuple:
        """One zeroed symmetric-memory area per rank: (tensor, handle, address array, bytes)."""
        import ctypes
        import torch.distributed._symmetric_memory as symmetric
        size = 1 << max(nbytes - 1, 1).bit_length()   # the same power of two on every rank
        group = self._owner.group if self._owner.group is not None else dist.group.WORLD
        enable = getattr(symmetric, "enable_symm_mem_for_group", None)
        if enable is not None:
            try:
                enable(group.group_name)
            except Exception:  # noqa: BLE001 - newer releases enable groups on rendezvous
                pass
        buffer = symmetric.empty(size // 4, dtype=torch.float32, device=device)
        buffer.zero_()
        handle = symmetric.rendezvous(buffer, group)
        handle.barrier()   # every area is zero before any rank's kernel can touch it
        pointers = (ctypes.c_void_p * self._owner.world_size)(*[int(p) for p in handle.buffer_ptrs])
        return buffer, handle, pointers, size

    def areas(self, nbytes: int, device: torch.device):
        """(array of the ranks' area addresses, bytes per area) with at least `nbytes` per area.
        The first call for a device (or a larger size) allocates and is a collective host operation:
        make it on every rank, outside CUDA-graph capture."""
        entry = self._areas.get(device.index)
        if entry is None or entry[3] < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    "the peer-memory exchange areas must be allocated before CUDA-graph capture: run one eager "
                    "step (or call SequenceParallel.prepare_peer_exchange) on every rank first")
            if entry is not None:
                torch.cuda.current_stream(device).synchronize()   # no kernel may still use the old area
            entry = self._areas[device.index] = self._allocate(max(nbytes, self.MINIMUM_BYTES), device)
        return entry[2], entry[3]

    def prepare(self, statistics_bytes: int, largest_gradient_numel: int, device: torch.device) -> None:
        """Allocate both kinds of areas once, outside capture (collective: call on every rank)."""
        from ..ball import cuda as backend
        self.areas(statistics_bytes, device)
        if largest_gradient_numel >= self.SUM_MINIMUM_NUMEL and device.index not in self._sum_areas:
            need = int(backend._LIB.ms_peer_sum_area_bytes(largest_gradient_numel))
            self._sum_areas[device.index] = self._allocate(max(need, 32 << 20), device)
            self._streams[device.index] = torch.cuda.Stream(device)

    # ---- in-place SUM of a gradient over the ranks, on a stream of its own
    SUM_MINIMUM_NUMEL = 1 << 18   # smaller gradients are latency-bound either way: leave them to NCCL

    def can_sum(self, tensor: torch.Tensor) -> bool:
        if not (tensor.is_cuda and tensor.dtype == torch.float32 and tensor.is_contiguous()
                and tensor.numel() >= self.SUM_MINIMUM_NUMEL and tensor.numel() % 4 == 0
                and tensor.data_ptr() % 16 == 0):
            return False
        entry = self._sum_areas.get(tensor.device.index)
        if entry is None:
            # the first SUM allocates (a collective host operation): not while a graph is being captured
            return not torch.cuda.is_current_stream_capturing()
        # an area is never replaced while work may be queued on it: what does not fit goes to NCCL
        from ..ball import cuda as backend
        return int(backend._LIB.ms_peer_sum_area_bytes(tensor.numel())) <= entry[3]

    def sum_async(self, tensor: torch.Tensor) -> "_StreamWork":
        """Launch the peer-memory SUM of `tensor` on the exchange's side stream, ordered after the
        work already queued on the current stream; the returned object's wait() makes the current
        stream wait for it.  The first call on a device allocates (see `areas`)."""
        from ..ball import cuda as backend
        device = tensor.device
        backend.require_available()
        lib = backend._LIB
        entry = self._sum_areas.get(device.index)
        need = int(lib.ms_peer_sum_area_bytes(tensor.numel()))
        if entry is None:
            entry = self._sum_areas[device.index] = self._allocate(max(need, 32 << 20), device)
            self._streams[device.index] = torch.cuda.Stream(device)
        elif entry[3] < need:
            raise RuntimeError("gradient larger than the peer-memory SUM area; can_sum() routes such tensors to NCCL")
        side = self._streams[device.index]
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            status = lib.ms_peer_sum(tensor.data_ptr(), tensor.numel(), entry[2], entry[3], self._owner.world_size,
                                     self._owner.rank, side.cuda_stream)
            if status != 0:
                raise RuntimeError(f"peer-memory gradient SUM failed: {lib.ms_status_string(status).decode()}")
            # the gradient stays alive in `parameter.grad` until the caller has waited for this work
            return _StreamWork(side.record_event(), device)


class _StreamWork:
    """Completion of work queued on a side stream (same role as a collective's Work object)."""

    def __init__(self, event: torch.cuda.Event, device: torch.device):
        self._event, self._device = event, device

    def wait(self) -> None:
        torch.cuda.current_stream(self._device).wait_event(self._event)


class SequenceParallel:
    """Layout of one sharded sequence: the process group, every rank's shard length, this rank."""

    __slots__ = ("group", "shard_lengths", "rank", "_starts", "_overlaps", "peer_exchange", "check_device_errors")

    def __init__(self, group, shard_lengths: Iterable[int], rank: int):
        self.group = group
        self.shard_lengths = tuple(int(length) for length in shard_lengths)
        self.rank = int(rank)
        self._starts = (0, *itertools.accumulate(self.shard_lengths))
        self._overlaps: dict[int, _GradientOverlap] = {}
        self.peer_exchange: _PeerExchange | None = None
        # read the kernels' error word at the end of reduce_gradients_ (one device synchronisation per step):
        # off unless asked for, because a peer that never arrives already turns the sums into NaN
        self.check_device_errors = os.environ.get("MEMSOLVE_CHECK_DEVICE_ERRORS", "") == "1"

    def __repr__(self) -> str:
        return f"SequenceParallel(shard_lengths={self.shard_lengths}, rank={self.rank})"

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, SequenceParallel):
            return NotImplemented
        return (self.group, self.shard_lengths, self.rank) == (other.group, other.shard_lengths, other.rank)

    def __hash__(self) -> int:
        return hash((id(self.group), self.shard_lengths, self.rank))

    # ---------------------------------------------------------------- layout
    @classmethod
    def create(cls, local_length: int, group=None) -> "SequenceParallel":
        """Collect the shard lengths of all ranks (one host-side object gather; call it once per
        layout and outside CUDA-graph capture)."""
        if not dist.is_initialized():
            raise RuntimeError("initialize torch.distributed before sequence parallelism")
        world = dist.get_world_size(group)
        gathered: list = [None for _ in range(world)]
        dist.all_gather_object(gathered, int(local_length), group=group)
        if min(gathered) < 1:
            raise ValueError("sequence shards must be nonempty")
        return cls(group, gathered, dist.get_rank(group))

    @property
    def world_size(self) -> int:
        return len(self.shard_lengths)

    @property
    def global_length(self) -> int:
        return self._starts[-1]

    @property
    def offset(self) -> int:
        """Global index of this rank's first token (where its rotary positions start)."""
        return self._starts[self.rank]

    @property
    def local_length(self) -> int:
        return self.shard_lengths[self.rank]

    def validate(self, local_length: int, operator_rank: int) -> None:
        if local_length != self.local_length:
            raise ValueError("local sequence length differs from the sequence-parallel layout")
        if self.global_length <= operator_rank:
            raise ValueError(
                "sequence parallelism requires global sequence length > rank; use an unsharded short sequence")

    # ---------------------------------------------------------------- collectives
    def sum_(self, tensor: torch.Tensor) -> torch.Tensor:
        """In-place SUM over the group (a no-op for a single rank)."""
        if self.world_size != 1:
            dist.all_reduce(tensor, op=_SUM, group=self.group)
        return tensor

    def sum_tensors(self, *tensors: torch.Tensor):
        """SUM several tensors with one collective.  A single contiguous tensor is summed in place;
        otherwise the values travel in one packed buffer and views of it are returned."""
        if self.world_size == 1:
            return tensors
        if len(tensors) == 1 and tensors[0].is_contiguous():
            self.sum_(tensors[0].view(-1))
            return tensors
        sizes = [t.numel() for t in tensors]
        packed = torch.empty(sum(sizes), dtype=tensors[0].dtype, device=tensors[0].device)
        slots = packed.split(sizes)
        for slot, t in zip(slots, tensors):
            slot.copy_(t.reshape(-1))
        self.sum_(packed)
        return tuple(slot.view_as(t) for slot, t in zip(slots, tensors))

    def valid_counts(self, mask, *, batch_size=None, device=None) -> torch.Tensor:
        """Valid tokens per sample over the whole sequence, FP32 ``[B]``, at least 1.

        Every rank must call this, also one whose own shard has no padding and passes
        ``mask=None``: the SUM is a collective.  The lower bound is applied after the SUM.
        """
        if mask is not None:
            if mask.dtype != torch.bool or mask.ndim != 2 or mask.shape[1] != self.local_length:
                raise ValueError("mask must be boolean [batch, local_length]")
            local = mask.sum(dim=-1, dtype=torch.float32)
        elif batch_size is None or device is None:
            raise ValueError("unmasked counts require batch_size and device")
        else:
            local = torch.full((batch_size,), float(self.local_length), dtype=torch.float32, device=device)
        return self.sum_(local).clamp_min_(1)

    def use_peer_exchange(self, enabled: bool = True) -> None:
        """Sum the token statistics of the CUDA layer with one kernel over NVLink peer memory instead
        of reduce + all-reduce (single node, at most 8 ranks, every GPU able to address its peers).
        Call it on every rank; the first layer call afterwards allocates the exchange areas and must
        run eagerly (not under CUDA-graph capture)."""
        if enabled and self.world_size > 8:
            raise ValueError("the peer-memory exchange supports at most 8 ranks")
        self.peer_exchange = _PeerExchange(self) if enabled and self.world_size > 1 else None

    def prepare_peer_exchange(self, module: torch.nn.Module, local_batch: int = 1) -> None:
        """Allocate the exchange areas for `module` (a MemSolve layer or a model containing such layers) once,
        before any CUDA-graph capture: the statistics areas from the largest layer shape, the gradient-SUM
        areas from the largest trainable parameter.  Collective host operation: call on every rank."""
        if self.peer_exchange is None:
            return
        import ctypes
        from ..ball import cuda as backend
        backend.require_available()
        params = [p for p in module.parameters() if p.requires_grad and p.is_cuda]
        if not params:
            return
        device = params[0].device
        need = 0
        for sub in module.modules():
            cfg = getattr(sub, "config", None)
            if cfg is None or not hasattr(cfg, "rank") or not hasattr(cfg, "num_heads"):
                continue
            shape = backend._Shape(local_batch, self.local_length, cfg.num_heads, cfg.rank,
                                   cfg.dim // cfg.num_heads, 0, 0, 0)
            need = max(need, int(backend._LIB.ms_exchange_area_bytes(ctypes.byref(shape))))
        largest = max(p.numel() for p in params)
        with torch.cuda.device(device):
            self.peer_exchange.prepare(max(need, _PeerExchange.MINIMUM_BYTES), largest, device)

    # ---------------------------------------------------------------- parameter gradients
    def overlap_gradient_sum(self, module: torch.nn.Module) -> _GradientOverlap:
        """Start the SUM of each parameter gradient of `module` as soon as autograd has written it.

        The all-reduces run on the communication stream of the process group and overlap the
        remaining backward kernels; ``reduce_gradients_(module)`` then only waits for them.  Use it
        when every ``reduce_gradients_`` follows exactly one backward pass: with gradient
        accumulation over several backward passes an early SUM would count the earlier passes once
        per rank.  Returns the handle whose ``remove()`` restores the plain behaviour.
        """
        overlap = self._overlaps.get(id(module))
        if overlap is None:
            overlap = self._overlaps[id(module)] = _GradientOverlap(self, module)
        return overlap

    @torch.no_grad()
    def reduce_gradients_(self, module: torch.nn.Module) -> None:
        """SUM the gradients of the replicated parameters over the group, in place.

        Call it once after the (accumulated) backward pass and before clipping or the optimizer
        step, and do not average over this group as well.  Every trainable parameter must have a
        gradient: the set of collectives is then the same on all ranks without any host check, and
        the call can be captured in a CUDA graph together with forward and backward.
        """
        trainable = [p for p in module.parameters() if p.requires_grad]
        if self.world_size == 1 or not trainable:
            return
        if not all(p.grad is not None for p in trainable):
            raise ValueError(
                "sequence gradient SUM requires a gradient for every trainable parameter; freeze unused parameters")
        overlap = self._overlaps.get(id(module))
        if overlap is not None and overlap._handles:
            overlap.finish(trainable)
        else:
            self._sum_in_place([p.grad for p in trainable])
        if self.check_device_errors and self.peer_exchange is not None and trainable[0].is_cuda:
            self.raise_on_device_error(trainable[0].device)

    def raise_on_device_error(self, device) -> None:
        """Synchronise `device` and raise if one of the library's kernels recorded an error since the last
        check: 0x200 means a rank waited for a peer longer than the limit (`ms_set_peer_wait_ms`) and its
        statistics or gradients of this step are NaN; 0x100 a shared-memory barrier timeout inside a kernel."""
        from ..ball import cuda as backend
        if torch.cuda.is_current_stream_capturing():
            return
        with torch.cuda.device(device):
            word = int(backend._LIB.ms_device_error())
        if word != 0:
            raise RuntimeError(
                f"MemSolve CUDA kernels reported device error {word:#x} on rank {self.rank}"
                + (": a peer did not publish its statistics or gradients within the wait limit; this step's "
                   "results are NaN" if word == 0x200 else ""))

    def _sum_in_place(self, tensors: Sequence[torch.Tensor]) -> None:
        """One coalesced collective over all tensors (no packing copies) where the backend offers
        it, else one packed buffer per (device, dtype)."""
        manager = getattr(dist, "_coalescing_manager", None)
        if manager is not None and tensors[0].is_cuda:
            with manager(group=self.group, device=tensors[0].device, async_ops=False):
                for t in tensors:
                    dist.all_reduce(t, op=_SUM, group=self.group)
            return
        groups: dict = {}
        for t in tensors:
            groups.setdefault((t.device, t.dtype), []).append(t)
        for members in groups.values():
            summed = self.sum_tensors(*members)
            for target, value in zip(members, summed):
                if target.data_ptr() != value.data_ptr():
                    target.copy_(value)


__all__ = ["SequenceParallel"]
