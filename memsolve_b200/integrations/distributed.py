"""Exact sequence parallelism for the MemSolve layer.

Each rank owns a contiguous slice of the token axis of the same samples and a
full copy of the weights.  Because the Gram/moment statistics ``(G, Q)`` and the
adjoint statistics ``(E, de)`` are sums over tokens, one SUM all-reduce of
``O(B*H*(r*r + r*d))`` floats per direction makes every rank's compact solve
identical to the unsharded one; nothing of size N crosses the interconnect.

API and semantics follow the reference's ``integrations.distributed.SequenceParallel``
(integrations/distributed.py:14-99): ``create``, ``world_size``, ``global_length``,
``offset``, ``validate``, ``sum_``, ``sum_tensors``, ``valid_counts``,
``reduce_gradients_``.  The collective is ``torch.distributed.all_reduce`` (NCCL
over NVLink on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class SequenceParallel:
    group: object
    shard_lengths: tuple[int, ...]
    rank: int

    @classmethod
    def create(cls, local_length: int, group=None) -> "SequenceParallel":
        """Exchange shard lengths once per layout (host-side object gather)."""
        if not dist.is_initialized():
            raise RuntimeError("initialize torch.distributed before sequence parallelism")
        lengths: list = [None] * dist.get_world_size(group)
        dist.all_gather_object(lengths, int(local_length), group=group)
        if any(length < 1 for length in lengths):
            raise ValueError("sequence shards must be nonempty")
        return cls(group, tuple(int(v) for v in lengths), dist.get_rank(group))

    @property
    def world_size(self) -> int:
        return len(self.shard_lengths)

    @property
    def global_length(self) -> int:
        return sum(self.shard_lengths)

    @property
    def offset(self) -> int:
        """Global index of this rank's first token (start of its rotary positions)."""
        return sum(self.shard_lengths[: self.rank])

    def validate(self, local_length: int, operator_rank: int) -> None:
        if local_length != self.shard_lengths[self.rank]:
            raise ValueError("local sequence length differs from the sequence-parallel layout")
        if self.global_length <= operator_rank:
            raise ValueError(
                "sequence parallelism requires global sequence length > rank; use an unsharded short sequence")

    def sum_(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor

    def sum_tensors(self, *tensors: torch.Tensor):
        """One collective for several tensors; returns views of the summed buffer."""
        if self.world_size == 1:
            return tensors
        if len(tensors) == 1 and tensors[0].is_contiguous():
            self.sum_(tensors[0].view(-1))
            return tensors
        flat = torch.cat([t.reshape(-1) for t in tensors])
        self.sum_(flat)
        parts = flat.split([t.numel() for t in tensors])
        return tuple(part.view_as(t) for part, t in zip(parts, tensors))

    def valid_counts(self, mask, *, batch_size=None, device=None) -> torch.Tensor:
        """Global max(valid tokens, 1) per sample as FP32 [B]; the clamp follows the SUM."""
        local = self.shard_lengths[self.rank]
        if mask is None:
            if batch_size is None or device is None:
                raise ValueError("unmasked counts require batch_size and device")
            counts = torch.full((batch_size,), float(local), device=device, dtype=torch.float32)
        else:
            if mask.dtype != torch.bool or mask.ndim != 2 or mask.shape[1] != local:
                raise ValueError("mask must be boolean [batch, local_length]")
            counts = mask.sum(-1, dtype=torch.float32)
        return self.sum_(counts).clamp_min_(1)

    @torch.no_grad()
    def reduce_gradients_(self, module: torch.nn.Module) -> None:
        """SUM the gradients of replicated parameters, one flat collective per (device, dtype)."""
        params = [p for p in module.parameters() if p.requires_grad]
        if self.world_size == 1 or not params:
            return
        if any(p.grad is None for p in params):
            raise ValueError(
                "sequence gradient SUM requires a gradient for every trainable parameter; freeze unused parameters")
        buckets: dict = {}
        for p in params:
            buckets.setdefault((p.device, p.dtype), []).append(p.grad)
        for grads in buckets.values():
            flat = torch.cat([g.reshape(-1) for g in grads])
            self.sum_(flat)
            parts = flat.split([g.numel() for g in grads])
            torch._foreach_copy_(grads, [part.view_as(g) for g, part in zip(grads, parts)])


__all__ = ["SequenceParallel"]
