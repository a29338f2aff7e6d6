"""Sequence-parallel host logic on CPU: two `gloo` ranks (no GPU involved).

Covers `SequenceParallel` (layout exchange, offsets, global counts with the clamp after the SUM,
packed SUM of several tensors, SUM of replicated gradients) and the algebra the CUDA path relies on:
per-shard statistics scaled by the GLOBAL count add up to the unsharded statistics, so the compact
stage and the local readout reproduce the unsharded result (checked with the CPU oracle's stages)."""
from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, path: str, lengths, results):
    sys.path.insert(0, ROOT)
    from memsolve_b200.integrations.distributed import SequenceParallel
    from oracle import memsolve_oracle as O

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    try:
        sp = SequenceParallel.create(lengths[rank])
        assert sp.world_size == world and sp.shard_lengths == tuple(lengths)
        assert sp.global_length == sum(lengths) and sp.offset == sum(lengths[:rank])
        sp.validate(lengths[rank], 16)
        with pytest.raises(ValueError, match="differs from the sequence-parallel layout"):
            sp.validate(lengths[rank] + 1, 16)
        with pytest.raises(ValueError, match="global sequence length > rank"):
            sp.validate(lengths[rank], sum(lengths))

        # counts: the clamp comes after the SUM; a rank without a mask still takes part
        batch = 3
        full_mask = torch.ones(batch, sum(lengths), dtype=torch.bool)
        full_mask[0, ::3] = False
        full_mask[2] = False
        local_mask = full_mask[:, sp.offset: sp.offset + lengths[rank]]
        counts = sp.valid_counts(local_mask)
        assert torch.equal(counts, full_mask.sum(-1).float().clamp_min(1))
        unmasked = sp.valid_counts(None, batch_size=batch, device=torch.device("cpu"))
        assert torch.equal(unmasked, torch.full((batch,), float(sum(lengths))))
        with pytest.raises(ValueError, match="batch_size and device"):
            sp.valid_counts(None)

        # packed SUM of several tensors returns views with the original shapes
        a = torch.full((2, 3), float(rank + 1))
        bvec = torch.arange(4, dtype=torch.float32) * (rank + 1)
        sa, sb = sp.sum_tensors(a, bvec)
        tot = sum(range(1, world + 1))
        assert sa.shape == (2, 3) and torch.equal(sa, torch.full((2, 3), float(tot)))
        assert torch.equal(sb, torch.arange(4, dtype=torch.float32) * tot)
        (single,) = sp.sum_tensors(torch.ones(5) * (rank + 1))
        assert torch.equal(single, torch.ones(5) * tot)

        # replicated-parameter gradients: SUM once over the group, frozen parameters skipped
        lin = torch.nn.Linear(3, 2)
        frozen = torch.nn.Parameter(torch.zeros(2), requires_grad=False)
        lin.register_parameter("frozen", frozen)
        for p in lin.parameters():
            if p.requires_grad:
                p.grad = torch.full_like(p, float(rank + 1))
        sp.reduce_gradients_(lin)
        assert torch.equal(lin.weight.grad, torch.full_like(lin.weight, float(tot)))
        lin.bias.grad = None
        with pytest.raises(ValueError, match="requires a gradient for every trainable parameter"):
            sp.reduce_gradients_(lin)

        # overlapped SUM: hooks launch the all-reduce of each gradient during backward, the call
        # afterwards only waits; a gradient written by hand (no hook) is summed by the call itself
        net = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Tanh(), torch.nn.Linear(3, 2))
        with torch.no_grad():
            for k, p in enumerate(net.parameters()):
                p.copy_(torch.linspace(-1, 1, p.numel()).reshape(p.shape) * (k + 1) / 4)
        data = torch.arange(8.0).reshape(2, 4) * (rank + 1)
        net(data).square().sum().backward()
        local = [p.grad.clone() for p in net.parameters()]
        net.zero_grad(set_to_none=True)
        handle = sp.overlap_gradient_sum(net)
        assert sp.overlap_gradient_sum(net) is handle
        net(data).square().sum().backward()
        sp.reduce_gradients_(net)
        for p, mine in zip(net.parameters(), local):
            both = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(both, mine)
            assert torch.allclose(p.grad, sum(both), rtol=1e-6, atol=1e-6)
        for p in net.parameters():
            p.grad = torch.full_like(p, float(rank + 1))
        sp.reduce_gradients_(net)
        assert all(torch.equal(p.grad, torch.full_like(p, float(tot))) for p in net.parameters())
        handle.remove()

        # algebra of the sharded mixer (CPU oracle stages): statistics scaled by the global count add up
        heads, rank_r, d = 2, 16, 8
        gen = torch.Generator().manual_seed(7)
        proj = torch.randn(2, sum(lengths), heads * (rank_r + d), generator=gen).bfloat16()
        base = torch.randn(heads, rank_r, rank_r, generator=gen) * 0.1
        eta_raw = torch.randn(heads, generator=gen) * 0.3
        pos = torch.arange(sum(lengths))[None]
        cos, sin = O.rotary_tables(pos, head_dim=d, train_length=16, context_length=sum(lengths))
        sl = slice(sp.offset, sp.offset + lengths[rank])
        gcount = sp.valid_counts(None, batch_size=2, device=torch.device("cpu")).double()
        g_loc, q_loc = O.stage_stats(proj[:, sl], heads, rank_r, gcount, cos[:, sl], sin[:, sl])
        g_sum, q_sum = sp.sum_tensors(g_loc.contiguous(), q_loc.contiguous())
        g_full, q_full = O.stage_stats(proj, heads, rank_r, None, cos, sin)
        assert torch.allclose(g_sum, g_full, rtol=1e-12, atol=1e-12)
        assert torch.allclose(q_sum, q_full, rtol=1e-12, atol=1e-12)
        _t, _z, _f, eta, w = O.stage_compact(g_sum, q_sum, base, eta_raw)
        y_loc = O.stage_readout(proj[:, sl], w, eta, heads, rank_r, gcount, cos[:, sl], sin[:, sl])
        y_full = O.fast_mix_frame(proj, base, eta_raw, None, cos, sin)
        assert torch.allclose(y_loc, y_full[:, sl], rtol=1e-9, atol=1e-9)
        results[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("lengths", [(19, 22), (40, 40)])
def test_two_gloo_ranks(tmp_path, lengths):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, str(tmp_path / "rendezvous"), lengths, results), nprocs=2, join=True)
    assert dict(results) == {0: 1, 1: 1}


def test_requires_initialised_process_group():
    from memsolve_b200.integrations.distributed import SequenceParallel
    if not dist.is_initialized():
        with pytest.raises(RuntimeError, match="initialize torch.distributed"):
            SequenceParallel.create(8)
