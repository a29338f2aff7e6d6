"""Two-rank sequence-parallel layer on two GPUs (NCCL): sharded forward/backward equals the unsharded
FP64 oracle and the unsharded CUDA layer (limits of the reference's tests/cuda/test_sequence_parallel.py:
output < 5e-3, gradients < 3e-2).  Skipped with fewer than two devices."""
from __future__ import annotations

import copy
import os
import sys
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).norm() / b.double().cpu().norm().clamp_min(1e-12))


def _worker(rank, path, results):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from memsolve_b200 import CoreMode, MemSolve, MemSolveConfig
    from memsolve_b200.ball import cuda
    from memsolve_b200.integrations.distributed import SequenceParallel
    from oracle import memsolve_oracle as O

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{path}", rank=rank, world_size=2,
                            timeout=timedelta(seconds=120), device_id=torch.device("cuda", rank))
    try:
        cuda.load()
        cases = [(16, (97, 100), False, False), (32, (512, 480), True, False), (64, (200, 184), True, True),
                 (32, (19, 22), False, True)]
        for case, (rank_r, lengths, rotary, masked) in enumerate(cases):
            sp = SequenceParallel.create(lengths[rank])
            torch.manual_seed(913 + rank_r)
            layer = MemSolve(MemSolveConfig(128, 2, rank=rank_r, bias=True, rotary=rotary)).cuda()
            if case % 2 == 0:
                sp.overlap_gradient_sum(layer)   # gradient SUMs start from autograd hooks
            if case in (1, 2):
                sp.use_peer_exchange()           # statistics summed by one kernel over peer memory
            with torch.no_grad():
                layer.core_base_raw.normal_(std=0.1)
            total = sum(lengths)
            full = torch.randn(2, total, 128).bfloat16().cuda()            # same seed on both ranks
            upstream = (torch.randn(2, total, 128) * 0.01).bfloat16().cuda()
            mask = torch.ones(2, total, dtype=torch.bool, device="cuda")
            if masked:
                mask[0, ::3] = False
                mask[1, : total // 2] = False
            sel = slice(sp.offset, sp.offset + lengths[rank])
            x = full[:, sel].clone().requires_grad_()
            local_mask = mask[:, sel] if masked else None
            counts = sp.valid_counts(local_mask, batch_size=2, device=x.device)
            kwargs = {}
            if rotary and masked:
                kwargs["rotary_context_length"] = total
            y = layer(x, local_mask, implementation="cuda", sequence_parallel=sp, valid_counts=counts, **kwargs)
            (y.float() * upstream[:, sel].float()).sum().backward()
            sp.reduce_gradients_(layer)
            torch.cuda.synchronize()

            # unsharded FP64 oracle
            p = O.LayerParams(layer.w_bc.weight.detach().cpu(), layer.w_o.weight.detach().cpu(),
                              layer.core_base_raw.detach().cpu(), layer.eta_raw.detach().cpu(),
                              layer.w_bc.bias.detach().cpu(), layer.w_o.bias.detach().cpu(),
                              heads=2, rank=rank_r).to(torch.float64)
            for t in p.tensors():
                t.requires_grad_()
            xr = full.double().cpu().requires_grad_()
            cos = sin = None
            if rotary:
                cos, sin = O.rotary_tables(torch.arange(total)[None], head_dim=64, context_length=total,
                                           dtype=torch.float64)
            yr = O.layer_forward(p, xr, mask.cpu() if masked else None, cos, sin)
            (yr * upstream.double().cpu()).sum().backward()
            assert _rel(y, yr[:, sel]) < 5e-3, (rank_r, "out")
            assert _rel(x.grad, xr.grad[:, sel]) < 3e-2, (rank_r, "dx")
            pairs = [(layer.w_bc.weight, p.w_bc), (layer.w_o.weight, p.w_o), (layer.core_base_raw, p.core_base_raw),
                     (layer.eta_raw, p.eta_raw), (layer.w_bc.bias, p.b_bc), (layer.w_o.bias, p.b_o)]
            for got, want in pairs:
                assert _rel(got.grad, want.grad) < 3e-2, (rank_r, tuple(got.shape), _rel(got.grad, want.grad))
            if masked:
                assert torch.count_nonzero(x.grad[~local_mask]) == 0

            # unsharded CUDA layer on this rank
            ref = copy.deepcopy(layer)
            ref.zero_grad(set_to_none=True)
            xf = full.clone().requires_grad_()
            yf = ref(xf, mask if masked else None, implementation="cuda", **kwargs)
            (yf.float() * upstream.float()).sum().backward()
            assert _rel(y, yf[:, sel]) < 5e-3 and _rel(x.grad, xf.grad[:, sel]) < 5e-3
            assert _rel(layer.core_base_raw.grad, ref.core_base_raw.grad) < 5e-3
        assert cuda._LIB.ms_device_error() == 0
        results[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="requires two CUDA devices")
def test_sharded_layer_matches_unsharded(tmp_path):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(str(tmp_path / "nccl"), results), nprocs=2, join=True)
    assert dict(results) == {0: 1, 1: 1}


def _peer_worker(rank, world, path, results):
    """Peer-memory kernels against NCCL on `world` GPUs: the statistics exchange (through the layer, both
    directions) and the in-place gradient SUM (`ms_peer_sum`: reduce-scatter + all-gather, two flag rounds)."""
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from memsolve_b200 import MemSolve, MemSolveConfig
    from memsolve_b200.ball import cuda
    from memsolve_b200.integrations.distributed import SequenceParallel

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{path}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=180), device_id=torch.device("cuda", rank))
    try:
        cuda.load()
        lib = cuda._LIB
        # --- gradient SUM: several calls in a row (both buffer parities), a length that is not a multiple of
        # world * 16, values that differ per rank and call
        sp = SequenceParallel.create(64)
        sp.use_peer_exchange()
        exchange = sp.peer_exchange
        for call, numel in enumerate((1 << 18, (1 << 18) + 4 * 37, 768 * 1152, 1 << 18)):
            torch.manual_seed(1000 * call + rank)
            values = torch.randn(numel, device="cuda")
            want = values.clone()
            dist.all_reduce(want)
            assert exchange.can_sum(values)
            exchange.sum_async(values).wait()
            torch.cuda.synchronize()
            # the kernel adds in rank order on every rank; NCCL's order differs: compare to rounding
            assert _rel(values, want) < 1e-6, (call, _rel(values, want))
            gathered = [torch.empty_like(values) for _ in range(world)]
            dist.all_gather(gathered, values)
            assert all(torch.equal(gathered[0], g) for g in gathered)      # identical bits on all ranks
        assert not exchange.can_sum(torch.randn(1 << 10, device="cuda"))   # small gradients stay on NCCL
        assert lib.ms_device_error() == 0

        # --- a layer whose weight gradients are large enough for the peer-memory SUM (dim 512): sharded step
        # with the peer exchange against the same step with NCCL for statistics and gradients
        local = 256 + 16 * rank
        torch.manual_seed(77)
        layer = MemSolve(MemSolveConfig(512, 8, rank=32, rotary=True)).cuda()
        with torch.no_grad():
            layer.core_base_raw.normal_(std=0.1)
        twin = copy.deepcopy(layer)
        total = sum(256 + 16 * r for r in range(world))
        full = torch.randn(1, total, 512).bfloat16().cuda()
        upstream = (torch.randn(1, total, 512) * 0.01).bfloat16().cuda()
        outs = []
        for module, peer in ((layer, True), (twin, False)):
            sp = SequenceParallel.create(local)
            sp.check_device_errors = True
            sp.overlap_gradient_sum(module)
            if peer:
                sp.use_peer_exchange()
                sp.prepare_peer_exchange(module)
            sel = slice(sp.offset, sp.offset + local)
            x = full[:, sel].clone().requires_grad_()
            counts = sp.valid_counts(None, batch_size=1, device=x.device)
            for _ in range(3):   # several steps: both parities of the double-buffered areas
                module.zero_grad(set_to_none=True)
                x.grad = None
                y = module(x, implementation="cuda", sequence_parallel=sp, valid_counts=counts)
                y.backward(upstream[:, sel])
                sp.reduce_gradients_(module)
            torch.cuda.synchronize()
            outs.append((y.detach(), x.grad.clone(), [p.grad.clone() for p in module.parameters()]))
        (y1, dx1, g1), (y2, dx2, g2) = outs
        assert _rel(y1, y2) < 1e-3 and _rel(dx1, dx2) < 1e-3
        for a, b in zip(g1, g2):
            assert _rel(a, b) < 1e-3, (tuple(a.shape), _rel(a, b))
        assert lib.ms_device_error() == 0
        results[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_memory_kernels_match_nccl(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"requires {world} CUDA devices")
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_peer_worker, args=(world, str(tmp_path / f"nccl{world}"), results), nprocs=world, join=True)
    assert dict(results) == {r: 1 for r in range(world)}
