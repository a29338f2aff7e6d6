#!/usr/bin/env python
"""MemSolve layer forward+backward throughput on B200 (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c5|c2|c4]

Workload on one GPU ("c3"): one MemSolve layer, dim 768, 12 heads (head dim 64), rank 32, rotary on,
BF16, x = [1, 32768, 768] ~ N(0,1), upstream gradient ~ N(0,1), seeded random-init weights
(core_base_raw ~ N(0, 0.1^2) so the core is exercised), recompute_readout=False -- the long-sequence
single-layer shape the headline metric is quoted on.  On N > 1 GPUs ("c5"): rank 64, one sequence of
262144 tokens split evenly over the ranks (sequence parallel, strong scaling) -- the reference's
multi-GPU shape; `--workload c3 --gpus N` instead gives every rank 32768 tokens of a 32768*N-token
sequence (weak scaling).

A step is layer forward + backward (+ the sequence-parallel gradient SUM when N > 1).  The timed region is
`--blocks` blocks of `--steps` steps each, every block bracketed by a barrier and a device synchronisation;
the median block is reported.  `value` is tokens/s of the whole job with inputs resident in HBM; `e2e`
repeats the step through the same public call with the inputs in pinned host memory (copied in every step)
and the output and the input gradient copied back to pinned host memory.  `roofline` is measured live: each
mixer kernel is timed alone with CUDA events on the launching stream after an L2 flush.  `--sweep` prints
one line per sequence length 128 ... 32768 (tokens/s of the layer and of the mix core).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    "c3": dict(dim=768, heads=12, rank=32, local_tokens=32768, strong=False),
    "c5": dict(dim=768, heads=12, rank=64, global_tokens=262144, strong=True),
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_layer(cfg, device, seed=0):
    from memsolve_b200 import MemSolve, MemSolveConfig
    torch.manual_seed(seed)
    layer = MemSolve(MemSolveConfig(dim=cfg["dim"], num_heads=cfg["heads"], rank=cfg["rank"], rotary=True,
                                    recompute_readout=False))
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    return layer.to(device)


# ---------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port of the reference's pure-PyTorch CPU path
# ---------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def reference_available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "memsolve", "__init__.py"))


def reference_layer_step(cfg, tokens, seed=0):
    """One forward+backward of the reference's own layer (`layer(x, implementation="reference")`, its pure
    PyTorch CPU path) on `tokens` tokens; the package is the copy that oracle/build_ref.py placed in oracle/_ref."""
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    from memsolve import MemSolve as RefLayer, MemSolveConfig as RefConfig
    torch.manual_seed(seed)
    layer = RefLayer(RefConfig(dim=cfg["dim"], num_heads=cfg["heads"], rank=cfg["rank"], rotary=True))
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    x = torch.randn(1, tokens, cfg["dim"]).bfloat16().requires_grad_()
    dout = torch.randn(1, tokens, cfg["dim"]).bfloat16()

    def step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        y = layer(x, implementation="reference")
        y.backward(dout)
        return y

    return step


def cpu_layer_step(cfg, tokens, seed=0):
    """Returns (closure running one CPU layer forward+backward on `tokens` tokens, kind): the reference's own
    package when it is present, else the oracle port of it."""
    if reference_available():
        return reference_layer_step(cfg, tokens, seed), "reference"
    return port_layer_step(cfg, tokens, seed), "port"


def port_layer_step(cfg, tokens, seed=0):
    """One oracle layer forward+backward on `tokens` tokens."""
    from oracle import memsolve_oracle as O
    from memsolve_b200 import MemSolve, MemSolveConfig
    torch.manual_seed(seed)
    layer = MemSolve(MemSolveConfig(dim=cfg["dim"], num_heads=cfg["heads"], rank=cfg["rank"], rotary=True))
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    params = O.LayerParams(layer.w_bc.weight.detach().clone(), layer.w_o.weight.detach().clone(),
                           layer.core_base_raw.detach().clone(), layer.eta_raw.detach().clone(),
                           heads=cfg["heads"], rank=cfg["rank"])
    for t in params.tensors():
        t.requires_grad_()
    x = torch.randn(1, tokens, cfg["dim"]).bfloat16().requires_grad_()
    dout = torch.randn(1, tokens, cfg["dim"]).bfloat16()
    d = cfg["dim"] // cfg["heads"]
    cos, sin = O.rotary_tables(torch.arange(tokens)[None], head_dim=d, train_length=128, context_length=tokens)

    def step():
        for t in params.tensors():
            t.grad = None
        x.grad = None
        y = O.layer_forward(params, x, None, cos, sin)
        y.backward(dout)
        return y

    return step


def time_cpu(cfg, tokens, steps, warmup):
    """(seconds per step, kind) of the CPU layer on `tokens` tokens."""
    step, kind = cpu_layer_step(cfg, tokens)
    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return sum(times) / len(times), kind


CPU_KIND_TEXT = {"reference": "the reference's own pure-PyTorch CPU layer (layer(x, implementation=\"reference\"))",
                 "port": "oracle port of the reference's pure-PyTorch CPU layer"}


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all the host threads this process may use (torchrun presets OMP_NUM_THREADS=1 for its workers)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    full = cfg.get("local_tokens", cfg.get("global_tokens"))
    # bounded sample: pick the largest token count whose (steps+warmup) run stays near two minutes
    probe, _ = time_cpu(cfg, 2048, 1, 1)
    steps = min(args.steps, 10)          # the CPU arm needs no more repetitions than that for a stable mean
    warmup = min(args.warmup, 2)
    budget = 150.0 / max(1, steps + warmup)
    tokens = full
    while tokens > 2048 and probe * (tokens / 2048.0) > budget:
        tokens //= 2
    dt, kind = time_cpu(cfg, tokens, steps, warmup)
    value = tokens / dt
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if cfg["strong"] else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, cfg, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind,
                         "sample": f"{tokens} of {full} tokens per step, {CPU_KIND_TEXT[kind]}"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, cfg, world):
    if cfg["strong"]:
        glob = cfg["global_tokens"]
    else:
        glob = cfg["local_tokens"] * world
    return {"workload": f"MemSolve layer fwd+bwd, config {args.workload}: dim {cfg['dim']}, {cfg['heads']} heads, "
                        f"rank {cfg['rank']}, rotary, B=1, N={glob} tokens"
                        + (f" sequence-parallel over {world} GPUs" if world > 1 else ""),
            "global_tokens": glob, "tokens_per_gpu": glob // world, "recompute_readout": False,
            "parallelism": f"sp{world}", "l2": "working set per step exceeds the 126 MB L2 (inputs larger than L2)"}


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------
def time_kernels(layer, cfg, tokens, device, reps=10, warm=3, with_graph=True, batch=1, rotary=True):
    """Each mixer kernel alone, CUDA events on the launching stream, L2 flushed before each launch."""
    import ctypes
    from memsolve_b200.ball import cuda as C
    lib = C._LIB
    heads, rank, dim = cfg["heads"], cfg["rank"], cfg["dim"]
    d = dim // heads
    width = heads * rank + dim
    g = torch.Generator(device="cpu").manual_seed(1)
    proj = (torch.randn(batch, tokens, width, generator=g) * 0.5).bfloat16().to(device)
    dy = torch.randn(batch, tokens, dim, generator=g).bfloat16().to(device)
    pos = torch.arange(tokens, device=device)[None]
    from memsolve_b200.ball.rotary import rotary_position_factors
    cos = sin = None
    if rotary:
        cos, sin = rotary_position_factors(pos, head_dim=d, base=10000.0, train_length=128,
                                           context_length=tokens, scaling="yarn")
    base, raw = layer.core_base_raw.detach(), layer.eta_raw.detach()
    shape, dims = C._make_shape(proj, base, cos)
    tape = C._alloc_tape(dims, device)
    tc = tape.as_struct()
    ws = C._workspace(shape, device)
    dpad = lib.ms_padded_head_dim(d)
    mixed = torch.empty(batch, tokens, dim, device=device, dtype=torch.bfloat16)
    gg = torch.empty(batch, heads, 2, rank, rank, device=device, dtype=torch.bfloat16)
    cg = torch.empty(batch, heads, 2, rank, dpad, device=device, dtype=torch.bfloat16)
    dproj = torch.empty_like(proj)
    dbase = torch.empty_like(base)
    draw = torch.empty_like(raw)
    st = torch.cuda.current_stream(device).cuda_stream
    S = ctypes.byref(shape)
    T = ctypes.byref(tc)
    cos_p = cos.data_ptr() if rotary else None
    sin_p = sin.data_ptr() if rotary else None
    calls = {
        "core_forward": lambda: lib.ms_core_forward(S, base.data_ptr(), raw.data_ptr(), T, st),
        "stats_forward": lambda: lib.ms_stats_forward(S, proj.data_ptr(), cos_p, sin_p, None,
                                                      ws.data_ptr(), ws.numel(), None, st),
        "compact_forward": lambda: lib.ms_compact_forward(S, None, ws.data_ptr(), ws.numel(), None, T, st),
        "readout": lambda: lib.ms_readout(S, proj.data_ptr(), cos_p, sin_p, None, T,
                                          mixed.data_ptr(), st),
        "stats_backward": lambda: lib.ms_stats_backward(S, proj.data_ptr(), dy.data_ptr(), cos_p,
                                                        sin_p, None, ws.data_ptr(), ws.numel(), None, st),
        "compact_backward": lambda: lib.ms_compact_backward(S, None, ws.data_ptr(), ws.numel(), None, T,
                                                            base.data_ptr(), raw.data_ptr(), 1.0, gg.data_ptr(),
                                                            cg.data_ptr(), dbase.data_ptr(), draw.data_ptr(), st),
        "token_backward": lambda: lib.ms_token_backward(S, proj.data_ptr(), dy.data_ptr(), cos_p,
                                                        sin_p, None, T, gg.data_ptr(), cg.data_ptr(),
                                                        dproj.data_ptr(), st),
    }
    bpt = {  # algorithmic bytes per token (BF16): packed row = 2*width, mixed row = 2*dim
        "stats_forward": 2 * width, "readout": 2 * width + 2 * dim,
        "stats_backward": 2 * width + 2 * dim, "token_backward": 4 * width + 2 * dim,
    }
    # the whole mix core (ms_mix_forward + ms_mix_backward: six launches) as one CUDA graph, replayed
    # back to back; its tensors (projected, mixed, dy, dprojected: 250 MB at 32768 tokens) exceed L2
    def mix_core():
        assert lib.ms_mix_forward(S, proj.data_ptr(), base.data_ptr(), raw.data_ptr(), cos_p,
                                  sin_p, None, ws.data_ptr(), ws.numel(), T, mixed.data_ptr(),
                                  torch.cuda.current_stream(device).cuda_stream) == 0
        assert lib.ms_mix_backward(S, proj.data_ptr(), dy.data_ptr(), base.data_ptr(), raw.data_ptr(),
                                   cos_p, sin_p, None, ws.data_ptr(), ws.numel(), T,
                                   gg.data_ptr(), cg.data_ptr(), dproj.data_ptr(), dbase.data_ptr(),
                                   draw.data_ptr(), torch.cuda.current_stream(device).cuda_stream) == 0

    mix_core_graph_s = 0.0
    if with_graph:
        mix_core()
        torch.cuda.synchronize(device)
        core_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(core_graph):
            mix_core()
        for _ in range(3):
            core_graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            core_graph.replay()
        e1.record()
        e1.synchronize()
        mix_core_graph_s = e0.elapsed_time(e1) * 1e-3 / 20

    flush = torch.empty(256 * 1024 * 1024, device=device, dtype=torch.uint8)
    out = {"mix_core_graph": {"s": mix_core_graph_s, "bytes": 0}}
    for name, fn in calls.items():
        for _ in range(warm):
            assert fn() == 0
        ts = []
        for _ in range(reps):
            # flush L2: write 256 MB, then read it back so that no dirty lines are left to be written out
            # while the timed kernel runs
            flush.zero_()
            flush.view(torch.int64).sum()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            assert fn() == 0
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3)
        out[name] = {"s": sum(ts) / len(ts), "bytes": bpt.get(name, 0) * tokens * batch}
    return out


TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.md")


def _ncu_traffic(workload, kernel, tokens):
    """DRAM bytes (read + write) of one launch of `kernel`, from the ncu captures summarised in
    profiles/dram_traffic_per_launch.md (lines `workload kernel tokens bytes`); the traffic of these streaming
    kernels grows in proportion to the tokens of a launch.  None when the file has no line for the kernel."""
    try:
        with open(TRAFFIC_FILE) as f:
            for line in f:
                parts = line.split()
                if len(parts) >= 4 and parts[0] == workload and parts[1] == kernel:
                    return float(parts[3]) * tokens / float(parts[2])
    except (OSError, ValueError):
        pass
    return None


def time_one_gpu(cfg, device, steps=10):
    """tokens/s of the whole `cfg` workload (all its tokens) on one GPU without sequence parallelism: CUDA-graph
    replays, median of three blocks."""
    tokens = cfg.get("global_tokens", cfg.get("local_tokens"))
    layer = build_layer(cfg, device)
    gen = torch.Generator().manual_seed(99)
    x = torch.randn(1, tokens, cfg["dim"], generator=gen).bfloat16().to(device).requires_grad_()
    dout = torch.randn(1, tokens, cfg["dim"], generator=gen).bfloat16().to(device)

    def step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        layer(x, implementation="cuda").backward(dout)

    for _ in range(3):
        step()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        graph.replay()
    blocks = []
    for _ in range(3):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        e1.synchronize()
        blocks.append(e0.elapsed_time(e1) * 1e-3 / steps)
    dt = statistics.median(blocks)
    graph.reset()
    del graph, x, dout, layer
    torch.cuda.empty_cache()
    return {"value": tokens / dt, "unit": "tokens/s", "ms_per_step": dt * 1e3, "n_gpus": 1,
            "note": "same workload on rank 0's GPU alone, measured in this run before the ranks join"}


def run_sweep(args):
    """One line per sequence length 128 ... 32768 (the reference benchmark's sweep, benchmarks/benchmark_ball.py:
    20-66): layer forward+backward as CUDA-graph replays, and the mix core (fast_mix forward + backward, six
    launches) alone with its fraction of the HBM roofline."""
    from memsolve_b200.ball import cuda as C
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    C.load(device=device)
    cfg = CONFIGS["c3"]
    hbm, _tc, which = _peaks()
    width = cfg["heads"] * cfg["rank"] + cfg["dim"]
    rows = []
    tokens = 128
    while tokens <= 32768:
        one = time_one_gpu(dict(cfg, local_tokens=tokens), device, steps=50)
        kern = time_kernels(build_layer(cfg, device), cfg, tokens, device, reps=3, warm=2, with_graph=True)
        core_s = kern["mix_core_graph"]["s"]
        core_bytes = 2 * (5 * width + 3 * cfg["dim"]) * tokens
        rows.append({"tokens": tokens, "layer_us": round(one["ms_per_step"] * 1e3, 2),
                     "layer_tokens_per_s": one["value"], "mix_core_us": round(core_s * 1e6, 2),
                     "mix_core_tokens_per_s": tokens / core_s,
                     "mix_core_frac_of_hbm": core_bytes / core_s / 1e9 / hbm})
        tokens *= 2
    print(json.dumps({"metric": "layer_fwd_bwd_tokens_per_s", "unit": "tokens/s", "sweep": rows, "dtype": "bf16",
                      "data": "synthetic", "peak_source": f"of {which}", "timing": "cuda_graph_replay",
                      "config": {"workload": "MemSolve layer fwd+bwd, dim 768, 12 heads, rank 32, rotary, B=1, "
                                             "N = 128 ... 32768"}}))


def run_ours(args, cfg):
    import torch.distributed as dist
    from memsolve_b200.ball import cuda as C
    from memsolve_b200.integrations.distributed import SequenceParallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    C.load(device=device)

    tokens = cfg["global_tokens"] // world if cfg["strong"] else cfg["local_tokens"]
    global_tokens = tokens * world
    layer = build_layer(cfg, device)
    gen = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(1, tokens, cfg["dim"], generator=gen).bfloat16().pin_memory()
    d_host = torch.randn(1, tokens, cfg["dim"], generator=gen).bfloat16().pin_memory()
    x = x_host.to(device).requires_grad_()
    dout = d_host.to(device)
    sp = counts = None
    peer_path = False
    one_gpu = None
    if world > 1 and cfg["strong"] and rank == 0 and not args.no_one_gpu:
        # the same strong-scaling workload on this GPU alone (no sequence parallelism), as the reference point of
        # the multi-GPU figure: measured before the ranks start working together
        one_gpu = time_one_gpu(cfg, device)
    if world > 1:
        sp = SequenceParallel.create(tokens)
        counts = sp.valid_counts(None, batch_size=1, device=device)
        sp.overlap_gradient_sum(layer)   # parameter-gradient SUMs overlap the rest of the backward pass
        # statistics and large gradients summed by kernels over NVLink peer memory (verified against the NCCL
        # path on 2, 4 and 8 GPUs); MEMSOLVE_BENCH_PEER_EXCHANGE=0 selects NCCL for both instead
        if os.environ.get("MEMSOLVE_BENCH_PEER_EXCHANGE", "") != "0":
            sp.use_peer_exchange()
            # both kinds of exchange areas sized for this layer (largest gradient included) before any capture
            sp.prepare_peer_exchange(layer)
            peer_path = True

    def step(xin, grad_out):
        layer.zero_grad(set_to_none=True)
        xin.grad = None
        if sp is None:
            y = layer(xin, implementation="cuda")
        else:
            y = layer(xin, implementation="cuda", sequence_parallel=sp, valid_counts=counts)
        y.backward(grad_out)
        if sp is not None:
            sp.reduce_gradients_(layer)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, finish=None, blocks=1):
        """Median over `blocks` blocks of `steps` calls; every block is bracketed by a barrier and a device
        synchronisation, timed with CUDA events on this rank and reduced with MAX over the ranks."""
        totals = []
        for _ in range(blocks):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            if finish is not None:
                finish()
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            totals.append(float(t.item()))
        return statistics.median(totals)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(x, dout)
    # The reference's own benchmark times CUDA-graph replays of the step; do the same here
    # (the step makes no host decisions, allocates through torch's graph pool and launches only
    # on the current stream).  Eager timing is kept beside it.
    graph = None
    if not args.eager:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(x, dout)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_y = step(x, dout)
            graph_dx = x.grad
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as error:  # noqa: BLE001 - report and fall back to eager timing
            print(f"graph capture failed, timing eagerly: {error}", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    eager_total = timed(lambda: step(x, dout), args.steps)
    total = timed(graph.replay, args.steps, blocks=args.blocks) if graph is not None else \
        timed(lambda: step(x, dout), args.steps, blocks=args.blocks)
    # nvidia-smi samples every 100 ms and the timed region lasts milliseconds: keep the same step
    # running (untimed) for about a second so that the clock record covers this load
    t_end = time.perf_counter() + 1.2
    while time.perf_counter() < t_end:
        for _ in range(20):
            graph.replay() if graph is not None else step(x, dout)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed steps + 1.2 s of the same step"

    # end to end: inputs start in pinned host memory every step; the layer output and the input gradient go back
    # to pinned host memory every step
    x_dev = torch.empty_like(x_host, device=device).requires_grad_()
    d_dev = torch.empty_like(d_host, device=device)
    y_host = torch.empty_like(x_host).pin_memory()
    dx_host = torch.empty_like(x_host).pin_memory()
    y_stage = torch.empty_like(x_host, device=device)
    dx_stage = torch.empty_like(x_host, device=device)
    back_stream = torch.cuda.Stream(device)
    results_staged = torch.cuda.Event()
    results_copied = torch.cuda.Event()
    results_copied.record()

    # The copies of step k+1 run on a copy stream into staging buffers while step k computes (what a
    # training loop with a prefetching loader does); the step then takes its inputs from the staging
    # buffers with a device-to-device copy.  Every step still moves its own inputs host -> device.
    copy_stream = torch.cuda.Stream(device)
    x_stage = torch.empty_like(x_host, device=device)
    d_stage = torch.empty_like(d_host, device=device)
    staged = torch.cuda.Event()
    consumed = torch.cuda.Event()
    consumed.record()

    def prefetch():
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed)          # the staging buffers are free again
            x_stage.copy_(x_host, non_blocking=True)
            d_stage.copy_(d_host, non_blocking=True)
            staged.record(copy_stream)

    def e2e_step():
        main = torch.cuda.current_stream()
        main.wait_event(staged)
        with torch.no_grad():
            if graph is not None:
                # the captured step reads its inputs from the static device tensors x and dout
                x.copy_(x_stage)
                dout.copy_(d_stage)
            else:
                x_dev.copy_(x_stage)
                d_dev.copy_(d_stage)
        consumed.record(main)
        prefetch()                                    # inputs of the next step
        if graph is not None:
            graph.replay()
            y, dx = graph_y, graph_dx
        else:
            y = step(x_dev, d_dev)
            dx = x_dev.grad
        with torch.no_grad():
            # results leave through staging buffers on a copy stream of their own (PCIe is full duplex), while
            # the next step already computes
            main.wait_event(results_copied)           # the staging buffers of the step before have been read
            y_stage.copy_(y)
            dx_stage.copy_(dx)
            results_staged.record(main)
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(results_staged)
                y_host.copy_(y_stage, non_blocking=True)
                dx_host.copy_(dx_stage, non_blocking=True)
                results_copied.record(back_stream)

    prefetch()
    for _ in range(2):
        e2e_step()
    # the timed region ends after the copy stream has drained too (steps + 1 input copies for `steps` steps)
    def drain():
        torch.cuda.current_stream().wait_stream(copy_stream)
        torch.cuda.current_stream().wait_stream(back_stream)

    e2e_total = timed(e2e_step, args.steps, finish=drain, blocks=min(args.blocks, 3))

    timing_mode = "cuda_graph_replay" if graph is not None else "eager"
    # a captured graph keeps references to the NCCL communicator: release it before the group goes away
    if graph is not None:
        torch.cuda.synchronize()
        graph.reset()
        graph = None
    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm, tc, which = _peaks()
    kern = time_kernels(layer, cfg, tokens, device)
    mix_core_graph_s = kern.pop("mix_core_graph")["s"]
    name = max((k for k in kern if kern[k]["bytes"]), key=lambda k: kern[k]["s"])
    achieved = kern[name]["bytes"] / kern[name]["s"] / 1e9
    mixer_time = sum(v["s"] for v in kern.values())
    width = cfg["heads"] * cfg["rank"] + cfg["dim"]
    core_bytes = 2 * (5 * width + 3 * cfg["dim"]) * tokens
    dt = total / args.steps
    value = global_tokens / dt
    layer_bytes_per_tok = 2 * (5 * width + 3 * cfg["dim"]) + 2 * (5 * cfg["dim"] + 2 * width + 3 * cfg["dim"])
    layer_flops_per_tok = 6 * cfg["dim"] * (width + cfg["dim"])
    tok_rate_gpu = tokens / dt
    bound = max(layer_bytes_per_tok * tok_rate_gpu / (hbm * 1e9), layer_flops_per_tok * tok_rate_gpu / (tc * 1e12))
    line = {
        "metric": "layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if cfg["strong"] else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, cfg, world), "clocks": clocks,
        "e2e": {"value": global_tokens / (e2e_total / args.steps), "unit": "tokens/s",
                "h2d_bytes_per_step": (x_host.numel() + d_host.numel()) * 2 * world,
                "d2h_bytes_per_step": (y_host.numel() + dx_host.numel()) * 2 * world},
        # own kernels per step: statistics (+ per-head core), compact, readout, and their three adjoints;
        # the sequence-parallel path adds a pack kernel per direction (the buffer that is all-reduced)
        # statistics (+ per-head core), compact, readout and their three adjoints; sequence parallel with the
        # peer-memory exchange adds one exchange kernel per direction and one SUM kernel per weight matrix
        # (on one GPU rank 64 adds a launch per direction that reduces the statistics' partials)
        "gpu_launches": ((8 if cfg["rank"] == 64 else 6) if world == 1 else (10 if peer_path else 8))
                        * args.steps * args.blocks,
        "timing": f"{timing_mode}, median of {args.blocks} blocks of {args.steps} steps",
        "eager_ms_per_step": eager_total / args.steps * 1e3,
        "collective": None if world == 1 else (
            "statistics: one kernel over NVLink peer memory per direction; weight gradients: peer-memory SUM kernel "
            "overlapped with backward; small gradients: NCCL all-reduce" if peer_path else
            "NCCL all-reduce of the packed statistics per direction; NCCL all-reduce of the gradients overlapped "
            "with backward"),
        "one_gpu_same_workload": one_gpu,
        "roofline": {
            "bound": "hbm", "kernel": name, "achieved": achieved, "peak": hbm, "unit": "GB/s",
            "frac": achieved / hbm, "traffic": _ncu_traffic(args.workload, name, tokens),
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                              "(profiles/dram_traffic_per_launch.md names the capture), scaled by tokens",
            "peak_source": f"of {which}",
            "per_kernel_us": {k: round(v["s"] * 1e6, 2) for k, v in kern.items()},
            "per_kernel_gbs": {k: round(v["bytes"] / v["s"] / 1e9, 1) for k, v in kern.items() if v["bytes"]},
            # fast_mix forward + backward: CUDA-graph replays of the six launches back to back, and the sum of
            # the launches timed alone after an L2 flush
            "mix_core": {"bytes_per_token": 2 * (5 * width + 3 * cfg["dim"]),
                         "us": round(mix_core_graph_s * 1e6, 2),
                         "achieved": core_bytes / mix_core_graph_s / 1e9,
                         "frac": core_bytes / mix_core_graph_s / 1e9 / hbm,
                         "isolated_sum_us": round(mixer_time * 1e6, 2),
                         "isolated_frac": core_bytes / mixer_time / 1e9 / hbm},
            "layer": {"frac_of_max_hbm_tensor_bound": bound},
        },
    }
    if world == 1 and not args.no_cpu:
        try:
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        except (AttributeError, RuntimeError):
            pass
        n_cpu = tokens   # the whole workload: about half a second per step on the box's cores
        t_cpu, kind = time_cpu(cfg, n_cpu, 3, 1)
        line["cpu_baseline"] = {"value": n_cpu / t_cpu, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                "kind": kind,
                                "sample": f"all {n_cpu} tokens of the workload, 3 timed steps after 1 warm-up, "
                                          f"{CPU_KIND_TEXT[kind]} forward+backward"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# encoder scaffolds (ViT-Small-shaped "c2", BERT-base-shaped "c4"): many short sequences, one GPU
# ---------------------------------------------------------------------------------------
SCAFFOLDS = {
    "c2": dict(kind="vision", batch=256, tokens=197, dim=384, heads=6, rank=32, depth=12),
    "c4": dict(kind="text", batch=64, tokens=128, dim=768, heads=12, rank=32, depth=12),
}


def run_scaffold(args):
    """Forward + backward of the ViT-Small-shaped / BERT-base-shaped scaffold under BF16 autocast, and one of
    its MemSolve layers alone at the same shape (CUDA-graph replays), on synthetic inputs."""
    from memsolve_b200.ball import cuda as C
    from memsolve_b200 import MemSolve, MemSolveConfig
    from memsolve_b200.integrations.scaffolds import TextScaffold, VisionScaffold
    spec = SCAFFOLDS[args.workload]
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    C.load(device=device)
    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(1)
    if spec["kind"] == "vision":
        model = VisionScaffold().to(device)
        images = torch.randn(spec["batch"], 3, 224, 224, generator=gen).to(device)
        labels = torch.randint(0, 1000, (spec["batch"],), generator=gen).to(device)

        def loss_fn():
            return torch.nn.functional.cross_entropy(model(images).float(), labels)
        units, unit = spec["batch"], "images/s"
    else:
        model = TextScaffold().to(device)
        ids = torch.randint(0, 30522, (spec["batch"], spec["tokens"]), generator=gen)
        chosen = torch.rand(ids.shape, generator=gen) < 0.15
        targets = torch.where(chosen, ids, torch.full_like(ids, -100)).to(device)
        ids = torch.where(chosen, torch.full_like(ids, 103), ids).to(device)

        positions = (targets.reshape(-1) != -100).nonzero().squeeze(1)
        wanted = targets.reshape(-1)[positions]

        def loss_fn():
            return model.masked_lm_loss(ids, positions, wanted)
        units, unit = spec["batch"] * spec["tokens"], "tokens/s"

    def step():
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = loss_fn()
        loss.backward()
        return loss

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / steps

    warm = max(args.warmup, 3)
    for _ in range(warm):
        loss = step()
    assert torch.isfinite(loss).item()
    sampler = ClockSampler(0)
    sampler.start()
    dt = timed(step, args.steps)
    clocks = sampler.stop()

    # one MemSolve layer of the scaffold alone: forward + backward, CUDA-graph replays
    layer = MemSolve(MemSolveConfig(dim=spec["dim"], num_heads=spec["heads"], rank=spec["rank"], rotary=False,
                                    recompute_readout=False)).to(device)
    with torch.no_grad():
        layer.core_base_raw.normal_(std=0.1)
    x = torch.randn(spec["batch"], spec["tokens"], spec["dim"], device=device).bfloat16().requires_grad_()
    dout = torch.randn_like(x)

    def layer_step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        layer(x, implementation="cuda").backward(dout)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            layer_step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer_step()
    for _ in range(3):
        graph.replay()
    layer_dt = timed(graph.replay, 50)

    # the same step as one CUDA graph (static shapes; gradients are written into the same tensors each replay)
    graph_dt = None
    del loss   # no autograd graph of an eager step may be alive while the step is captured
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            step()
        for _ in range(3):
            step_graph.replay()
        graph_dt = timed(step_graph.replay, args.steps)
    except Exception as error:   # capture is an extra; the eager figure above stands on its own
        print(f"graph capture of the scaffold step failed: {error}", file=sys.stderr)
        torch.cuda.synchronize()

    width = spec["heads"] * spec["rank"] + spec["dim"]
    n_tok = spec["batch"] * spec["tokens"]
    hbm, _tc, which = _peaks()
    print(json.dumps({
        "metric": f"scaffold_fwd_bwd_{unit.split('/')[0]}_per_s", "value": units / dt, "unit": unit, "n_gpus": 1,
        "steps": args.steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "timing": "eager, BF16 autocast",
        "config": {"workload": f"{args.workload}: {spec['kind']} scaffold, {spec['depth']} layers, "
                               f"dim {spec['dim']}, {spec['heads']} heads, rank {spec['rank']}, batch {spec['batch']}"
                               f" x {spec['tokens']} tokens", "parallelism": "sp1"},
        "clocks": clocks, "gpu_launches": 6 * spec["depth"] * args.steps,
        "graph_replay": None if graph_dt is None else {"ms_per_step": graph_dt * 1e3, "value": units / graph_dt,
                                                         "unit": unit},
        "layer_alone": {"us": round(layer_dt * 1e6, 1), "tokens_per_s": n_tok / layer_dt,
                        "systems": spec["batch"] * spec["heads"],
                        "frac_of_layer_hbm_bound": 2 * (5 * width + 3 * spec["dim"] + 8 * spec["dim"] + 2 * width)
                        * n_tok / layer_dt / 1e9 / hbm, "peak_source": f"of {which}"},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=7, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=tuple(CONFIGS) + tuple(SCAFFOLDS), default=None,
                    help="default: c3 on one GPU, c5 (strong scaling) on several")
    ap.add_argument("--sweep", action="store_true", help="sequence lengths 128 ... 32768 on one GPU")
    ap.add_argument("--no-one-gpu", action="store_true",
                    help="skip the one-GPU measurement of the same workload in a multi-GPU strong-scaling run")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--kernels-only", action="store_true",
                    help="launch each mixer kernel alone (--reps times) and print their timings; used for ncu")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--kernel-warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=0, help="with --kernels-only: tokens per launch instead of the workload's")
    args = ap.parse_args()
    if args.workload is None:
        args.workload = "c3" if args.gpus <= 1 else "c5"
    if args.sweep:
        run_sweep(args)
        return
    if args.workload in SCAFFOLDS:
        if args.impl != "ours" or args.gpus != 1:
            raise SystemExit("the scaffold workloads run the CUDA arm on one GPU")
        if args.kernels_only:
            from memsolve_b200.ball import cuda as C
            spec = SCAFFOLDS[args.workload]
            device = torch.device("cuda", 0)
            torch.cuda.set_device(device)
            C.load(device=device)
            cfg = dict(dim=spec["dim"], heads=spec["heads"], rank=spec["rank"])
            kern = time_kernels(build_layer(cfg, device), cfg, spec["tokens"], device, reps=args.reps,
                                warm=args.kernel_warmup, with_graph=args.reps > 1, batch=spec["batch"], rotary=False)
            print(json.dumps({k: {"us": round(v["s"] * 1e6, 2), "gbs": round(v["bytes"] / v["s"] / 1e9, 1)}
                              for k, v in kern.items() if v["s"] > 0}))
            return
        run_scaffold(args)
        return
    cfg = CONFIGS[args.workload]
    if args.kernels_only:
        from memsolve_b200.ball import cuda as C
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        C.load(device=device)
        tokens = cfg["global_tokens"] // args.gpus if cfg["strong"] else cfg["local_tokens"]
        if args.tokens > 0:
            tokens = args.tokens
        kern = time_kernels(build_layer(cfg, device), cfg, tokens, device, reps=args.reps, warm=args.kernel_warmup,
                            with_graph=args.reps > 1)
        print(json.dumps({k: {"us": round(v["s"] * 1e6, 2), "gbs": round(v["bytes"] / v["s"] / 1e9, 1)}
                          for k, v in kern.items() if v["s"] > 0}))
        return
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
