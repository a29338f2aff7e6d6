"""CPU-side checks: configuration, module contract, loader errors, exported C symbols."""
from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from memsolve_b200 import CoreMode, MemSolve, MemSolveConfig
from memsolve_b200.ball import cuda
from memsolve_b200.ball.rotary import axial_rotary_position_factors, rotary_position_factors
from oracle import memsolve_oracle as O


def test_config_validation_matches_reference_rules():
    cfg = MemSolveConfig(dim=384, num_heads=6, rank=32)
    assert cfg.head_dim == 64 and cfg.core_mode is CoreMode.EQUILIBRIUM and cfg.recompute_readout == "auto"
    assert MemSolveConfig(dim=8, num_heads=2, core_mode="complement").core_mode is CoreMode.COMPLEMENT
    with pytest.raises(ValueError, match="divisible"):
        MemSolveConfig(dim=10, num_heads=3)
    with pytest.raises(TypeError, match="must be an integer"):
        MemSolveConfig(dim=8.0, num_heads=2)
    with pytest.raises(ValueError, match="core_mode"):
        MemSolveConfig(dim=8, num_heads=2, core_mode="other")
    with pytest.raises(ValueError, match="even head_dim"):
        MemSolveConfig(dim=6, num_heads=2, rotary=True)
    with pytest.raises(ValueError, match="recompute_readout"):
        MemSolveConfig(dim=8, num_heads=2, recompute_readout="never")
    with pytest.raises(TypeError, match="recompute_readout"):
        MemSolveConfig(dim=8, num_heads=2, recompute_readout=1)
    with pytest.raises(ValueError, match="rotary_scaling"):
        MemSolveConfig(dim=8, num_heads=2, rotary_scaling="ntk")


def test_module_parameters_and_checkpoint_contract():
    layer = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=16, rotary=True))
    assert layer.w_bc.weight.shape == (2 * 16 + 32, 32) and layer.w_o.weight.shape == (32, 32)
    assert layer.core_base_raw.shape == (2, 16, 16) and torch.count_nonzero(layer.core_base_raw) == 0
    assert torch.allclose(layer.complement(), torch.full((2,), 0.9), atol=1e-6)
    state = layer.state_dict()
    extra = state["_extra_state"]
    assert extra["version"] == 26 and extra["rotary"]["yarn_beta"] == [32, 1]
    other = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=16, rotary=True))
    other.load_state_dict(state)
    mismatched = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=16, rotary=False))
    with pytest.raises(RuntimeError, match="incompatible MemSolve checkpoint contract"):
        mismatched.load_state_dict(state)
    del state["_extra_state"]
    with pytest.raises(RuntimeError, match="missing its configuration contract"):
        other.load_state_dict(state, strict=False)
    comp = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=16, core_mode="complement"))
    assert comp.core_base_raw is None
    layer.recompute_readout = True
    assert layer.recompute_readout is True
    with pytest.raises(ValueError):
        layer.recompute_readout = "sometimes"


def test_forward_dispatch_errors_on_cpu():
    layer = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=16))
    x = torch.randn(1, 5, 32)
    with pytest.raises(ValueError, match="requires x to be a CUDA tensor"):
        layer(x, implementation="cuda")
    with pytest.raises(ValueError, match="implementation must be"):
        layer(x, implementation="triton")
    with pytest.raises(RuntimeError, match="ships only the sm_100a CUDA path"):
        layer(x)
    with pytest.raises(ValueError, match=r"x must have shape \[B, N, 32\]"):
        layer(torch.randn(1, 5, 31), implementation="cuda")
    with pytest.raises(ValueError, match="rotary=True"):
        layer(x, implementation="cuda", rotary_factors=(x, x))
    bad = MemSolve(MemSolveConfig(dim=32, num_heads=2, rank=8))
    with pytest.raises(ValueError, match="rank in"):
        bad._forward_cuda(x, None)


def test_rotary_tables_match_oracle():
    pos = torch.arange(3, 500, 11)[None]
    for kw in (dict(head_dim=64, base=10000.0, train_length=128, context_length=32768, scaling="yarn"),
               dict(head_dim=24, base=500.0, train_length=64, context_length=torch.tensor([40, 400]), scaling="yarn"),
               dict(head_dim=8, base=10000.0, train_length=128, context_length=77, scaling="none")):
        c, s = rotary_position_factors(pos, **kw)
        oc, os_ = O.rotary_tables(pos, **kw)
        assert torch.equal(c, oc) and torch.equal(s, os_)
    coords = torch.stack(torch.meshgrid(torch.arange(4), torch.arange(5), indexing="ij"), -1).reshape(1, 20, 2)
    c, s = axial_rotary_position_factors(coords, head_dim=16)
    assert c.shape == (1, 20, 8) and torch.allclose(c * c + s * s, torch.ones_like(c))
    with pytest.raises(ValueError, match="divisible by four"):
        axial_rotary_position_factors(coords, head_dim=6)


def test_loader_refuses_without_device_and_bad_names(tmp_path, monkeypatch):
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="requires an available CUDA device"):
            cuda.load()
    if not cuda.is_available():
        with pytest.raises(RuntimeError, match="extension is not loaded"):
            cuda.require_available()
        with pytest.raises(RuntimeError, match="extension is not loaded"):
            cuda.fast_mix(torch.zeros(1, 4, 48), torch.zeros(2, 16, 16), torch.zeros(2))
    with pytest.raises(RuntimeError, match="must be named"):
        cuda._resolve_library_path(tmp_path / "libother.so")
    with pytest.raises(RuntimeError, match="is not built"):
        cuda._resolve_library_path(tmp_path / "memsolve_equilibrium_sm100.so")
    monkeypatch.setenv("MEMSOLVE_CUDA_LIBRARY", str(tmp_path / "memsolve_equilibrium.so"))
    with pytest.raises(RuntimeError, match="is not built"):
        cuda._resolve_library_path(None)


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "memsolve_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ms_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    """The built library loads without a GPU and exports exactly what the header declares."""
    path = cuda.default_library_path()
    if not path.exists():
        from memsolve_b200.csrc.build import build
        build()
    lib = cuda._open_library(path)
    declared = _header_symbols()
    assert declared == sorted(cuda.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.ms_abi_version() == 1
    buf = (ctypes.c_int32 * 4)()
    assert lib.ms_supported_architectures(buf, 4) == 1 and buf[0] == 100
    assert lib.ms_padded_head_dim(17) == 24 and lib.ms_padded_head_dim(64) == 64
    assert b"rank" in lib.ms_status_string(2)
    shape = cuda._Shape(1, 32768, 12, 32, 64, 0, 1, 0)
    assert lib.ms_packed_stats_floats(ctypes.byref(shape), 0) == 12 * (32 * 32 + 32 * 64)
    assert lib.ms_packed_stats_floats(ctypes.byref(shape), 1) == 12 * (32 * 64 + 1)
    assert lib.ms_workspace_bytes(ctypes.byref(shape)) > 0
    bad = cuda._Shape(1, 10, 2, 20, 8, 0, 0, 0)
    assert lib.ms_workspace_bytes(ctypes.byref(bad)) == 0


def test_stale_contract_version_is_rejected():
    class Fake:
        @staticmethod
        def ms_abi_version():
            return 0
    with pytest.raises(RuntimeError, match="native contract version"):
        cuda._check_native_contract(Fake())


def test_scaffolds_construct_and_refuse_cpu_input():
    """The encoder scaffolds build without a GPU; their mixer has no CPU path."""
    from memsolve_b200.integrations.scaffolds import TextScaffold, VisionScaffold
    vision = VisionScaffold(depth=1)
    assert vision.tokens == 197 and vision.blocks[0].attn.mixer.config.rank == 32
    text = TextScaffold(depth=1, vocab_size=100)
    assert text.blocks[0].attention.mixer.w_bc.weight.shape == (12 * 32 + 768, 768)
    with pytest.raises(ValueError, match="requires x to be a CUDA tensor"):
        text(torch.zeros(1, 8, dtype=torch.long))
    with pytest.raises(ValueError, match="multiple of patch_size"):
        VisionScaffold(image_size=100)
