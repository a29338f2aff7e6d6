"""Build memsolve_equilibrium_sm100.so from the .cu files beside this script.

    python -m memsolve_b200.csrc.build        (or: python memsolve_b200/csrc/build.py)

Each translation unit is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``)
and linked into ``memsolve_b200/lib/memsolve_equilibrium_sm100.so``.  The ptxas resource report
(registers, spills, shared memory per kernel) is kept in ``memsolve_b200/lib/ptxas.log``.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(HERE), "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_NAME = "memsolve_equilibrium_sm100.so"
SOURCES = ["ms_api.cu", "ms_stats.cu", "ms_compact.cu", "ms_token.cu", "ms_readout_tma.cu", "ms_token_bwd_tma.cu",
           "ms_stats_tma.cu", "ms_exchange.cu", "ms_token_bwd_tc.cu", "ms_readout_tc.cu", "ms_stats_tc.cu", "ms_linear_tc.cu",
           "ms_short.cu", "ms_linear_wgrad_tc.cu"]
HEADERS = ["ms_common.cuh", "ms_core.cuh", "ms_tma.cuh", "ms_frag.cuh", "ms_tc.cuh", os.path.join("..", "..", "include", "memsolve_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _digest(paths) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _compile(src: str, force: bool) -> tuple[str, str]:
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    stamp = obj + ".sha"
    deps = [os.path.join(HERE, src)] + [os.path.join(HERE, h) for h in HEADERS]
    digest = _digest(deps)
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return obj, proc.stderr


def library_path() -> str:
    return os.path.join(LIB_DIR, LIB_NAME)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda s: _compile(s, force), SOURCES))
    objs = [r[0] for r in results]
    logs = [r[1] for r in results if r[1]]
    out = library_path()
    stale = not os.path.exists(out) or any(os.path.getmtime(o) > os.path.getmtime(out) for o in objs)
    if logs or stale:
        cmd = [_nvcc(), "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        if logs:
            with open(os.path.join(LIB_DIR, "ptxas.log"), "w") as f:
                f.write("\n".join(logs))
    if verbose:
        print(out)
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
