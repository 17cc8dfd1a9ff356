"""Build the sm_100a shared library in-tree with nvcc (no torch involved).

    python -m nanoserve_b200.build            # build if sources are newer than the library
    python -m nanoserve_b200.build --force
    python -m nanoserve_b200.build --debug-hooks   # a second library with the profiling hooks (not loaded by default)

The library is one C-ABI .so (include/nanoserve_b200.h); the Python package loads it with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libnanoserve_b200.so"
SOURCES = ["c_api.cu", "fused_ops.cu", "attn_plan.cu", "attn_decode.cu", "attn_decode_static.cu", "attn_prefill_mma.cu", "attn_prefill_tc.cu", "attn_simple.cu",
           "metadata.cu", "sampling.cu", "skinny_gemm.cu", "thin_gemm.cu", "stream_gemm.cu", "umma_gemm.cu", "tp_allreduce.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "nanoserve_b200.h"]
    return any(p.stat().st_mtime > built for p in deps)


DEBUG_LIB_PATH = LIB_DIR / "libnanoserve_b200_dbg.so"


def build(force: bool = False, verbose: bool = False, debug_hooks: bool = False) -> Path:
    """debug_hooks=True builds lib/libnanoserve_b200_dbg.so with -DNS_DEBUG_HOOKS: the same library plus the profiling
    entry points (ns_debug_*: in-kernel time stamps) that the shipping library does not export. NS_DEBUG_LIB=1 makes
    the Python binding load it."""
    if debug_hooks:
        return _build(DEBUG_LIB_PATH, PKG / "build_dbg", ["-DNS_DEBUG_HOOKS"], verbose)
    if not force and not needs_build():
        return LIB_PATH
    return _build(LIB_PATH, PKG / "build", [], verbose)


def _build(lib_path: Path, obj_dir: Path, extra_flags: list, verbose: bool) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    procs = []
    obj_dir.mkdir(exist_ok=True)
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")] + extra_flags
    for src in SOURCES:
        obj = obj_dir / (src[:-3] + ".o")
        cmd = [_nvcc(), *flags, "-Xcompiler", "-fPIC", "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src} ---\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = lib_path.with_suffix(".so.tmp")
    subprocess.run([_nvcc(), "-shared", "-o", str(tmp), *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"], check=True)
    os.replace(tmp, lib_path)
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_hooks="--debug-hooks" in sys.argv)
    print(path)
