"""The C-ABI library loads and exports every entry point include/nanoserve_b200.h declares (no compute calls)."""
import ctypes
import re
from pathlib import Path

from nanoserve_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "nanoserve_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ns_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ["ns_ragged_paged_attn", "ns_paged_attn_decode", "ns_rope_qkv_kvwrite", "ns_add_rmsnorm", "ns_silu_mul",
                 "ns_build_step_metadata", "ns_attn_plan", "ns_last_error"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but missing from the library"


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert _lib.load().ns_version() >= 100


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from nanoserve_b200.kernels.fused import silu_mul
    with pytest.raises(_lib.NanoserveB200Error):
        silu_mul(torch.zeros(2, 16))


def test_decode_gemm_entry_points_validate_before_touching_the_device():
    """Shape, alignment and epilogue checks of the decode-sized GEMMs come before any CUDA call: they return a status
    and leave a message, with or without a GPU (the pointers below are never dereferenced)."""
    lib, P = _lib.load(), ctypes.c_void_p
    msg = lambda: lib.ns_last_error().decode()
    x, w, out = P(256), P(512), P(1024)
    nul = None
    INVALID, UNSUPPORTED = 1, 2
    assert lib.ns_thin_gemm(x, w, nul, out, 0, 1152, 896, 0, nul, nul, nul, nul, nul, 0, 0, nul) == 0          # empty step
    assert lib.ns_thin_gemm(x, w, nul, out, 65, 896, 896, 0, nul, nul, nul, nul, nul, 0, 0, nul) == UNSUPPORTED and "65 token rows" in msg()
    assert lib.ns_thin_gemm(x, w, nul, out, 8, 896, 900, 0, nul, nul, nul, nul, nul, 0, 0, nul) == UNSUPPORTED and "multiple of 128" in msg()
    assert lib.ns_thin_gemm(x, w, nul, out, 64, 4608, 3584, 0, nul, nul, nul, nul, nul, 0, 0, nul) == UNSUPPORTED and "shared memory" in msg()
    assert lib.ns_thin_gemm(x, w, nul, out, 8, 1152, 896, 2, nul, nul, nul, nul, nul, 14, 2, nul) == INVALID and "RoPE epilogue needs" in msg()
    assert lib.ns_thin_gemm(x, w, nul, out, 8, 1160, 896, 2, x, x, x, x, x, 14, 2, nul) == INVALID and "head_dim" in msg()
    assert lib.ns_thin_gemm(x, w, nul, out, 8, 1152, 896, 7, nul, nul, nul, nul, nul, 14, 2, nul) == INVALID and "unknown epilogue" in msg()
    assert lib.ns_thin_gemm(x, nul, nul, out, 8, 1152, 896, 0, nul, nul, nul, nul, nul, 0, 0, nul) == INVALID and "null pointer" in msg()
    assert lib.ns_thin_swiglu_gemm(x, w, out, 33, 4864, 896, nul) == UNSUPPORTED and "33 token rows" in msg()
    assert lib.ns_thin_swiglu_gemm(x, w, out, 8, 8960, 1536, nul) == UNSUPPORTED and "shared memory" in msg()
    assert lib.ns_thin_swiglu_gemm(x, w, P(1028), 8, 4864, 896, nul) == INVALID and "aligned" in msg()
    assert lib.ns_thin_swiglu_gemm(x, w, out, 8, 4866, 896, nul) == UNSUPPORTED
    assert lib.ns_skinny_gemm(x, nul, nul, nul, w, nul, out, 65, 896, 896, 8, ctypes.c_float(1e-6), 0, 0, nul, nul, nul, nul, nul,
                              0, 0, nul) == UNSUPPORTED and "65 token rows" in msg()
    ss, eps = ctypes.cast(P(2048), ctypes.POINTER(ctypes.c_float)), ctypes.c_float(1e-6)
    assert lib.ns_thin_gemm_residual(x, w, x, out, ss, 0, 896, 896, nul) == 0                                  # empty step
    assert lib.ns_thin_gemm_residual(x, w, nul, out, ss, 8, 896, 896, nul) == INVALID and "null pointer" in msg()
    assert lib.ns_thin_gemm_residual(x, w, x, out, ss, 65, 896, 896, nul) == UNSUPPORTED and "65 token rows" in msg()
    assert lib.ns_thin_gemm_residual(x, w, x, out, ss, 64, 3584, 3584, nul) == UNSUPPORTED and "shared memory" in msg()
    assert lib.ns_thin_swiglu_gemm_norm(x, ss, 112, w, eps, w, out, 33, 4864, 896, nul) == UNSUPPORTED and "33 token rows" in msg()
    assert lib.ns_thin_swiglu_gemm_norm(x, ss, 0, w, eps, w, out, 8, 4864, 896, nul) == INVALID and "bad shape" in msg()
    assert lib.ns_thin_swiglu_gemm_norm(x, ss, 192, w, eps, w, out, 8, 8960, 1536, nul) == UNSUPPORTED and "shared memory" in msg()
    assert lib.ns_thin_swiglu_gemm_norm(x, nul, 112, w, eps, w, out, 8, 4864, 896, nul) == INVALID and "null pointer" in msg()


def test_no_undeclared_entry_point_is_exported():
    """The shipping library exports exactly the header's surface: profiling hooks exist only in a -DNS_DEBUG_HOOKS build."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if " T ns_" in line})
    assert exported == declared_symbols()


def test_tuning_knobs_round_trip_without_a_device():
    lib = _lib.load()
    assert lib.ns_get_tuning(_lib.TUNE_PREFILL_OVERLAP) == 1 and lib.ns_get_tuning(_lib.TUNE_DECODE_SPLIT_BLOCKS) == -1
    assert _lib.set_tuning(_lib.TUNE_DECODE_MIN_BLOCKS, 8) == 0
    assert lib.ns_get_tuning(_lib.TUNE_DECODE_MIN_BLOCKS) == 8
    _lib.set_tuning(_lib.TUNE_DECODE_MIN_BLOCKS, 0)
    assert lib.ns_set_tuning(99, 1) == 1 and "unknown knob" in lib.ns_last_error().decode()
