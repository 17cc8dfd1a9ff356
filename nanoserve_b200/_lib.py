"""ctypes binding of libnanoserve_b200.so (the C ABI declared in include/nanoserve_b200.h).

There is no fallback: if the library is missing or a call fails, the caller gets an exception. The product
path never routes through PyTorch ops or CPU code for work this library owns.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

import os

# NS_DEBUG_LIB=1 loads the -DNS_DEBUG_HOOKS build (python -m nanoserve_b200.build --debug-hooks) instead: the same
# entry points plus the profiling hooks
LIB_PATH = Path(__file__).resolve().parent / "lib" / ("libnanoserve_b200_dbg.so" if os.environ.get("NS_DEBUG_LIB") == "1"
                                                      else "libnanoserve_b200.so")

NS_BF16, NS_F32 = 0, 1
# ns_tuning_knob
(TUNE_PREFILL_IMPL, TUNE_PREFILL_OVERLAP, TUNE_DECODE_SPLIT_BLOCKS, TUNE_DECODE_MIN_BLOCKS, TUNE_DECODE_SNAP_BLOCKS,
 TUNE_DECODE_BALANCE, TUNE_DECODE_CLUSTER, TUNE_DECODE_CLUSTER_BLOCKS, TUNE_PREFILL_CLUSTER) = range(9)

# name -> (restype, argtypes); mirrors include/nanoserve_b200.h declaration by declaration.
_P, _I32, _I64, _F = c_void_p, c_int32, c_int64, c_float
SIGNATURES: dict[str, tuple] = {
    "ns_version": (c_int, []),
    "ns_last_error": (c_char_p, []),
    "ns_sm_count": (c_int, []),
    "ns_set_tuning": (c_int, [c_int, c_int]),
    "ns_get_tuning": (c_int, [c_int]),
    "ns_collect_status": (c_int, [_P, _P, _P]),
    "ns_tp_allreduce_add_rmsnorm": (c_int, [_P, _P, _P, _P, _P, _P, _P, _I64, _I32, _F, _I32, _I32, _P]),
    "ns_peer_alloc": (c_int, [_I64, _P]),
    "ns_peer_free": (c_int, [_P]),
    "ns_peer_export": (c_int, [_P, _P]),
    "ns_peer_open": (c_int, [_P, _P]),
    "ns_peer_close": (c_int, [_P]),
    "ns_check_step_metadata": (c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P]),
    "ns_add_rmsnorm": (c_int, [_P, _P, _P, _P, _P, _I64, _I32, _F, c_int, _P]),
    "ns_silu_mul": (c_int, [_P, _P, _I64, _I32, c_int, _P]),
    "ns_rope_cos_sin": (c_int, [_P, _P, _P, _P, _I64, _I32, c_int, _P]),
    "ns_rope_qkv_kvwrite": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, c_int, _P]),
    "ns_kv_write": (c_int, [_P, _P, _P, _P, _P, _I64, _I32, c_int, _P]),
    "ns_skinny_gemm": (c_int, [_P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _F, _I32, _I32, _P, _P, _P, _P, _P, _I32,
                               _I32, _P]),
    "ns_thin_gemm": (c_int, [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P, _I32, _I32, _P]),
    "ns_thin_swiglu_gemm": (c_int, [_P, _P, _P, _I32, _I32, _I32, _P]),
    "ns_thin_gemm_residual": (c_int, [_P, _P, _P, _P, _P, _I32, _I32, _I32, _P]),
    "ns_thin_swiglu_gemm_norm": (c_int, [_P, _P, _I32, _P, _F, _P, _P, _I32, _I32, _I32, _P]),
    "ns_thin_gemm_errors": (c_int, [_P]),
    "ns_stream_gemm": (c_int, [_P, _P, _P, _P, _P, _I32, _P, _P, _P, _P, _P, _I32, _I32, _I32, _F, _I32, _P]),
    "ns_stream_gemm_errors": (c_int, [_P]),
    "ns_swiglu_gemm": (c_int, [_P, _P, _P, _I32, _I32, _I32, _P]),
    "ns_umma_gemm_errors": (c_int, [_P]),
    "ns_attn_workspace_bytes": (_I64, [_I32, _I32, _I32, _I32]),
    "ns_attn_plan": (c_int, [_P, _P, _P, _I32, _I32, _I32, _I32, _P, _I64, _I32, _I32, _P]),
    "ns_ragged_paged_attn": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _I32, _I64, _I64,
                                     _I64, _I64, _I64, _I64, _F, c_int, _P, _I64, _I32, _I32, _P]),
    "ns_paged_attn_decode": (c_int, [_P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _I64, _I64, _I64, _I64,
                                     _I64, _I64, _F, c_int, _P, _I64, _I32, _I32, _P]),
    "ns_paged_attn_decode_static_bytes": (_I64, []),
    "ns_paged_attn_decode_static": (c_int, [_P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _I64, _I64, _I64, _I64,
                                            _I64, _I64, _F, c_int, _P]),
    "ns_ragged_paged_attn_simple": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _I32, _I64,
                                            _I64, _I64, _I64, _I64, _I64, _F, c_int, _P]),
    "ns_build_step_metadata": (c_int, [_P, _I32, _P, _P, _I32, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _P]),
    "ns_argmax_rows": (c_int, [_P, _I64, _I32, _I32, _P, _P, _P, c_int, _P]),
    "ns_sample_rows": (c_int, [_P, _I64, _I32, _I32, _P, _P, _P, _P, _P, _P, c_int, _P]),
}

_lib = None

# Kernel launches issued through this binding (eager calls and, via note_graph_replay, launches replayed from CUDA
# graphs). Benchmarks read it to report how many of this library's kernels ran in a timed region.
launch_count = 0
_LAUNCHES_PER_CALL = {"ns_paged_attn_decode": 2, "ns_paged_attn_decode_static": 2}       # plan + decode; ns_ragged_paged_attn is counted by its wrapper


class NanoserveB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built (no CPU / PyTorch fallback exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NanoserveB200Error(
                f"{LIB_PATH} is missing: build it with `python -m nanoserve_b200.build` "
                "(the sm_100a kernels are the only implementation of these ops)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)      # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Invoke a status-returning entry point; raise with the library's message on failure."""
    global launch_count
    lib = load()
    status = getattr(lib, name)(*args)
    launch_count += _LAUNCHES_PER_CALL.get(name, 1)
    if status != 0:
        raise NanoserveB200Error(f"{name} failed (status {status}): {lib.ns_last_error().decode()}")


def set_tuning(knob: int, value: int) -> int:
    """Set a process-wide tuning knob (ns_set_tuning); returns the previous value."""
    lib = load()
    old = lib.ns_get_tuning(knob)
    if lib.ns_set_tuning(knob, value) != 0:
        raise NanoserveB200Error(f"ns_set_tuning failed: {lib.ns_last_error().decode()}")
    return old


def note_launches(n: int) -> None:
    """Account for launches that did not go through call(): graph replays, a second kernel behind one entry point."""
    global launch_count
    launch_count += n


def dtype_code(dtype) -> int:
    import torch
    if dtype == torch.bfloat16:
        return NS_BF16
    if dtype == torch.float32:
        return NS_F32
    raise NotImplementedError(f"nanoserve_b200 kernels handle bfloat16 and float32, not {dtype}")


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NanoserveB200Error("nanoserve_b200 kernels run on CUDA tensors only (there is no CPU path)")
