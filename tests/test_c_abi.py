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
