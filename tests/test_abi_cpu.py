"""The C-ABI library without a GPU: it loads, exports every declared symbol, and answers the
host-only questions (geometry, pre-flight refusals). No compute call is made here."""
import ctypes as C
import os
import re

import pytest

from kraken_b200 import capi, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "krk_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(krk_(?:cuda|gguf)_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(capi.lib, n), f"{n} is declared in krk_cuda.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature in capi.py"
    assert set(capi.SIGNATURES) <= set(names), "capi binds a symbol the header does not declare"


def test_geometry_matches_reference_tables():
    # tests/test_kraken.cpp:396-403 and src/quant.cpp:1805-1900
    assert capi.lib.krk_cuda_block_size(capi.Q4_0) == 32 and capi.lib.krk_cuda_block_bytes(capi.Q4_0) == 18
    assert capi.lib.krk_cuda_block_size(capi.Q6_K) == 256 and capi.lib.krk_cuda_block_bytes(capi.Q6_K) == 210
    assert capi.row_bytes(capi.Q8_0, 64) == 68
    assert capi.row_bytes(capi.Q4_K, 4096) == 2304 and capi.row_bytes(capi.Q6_K, 4096) == 3360
    assert capi.row_bytes(capi.Q8_0, 4096) == 4352 and capi.row_bytes(capi.Q6_K, 1536) == 1260
    for wt in synth.FORMATS + synth.MORE_FORMATS:
        assert capi.lib.krk_cuda_dtype_ok(wt) == 1
        assert capi.row_bytes(wt, 2048) == synth.row_bytes(wt, 2048)
    assert capi.row_bytes(capi.Q5_0, 4096) == 2816 and capi.row_bytes(capi.Q5_K, 4096) == 2816 and capi.row_bytes(capi.Q5_1, 64) == 48
    for wt in (0, 1, 3, 9, 15, 16, 19, 99, -1):
        assert capi.lib.krk_cuda_dtype_ok(wt) == 0 and capi.row_bytes(wt, 256) == 0


def test_gemm_k_ok():
    assert capi.gemm_k_ok(capi.Q8_0, 32) and capi.gemm_k_ok(capi.Q4_0, 4096)
    assert not capi.gemm_k_ok(capi.Q8_0, 0) and not capi.gemm_k_ok(capi.Q8_0, 48)
    assert capi.gemm_k_ok(capi.Q4_K, 11008) and not capi.gemm_k_ok(capi.Q4_K, 100)   # tests/test_kraken.cpp:401
    assert not capi.gemm_k_ok(capi.Q6_K, 32) and not capi.gemm_k_ok(77, 256) and not capi.gemm_k_ok(capi.Q6_K, -256)


def test_preflight_refusals_launch_nothing():
    """Bad arguments are refused with a code before any device is touched."""
    L = capi.lib
    before = L.krk_cuda_launch_count()
    a = C.c_void_p(0x1000)   # never dereferenced: the checks below all fail first
    assert L.krk_cuda_gemv(a, a, a, 99, 8, 256, 1, 0, None) == -1            # EDTYPE
    assert L.krk_cuda_gemv(a, a, a, capi.Q4_K, 8, 100, 1, 0, None) == -2     # ESHAPE: K not whole blocks
    assert L.krk_cuda_gemv(a, a, a, capi.Q4_K, -1, 256, 1, 0, None) == -2
    assert L.krk_cuda_gemv(a, a, a, capi.Q4_K, 8, 256, 9, 0, None) == -2     # rows > 8
    assert L.krk_cuda_gemv(None, a, a, capi.Q4_K, 8, 256, 1, 0, None) == -3  # ENULL
    assert L.krk_cuda_gemv(a, a, C.c_void_p(0x1008), capi.Q4_K, 8, 256, 1, 0, None) == -4  # EALIGN
    assert L.krk_cuda_gemv(a, C.c_void_p(0x1004), a, capi.Q4_K, 8, 256, 1, 0, None) == -4
    assert L.krk_cuda_dequant_rows(a, a, 5, 1, 256, None) == -1
    assert L.krk_cuda_dequant_rows(a, a, capi.Q6_K, 1, 100, None) == -2
    assert L.krk_cuda_gemm(a, a, 7, a, capi.Q4_K, 8, 256, 16, None, 0, None) == -8       # EARG: x dtype
    assert L.krk_cuda_gemm(a, a, capi.X_F16, a, capi.Q8_0, 8, 96, 16, None, 0, None) == -2
    assert L.krk_cuda_gemv_group(None, None, None, None, None, 256, 17, 0, None) == -8
    assert L.krk_cuda_gemv_group(None, None, None, None, None, 256, 2, 0, None) == -3
    # empty problems are a no-op success (the reference walks zero outputs without complaint)
    assert L.krk_cuda_gemv(None, None, None, capi.Q4_K, 0, 256, 1, 0, None) == 0
    assert L.krk_cuda_dequant_rows(None, None, capi.Q8_0, 0, 256, None) == 0
    assert L.krk_cuda_launch_count() == before
    assert b"whole number of blocks" in L.krk_cuda_strerror(-2)
