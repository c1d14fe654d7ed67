"""The C-ABI library loads and exports every symbol include/rocwmma_b200.h declares; argument checks
that precede any device work return the documented codes.  No GPU needed, no compute calls."""
import ctypes as C
import os
import re

import pytest

from rocwmma_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rocwmma_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200wmma_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    handle = C.CDLL(_lib.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(handle, s)]
    assert not missing, f"librocwmma_b200.so lacks: {missing}"
    assert _lib.lib().b200wmma_version() >= 100


def test_no_cpu_fallback_in_product_sources():
    """The product must not reach the CPU checker: nothing under rocwmma_b200/ or include/ names oracle/."""
    bad = []
    for base in ("rocwmma_b200", "include"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            if "_obj" in dirpath or "__pycache__" in dirpath:
                continue
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                    src = open(os.path.join(dirpath, f), errors="ignore").read()
                    if re.search(r"\boracle\b|ref_port|cpu_ref", src):
                        bad.append(os.path.join(dirpath, f))
    assert not bad, bad


@pytest.mark.parametrize("call,code", [
    (lambda L: L.b200wmma_gemm_f16(128, 128, 64, None, None, None, None, 64, 64, 128, 128, 1.0, 0.0, 2, 1, 0, 0, None), 1),
    (lambda L: L.b200wmma_gemm_f16(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 1, 1, 0, 0, None), 1),
    (lambda L: L.b200wmma_gemm_f16(0, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 0, 1, 0, 0, None), 1),
    (lambda L: L.b200wmma_gemm_f16(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 1.0, 0, 1, 0, 0, None), 1),
    (lambda L: L.b200wmma_gemm_i8(128, 128, 64, 16, 16, None, 16, 60, 64, 128, 128, 1, 0, 0, 1, 0, None), 1),
    (lambda L: L.b200wmma_gemm_i8(128, 128, 64, 16, 16, None, 16, 72, 64, 128, 128, 1, 0, 0, 1, 0, None), 3),
    (lambda L: L.b200wmma_gemm_f64(8, 8, 7, 16, 16, None, 16, 8, 8, 8, 8, 1.0, 0.0, 0, 1, 0, None), 3),
    (lambda L: L.b200wmma_gemv_f32(0, 8, 16, 8, 0, 16, 16, 1.0, 0.0, None), 1),
    (lambda L: L.b200wmma_gemv_f64(8, 8, 16, 4, 0, 16, 16, 1.0, 0.0, None), 1),
    (lambda L: L.b200wmma_dlrm_fwd(16, 16, 40, 40, 128, 4, 1024, None), 2),
    (lambda L: L.b200wmma_dlrm_fwd(16, 16, 27, 32, 100, 4, 480, None), 2),
    (lambda L: L.b200wmma_dlrm_fwd(16, 16, 27, 32, 128, 4, 100, None), 1),
    (lambda L: L.b200wmma_dlrm_bwd(16, None, 16, None, 27, 32, 128, 4, 480, 0, None), 1),
    (lambda L: L.b200wmma_gemm_i8_sp24(64, 64, 48, 16, 16, 16, None, 16, 24, 8, 48, 64, 64, 1, 0, 16, 1 << 20, None), 2),
    (lambda L: L.b200wmma_gemm_i4(64, 64, 48, 16, 16, None, 16, 32, 32, 64, 64, 1, 0, None, 0, None), 2),
    (lambda L: L.b200wmma_ctx_create(None), 1),
    (lambda L: L.b200wmma_gemm_bf16(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 0, 3, 0, None), 1),
    (lambda L: L.b200wmma_gemm_fp8(128, 128, 64, 16, 16, None, 16, 60, 64, 128, 128, 1.0, 0.0, 0, 1, 0, 0, None), 1),
    (lambda L: L.b200wmma_gemm_fp8(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 0, 1, 0, 7, None), 1),
    (lambda L: L.b200wmma_gemm_f32(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 1, 1, 0, 16, 1 << 30, None), 1),
    (lambda L: L.b200wmma_gemm_f32(128, 128, 64, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 0, 1, 0, 16, 1024, None), 1),
    (lambda L: L.b200wmma_gemm_f32(128, 128, 62, 16, 16, None, 16, 64, 64, 128, 128, 1.0, 0.0, 0, 1, 0, 16, 1 << 30, None), 2),
    (lambda L: L.b200wmma_sp24_repack_meta(256, 192, 16, 32, 16, 1 << 20, None), 2),
    (lambda L: L.b200wmma_sp24_repack_meta(256, 256, 16, 32, 16, 64, None), 1),
    (lambda L: L.b200wmma_gemm_i8_sp24_packed(256, 256, 192, 16, 16, 16, None, 16, 96, 192, 256, 256, 1, 0, None), 2),
    (lambda L: L.b200wmma_gemm_i8_sp24_packed(256, 256, 256, 16, None, 16, None, 16, 128, 256, 256, 256, 1, 0, None), 1),
    (lambda L: L.b200wmma_simple_sgemm(100, 64, 64, 16, 16, 16, 16, 64, 64, 64, 64, 1.0, 1.0, None), 2),
    (lambda L: L.b200wmma_simple_dgemm(64, 64, 64, 16, 16, None, 16, 64, 64, 64, 64, 1.0, 1.0, None), 1),
    (lambda L: L.b200wmma_mg_unique_id(None), 1),
    (lambda L: L.b200wmma_mg_create(None, None, 0, 1), 1),
    (lambda L: L.b200wmma_mg_broadcast(None, 16, 16, 0, None), 1),
    (lambda L: L.b200wmma_mg_allgather(None, 16, 16, None), 1),
    (lambda L: L.b200wmma_set_tuning(b"no_such_key", 1), 1),
    (lambda L: L.b200wmma_set_tuning(b"gemm_tile_variant", 9), 1),
    (lambda L: L.b200wmma_ctx_last_stage_ms(None, None), 1),
    (lambda L: L.b200wmma_shard_range(1000, 8, 0, 16, C.byref(C.c_uint64()), C.byref(C.c_uint64())), 2),
    (lambda L: L.b200wmma_shard_range(1024, 8, 8, 16, C.byref(C.c_uint64()), C.byref(C.c_uint64())), 1),
], ids=["bad_layout_flag", "col_major_a_lda_lt_m", "zero_m", "null_c_with_beta", "lda_too_small",
        "lda_not_16B", "f64_odd_k", "gemv_zero_m", "gemv_lda_small", "dlrm_rows_beyond_stride", "dlrm_k_not_16",
        "dlrm_out_stride_small", "dlrm_bwd_null_upstream", "sp24_k_not_32", "i4_k_not_32", "ctx_null",
        "bf16_bad_layout_flag", "fp8_lda_too_small", "fp8_bad_format", "f32_col_major_a_lda_lt_m", "f32_workspace_small",
        "f32_k_not_4", "repack_k_not_128", "repack_dest_small", "sp24_packed_k_not_128", "sp24_packed_null_meta",
        "simple_sgemm_m_not_16", "simple_dgemm_null_c", "mg_id_null", "mg_create_null", "mg_broadcast_null_handle",
        "mg_allgather_null_handle", "tuning_unknown_key", "tuning_out_of_range", "stage_ms_null",
        "shard_uneven", "shard_bad_index"])
def test_argument_checks(call, code):
    L = _lib.lib()
    assert call(L) == code
    assert L.b200wmma_last_error_string()  # a message is always recorded


def test_set_tuning_round_trip():
    """Every key the header documents is accepted at a legal value and reset; unknown keys and values out of range are
    argument errors."""
    L = _lib.lib()
    keys = {b"gemm_tile_variant": 1, b"gemm_group_m": 4, b"sp24_force_expand": 1, b"gemm_mma_order": 2, b"gemm_split_tail": 2,
            b"gemm_split_fixup": 16, b"dlrm_bwd_stages": 3, b"dlrm_bwd_warps": 8, b"dlrm_fwd_stages": 3, b"dlrm_fwd_warps": 8,
            b"gemm_f64_kernel": 1, b"frag_perf_slab_k": 32, b"gemv_rows": 4, b"gemv_col_vn": 2}
    header = open(os.path.join(ROOT, "include", "rocwmma_b200.h")).read()
    for key, value in keys.items():
        assert f'"{key.decode()}"' in header, f"{key} is not documented in the header"
        assert L.b200wmma_set_tuning(key, value) == 0
        assert L.b200wmma_set_tuning(key, 0) == 0
    assert L.b200wmma_set_tuning(b"no_such_key", 1) == 1
    assert L.b200wmma_set_tuning(b"gemm_f64_kernel", 7) == 1
    assert L.b200wmma_set_tuning(None, 1) == 1


def test_measure_mma_sync_rate_argument_checks():
    L = _lib.lib()
    out = C.c_double(0.0)
    assert L.b200wmma_measure_mma_sync_rate(2, C.byref(out), None) == 1   # kinds are 0 and 1
    assert L.b200wmma_measure_mma_sync_rate(0, None, None) == 1


def test_shard_range_and_destroy_of_null():
    L = _lib.lib()
    begin, count = C.c_uint64(), C.c_uint64()
    assert L.b200wmma_shard_range(8192, 8, 3, 16, C.byref(begin), C.byref(count)) == 0
    assert (begin.value, count.value) == (3072, 1024)
    assert L.b200wmma_mg_destroy(None) == 0  # like free(NULL)
    assert L.b200wmma_mg_rank(None) == -1 and L.b200wmma_mg_size(None) == 0
