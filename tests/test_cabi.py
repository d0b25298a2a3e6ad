"""The C-ABI library loads and exports every symbol the header declares.  CPU only:
no compute entry point is called."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "awq_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"AWQ_B200_API\s+[\w\s\*]+?\b(awq_b200_\w+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = declared_symbols()
    for must in ("awq_b200_repack", "awq_b200_dequant", "awq_b200_gemv", "awq_b200_gemm", "awq_b200_linear"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from llmrqt_sdv1_b200 import _lib
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} declared in awq_b200.h but not exported"
    # and the Python binding table covers the header exactly
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_stateless_queries():
    from llmrqt_sdv1_b200._lib import lib
    assert lib.awq_b200_version() >= 1000
    assert lib.awq_b200_status_string(0) == b"ok"
    assert b"128" in lib.awq_b200_status_string(4)
    assert lib.awq_b200_packed_bytes(2048, 6144) == 2048 * 6144 // 2
    assert lib.awq_b200_gemv_max_rows() == 64
    assert lib.awq_b200_gemv_counter_bytes(6144) == lib.awq_b200_gemv_counter_bytes(57344) == 16384
    ws1 = lib.awq_b200_gemv_workspace_bytes(1, 2048, 6144)
    ws16 = lib.awq_b200_gemv_workspace_bytes(16, 2048, 6144)
    assert 0 < ws1 <= ws16 <= lib.awq_b200_gemv_workspace_bytes_max(16, 2048, 6144)
    assert lib.awq_b200_linear_workspace_bytes(4096, 2048, 6144) >= 256


def test_argument_errors_need_no_gpu():
    """Validation happens before any CUDA call, so it is checkable here."""
    from llmrqt_sdv1_b200._lib import lib, ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_GROUP
    assert lib.awq_b200_repack(None, None, 128, 8, None) == ERR_NULL
    assert lib.awq_b200_repack(16, 32, 100, 8, None) == ERR_SHAPE
    assert lib.awq_b200_repack(16, 36, 128, 8, None) == ERR_ALIGN
    assert lib.awq_b200_gemv(16, 16, 16, 16, None, 16, 1, 128, 8, 64, None, 0, None) == ERR_GROUP
    assert lib.awq_b200_gemv(16, 16, 16, 16, None, 16, 65, 128, 8, 128, None, 0, None) == ERR_SHAPE
    assert lib.awq_b200_gemm(16, 16, 16, 16, None, 16, 0, 128, 8, 128, None, 0, None) == ERR_SHAPE
