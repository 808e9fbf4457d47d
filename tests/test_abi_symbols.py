"""CPU: the C-ABI library builds, loads, and exports every function include/gemlite_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gemlite_b200.h")).read()
    return sorted(set(re.findall(r"GL_API\s+[\w\s\*]+?\b(gl_\w+)\s*\(", text)))


def test_header_functions_are_exported(lib):
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), "missing export: " + n


def test_binding_table_matches_header():
    from gemlite_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_struct_size_matches_c_layout(lib):
    # 10 pointers/u64 (80) + 16 int32 (64) + 4 int64 (32) + 4 int32 (16) + 1 pointer (8)
    from gemlite_b200 import _lib
    assert ctypes.sizeof(_lib.GLMatmulArgs) == 200


def test_version_and_dispatch_rules(lib):
    assert lib.gl_abi_version() == 1
    assert b"sm_100a" in lib.gl_build_info()
    # get_matmul_type of the reference (gemlite/core.py:171-179)
    names = ["GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"]
    def ref(M, nbits, mx):
        if M >= 64:
            return "GEMM"
        limit = 4 if (nbits < 8 and not mx) else 2
        if M > limit:
            return "GEMM_SPLITK"
        if mx:
            return "GEMM_SPLITK"
        return "GEMV_REVSPLITK" if nbits < 8 else "GEMV_SPLITK"
    for M in (1, 2, 3, 4, 5, 16, 63, 64, 4096):
        for nbits in (1, 2, 4, 8, 16):
            for mx in (0, 1):
                assert names[lib.gl_get_matmul_type(M, nbits, mx)] == ref(M, nbits, mx)


def test_invalid_arguments_are_rejected_without_a_gpu(lib):
    from gemlite_b200 import _lib
    a = _lib.GLMatmulArgs()
    assert lib.gl_matmul(ctypes.byref(a), None) == _lib.GL_E_INVALID
    assert b"gl_matmul" in lib.gl_last_error()
    assert lib.gl_pack_over_cols(None, None, 4, 8, 3, 32, None) == _lib.GL_E_INVALID
    assert lib.gl_scale_activations_mxfp4(None, None, None, 4, 48, 2, 0, None) == _lib.GL_E_INVALID
