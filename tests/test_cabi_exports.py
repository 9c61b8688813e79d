"""Without a GPU: the C-ABI library loads and exports every symbol include/spk.h declares, and
host-side validation answers with status codes (no kernel is launched here)."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "5090-blackwell-kernels_b200", "lib", "libspark_b200.so")


def _declared():
    text = open(os.path.join(ROOT, "include", "spk.h")).read()
    return sorted(set(re.findall(r"SPK_API\s+[\w\s\*]+?\b(spk_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    assert os.path.exists(LIB), "build the library first: python 5090-blackwell-kernels_b200/build.py"
    lib = ctypes.CDLL(LIB)
    names = _declared()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/spk.h but not exported"


def test_host_validation_returns_status_codes():
    lib = ctypes.CDLL(LIB)
    lib.spk_last_error.restype = ctypes.c_char_p
    p = ctypes.c_void_p
    lib.spk_w4gemm_bf16.argtypes = [p, p, p, p, p] + [ctypes.c_int] * 4 + [p]
    buf = ctypes.create_string_buffer(64)
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16
    # K not a multiple of 128 -> SPK_INVALID before anything touches CUDA
    assert lib.spk_w4gemm_bf16(addr, addr, addr, None, addr, 1, 16, 100, 2, None) == 1
    assert b"128" in lib.spk_last_error()
    assert lib.spk_w4gemm_bf16(addr, addr, addr, None, addr, 1, 16, 128, 9, None) == 1  # variant
    assert lib.spk_w4gemm_bf16(None, addr, addr, None, addr, 1, 16, 128, 2, None) == 1  # null
    assert lib.spk_w4gemm_bf16(addr + 2, addr, addr, None, addr, 1, 16, 128, 2, None) == 1  # alignment
    lib.spk_w4_repack.argtypes = [p, p, ctypes.c_int, ctypes.c_int, p]
    assert lib.spk_w4_repack(addr, addr, 64, 16, None) == 1  # in place is refused
    assert lib.spk_w4gemm_num_variants() == 4 and lib.spk_w4gemm_default_variant() == 2
    assert lib.spk_w4gemm_supports(1, 4096, 4096, 2) == 1 and lib.spk_w4gemm_supports(1, 40, 4096, 2) == 0
