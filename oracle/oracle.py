"""ctypes/numpy front end of the CPU oracle (oracle/spark_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's CPU
baseline leg. The product package never imports it.

Arrays are numpy; bf16 travels as uint16 bit patterns, e4m3 / e2m1 / scale bytes as uint8.
`t2n` / `n2t` convert torch tensors (any of bf16, float8_e4m3fn, uint8, int32, float32) to and
from that convention.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libspark_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, a second or two)."""
    src = os.path.join(_HERE, "spark_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        L = _lib
        c_i, c_f, c_p, c_i64 = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64
        L.orc_bf16_from_f32.restype = ctypes.c_uint16
        L.orc_bf16_from_f32.argtypes = [c_f]
        L.orc_bf16_to_f32.restype = c_f
        L.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_e4m3_to_f32.restype = c_f
        L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_e4m3_from_f32.restype = ctypes.c_uint8
        L.orc_e4m3_from_f32.argtypes = [c_f]
        L.orc_e2m1_code.restype = ctypes.c_uint8
        L.orc_e2m1_code.argtypes = [c_f]
        L.orc_e2m1_value.restype = c_f
        L.orc_e2m1_value.argtypes = [ctypes.c_uint8]
        L.orc_w4_locate.restype = None
        L.orc_w4_locate.argtypes = [c_i, c_i, c_i, ctypes.POINTER(c_i64), ctypes.POINTER(c_i)]
        for name, n in (("orc_w4_repack", 2), ("orc_w4_unpack", 2), ("orc_w4_pack_gptq", 2)):
            f = getattr(L, name)
            f.restype = None
            f.argtypes = [c_p] * n + [c_i, c_i]
        L.orc_w4_quantize.restype = None
        L.orc_w4_quantize.argtypes = [c_p, c_p, c_p, c_p, c_i, c_i]
        L.orc_w4_dequantize.restype = None
        L.orc_w4_dequantize.argtypes = [c_p, c_p, c_p, c_p, c_i, c_i]
        L.orc_w4gemm.restype = None
        L.orc_w4gemm.argtypes = [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i]
        L.orc_fp8_quantize.restype = None
        L.orc_fp8_quantize.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i]
        L.orc_fp8_quantize_per_tensor.restype = None
        L.orc_fp8_quantize_per_tensor.argtypes = [c_p, c_p, c_p, c_i64]
        L.orc_fp8gemm.restype = None
        L.orc_fp8gemm.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i, c_f, c_f, c_p, c_p, c_i]
        L.orc_fp8_block128_quantize.restype = None
        L.orc_fp8_block128_quantize.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i]
        L.orc_fp8gemm_block128.restype = None
        L.orc_fp8gemm_block128.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_i]
        L.orc_fp4_scale_bytes.restype = c_i64
        L.orc_fp4_scale_bytes.argtypes = [c_i, c_i, c_i]
        L.orc_fp4_sf_offset.restype = c_i64
        L.orc_fp4_sf_offset.argtypes = [c_i, c_i, c_i]
        L.orc_fp4_quantize.restype = None
        L.orc_fp4_quantize.argtypes = [c_p, c_p, c_p, c_i, c_i, c_p, c_p, c_i]
        L.orc_fp4_dequantize.restype = None
        L.orc_fp4_dequantize.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i]
        L.orc_fp4gemm.restype = None
        L.orc_fp4gemm.argtypes = [c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_f, c_f, c_i, c_i]
        L.orc_max_threads.restype = c_i
        L.orc_max_threads.argtypes = []
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


# ---- torch <-> numpy convention -------------------------------------------------------------

def t2n(t):
    """torch tensor -> numpy in the oracle's convention (bf16 -> uint16 bits, fp8 -> uint8)."""
    import torch

    if t is None:
        return None
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, getattr(torch, "float8_e8m0fnu", None),
                   getattr(torch, "float4_e2m1fn_x2", None)):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def n2t(a, kind=None):
    """numpy -> torch; kind 'bf16' reinterprets uint16 bits, 'e4m3' uint8 bytes."""
    import torch

    if kind == "bf16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    if kind == "e4m3":
        return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)
    return torch.from_numpy(a.copy())


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 array -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


_E4M3_TABLE = None


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        L = lib()
        _E4M3_TABLE = np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return _E4M3_TABLE[b]


# ---- int4 -------------------------------------------------------------------------------------

def w4_quantize(w_bits: np.ndarray, asym: bool = False):
    """bf16 bits [K, N] -> (qweight int32 [K/8, N], scales uint16 [K/128, N], zeros u8 | None)."""
    w_bits = _c(w_bits, np.uint16)
    K, N = w_bits.shape
    q = np.empty((K // 8, N), np.int32)
    s = np.empty((K // 128, N), np.uint16)
    z = np.empty((K // 128, N), np.uint8) if asym else None
    lib().orc_w4_quantize(_p(w_bits), _p(q), _p(s), _p(z), K, N)
    return q, s, z


def w4_pack_gptq(codes: np.ndarray) -> np.ndarray:
    codes = _c(codes, np.uint8)
    K, N = codes.shape
    q = np.empty((K // 8, N), np.int32)
    lib().orc_w4_pack_gptq(_p(codes), _p(q), K, N)
    return q


def w4_repack(qweight: np.ndarray) -> np.ndarray:
    qweight = _c(qweight, np.int32)
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    out = np.empty((N // 16, 2 * K), np.int32)
    lib().orc_w4_repack(_p(qweight), _p(out), K, N)
    return out


def w4_unpack(packed: np.ndarray) -> np.ndarray:
    packed = _c(packed, np.int32)
    K, N = packed.shape[1] // 2, packed.shape[0] * 16
    out = np.empty((K, N), np.uint8)
    lib().orc_w4_unpack(_p(packed), _p(out), K, N)
    return out


def w4_locate(n: int, k: int, K: int):
    w, p = ctypes.c_int64(), ctypes.c_int()
    lib().orc_w4_locate(n, k, K, ctypes.byref(w), ctypes.byref(p))
    return w.value, p.value


def w4_dequantize(packed, scales, zeros=None) -> np.ndarray:
    packed, scales = _c(packed, np.int32), _c(scales, np.uint16)
    zeros = None if zeros is None else _c(zeros, np.uint8)
    K, N = packed.shape[1] // 2, packed.shape[0] * 16
    out = np.empty((K, N), np.uint16)
    lib().orc_w4_dequantize(_p(packed), _p(scales), _p(zeros), _p(out), K, N)
    return out


def w4gemm(a_bits, packed, scales, zeros=None, threads: int = 0) -> np.ndarray:
    a_bits, packed, scales = _c(a_bits, np.uint16), _c(packed, np.int32), _c(scales, np.uint16)
    zeros = None if zeros is None else _c(zeros, np.uint8)
    M, K = a_bits.shape
    N = packed.shape[0] * 16
    assert packed.shape[1] == 2 * K
    out = np.empty((M, N), np.uint16)
    lib().orc_w4gemm(_p(a_bits), _p(packed), _p(scales), _p(zeros), _p(out), M, N, K, threads)
    return out


# ---- fp8 --------------------------------------------------------------------------------------

def fp8_quantize(x_bits: np.ndarray, mode: str = "tensor"):
    x_bits = _c(x_bits, np.uint16)
    rows, K = x_bits.shape
    q = np.empty((rows, K), np.uint8)
    m = {"tensor": 0, "row": 1, "mx": 2}[mode]
    if m == 0:
        s = np.empty((1,), np.float32)
    elif m == 1:
        s = np.empty((rows, 1), np.float32)
    else:
        s = np.empty((rows, K // 32), np.uint8)
    lib().orc_fp8_quantize(_p(x_bits), _p(q), _p(s), rows, K, m)
    return q, s


def fp8_quantize_per_tensor(x: np.ndarray):
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    s = np.empty((1,), np.float32)
    lib().orc_fp8_quantize_per_tensor(_p(x), _p(q), _p(s), x.size)
    return q, s


def fp8gemm(a, bt, sa: float = 1.0, sb: float = 1.0, sfa=None, sfb=None, threads: int = 0):
    a, bt = _c(a, np.uint8), _c(bt, np.uint8)
    M, K = a.shape
    N = bt.shape[0]
    if sfa is not None:
        sfa, sfb = _c(sfa, np.uint8), _c(sfb, np.uint8)
    out = np.empty((M, N), np.uint16)
    lib().orc_fp8gemm(_p(a), _p(bt), _p(out), M, N, K, float(sa), float(sb), _p(sfa), _p(sfb), threads)
    return out


def fp8_block128_quantize(x: np.ndarray, block_rows: int):
    """fp32 [rows, K] -> (e4m3 bytes, fp32 scales [cdiv(rows, block_rows), K/128]).
    block_rows = 1 for activations (1x128), 128 for weights (128x128). Not in the reference."""
    x = _c(x, np.float32)
    rows, K = x.shape
    q = np.empty((rows, K), np.uint8)
    s = np.empty(((rows + block_rows - 1) // block_rows, K // 128), np.float32)
    lib().orc_fp8_block128_quantize(_p(x), _p(q), _p(s), rows, K, block_rows)
    return q, s


def fp8gemm_block128(a, bt, sA, sB, threads: int = 0):
    a, bt, sA, sB = _c(a, np.uint8), _c(bt, np.uint8), _c(sA, np.float32), _c(sB, np.float32)
    M, K = a.shape
    N = bt.shape[0]
    out = np.empty((M, N), np.uint16)
    lib().orc_fp8gemm_block128(_p(a), _p(bt), _p(out), M, N, K, _p(sA), _p(sB), threads)
    return out


# ---- fp4 --------------------------------------------------------------------------------------

FMT = {"nvfp4": 0, "mxfp4": 1}


def fp4_scale_bytes(rows: int, K: int, fmt: str = "nvfp4") -> int:
    return int(lib().orc_fp4_scale_bytes(rows, K, FMT[fmt]))


def fp4_sf_offset(r: int, j: int, cols: int) -> int:
    return int(lib().orc_fp4_sf_offset(r, j, cols))


def fp4_quantize(x_bits: np.ndarray, fmt: str = "nvfp4", scale: float | None = None):
    """-> (q u8 [rows, K/2], sf u8 flat blocked, scale float32 | None)."""
    x_bits = _c(x_bits, np.uint16)
    rows, K = x_bits.shape
    q = np.empty((rows, K // 2), np.uint8)
    sf = np.empty((fp4_scale_bytes(rows, K, fmt),), np.uint8)
    s_out = np.zeros((1,), np.float32)
    s_in = None if scale is None else np.array([scale], np.float32)
    lib().orc_fp4_quantize(_p(x_bits), _p(q), _p(sf), rows, K, _p(s_in), _p(s_out), FMT[fmt])
    return q, sf, (s_out[0] if fmt == "nvfp4" else None)


def fp4_dequantize(q, sf, fmt: str = "nvfp4") -> np.ndarray:
    q, sf = _c(q, np.uint8), _c(sf, np.uint8)
    rows, K = q.shape[0], q.shape[1] * 2
    out = np.empty((rows, K), np.float32)
    lib().orc_fp4_dequantize(_p(q), _p(sf), _p(out), rows, K, FMT[fmt])
    return out


def fp4gemm(a, bt, sfa, sfb, sa: float = 1.0, sb: float = 1.0, fmt: str = "nvfp4", threads: int = 0):
    a, bt, sfa, sfb = _c(a, np.uint8), _c(bt, np.uint8), _c(sfa, np.uint8), _c(sfb, np.uint8)
    M, K = a.shape[0], a.shape[1] * 2
    N = bt.shape[0]
    out = np.empty((M, N), np.uint16)
    lib().orc_fp4gemm(_p(a), _p(bt), _p(out), M, N, K, _p(sfa), _p(sfb), float(sa), float(sb),
                      FMT[fmt], threads)
    return out


def max_threads() -> int:
    return int(lib().orc_max_threads())
