"""The `spark_kernels._C` operator module: same op names, argument order, defaults, return shapes
and error behaviour as the reference's pybind extension for the quantized-GEMM path
(reference python/csrc/bindings.cpp:333-651, defs :1943-1990), implemented over the C-ABI of
libspark_b200.so with ctypes.

Each op validates like the reference binding does (a failed check raises RuntimeError, as
TORCH_CHECK does), allocates its outputs with torch on the inputs' device, and launches on
torch's current CUDA stream. A status SPK_INVALID from the library raises ValueError
(the reference's std::invalid_argument), any other non-zero status RuntimeError.

There is no CPU or eager fallback: if the shared library is missing this module fails to import.
"""

from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get(
    "SPARK_B200_LIB",
    os.path.normpath(os.path.join(_HERE, "..", "..", "lib", "libspark_b200.so")),
)
if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} not found: build it with `python 5090-blackwell-kernels_b200/build.py` "
        "(there is no fallback path)"
    )
_lib = ctypes.CDLL(_LIB_PATH)

_i, _p, _i64, _f = ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_float
_lib.spk_last_error.restype = ctypes.c_char_p
_lib.spk_version.restype = ctypes.c_char_p


def _sig(name, argtypes, restype=_i):
    fn = getattr(_lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


_spk_init = _sig("spk_init", [])
_spk_device_status = _sig("spk_device_status", [_p, ctypes.POINTER(_i)])
_spk_w4_quantize = _sig("spk_w4_quantize_bf16", [_p, _p, _p, _p, _i, _i, _p])
_spk_w4_repack = _sig("spk_w4_repack", [_p, _p, _i, _i, _p])
_spk_w4gemm = _sig("spk_w4gemm_bf16", [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p])
_spk_w4gemm_noalloc = _sig("spk_w4gemm_bf16_noalloc", [_p, _p, _p, _p, _p, _i, _i, _i, _p])
_sig("spk_w4gemm_num_variants", [])
_sig("spk_w4gemm_default_variant", [])
_sig("spk_w4gemm_supports", [_i, _i, _i, _i])

W4_GROUP = 128


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _status(rc: int) -> None:
    if rc == 0:
        return
    msg = _lib.spk_last_error().decode()
    if rc == 1:
        raise ValueError(msg)
    raise RuntimeError(f"[spk status {rc}] {msg}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _check_cuda_contig(t: torch.Tensor, name: str) -> None:
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _aligned16(t: torch.Tensor) -> bool:
    return t.data_ptr() % 16 == 0


def _ptr(t):
    return None if t is None else t.data_ptr()


def _resolve_variant(variant: int, n: int) -> int:
    """variant < 0 -> the highest rung; a variant past the ladder is a binding-level error
    (reference python/csrc/bindings.cpp:48-52)."""
    if variant < 0:
        return n - 1
    _check(variant < n, f"variant {variant} out of range [0, {n})")
    return variant


def lib_path() -> str:
    return _LIB_PATH


def version() -> str:
    return _lib.spk_version().decode()


def init(device=None) -> None:
    """Allocate the library's per-device scratch now (do this before capturing a CUDA graph)."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _status(_spk_init())


def device_status(device=None) -> int:
    """Synchronize and return the device status word (0, or 3 after a bounded wait timed out)."""
    code = _i(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _status(_spk_device_status(torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(code)))
    return code.value


def num_variants(name: str) -> int:
    fn = {"w4gemm": "spk_w4gemm_num_variants", "fp8gemm": "spk_fp8gemm_num_variants",
          "fp4gemm": "spk_fp4gemm_num_variants"}.get(name)
    if fn is None or not hasattr(_lib, fn):
        raise ValueError(f"unknown kernel: {name}")
    return int(getattr(_lib, fn)())


# ---- W4A16 ----------------------------------------------------------------------------------

def w4_quantize(w: torch.Tensor, asym: bool = False):
    """(qweight int32 [K/8, N], scales bf16 [K/128, N], zeros uint8 [K/128, N] | None)."""
    _check_cuda_contig(w, "w")
    _check(w.dtype == torch.bfloat16, "w4_quantize expects a bfloat16 weight")
    _check(w.dim() == 2, "w4_quantize expects a 2-D [K, N] weight")
    K, N = w.shape
    _check(K % W4_GROUP == 0 and N % 16 == 0 and K > 0 and N > 0,
           f"w4_quantize needs K a multiple of 128 and N a multiple of 16, got {K}x{N}")
    with torch.cuda.device(w.device):
        q = torch.empty((K // 8, N), dtype=torch.int32, device=w.device)
        sc = torch.empty((K // W4_GROUP, N), dtype=torch.bfloat16, device=w.device)
        z = torch.empty((K // W4_GROUP, N), dtype=torch.uint8, device=w.device) if asym else None
        _status(_spk_w4_quantize(w.data_ptr(), q.data_ptr(), sc.data_ptr(), _ptr(z), K, N, _stream(w)))
    return q, sc, z


def w4_repack(qweight: torch.Tensor) -> torch.Tensor:
    """qweight [K/8, N] int32 -> the kernel layout, int32 [N/16, 2K]."""
    _check_cuda_contig(qweight, "qweight")
    _check(qweight.dtype == torch.int32 and qweight.dim() == 2,
           "w4_repack expects a 2-D int32 qweight [K/8, N]")
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    _check(K % 64 == 0 and N % 16 == 0 and K > 0 and N > 0,
           f"w4_repack needs K a multiple of 64 and N a multiple of 16, got {K}x{N}")
    with torch.cuda.device(qweight.device):
        packed = torch.empty((N // 16, 2 * K), dtype=torch.int32, device=qweight.device)
        _status(_spk_w4_repack(qweight.data_ptr(), packed.data_ptr(), K, N, _stream(qweight)))
    return packed


def w4gemm(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, zeros=None,
           variant: int = -1, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] bf16 times the weight in `packed` [N/16, 2K] (w4_repack), `scales` [K/128, N]
    bf16 and `zeros` [K/128, N] uint8 (None: symmetric) -> [M, N] bf16. `out` (an addition to
    the reference signature) receives the result without an allocation."""
    _check_cuda_contig(a, "a")
    _check_cuda_contig(packed, "packed")
    _check_cuda_contig(scales, "scales")
    _check(a.dtype == torch.bfloat16 and a.dim() == 2, "w4gemm expects a 2-D bfloat16 a")
    _check(packed.dtype == torch.int32 and packed.dim() == 2,
           "w4gemm expects packed as the int32 [N/16, 2K] tensor from w4_repack")
    M, K = a.shape
    N = packed.shape[0] * 16
    _check(packed.shape[1] == 2 * K,
           f"packed is {list(packed.shape)}, expected [N/16, 2K] = [{packed.shape[0]}, {2 * K}] for K = {K}")
    _check(K % W4_GROUP == 0, f"w4gemm needs K a multiple of 128, got {K}")
    _check(M >= 1, "w4gemm needs at least one row")
    _check(scales.dtype == torch.bfloat16 and scales.dim() == 2 and tuple(scales.shape) == (K // W4_GROUP, N),
           f"scales must be bfloat16 [{K // W4_GROUP}, {N}], got {list(scales.shape)}")
    if zeros is not None:
        _check_cuda_contig(zeros, "zeros")
        _check(zeros.dtype == torch.uint8 and zeros.dim() == 2 and tuple(zeros.shape) == (K // W4_GROUP, N),
               f"zeros must be uint8 [{K // W4_GROUP}, {N}], got {list(zeros.shape)}")
        _check(zeros.device == a.device, "zeros must be on a's device")
    _check(packed.device == a.device and scales.device == a.device, "packed and scales must be on a's device")
    _check(_aligned16(a) and _aligned16(packed) and _aligned16(scales) and (zeros is None or _aligned16(zeros)),
           "w4gemm needs 16-byte aligned a, packed, scales and zeros storage")
    with torch.cuda.device(a.device):
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        else:
            _check(out.is_cuda and out.is_contiguous() and out.dtype == torch.bfloat16
                   and tuple(out.shape) == (M, N) and out.device == a.device, "out must be bf16 [M, N] on a's device")
        v = _lib.spk_w4gemm_default_variant() if variant < 0 else _resolve_variant(
            variant, _lib.spk_w4gemm_num_variants())
        _status(_spk_w4gemm(a.data_ptr(), packed.data_ptr(), scales.data_ptr(), _ptr(zeros), out.data_ptr(),
                            M, N, K, v, _stream(a)))
    return out


def w4gemm_noalloc(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, zeros, out: torch.Tensor) -> torch.Tensor:
    """w4gemm for callers that must not allocate device memory (no counterpart in the reference):
    the caller passes `out` [M, N] bf16, and the library's split-K scratch is a fixed array inside
    the library image instead of lazily allocated memory. Limits: M <= 64, N <= 32768 (ValueError
    beyond). Calls on one device share that array, so calls that could overlap on the GPU must be
    ordered by the caller; make the first call on a device before any stream capture."""
    for t, name in ((a, "a"), (packed, "packed"), (scales, "scales"), (out, "out")):
        _check_cuda_contig(t, name)
    _check(a.dtype == torch.bfloat16 and a.dim() == 2, "w4gemm_noalloc expects a 2-D bfloat16 a")
    _check(packed.dtype == torch.int32 and packed.dim() == 2, "packed must be the int32 [N/16, 2K] tensor from w4_repack")
    M, K = a.shape
    N = packed.shape[0] * 16
    _check(packed.shape[1] == 2 * K, f"packed is {list(packed.shape)}, expected [N/16, {2 * K}]")
    _check(scales.dtype == torch.bfloat16 and tuple(scales.shape) == (K // W4_GROUP, N),
           f"scales must be bfloat16 [{K // W4_GROUP}, {N}]")
    if zeros is not None:
        _check_cuda_contig(zeros, "zeros")
        _check(zeros.dtype == torch.uint8 and tuple(zeros.shape) == (K // W4_GROUP, N), "zeros must be uint8 [K/128, N]")
    _check(out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N) and out.device == a.device,
           "out must be bfloat16 [M, N] on a's device")
    with torch.cuda.device(a.device):
        _status(_spk_w4gemm_noalloc(a.data_ptr(), packed.data_ptr(), scales.data_ptr(), _ptr(zeros),
                                    out.data_ptr(), M, N, K, _stream(a)))
    return out
