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
_spk_w4_interleave_gate_up = _sig("spk_w4_interleave_gate_up", [_p, _p, _p, _p, _p, _p, _i, _i, _p])
_spk_w4gemm_swiglu = _sig("spk_w4gemm_swiglu_bf16", [_p, _p, _p, _p, _p, _i, _i, _i, _p])
_spk_w4_prefill_reserve = _sig("spk_w4_prefill_reserve", [ctypes.c_longlong])
_spk_w4gemm_noalloc_status = _sig("spk_w4gemm_noalloc_status", [_p, ctypes.POINTER(_i)])
_spk_debug_expire_wait = _sig("spk_debug_expire_wait", [_i, _p])
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


def w4_interleave_gate_up(qweight: torch.Tensor, scales: torch.Tensor, zeros=None):
    """GPTQ-order tensors of a fused [gate | up] weight -> the same tensors with their 16-column strips
    alternating gate, up (what `w4gemm_swiglu` expects after `w4_repack`). An addition to the reference's surface."""
    for t, name in ((qweight, "qweight"), (scales, "scales")):
        _check_cuda_contig(t, name)
    _check(qweight.dtype == torch.int32 and qweight.dim() == 2, "qweight must be int32 [K/8, N]")
    K, N2 = qweight.shape[0] * 8, qweight.shape[1]
    _check(scales.dtype == torch.bfloat16 and tuple(scales.shape) == (K // W4_GROUP, N2), "scales must be bfloat16 [K/128, N]")
    if zeros is not None:
        _check_cuda_contig(zeros, "zeros")
        _check(zeros.dtype == torch.uint8 and tuple(zeros.shape) == (K // W4_GROUP, N2), "zeros must be uint8 [K/128, N]")
    with torch.cuda.device(qweight.device):
        q2, s2 = torch.empty_like(qweight), torch.empty_like(scales)
        z2 = None if zeros is None else torch.empty_like(zeros)
        _status(_spk_w4_interleave_gate_up(qweight.data_ptr(), scales.data_ptr(), _ptr(zeros), q2.data_ptr(), s2.data_ptr(),
                                           _ptr(z2), K, N2, _stream(qweight)))
    return q2, s2, z2


def w4gemm_swiglu(a: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, zeros=None, out=None) -> torch.Tensor:
    """bf16 [M, N/2] = silu(a Wgate) * (a Wup) for a gate|up weight whose strips were interleaved with
    `w4_interleave_gate_up` before `w4_repack`. An addition to the reference's surface."""
    for t, name in ((a, "a"), (packed, "packed"), (scales, "scales")):
        _check_cuda_contig(t, name)
    _check(a.dtype == torch.bfloat16 and a.dim() == 2, "w4gemm_swiglu expects a 2-D bfloat16 a")
    _check(packed.dtype == torch.int32 and packed.dim() == 2, "packed must be the int32 [N/16, 2K] tensor from w4_repack")
    M, K = a.shape
    N2 = packed.shape[0] * 16
    _check(packed.shape[1] == 2 * K, f"packed is {list(packed.shape)}, expected [N/16, {2 * K}]")
    _check(scales.dtype == torch.bfloat16 and tuple(scales.shape) == (K // W4_GROUP, N2), f"scales must be bfloat16 [{K // W4_GROUP}, {N2}]")
    if zeros is not None:
        _check_cuda_contig(zeros, "zeros")
        _check(zeros.dtype == torch.uint8 and tuple(zeros.shape) == (K // W4_GROUP, N2), "zeros must be uint8 [K/128, N]")
    with torch.cuda.device(a.device):
        if out is None:
            out = torch.empty((M, N2 // 2), dtype=torch.bfloat16, device=a.device)
        else:
            _check(out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N2 // 2) and out.is_contiguous(), "out must be contiguous bfloat16 [M, N/2]")
        _status(_spk_w4gemm_swiglu(a.data_ptr(), packed.data_ptr(), scales.data_ptr(), _ptr(zeros), out.data_ptr(), M, N2, K, _stream(a)))
    return out


def w4_prefill_reserve(nbytes: int, device=None) -> None:
    """Size the bf16 scratch of the many-token route of w4gemm (N * K * 2 bytes of the largest weight) now,
    e.g. before capturing a CUDA graph."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _status(_spk_w4_prefill_reserve(int(nbytes)))


def w4gemm_noalloc_status(device=None) -> int:
    """Waits for the current stream and returns the status word of `w4gemm_noalloc` on the device
    (0, or 3 after a bounded wait of its kernel gave up), clearing it. Allocates nothing; it is not
    the word `device_status` reads."""
    code = _i(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _status(_spk_w4gemm_noalloc_status(torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(code)))
    return code.value


def debug_expire_wait(dirty: int = 0, device=None) -> None:
    """Test hook: a kernel whose bounded wait runs out (status 3 afterwards) and that leaves `dirty`
    words of the split-K scratch non-zero, as an interrupted GEMM would."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _status(_spk_debug_expire_wait(int(dirty), torch.cuda.current_stream(dev).cuda_stream))


_spk_stream_probe = _sig("spk_stream_probe", [_p, ctypes.c_longlong, _i, _i, _p])


def stream_probe(buf: torch.Tensor, ctas: int, depth: int) -> None:
    """Read-only stream over `buf` (CUDA, contiguous, a multiple of 4096 bytes) by `ctas` CTAs with
    `depth` 4 KiB bulk copies in flight each; time it with CUDA events (launch-rule calibration, read floor)."""
    _check_cuda_contig(buf, "buf")
    nbytes = buf.numel() * buf.element_size()
    with torch.cuda.device(buf.device):
        _status(_spk_stream_probe(buf.data_ptr(), nbytes, int(ctas), int(depth), _stream(buf)))


# ---- fp8 --------------------------------------------------------------------------------------

_u8p = _p
_spk_fp8_quantize = _sig("spk_fp8_quantize", [_p, _p, _p, _p, _i, _i, _i, _p])
_spk_fp8gemm = _sig("spk_fp8gemm", [_p, _p, _p, _i, _i, _i, _p, _p, _i, _p])
_spk_fp8gemm_mx = _sig("spk_fp8gemm_mx", [_p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _i, _p])
_spk_fp8gemm_block128 = _sig("spk_fp8gemm_block128", [_p, _p, _p, _i, _i, _i, _p, _p, _p])
_spk_fp8_quantize_block128 = _sig("spk_fp8_quantize_block128", [_p, _p, _p, _i, _i, _i, _p])
_sig("spk_fp8gemm_num_variants", [])
_sig("spk_fp8gemm_default_variant", [])
_sig("spk_fp8gemm_supports", [_i, _i, _i, _i])
_sig("spk_fp8gemm_mx_supports", [_i, _i, _i, _i])
_sig("spk_fp8gemm_v3_set_route", [_i], None)
_sig("spk_fp8gemm_v3_route", [])
_sig("spk_fp8gemm_v3_num_tiles", [])
_sig("spk_fp8gemm_v3_route_name", [_i, _i, _i, _i], ctypes.c_char_p)
_sig("spk_fp8gemm_v4_route_name", [_i, _i, _i], ctypes.c_char_p)
_spk_grouped_gemm_fp8 = _sig("spk_grouped_gemm_fp8", [_p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p])
_spk_grouped_gemm_swiglu_fp8 = _sig("spk_grouped_gemm_swiglu_fp8", [_p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p])
_sig("spk_grouped_gemm_supports", [_i, _i, _i])
_spk_fp4_scale_bytes = _sig("spk_fp4_scale_bytes", [_i, _i, _i], ctypes.c_size_t)
_spk_fp4_quantize = _sig("spk_fp4_quantize", [_p, _p, _p, _i, _i, _p, _i, _p, _p, _p])
_spk_fp4gemm = _sig("spk_fp4gemm", [_p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p])
_sig("spk_fp4gemm_num_variants", [])
_sig("spk_fp4gemm_supports", [_i, _i, _i, _i])

_FP8 = torch.float8_e4m3fn


def _scalar_ptrs(scale_a, scale_b, like, op):
    if scale_a is None:
        return None, None
    for sc in (scale_a, scale_b):
        _check(sc.is_cuda and sc.dtype == torch.float32 and sc.numel() == 1,
               "scale_a and scale_b must be float32 CUDA tensors with one element")
        _check(sc.device == like.device, "scales must be on a's device")
    return scale_a.data_ptr(), scale_b.data_ptr()


def fp8gemm(a, b_t, scale_a=None, scale_b=None, variant: int = -1, sfa=None, sfb=None):
    """(scale_a * scale_b) * (a @ b_t.T) -> bf16 [M, N]; a [M, K], b_t [N, K] float8_e4m3fn. With
    sfa [M, K/32] / sfb [N, K/32] uint8: MX mode (reference python/csrc/bindings.cpp:333-400)."""
    _check_cuda_contig(a, "a")
    _check_cuda_contig(b_t, "b_t")
    _check(a.dtype == _FP8 and b_t.dtype == _FP8, "fp8gemm expects float8_e4m3fn inputs")
    _check(a.dim() == 2 and b_t.dim() == 2, "fp8gemm expects 2-D tensors")
    _check(a.shape[1] == b_t.shape[1],
           f"inner dimensions mismatch: a is {a.shape[0]}x{a.shape[1]}, b_t is {b_t.shape[0]}x{b_t.shape[1]} (b_t is [N, K])")
    mx = sfa is not None or sfb is not None
    _check(not mx or (sfa is not None and sfb is not None),
           "fp8gemm: sfa and sfb must both be given (MX mode) or both be None")
    _check(mx or (scale_a is not None and scale_b is not None),
           "fp8gemm: scale_a and scale_b are required without block scales")
    _check((scale_a is None) == (scale_b is None), "fp8gemm: scale_a and scale_b must both be given or both be None")
    sa, sb = _scalar_ptrs(scale_a, scale_b, a, "fp8gemm")
    _check(_aligned16(a) and _aligned16(b_t), "fp8gemm needs 16-byte aligned a and b_t storage")
    M, K = a.shape
    N = b_t.shape[0]
    if mx:
        _check(K % 256 == 0, f"fp8gemm with block scales needs K a multiple of 256, got {K}")
        for sf, name, rows in ((sfa, "sfa", M), (sfb, "sfb", N)):
            _check_cuda_contig(sf, name)
            _check(sf.dtype == torch.uint8, f"{name} must be uint8 (ue8m0: exponent + 127)")
            _check(sf.dim() == 2 and tuple(sf.shape) == (rows, K // 32), f"{name} must be [{rows}, {K // 32}], got {list(sf.shape)}")
            _check(sf.device == a.device, f"{name} must be on a's device")
            _check(_aligned16(sf), f"{name} needs 16-byte aligned storage")
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        sup = _lib.spk_fp8gemm_mx_supports if mx else _lib.spk_fp8gemm_supports
        v = _lib.spk_fp8gemm_default_variant() if variant < 0 else _resolve_variant(variant, _lib.spk_fp8gemm_num_variants())
        while variant < 0 and v > 0 and not sup(M, N, K, v):
            v -= 1
        if mx:
            _status(_spk_fp8gemm_mx(a.data_ptr(), b_t.data_ptr(), c.data_ptr(), M, N, K, sa, sb, sfa.data_ptr(),
                                    sfb.data_ptr(), v, _stream(a)))
        else:
            _status(_spk_fp8gemm(a.data_ptr(), b_t.data_ptr(), c.data_ptr(), M, N, K, sa, sb, v, _stream(a)))
    return c


def grouped_gemm_fp8(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, scale_a=None, scale_b=None, swiglu: bool = False):
    """Every expert's fp8 GEMM in one launch (reference python/csrc/bindings.cpp grouped_gemm_fp8 /
    grouped_gemm_swiglu_fp8): a e4m3 [T, K] with rows sorted by expert, w e4m3 [E, N, K], offsets int32 [E + 1] on the
    device, scale_a f32 [1] and scale_b f32 [E] (or None) -> bf16 [T, N], or [T, N / 2] = silu(gate) * up with `swiglu`
    (w rows alternating gate_j, up_j)."""
    for t, name in ((a, "a"), (w, "w"), (offsets, "offsets")):
        _check_cuda_contig(t, name)
    _check(a.dtype == _FP8 and w.dtype == _FP8 and a.dim() == 2 and w.dim() == 3, "grouped_gemm_fp8 expects float8_e4m3fn a [T, K] and w [E, N, K]")
    T, K = a.shape
    E, N, K2 = w.shape
    _check(K2 == K, "inner dimensions mismatch")
    _check(offsets.dtype == torch.int32 and tuple(offsets.shape) == (E + 1,), "offsets must be int32 [E + 1]")
    for sc, n, name in ((scale_a, 1, "scale_a"), (scale_b, E, "scale_b")):
        if sc is not None:
            _check_cuda_contig(sc, name)
            _check(sc.dtype == torch.float32 and sc.numel() == n, f"{name} must be float32 with {n} element(s)")
    with torch.cuda.device(a.device):
        out = torch.empty((T, N // 2 if swiglu else N), dtype=torch.bfloat16, device=a.device)
        fn = _spk_grouped_gemm_swiglu_fp8 if swiglu else _spk_grouped_gemm_fp8
        _status(fn(a.data_ptr(), w.data_ptr(), offsets.data_ptr(), out.data_ptr(), T, E, N, K, _ptr(scale_a), _ptr(scale_b), _stream(a)))
    return out


def fp8gemm_v3_set_route(route: int) -> int:
    prev = _lib.spk_fp8gemm_v3_route()
    n = _lib.spk_fp8gemm_v3_num_tiles()
    _check(-2 <= route < n, f"fp8gemm_v3_set_route: {route} is not -1, -2 or a tile in [0, {n})")
    _lib.spk_fp8gemm_v3_set_route(route)
    return prev


def fp8gemm_v3_route_name(M: int, N: int, K: int, mx: bool = False) -> str:
    return _lib.spk_fp8gemm_v3_route_name(M, N, K, int(mx)).decode()


def fp8gemm_v3_num_tiles() -> int:
    return _lib.spk_fp8gemm_v3_num_tiles()


def fp8gemm_v4_route_name(M: int, N: int, K: int) -> str:
    return _lib.spk_fp8gemm_v4_route_name(M, N, K).decode()


def fp8_quantize(x: torch.Tensor, mode: str = "tensor"):
    """bf16 [rows, K] -> (e4m3 [rows, K], scales): f32 [1] ("tensor"), f32 [rows, 1] ("row") or
    uint8 [rows, K/32] ("mx") (reference python/csrc/bindings.cpp:489-527)."""
    _check_cuda_contig(x, "x")
    _check(x.dtype == torch.bfloat16, "fp8_quantize expects bfloat16 x")
    _check(x.dim() == 2, "fp8_quantize expects a 2-D [rows, K] tensor")
    _check(_aligned16(x), "fp8_quantize needs 16-byte aligned x storage")
    rows, K = x.shape
    _check(mode in ("tensor", "row", "mx"), f"fp8_quantize mode must be 'tensor', 'row' or 'mx', got {mode}")
    m = {"tensor": 0, "row": 1, "mx": 2}[mode]
    _check(K % (32 if m == 2 else 8) == 0, f"fp8_quantize needs K a multiple of 8 (32 for mx), got {K}")
    _check(rows > 0 and K > 0, "fp8_quantize needs a non-empty x")
    with torch.cuda.device(x.device):
        q = torch.empty((rows, K), dtype=_FP8, device=x.device)
        work = None
        if m == 0:
            work = torch.zeros(2, dtype=torch.float32, device=x.device)  # [amax bits, scale]
            scale = work[1:2]
        elif m == 1:
            scale = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
        else:
            scale = torch.empty((rows, K // 32), dtype=torch.uint8, device=x.device)
        _status(_spk_fp8_quantize(x.data_ptr(), q.data_ptr(), scale.data_ptr(), _ptr(work), rows, K, m, _stream(x)))
    return q, scale


def fp8_quantize_block128(x: torch.Tensor, block_rows: int):
    """float32 [rows, K] -> (e4m3 [rows, K], f32 scales [cdiv(rows, block_rows), K/128]); an
    addition to the reference's surface (fp32 block scales: 1 for activations, 128 for weights)."""
    _check_cuda_contig(x, "x")
    _check(x.dtype == torch.float32 and x.dim() == 2, "fp8_quantize_block128 expects a 2-D float32 x")
    rows, K = x.shape
    with torch.cuda.device(x.device):
        q = torch.empty((rows, K), dtype=_FP8, device=x.device)
        s = torch.empty(((rows + block_rows - 1) // block_rows, K // 128), dtype=torch.float32, device=x.device)
        _status(_spk_fp8_quantize_block128(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, K, block_rows, _stream(x)))
    return q, s


def fp8gemm_block128(a, b_t, scale_a_blocks, scale_b_blocks):
    """fp8 GEMM with fp32 block scales (a: 1x128 blocks [M, K/128], b_t: 128x128 blocks
    [cdiv(N,128), K/128]) -> bf16 [M, N]; an addition to the reference's surface."""
    for t, name in ((a, "a"), (b_t, "b_t"), (scale_a_blocks, "scale_a_blocks"), (scale_b_blocks, "scale_b_blocks")):
        _check_cuda_contig(t, name)
    _check(a.dtype == _FP8 and b_t.dtype == _FP8 and a.dim() == 2 and b_t.dim() == 2, "fp8gemm_block128 expects 2-D float8_e4m3fn a, b_t")
    M, K = a.shape
    N = b_t.shape[0]
    _check(b_t.shape[1] == K, "inner dimensions mismatch")
    _check(K % 128 == 0, f"fp8gemm_block128 needs K a multiple of 128, got {K}")
    _check(scale_a_blocks.dtype == torch.float32 and tuple(scale_a_blocks.shape) == (M, K // 128), "scale_a_blocks must be f32 [M, K/128]")
    _check(scale_b_blocks.dtype == torch.float32 and tuple(scale_b_blocks.shape) == ((N + 127) // 128, K // 128),
           "scale_b_blocks must be f32 [cdiv(N,128), K/128]")
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        _status(_spk_fp8gemm_block128(a.data_ptr(), b_t.data_ptr(), c.data_ptr(), M, N, K, scale_a_blocks.data_ptr(),
                                      scale_b_blocks.data_ptr(), _stream(a)))
    return c


# ---- fp4 --------------------------------------------------------------------------------------

def _fp4_format(fmt: str) -> int:
    _check(fmt in ("nvfp4", "mxfp4"), f"fp4 format must be 'nvfp4' or 'mxfp4', got '{fmt}'")
    return 0 if fmt == "nvfp4" else 1


_FP4X2 = getattr(torch, "float4_e2m1fn_x2", None)
_E8M0 = getattr(torch, "float8_e8m0fnu", None)


def fp4_scale_bytes(rows: int, K: int, fmt: str = "nvfp4") -> int:
    return int(_spk_fp4_scale_bytes(rows, K, _fp4_format(fmt)))


def _check_fp4_bytes(t, name):
    _check_cuda_contig(t, name)
    _check(t.dtype == torch.uint8 or (_FP4X2 is not None and t.dtype == _FP4X2),
           f"{name} must be uint8 or float4_e2m1fn_x2 (packed e2m1), got {t.dtype}")
    _check(t.dim() == 2, f"{name} must be 2-D [rows, K / 2]")
    _check(_aligned16(t), f"{name} needs 16-byte aligned storage")


def _check_fp4_scales(t, name, rows, K, format, like):
    _check_cuda_contig(t, name)
    ok = t.dtype == torch.uint8 or (format == 0 and t.dtype == _FP8) or (format == 1 and _E8M0 is not None and t.dtype == _E8M0)
    _check(ok, f"{name} must be uint8 or the format's float8 scale type, got {t.dtype}")
    want = int(_spk_fp4_scale_bytes(rows, K, format))
    _check(t.numel() == want, f"{name} must hold the blocked scale layout of {rows} rows ({want} bytes, rows padded to 128), got {t.numel()}")
    _check(t.device == like.device, f"{name} must be on a's device")
    _check(_aligned16(t), f"{name} needs 16-byte aligned storage")


def fp4_quantize(x: torch.Tensor, fmt: str = "nvfp4", scale=None):
    """(q uint8 [rows, K/2], sf uint8 flat blocked, scale 0-dim f32 | None)
    (reference python/csrc/bindings.cpp:446-487)."""
    _check_cuda_contig(x, "x")
    _check(x.dtype == torch.bfloat16, "fp4_quantize expects bfloat16 x")
    _check(x.dim() == 2, "fp4_quantize expects a 2-D [rows, K] tensor")
    _check(_aligned16(x), "fp4_quantize needs 16-byte aligned x storage")
    format = _fp4_format(fmt)
    rows, K = x.shape
    _check(K % (128 if format == 1 else 64) == 0, f"fp4_quantize needs K a multiple of 64 (nvfp4) or 128 (mxfp4), got {K}")
    with torch.cuda.device(x.device):
        s, work = None, None
        if format == 0:
            if scale is not None:
                _check(scale.is_cuda and scale.dtype == torch.float32 and scale.numel() == 1 and scale.device == x.device,
                       "scale must be a float32 CUDA tensor with one element on x's device")
                s = scale.reshape(()).contiguous()
            else:
                work = torch.zeros(2, dtype=torch.float32, device=x.device)  # [amax bits, scale]
                s = work[1].reshape(())
        q = torch.empty((rows, K // 2), dtype=torch.uint8, device=x.device)
        sf = torch.empty((int(_spk_fp4_scale_bytes(rows, K, format)),), dtype=torch.uint8, device=x.device)
        _status(_spk_fp4_quantize(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, K, _ptr(s), format, _stream(x),
                                  _ptr(work), _ptr(s) if work is not None else None))
    return q, sf, s


def fp4gemm(a, b_t, sfa, sfb, scale_a=None, scale_b=None, fmt: str = "nvfp4", variant: int = -1):
    """scale_a * scale_b * (A @ B_t.T) for packed e2m1 a [M, K/2], b_t [N, K/2] with blocked block
    scales -> bf16 [M, N] (reference python/csrc/bindings.cpp:529-568)."""
    _check_fp4_bytes(a, "a")
    _check_fp4_bytes(b_t, "b_t")
    format = _fp4_format(fmt)
    _check(a.shape[1] == b_t.shape[1],
           f"inner dimensions mismatch: a is {a.shape[0]}x{a.shape[1]} bytes, b_t is {b_t.shape[0]}x{b_t.shape[1]} (both [rows, K / 2])")
    _check(b_t.device == a.device, "b_t must be on a's device")
    M, N, K = a.shape[0], b_t.shape[0], 2 * a.shape[1]
    _check((scale_a is None) == (scale_b is None), "fp4gemm: scale_a and scale_b must both be given or both be None")
    sa, sb = _scalar_ptrs(scale_a, scale_b, a, "fp4gemm")
    _check_fp4_scales(sfa, "sfa", M, K, format, a)
    _check_fp4_scales(sfb, "sfb", N, K, format, a)
    with torch.cuda.device(a.device):
        c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        v = _resolve_variant(variant, _lib.spk_fp4gemm_num_variants())
        while variant < 0 and v > 0 and not _lib.spk_fp4gemm_supports(M, N, K, v):
            v -= 1
        _status(_spk_fp4gemm(a.data_ptr(), b_t.data_ptr(), c.data_ptr(), M, N, K, sfa.data_ptr(), sfb.data_ptr(), sa, sb,
                             format, v, _stream(a)))
    return c


# ---- launch rules of the decode kernels (reference python/csrc/bindings.cpp:1797-1829) ----------

_sig("spk_device_shape_sm_count", [])
_sig("spk_device_shape_l2_bytes", [], _i64)
_sig("spk_device_shape_spec_gbps", [], ctypes.c_double)
_sig("spk_device_shape_bytes_in_flight", [], _i64)
_sig("spk_device_shape_forced", [])
_sig("spk_decode_split_k", [_i64, _i, _i, _i64, _i, _i])
_sig("spk_decode_need_ctas", [_i64, _i])
_sig("spk_decode_fits_l2", [_i64, _i])
_sig("spk_decode_force_split_k", [_i], None)
_sig("spk_decode_forced_split_k", [])


def _decode_device(device: str) -> int:
    table = {"": 0, "current": 0, "gb10": 1, "rtx5090": 2, "b200": 3}
    if device not in table:
        raise ValueError(f"device must be '', 'gb10', 'rtx5090' or 'b200', got '{device}'")
    return table[device]


def device_shape() -> dict:
    return {"sm_count": _lib.spk_device_shape_sm_count(), "l2_bytes": _lib.spk_device_shape_l2_bytes(),
            "spec_gbps": _lib.spk_device_shape_spec_gbps(), "bytes_in_flight": _lib.spk_device_shape_bytes_in_flight(),
            "forced": bool(_lib.spk_device_shape_forced())}


def split_k_for(weight_bytes: int, tiles: int, max_split: int, per_cta_in_flight: int, slots: int, device: str = "") -> int:
    _check(tiles >= 1 and max_split >= 1 and per_cta_in_flight >= 1 and slots >= 0,
           "split_k_for: tiles, max_split and per_cta_in_flight must be >= 1, slots >= 0")
    return _lib.spk_decode_split_k(weight_bytes, tiles, max_split, per_cta_in_flight, slots, _decode_device(device))


def need_ctas(per_cta_in_flight: int, device: str = "") -> int:
    _check(per_cta_in_flight >= 1, "need_ctas: per_cta_in_flight must be >= 1")
    return _lib.spk_decode_need_ctas(per_cta_in_flight, _decode_device(device))


def fits_l2(nbytes: int, device: str = "") -> bool:
    return bool(_lib.spk_decode_fits_l2(nbytes, _decode_device(device)))


def decode_force_split_k(split: int) -> None:
    _lib.spk_decode_force_split_k(split)


# ---- push all-reduce across the GPUs of one node (no counterpart in the reference) ---------------

_sig("spk_comm_buffer_bytes", [_i, ctypes.c_longlong], ctypes.c_longlong)
_sig("spk_comm_alloc", [ctypes.c_longlong, ctypes.POINTER(_p)])
_sig("spk_comm_free", [_p])
_sig("spk_comm_export", [_p, ctypes.c_char_p])
_sig("spk_comm_open", [ctypes.c_char_p, ctypes.POINTER(_p)])
_sig("spk_comm_close", [_p])
_sig("spk_comm_status", [_p, ctypes.POINTER(_i)])
_sig("spk_allreduce_push_bf16", [_p, ctypes.c_longlong, ctypes.POINTER(_p), _i, _i, ctypes.c_longlong, _p])
_sig("spk_allreduce_push_bf16_mode", [_p, ctypes.c_longlong, ctypes.POINTER(_p), _i, _i, ctypes.c_longlong, _i, _p])


def comm_alloc(world: int, slot_elems: int) -> int:
    """A zeroed device buffer for `world` ranks and tensors of up to slot_elems bf16 elements."""
    nbytes = _lib.spk_comm_buffer_bytes(world, slot_elems)
    _check(nbytes > 0, f"comm_alloc: world={world} slot_elems={slot_elems} not supported")
    ptr = _p()
    _status(_lib.spk_comm_alloc(nbytes, ctypes.byref(ptr)))
    return ptr.value


def comm_free(ptr: int) -> None:
    _status(_lib.spk_comm_free(ptr))


def comm_export(ptr: int) -> bytes:
    buf = ctypes.create_string_buffer(64)
    _status(_lib.spk_comm_export(ptr, buf))
    return buf.raw


def comm_open(handle: bytes) -> int:
    _check(len(handle) == 64, "comm_open: a CUDA IPC handle is 64 bytes")
    ptr = _p()
    _status(_lib.spk_comm_open(handle, ctypes.byref(ptr)))
    return ptr.value


def comm_close(ptr: int) -> None:
    _status(_lib.spk_comm_close(ptr))


def comm_status(local_ptr: int) -> int:
    code = _i(0)
    _status(_lib.spk_comm_status(local_ptr, ctypes.byref(code)))
    return code.value


def allreduce_push(t: torch.Tensor, ptrs, rank: int, slot_elems: int, mode: int = 0) -> torch.Tensor:
    """In-place sum of the contiguous bf16 tensor t over the ranks whose buffers are `ptrs`.
    mode 0: the library picks the form, 1: one phase, 2: two phases (reduce-scatter + all-gather), 3: two phases of
    flagged words, 4: one hop of flagged words."""
    _check_cuda_contig(t, "t")
    _check(t.dtype == torch.bfloat16, "allreduce_push: bf16 only")
    arr = (_p * len(ptrs))(*ptrs)
    with torch.cuda.device(t.device):
        _status(_lib.spk_allreduce_push_bf16_mode(t.data_ptr(), t.numel(), arr, rank, len(ptrs), slot_elems, int(mode), _stream(t)))
    return t
