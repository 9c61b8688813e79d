"""Python-level wrappers of the quantized-GEMM ops: the surface of the reference's
python/spark_kernels/ops.py:196-353 for this path (same names, arguments and defaults)."""

from __future__ import annotations

import torch

from . import _C

W4_GROUP = 128  # k per scale (and zero point) of the int4 weights


def w4_quantize(w: torch.Tensor, asym: bool = False):
    """Round-to-nearest int4 quantization of a [K, N] bfloat16 weight (the x @ w layout), one
    scale per 128 consecutive k of a column, computed in fp32.

    Symmetric: s = bf16(max|w| / 7), q = clamp(rint(w / s), -8, 7) + 8, so w ~ (q - 8) s.
    asym=True: lo = min(min w, 0), hi = max(max w, 0), s = bf16((hi - lo) / 15),
    z = clamp(rint(-lo / s), 0, 15), q = clamp(rint(w / s) + z, 0, 15), so w ~ (q - z) s.
    Returns (qweight [K/8, N] int32 in GPTQ's packing, scales [K/128, N] bf16, zeros uint8 or
    None). K must be a multiple of 128 and N of 16."""
    return _C.w4_quantize(w, asym)


def w4_repack(qweight: torch.Tensor) -> torch.Tensor:
    """qweight [K/8, N] int32 -> the layout `w4gemm` streams, int32 [N/16, 2K]. Once per weight."""
    return _C.w4_repack(qweight)


class W4Weight:
    """An int4 weight ready for `w4gemm`: repacked codes, scales and optional zero points of a
    [K, N] (in_features x out_features) matrix."""

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor | None = None):
        self.packed = packed
        self.scales = scales
        self.zeros = zeros

    @staticmethod
    def quantize(w: torch.Tensor, asym: bool = False) -> "W4Weight":
        qweight, scales, zeros = w4_quantize(w, asym)
        return W4Weight(w4_repack(qweight), scales, zeros)

    @property
    def shape(self) -> tuple[int, int]:
        """(K, N) of the weight it stands for."""
        return self.packed.shape[1] // 2, self.packed.shape[0] * 16

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.packed, self.scales, self.zeros) if t is not None)


def w4gemm(a: torch.Tensor, w, scales: torch.Tensor | None = None, zeros: torch.Tensor | None = None,
           variant: int = -1, out: torch.Tensor | None = None) -> torch.Tensor:
    """W4A16 GEMM: a [M, K] bf16 @ int4 weight [K, N] -> [M, N] bf16, fp32 accumulate. `w` is a
    `W4Weight`, or the packed codes with `scales` (and `zeros`) given separately. Every product
    uses the weight bf16((q - z) s), rounded once. K % 128 == 0, N % 16 == 0, any M >= 1.
    Variant 2 (default) is the bulk-copy weight stream, 3 its batch-invariant form, 0 and 1
    the simple rungs below."""
    if isinstance(w, W4Weight):
        if scales is not None or zeros is not None:
            raise ValueError("pass scales and zeros inside the W4Weight, not separately")
        w, scales, zeros = w.packed, w.scales, w.zeros
    if scales is None:
        raise ValueError("w4gemm needs the scales of the packed weight")
    return _C.w4gemm(a, w, scales, zeros, variant, out)


class W4GateUpWeight(W4Weight):
    """The fused [gate | up] weight of an MLP, [K, 2 I], quantized and repacked with its 16-column strips
    alternating gate, up, so that `w4gemm_swiglu` can apply SwiGLU in the GEMM's epilogue. Not usable with
    plain `w4gemm` (the column order differs). An addition to the reference's surface."""

    @staticmethod
    def quantize(w_gate_up: torch.Tensor, asym: bool = False) -> "W4GateUpWeight":
        qweight, scales, zeros = w4_quantize(w_gate_up, asym)
        q2, s2, z2 = _C.w4_interleave_gate_up(qweight, scales, zeros)
        return W4GateUpWeight(w4_repack(q2), s2, z2)


def w4gemm_swiglu(a: torch.Tensor, w: W4GateUpWeight, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] bf16 @ fused int4 gate|up weight [K, 2 I] -> silu(gate) * up, [M, I] bf16, in one GEMM launch
    per 64 tokens: the activation runs in the GEMM's epilogue on the fp32 sums (the reference runs `w4gemm`
    and then `swiglu` on its bf16 output, python/spark_kernels/engine.py:447-451). I % 64 == 0, K % 256 == 0."""
    if not isinstance(w, W4GateUpWeight):
        raise ValueError("w4gemm_swiglu needs a W4GateUpWeight (strips interleaved gate, up)")
    return _C.w4gemm_swiglu(a, w.packed, w.scales, w.zeros, out)


def num_variants(name: str) -> int:
    return _C.num_variants(name)


def fp8gemm(a, b_t, scale_a=None, scale_b=None, variant: int = -1, sfa=None, sfb=None):
    """fp8 GEMM: (scale_a * scale_b) * (a @ b_t.T) -> [M, N] bf16, fp32 accumulate. a [M, K] and
    b_t [N, K] are float8_e4m3fn, K-contiguous (b_t as nn.Linear stores a weight). scale_a / scale_b
    are one-element float32 CUDA tensors. With `sfa` [M, K/32] and `sfb` [N, K/32] (uint8 E8M0,
    exponent + 127) every product is also scaled by its two block scales (MXFP8; K % 256 == 0) and
    the per-tensor scales may be omitted. N and K multiples of 64, any M >= 1 (variant 1, 3, 4)."""
    return _C.fp8gemm(a, b_t, scale_a, scale_b, variant, sfa, sfb)


def fp8_quantize(x, mode: str = "tensor"):
    """bf16 [rows, K] -> (e4m3, scale): "tensor" one power-of-two fp32 scale [1], "row" one per row
    [rows, 1], "mx" a uint8 E8M0 byte per 32 values [rows, K/32] (the OCP recipe). Elements are
    x / scale rounded to nearest even, saturating at 448."""
    return _C.fp8_quantize(x, mode)


def fp4_quantize(x, fmt: str = "nvfp4", scale=None):
    """bf16 [rows, K] -> (q uint8 [rows, K/2], sf blocked uint8, scale). nvfp4: e4m3 scale per 16 on
    a per-tensor fp32 decode scale (`scale`, or max|x| / (6 * 448) computed on the device);
    mxfp4: E8M0 scale per 32, scale None."""
    return _C.fp4_quantize(x, fmt, scale)


def fp4gemm(a, b_t, sfa, sfb, scale_a=None, scale_b=None, fmt: str = "nvfp4", variant: int = -1):
    """fp4 block-scaled GEMM: scale_a * scale_b * (A @ B_t.T) -> [M, N] bf16. a [M, K/2], b_t [N, K/2]
    packed e2m1, sfa / sfb blocked block scales. N % 64 == 0, K % 256 == 0, any M (variant 1)."""
    return _C.fp4gemm(a, b_t, sfa, sfb, scale_a, scale_b, fmt, variant)


def grouped_gemm_fp8(a, w, offsets, scale_a=None, scale_b=None):
    """Grouped fp8 GEMM over the experts of a mixture-of-experts layer, one launch, no host sync: row r of a [T, K]
    (sorted by expert, expert e owning rows offsets[e] .. offsets[e + 1] - 1) times w[e]^T, w [E, N, K] -> bf16 [T, N]
    scaled by scale_a [1] * scale_b[e]. N % 128 == 0, K % 128 == 0, E <= 512."""
    return _C.grouped_gemm_fp8(a, w, offsets, scale_a, scale_b, False)


def grouped_gemm_swiglu_fp8(a, w, offsets, scale_a=None, scale_b=None):
    """The same with the SwiGLU of an expert's MLP in the epilogue: w rows alternate gate_j, up_j; -> bf16 [T, N / 2]."""
    return _C.grouped_gemm_fp8(a, w, offsets, scale_a, scale_b, True)


def fp8_quantize_block128(x, block_rows: int):
    return _C.fp8_quantize_block128(x, block_rows)


def fp8gemm_block128(a, b_t, scale_a_blocks, scale_b_blocks):
    return _C.fp8gemm_block128(a, b_t, scale_a_blocks, scale_b_blocks)
