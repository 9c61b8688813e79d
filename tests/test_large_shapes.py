"""GPU parity of the fp8 / fp4 tensor-core GEMMs at the sizes the headline numbers are quoted on
(4096^3 and 8192^3) and on shapes that give every persistent CTA many tiles.

A full CPU product at 8192^3 is hours of oracle time, so each case runs the GPU GEMM once and
checks sampled rows of the result over ALL columns against the oracle computed on exactly those
rows (a row of C depends on one row of A and all of Bt, so a row subset of A gives the same
numbers; the reference's own bench samples 4,096 outputs at these sizes,
src/bench/bench_fp8gemm.cu:316-333). The sample always holds the first and last row of the first
and last row tile, so the last row tile and (all columns being compared) the last column tile are
covered. Operands come from the CUDA quantizers, which the quantizer tests pin byte for byte.
Tolerance: tests/parity.py (1e-2 relative or 2 bf16 ulps).
"""

import numpy as np
import pytest
import torch

from tests.parity import assert_bf16_close, t2n

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
SQUARES = [4096, 8192]
# (M, N, K): many tiles per persistent CTA with odd tile counts, a ragged last row tile, and one N that
# is not a multiple of 256 (128-column tiles): 19 x 125 = 2375 and 19 x 251 = 4769 tiles on 148 / 296 CTAs
MANY_TILES = [(2400, 32000, 512), (2432, 32128, 256)]


def _rows(M: int, n: int = 64, seed: int = 0) -> np.ndarray:
    fixed = {0, min(127, M - 1), max(0, M - 128), M - 1, M // 2}
    rng = np.random.default_rng(seed + M)
    more = rng.choice(M, size=min(M, n), replace=False)
    return np.array(sorted(fixed | set(int(r) for r in more)), dtype=np.int64)


def _randn_bf16(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)


def _reblock(sf: np.ndarray, rows: np.ndarray, total_rows: int, cols: int, orc) -> np.ndarray:
    """Blocked scale bytes of the sampled `rows` of a [total_rows][cols] scale matrix, re-laid out as
    the blocked scales of a matrix that holds only those rows."""
    j = np.arange(cols)

    def offsets(r, nrows):
        tile = (r[:, None] // 128) * ((cols + 3) // 4) + j[None, :] // 4
        return tile * 512 + (r[:, None] % 32) * 16 + ((r[:, None] // 32) % 4) * 4 + j[None, :] % 4

    out = np.zeros(((len(rows) + 127) // 128) * 128 * cols, np.uint8)
    out[offsets(np.arange(len(rows)), len(rows))] = sf[offsets(rows, total_rows)]
    assert orc.fp4_sf_offset(int(rows[-1]), cols - 1, cols) == int(offsets(rows[-1:], total_rows)[0, -1])
    return out


def _check_rows(got: torch.Tensor, rows: np.ndarray, want_bits: np.ndarray, what: str):
    assert_bf16_close(got[torch.from_numpy(rows).cuda()], want_bits, what)


def _shapes():
    return [(s, s, s) for s in SQUARES] + MANY_TILES


@pytest.mark.parametrize("shape", _shapes(), ids=lambda s: "x".join(map(str, s)))
def test_fp8gemm_per_tensor_sampled_rows(sk, orc, shape):
    M, N, K = shape
    qa, sa = sk.fp8_quantize(_randn_bf16(M, K, 1), "tensor")
    qb, sb = sk.fp8_quantize(_randn_bf16(N, K, 2), "tensor")
    got = sk.fp8gemm(qa, qb, sa, sb)
    assert sk._C.device_status() == 0
    rows = _rows(M)
    want = orc.fp8gemm(t2n(qa)[rows], t2n(qb), float(sa.item()), float(sb.item()))
    _check_rows(got, rows, want, f"fp8 per-tensor {shape}")


@pytest.mark.parametrize("shape", _shapes(), ids=lambda s: "x".join(map(str, s)))
def test_fp8gemm_mx_sampled_rows(sk, orc, shape):
    M, N, K = shape
    qa, sfa = sk.fp8_quantize(_randn_bf16(M, K, 3) * 8, "mx")
    qb, sfb = sk.fp8_quantize(_randn_bf16(N, K, 4) * 8, "mx")
    got = sk.fp8gemm(qa, qb, sfa=sfa, sfb=sfb)
    assert sk._C.device_status() == 0
    rows = _rows(M)
    want = orc.fp8gemm(t2n(qa)[rows], t2n(qb), 1.0, 1.0, np.ascontiguousarray(t2n(sfa)[rows]), t2n(sfb))
    _check_rows(got, rows, want, f"fp8 mx {shape}")


@pytest.mark.parametrize("shape", [(4096, 4096, 4096), (8192, 8192, 8192), (2400, 32000, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fp8gemm_block128_sampled_rows(sk, orc, shape):
    """fp32 1 x 128 / 128 x 128 block scales (no such mode in the reference: parity unpinned, the
    oracle is the definition)."""
    M, N, K = shape
    qa, sa = sk.fp8_quantize_block128(_randn_bf16(M, K, 5).float(), 1)
    qb, sb = sk.fp8_quantize_block128(_randn_bf16(N, K, 6).float(), 128)
    got = sk.fp8gemm_block128(qa, qb, sa, sb)
    assert sk._C.device_status() == 0
    rows = _rows(M, n=24)
    want = orc.fp8gemm_block128(t2n(qa)[rows], t2n(qb), np.ascontiguousarray(t2n(sa)[rows]), t2n(sb))
    _check_rows(got, rows, want, f"fp8 block128 {shape}")


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("shape", _shapes(), ids=lambda s: "x".join(map(str, s)))
def test_fp4gemm_sampled_rows(sk, orc, shape, fmt):
    M, N, K = shape
    qa, sfa, sa = sk.fp4_quantize(_randn_bf16(M, K, 7) * 2, fmt)
    qb, sfb, sb = sk.fp4_quantize(_randn_bf16(N, K, 8) * 2, fmt)
    kw = {} if fmt == "mxfp4" else dict(scale_a=sa.reshape(1), scale_b=sb.reshape(1))
    got = sk.fp4gemm(qa, qb, sfa, sfb, fmt=fmt, **kw)
    assert sk._C.device_status() == 0
    rows = _rows(M)
    cols = K // (16 if fmt == "nvfp4" else 32)
    sfa_rows = _reblock(t2n(sfa), rows, M, cols, orc)
    fa, fb = (1.0, 1.0) if fmt == "mxfp4" else (float(sa.item()), float(sb.item()))
    want = orc.fp4gemm(t2n(qa)[rows], t2n(qb), sfa_rows, t2n(sfb), fa, fb, fmt)
    _check_rows(got, rows, want, f"fp4 {fmt} {shape}")


def test_block128_recipe_against_plain_fp32_torch(sk, orc):
    """The fp32-block recipe restated a second time, independently of the C oracle, in plain fp32 torch
    on the CPU: dequantize both operands with their block scales and multiply. Pins the oracle's
    definition (and so the kernel) to the formula in the header: C = sum_kb (A8 B8^T)_kb sA sB."""
    rng = np.random.default_rng(21)
    M, N, K = 48, 256, 512
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((N, K)).astype(np.float32)
    qa, sa = orc.fp8_block128_quantize(a, 1)
    qb, sb = orc.fp8_block128_quantize(b, 128)
    # independent quantizer check: s = amax / 448 per block, q = e4m3(x / s)
    amax_a = np.abs(a.reshape(M, K // 128, 128)).max(-1)
    assert np.array_equal(sa, np.where(amax_a > 0, amax_a / np.float32(448.0), np.float32(1.0)).astype(np.float32))
    da = torch.from_numpy(orc.e4m3_to_f32(qa)).double() * torch.from_numpy(np.repeat(sa, 128, axis=1)).double()
    db = torch.from_numpy(orc.e4m3_to_f32(qb)).double() * torch.from_numpy(np.repeat(np.repeat(sb, 128, axis=0), 128, axis=1)).double()
    want = (da @ db.T).float()
    oracle_out = torch.from_numpy(orc.bf16_to_f32(orc.fp8gemm_block128(qa, qb, sa, sb)))
    assert torch.allclose(oracle_out, want, rtol=1e-2, atol=1e-2)
    got = sk.fp8gemm_block128(torch.from_numpy(qa).cuda().view(E4M3), torch.from_numpy(qb).cuda().view(E4M3),
                              torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda())
    assert torch.allclose(got.float().cpu(), want, rtol=1e-2, atol=1e-2)
