"""The fused gate|up GEMM + SwiGLU epilogue against fp32 arithmetic on the oracle's dequantized weights.

No counterpart in the reference (it runs w4gemm and then a swiglu kernel on the bf16 output,
python/spark_kernels/engine.py:447-451); the definition checked here is
H = bf16( silu(g) * u ), g = A Wg, u = A Wu accumulated in fp32 on the bit-exact dequantized weights,
silu(x) = x / (1 + exp(-x)). Tolerance: tests/parity.py (1e-2 relative or 2 bf16 ulps, plus 2^-14 of the
output range); the unfused product path is checked to agree with the fused one to bf16 rounding of g and u."""

import numpy as np
import pytest
import torch

from tests.parity import assert_bf16_close, seeded_acts, seeded_weight, t2n

pytestmark = pytest.mark.gpu


def _reference(orc, a_bits, w: "torch.Tensor", asym: bool):
    """fp64 on the oracle's quantize -> repack -> dequantize of the fused [gate | up] weight."""
    qw, sc, z = orc.w4_quantize(t2n(w), asym)
    deq = orc.bf16_to_f32(orc.w4_dequantize(orc.w4_repack(qw), sc, z)).astype(np.float64)   # [K, 2 I]
    c = orc.bf16_to_f32(a_bits).astype(np.float64) @ deq
    inter = c.shape[1] // 2
    g, u = c[:, :inter], c[:, inter:]
    return orc.bf16_bits((g / (1.0 + np.exp(-g)) * u).astype(np.float32))


@pytest.mark.parametrize("asym", [False, True], ids=["sym", "asym"])
@pytest.mark.parametrize("M", [1, 5, 16, 33, 64, 100])
@pytest.mark.parametrize("K,inter", [(256, 64), (1024, 448), (4096, 1792)])
def test_w4gemm_swiglu_matches_fp32_reference(sk, orc, K, inter, M, asym):
    w = seeded_weight(K, 2 * inter, seed=31)
    ww = sk.W4GateUpWeight.quantize(w.cuda(), asym=asym)
    a = seeded_acts(M, K, seed=32)
    got = sk.w4gemm_swiglu(a.cuda(), ww)
    assert got.shape == (M, inter) and got.dtype == torch.bfloat16
    assert sk._C.device_status() == 0
    assert_bf16_close(got, _reference(orc, t2n(a), w, asym), f"w4gemm_swiglu M={M} K={K} I={inter}")


def test_interleaved_weight_is_a_column_permutation(sk, orc):
    """The interleave moves columns only: strip 2 i of the result is gate strip i, strip 2 i + 1 up strip i."""
    K, inter = 256, 128
    w = seeded_weight(K, 2 * inter, seed=33).cuda()
    qw, sc, z = sk.w4_quantize(w, True)
    q2, s2, z2 = sk._C.w4_interleave_gate_up(qw, sc, z)
    cols = []
    for i in range(inter // 16):
        cols += list(range(16 * i, 16 * i + 16)) + list(range(inter + 16 * i, inter + 16 * i + 16))
    idx = torch.tensor(cols, device="cuda")
    assert torch.equal(q2, qw[:, idx]) and torch.equal(s2, sc[:, idx]) and torch.equal(z2, z[:, idx])


def test_fused_agrees_with_gemm_then_swiglu(sk):
    """The fused epilogue against the two-step path (w4gemm, then silu(g) * u in fp32 on its bf16 output):
    equal up to the bf16 rounding of g and u that the fusion skips."""
    K, inter, M = 1024, 512, 64
    w = seeded_weight(K, 2 * inter, seed=34).cuda()
    a = seeded_acts(M, K, seed=35).cuda()
    fused = sk.w4gemm_swiglu(a, sk.W4GateUpWeight.quantize(w)).float()
    gu = sk.w4gemm(a, sk.W4Weight.quantize(w)).float()
    two_step = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    assert torch.allclose(fused, two_step, rtol=3e-2, atol=3e-2 * two_step.abs().max().item())


def test_w4gemm_swiglu_rejects_bad_input(sk):
    w = seeded_weight(256, 128).cuda()
    a = seeded_acts(4, 256).cuda()
    with pytest.raises(ValueError):
        sk.w4gemm_swiglu(a, sk.W4Weight.quantize(w))          # not interleaved
    with pytest.raises(ValueError):
        sk.W4GateUpWeight.quantize(seeded_weight(256, 96).cuda())   # fused width must be a multiple of 128
