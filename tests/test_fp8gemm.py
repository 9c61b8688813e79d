"""GPU parity of the fp8 path (activation quantizers, per-tensor / MX / fp32-block GEMMs) against
the CPU oracle and the golden vectors. Mirrors the reference's tests/test_fp8gemm.py cases."""

import numpy as np
import pytest
import torch

from tests.parity import assert_bf16_close, bf16_from_bits, t2n

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
# (M, N, K): small, ragged M, decode shapes, one tile-able square
SHAPES = [(16, 64, 64), (1, 128, 256), (3, 64, 192), (64, 256, 512), (100, 128, 256), (16, 4096, 4096),
          (128, 256, 256), (256, 512, 1024)]


def _e4m3(a: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(a.copy()).to(device).view(E4M3)


def _inputs(orc, M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((N, K)).astype(np.float32)
    qa, sa = orc.fp8_quantize_per_tensor(a)
    qb, sb = orc.fp8_quantize_per_tensor(b)
    return qa, sa, qb, sb


@pytest.mark.parametrize("shape", [(1, 4096), (3, 72), (64, 14336), (300, 1024)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("mode", ["tensor", "row", "mx"])
def test_fp8_quantize_matches_oracle(sk, orc, shape, mode):
    rows, K = shape
    if mode == "mx" and K % 32:
        pytest.skip("mx needs K % 32 == 0")
    g = torch.Generator(device="cpu").manual_seed(rows * K)
    x = (torch.randn(rows, K, generator=g) * 3).to(torch.bfloat16)
    x[0, K // 2] = 900.0  # an outlier
    if rows > 2:
        x[1] = 0          # an all-zero row
        x[2] *= 1e-30     # a tiny row
    q, s = sk.fp8_quantize(x.cuda(), mode)
    q_ref, s_ref = orc.fp8_quantize(t2n(x), mode)
    assert q.dtype == E4M3 and q.shape == x.shape
    assert np.array_equal(t2n(q), q_ref)
    assert tuple(s.shape) == s_ref.shape and np.array_equal(t2n(s), s_ref)


@pytest.mark.parametrize("mode", ["tensor", "row", "mx"])
def test_fp8_quantize_golden(sk, golden, mode):
    g = golden("fp8")
    q, s = sk.fp8_quantize(bf16_from_bits(g["x"]), mode)
    assert np.array_equal(t2n(q), g[f"{mode}_q"])
    want = g["mx_sf"] if mode == "mx" else g[f"{mode}_s"]
    assert np.array_equal(t2n(s).reshape(-1), want.reshape(-1))


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fp8gemm_matches_oracle(sk, orc, shape, variant):
    M, N, K = shape
    if not sk._C._lib.spk_fp8gemm_supports(M, N, K, variant):
        with pytest.raises(ValueError):
            qa, sa, qb, sb = _inputs(orc, M, N, K, 1)
            sk.fp8gemm(_e4m3(qa), _e4m3(qb), torch.tensor(sa).cuda(), torch.tensor(sb).cuda(), variant=variant)
        return
    qa, sa, qb, sb = _inputs(orc, M, N, K, M + N + K)
    got = sk.fp8gemm(_e4m3(qa), _e4m3(qb), torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda(), variant=variant)
    assert got.shape == (M, N) and got.dtype == torch.bfloat16
    assert_bf16_close(got, orc.fp8gemm(qa, qb, sa[0], sb[0]), f"fp8gemm v{variant} {shape}")


def test_fp8gemm_exact_sums_are_bitwise(sk, orc):
    """K = 64 with small integer-valued e4m3 operands: every partial sum is exact in fp32, so any
    summation order gives the oracle's bits (reference tests/test_fp8gemm.py:108-113)."""
    rng = np.random.default_rng(3)
    M, N, K = 32, 128, 64
    a = rng.integers(-4, 5, (M, K)).astype(np.float32)
    b = rng.integers(-4, 5, (N, K)).astype(np.float32)
    L = orc.lib()
    qa = np.vectorize(lambda v: L.orc_e4m3_from_f32(float(v)), otypes=[np.uint8])(a)
    qb = np.vectorize(lambda v: L.orc_e4m3_from_f32(float(v)), otypes=[np.uint8])(b)
    one = torch.ones(1, device="cuda")
    want = orc.fp8gemm(qa, qb)
    for v in (0, 1, 3, 4):
        assert np.array_equal(t2n(sk.fp8gemm(_e4m3(qa), _e4m3(qb), one, one, variant=v)), want), v


def test_fp8gemm_golden(sk, golden):
    g = golden("fp8")
    got = sk.fp8gemm(_e4m3(g["pt_a"]), _e4m3(g["pt_b"]), torch.from_numpy(g["pt_sa"]).cuda(), torch.from_numpy(g["pt_sb"]).cuda())
    assert_bf16_close(got, g["pt_c"], "golden per-tensor")
    got = sk.fp8gemm(_e4m3(g["mxg_a"]), _e4m3(g["mxg_b"]), sfa=torch.from_numpy(g["mxg_sfa"]).cuda(),
                     sfb=torch.from_numpy(g["mxg_sfb"]).cuda())
    assert_bf16_close(got, g["mxg_c"], "golden mx")


MX_SHAPES = [(16, 64, 256), (1, 128, 512), (5, 64, 256), (64, 256, 1024), (128, 256, 512), (16, 4096, 4096),
             (256, 384, 512), (300, 512, 768)]


def _mx_inputs(orc, M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = orc.bf16_bits(rng.standard_normal((M, K)).astype(np.float32) * 8)
    b = orc.bf16_bits(rng.standard_normal((N, K)).astype(np.float32) * 8)
    qa, sfa = orc.fp8_quantize(a, "mx")
    qb, sfb = orc.fp8_quantize(b, "mx")
    return qa, sfa, qb, sfb


@pytest.mark.parametrize("variant", [1, 3, 4])
@pytest.mark.parametrize("shape", MX_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fp8gemm_mx_matches_oracle(sk, orc, shape, variant):
    M, N, K = shape
    qa, sfa, qb, sfb = _mx_inputs(orc, M, N, K, M * 7 + K)
    got = sk.fp8gemm(_e4m3(qa), _e4m3(qb), sfa=torch.from_numpy(sfa).cuda(), sfb=torch.from_numpy(sfb).cuda(), variant=variant)
    assert_bf16_close(got, orc.fp8gemm(qa, qb, 1.0, 1.0, sfa, sfb), f"fp8gemm mx v{variant} {shape}")


def test_fp8gemm_mx_unit_scales_equal_per_tensor(sk, orc):
    """MX with every scale byte 127 (2^0) is the per-tensor GEMM bit for bit on exact inputs
    (reference tests/test_fp8gemm.py:379-406)."""
    rng = np.random.default_rng(9)
    M, N, K = 64, 128, 256
    L = orc.lib()
    enc = np.vectorize(lambda v: L.orc_e4m3_from_f32(float(v)), otypes=[np.uint8])
    qa, qb = enc(rng.integers(-3, 4, (M, K))), enc(rng.integers(-3, 4, (N, K)))
    ones_a = torch.full((M, K // 32), 127, dtype=torch.uint8, device="cuda")
    ones_b = torch.full((N, K // 32), 127, dtype=torch.uint8, device="cuda")
    one = torch.ones(1, device="cuda")
    for v in (1, 3):
        pt = sk.fp8gemm(_e4m3(qa), _e4m3(qb), one, one, variant=v)
        mx = sk.fp8gemm(_e4m3(qa), _e4m3(qb), sfa=ones_a, sfb=ones_b, variant=v)
        assert torch.equal(pt, mx), v


def test_fp8gemm_same_bits_every_run(sk, orc):
    qa, sa, qb, sb = _inputs(orc, 256, 512, 1024, 4)
    args = (_e4m3(qa), _e4m3(qb), torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda())
    first = sk.fp8gemm(*args, variant=3)
    for _ in range(3):
        assert torch.equal(sk.fp8gemm(*args, variant=3), first)


def test_fp8gemm_batch_invariant_rows(sk, orc):
    """Variant 4: row i has the same bits whatever M is."""
    qa, sa, qb, sb = _inputs(orc, 513, 256, 512, 5)
    B, SA, SB = _e4m3(qb), torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda()
    full = sk.fp8gemm(_e4m3(qa), B, SA, SB, variant=4)
    ms = (1, 3, 16, 17, 64, 65, 129, 257, 512)  # the reference's list goes to 513 (tests/test_batch_invariant.py:99-152)
    for M in ms:
        assert torch.equal(sk.fp8gemm(_e4m3(qa[:M]), B, SA, SB, variant=4), full[:M]), M
    # and with MX block scales
    qa, sfa, qb, sfb = _mx_inputs(orc, 513, 256, 512, 6)
    B, SFB = _e4m3(qb), torch.from_numpy(sfb).cuda()
    full = sk.fp8gemm(_e4m3(qa), B, sfa=torch.from_numpy(sfa).cuda(), sfb=SFB, variant=4)
    for M in ms:
        got = sk.fp8gemm(_e4m3(qa[:M]), B, sfa=torch.from_numpy(np.ascontiguousarray(sfa[:M])).cuda(), sfb=SFB, variant=4)
        assert torch.equal(got, full[:M]), ("mx", M)


def test_fp8gemm_block128_matches_oracle(sk, orc):
    """fp32 1x128 / 128x128 block scales: no counterpart in the reference (parity unpinned); the
    CUDA quantizer and GEMM are held to the oracle's definition."""
    rng = np.random.default_rng(6)
    # the last shape has enough 128 x 256 tiles to take the wide-tile kernel
    for (M, N, K) in [(16, 4096, 4096), (4, 256, 512), (130, 192, 384), (2048, 2560, 256)]:
        a = rng.standard_normal((M, K)).astype(np.float32)
        b = rng.standard_normal((N, K)).astype(np.float32)
        a[0, :128] = 0  # an all-zero block
        qa, sa = sk.fp8_quantize_block128(torch.from_numpy(a).cuda(), 1)
        qb, sb = sk.fp8_quantize_block128(torch.from_numpy(b).cuda(), 128)
        qa_ref, sa_ref = orc.fp8_block128_quantize(a, 1)
        qb_ref, sb_ref = orc.fp8_block128_quantize(b, 128)
        assert np.array_equal(t2n(qa), qa_ref) and np.array_equal(t2n(sa), sa_ref)
        assert np.array_equal(t2n(qb), qb_ref) and np.array_equal(t2n(sb), sb_ref)
        got = sk.fp8gemm_block128(qa, qb, sa, sb)
        assert_bf16_close(got, orc.fp8gemm_block128(qa_ref, qb_ref, sa_ref, sb_ref), f"block128 {M}x{N}x{K}")


def test_fp8gemm_rejects_bad_input(sk):
    a = torch.zeros(16, 128, device="cuda").to(E4M3)
    b = torch.zeros(64, 128, device="cuda").to(E4M3)
    one = torch.ones(1, device="cuda")
    with pytest.raises(RuntimeError):
        sk.fp8gemm(a, b)  # scales required without block scales
    with pytest.raises(RuntimeError):
        sk.fp8gemm(a.float(), b, one, one)
    with pytest.raises(RuntimeError):
        sk.fp8gemm(a, b[:, :64].contiguous(), one, one)
    with pytest.raises((RuntimeError, ValueError)):
        sk.fp8gemm(a, b, sfa=torch.zeros(16, 4, dtype=torch.uint8, device="cuda"),
                   sfb=torch.zeros(64, 4, dtype=torch.uint8, device="cuda"))  # K % 256 != 0
    with pytest.raises(ValueError):
        sk.fp8gemm(a[:5].contiguous(), b, one, one, variant=0)  # M % 16
    with pytest.raises(RuntimeError):
        sk.fp8gemm(a, b, one, one, variant=5)
    assert sk.num_variants("fp8gemm") == 5
    assert isinstance(sk._C.fp8gemm_v4_route_name(64, 4096, 4096), str)


def test_fp8gemm_v3_route_changes_what_runs(sk, orc):
    """The route knob of variant 3 (reference include/spark/kernels.h:281-294): -1 is the per-shape rule,
    -2 the legacy route (variant 2 where its tile rule holds, else the CUDA cores). The name reports the
    kernel the launcher's own predicate picks, and the legacy route really runs the other kernel: its
    bits equal variant 1's."""
    name = sk._C.fp8gemm_v3_route_name
    assert name(4096, 4096, 4096) == "umma_128x256" and name(16, 4096, 4096) == "umma_decode_splitk"
    assert name(100, 128, 256) == "umma_128x128" and name(100, 100, 256) == "unsupported"
    qa, sa, qb, sb = _inputs(orc, 100, 128, 256, 8)
    args = (_e4m3(qa), _e4m3(qb), torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda())
    v1 = sk.fp8gemm(*args, variant=1)
    prev = sk._C.fp8gemm_v3_set_route(-2)
    try:
        assert sk._C._lib.spk_fp8gemm_v3_route() == -2
        assert name(100, 128, 256) == "simt" and name(16, 4096, 4096) == "simt_decode"
        assert name(4096, 4096, 4096) == "umma_128x256"  # variant 2's tile rule holds there
        legacy = sk.fp8gemm(*args, variant=3)
    finally:
        sk._C.fp8gemm_v3_set_route(prev)
    assert torch.equal(legacy, v1)
    assert_bf16_close(sk.fp8gemm(*args, variant=3), orc.fp8gemm(qa, qb, sa[0], sb[0]), "default route")
