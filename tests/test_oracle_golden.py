"""Pins the CPU oracle (oracle/spark_oracle.c) to golden vectors produced by the reference's own
python/spark_kernels/reference.py (tests/golden/make_golden.py) and to the known-answer values
of the reference's tests. Runs without a GPU."""

import numpy as np
import pytest


# ---- int4 ---------------------------------------------------------------------------------

@pytest.mark.parametrize("tag", ["sym", "asym"])
def test_w4_quantize_bits(orc, golden, tag):
    g = golden("w4")
    q, s, z = orc.w4_quantize(g["w"], asym=tag == "asym")
    assert np.array_equal(q, g[f"{tag}_qweight"])
    assert np.array_equal(s, g[f"{tag}_scales"])
    if tag == "asym":
        assert np.array_equal(z, g["asym_zeros"])
    else:
        assert z is None
    # the all-zero group: scale 0 and every code the zero point (tests/test_w4gemm.py:40)
    codes = orc.w4_unpack(orc.w4_repack(q))
    assert np.array_equal(codes, g[f"{tag}_codes"])
    assert (s[0, :16] == 0).all()
    zp = 8 if tag == "sym" else 0
    assert (codes[:128, :16] == zp).all()


@pytest.mark.parametrize("tag", ["sym", "asym", "rand"])
def test_w4_pack_and_repack_bits(orc, golden, tag):
    g = golden("w4")
    codes = g[f"{tag}_codes"]
    qweight = orc.w4_pack_gptq(codes)
    assert np.array_equal(qweight, g[f"{tag}_qweight"])
    packed = orc.w4_repack(qweight)
    assert packed.shape == g[f"{tag}_packed"].shape
    assert np.array_equal(packed, g[f"{tag}_packed"])
    assert np.array_equal(orc.w4_unpack(packed), codes)


def test_w4_locate_is_the_inverse_of_the_repack(orc, golden):
    g = golden("w4")
    codes, packed = g["rand_codes"], g["rand_packed"].reshape(-1).view(np.uint32)
    K, N = codes.shape
    rng = np.random.default_rng(0)
    for _ in range(500):
        n, k = int(rng.integers(N)), int(rng.integers(K))
        w, p = orc.w4_locate(n, k, K)
        assert (int(packed[w]) >> (4 * p)) & 15 == codes[k, n]


@pytest.mark.parametrize("tag", ["sym", "asym"])
def test_w4_dequantize_bits(orc, golden, tag):
    g = golden("w4")
    z = g["asym_zeros"] if tag == "asym" else None
    deq = orc.w4_dequantize(g[f"{tag}_packed"], g[f"{tag}_scales"], z)
    assert np.array_equal(deq, g[f"{tag}_deq"])


@pytest.mark.parametrize("tag", ["sym", "asym"])
def test_w4gemm_against_reference(orc, golden, tag):
    g = golden("w4")
    z = g["asym_zeros"] if tag == "asym" else None
    c = orc.bf16_to_f32(orc.w4gemm(g["a"], g[f"{tag}_packed"], g[f"{tag}_scales"], z))
    want = orc.bf16_to_f32(g[f"{tag}_c"])
    # same weights bit for bit; the fp32 summation order differs from torch's matmul, so the
    # outputs agree to bf16 rounding (the reference's own tolerance is 3e-2, test_w4gemm.py:18)
    np.testing.assert_allclose(c, want, rtol=2 ** -7, atol=1e-3)
    # identity activations return the dequantized weight exactly (tests/test_w4gemm.py:116-127)
    K = g[f"{tag}_packed"].shape[1] // 2
    eye = orc.bf16_bits(np.eye(K, dtype=np.float32))
    out = orc.w4gemm(eye, g[f"{tag}_packed"], g[f"{tag}_scales"], z)
    assert np.array_equal(out, g[f"{tag}_deq"])


def test_w4gemm_threads_agree(orc, golden):
    g = golden("w4")
    a = orc.w4gemm(g["a"], g["sym_packed"], g["sym_scales"], None, threads=1)
    b = orc.w4gemm(g["a"], g["sym_packed"], g["sym_scales"], None, threads=0)
    assert np.array_equal(a, b)


# ---- fp8 ----------------------------------------------------------------------------------

def test_e4m3_codec(orc, golden):
    g = golden("fp8")
    L = orc.lib()
    got = np.array([L.orc_e4m3_from_f32(float(v)) for v in g["edge_x"].reshape(-1)], np.uint8)
    assert np.array_equal(got, g["edge_q"].reshape(-1))
    # decode(encode) is the identity on every finite byte
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        assert L.orc_e4m3_from_f32(L.orc_e4m3_to_f32(b)) == b
    assert L.orc_e4m3_to_f32(0x7E) == 448.0 and L.orc_e4m3_from_f32(1e9) == 0x7E
    assert L.orc_e4m3_from_f32(-1e9) == 0xFE


@pytest.mark.parametrize("mode", ["tensor", "row", "mx"])
def test_fp8_quantize_bytes(orc, golden, mode):
    g = golden("fp8")
    q, s = orc.fp8_quantize(g["x"], mode)
    assert np.array_equal(q, g[f"{mode}_q"])
    if mode == "mx":
        assert np.array_equal(s, g["mx_sf"])
        assert (q[1] == 0).all() and (s[1] == 0).all()  # all-zero row: smallest scale
    else:
        assert np.array_equal(s.reshape(-1), g[f"{mode}_s"].reshape(-1))


def test_fp8_per_tensor_weight_quantizer(orc, golden):
    g = golden("fp8")
    for t in ("a", "b"):
        q, s = orc.fp8_quantize_per_tensor(g[f"pt_{t}_f32"])
        assert np.array_equal(q, g[f"pt_{t}"]) and s[0] == g[f"pt_s{t}"][0]


def test_fp8gemm_against_reference(orc, golden):
    g = golden("fp8")
    c = orc.bf16_to_f32(orc.fp8gemm(g["pt_a"], g["pt_b"], g["pt_sa"][0], g["pt_sb"][0]))
    np.testing.assert_allclose(c, orc.bf16_to_f32(g["pt_c"]), rtol=2 ** -7, atol=1e-2)
    c = orc.bf16_to_f32(orc.fp8gemm(g["mxg_a"], g["mxg_b"], 1.0, 1.0, g["mxg_sfa"], g["mxg_sfb"]))
    np.testing.assert_allclose(c, orc.bf16_to_f32(g["mxg_c"]), rtol=2 ** -7, atol=1e-2)


def test_fp8_mx_unit_scales_equal_per_tensor(orc, golden):
    """MX with every scale byte 127 is the per-tensor GEMM bit for bit (tests/test_fp8gemm.py:379-406)."""
    g = golden("fp8")
    a, b = g["pt_a"], g["pt_b"]
    ones_a = np.full((a.shape[0], a.shape[1] // 32), 127, np.uint8)
    ones_b = np.full((b.shape[0], b.shape[1] // 32), 127, np.uint8)
    assert np.array_equal(orc.fp8gemm(a, b), orc.fp8gemm(a, b, 1.0, 1.0, ones_a, ones_b))


def test_fp8_block128_mode_is_self_consistent(orc):
    """The fp32 block-scale mode has no counterpart in the reference (parity unpinned): check
    the oracle's definition against a float64 evaluation of the same formula."""
    rng = np.random.default_rng(5)
    M, N, K = 4, 256, 512
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((N, K)).astype(np.float32)
    qa, sa = orc.fp8_block128_quantize(a, 1)
    qb, sb = orc.fp8_block128_quantize(b, 128)
    assert sa.shape == (M, K // 128) and sb.shape == (N // 128, K // 128)
    c = orc.bf16_to_f32(orc.fp8gemm_block128(qa, qb, sa, sb))
    da = orc.e4m3_to_f32(qa).astype(np.float64) * np.repeat(sa, 128, axis=1)
    db = orc.e4m3_to_f32(qb).astype(np.float64) * np.repeat(np.repeat(sb, 128, axis=0), 128, axis=1)
    want = da @ db.T
    np.testing.assert_allclose(c, want, rtol=2 ** -7, atol=1e-2)
    exact = a.astype(np.float64) @ b.T.astype(np.float64)
    assert np.linalg.norm(want - exact) / np.linalg.norm(exact) < 0.05  # e4m3 keeps 3 mantissa bits


# ---- fp4 ----------------------------------------------------------------------------------

def test_e2m1_rounding_table(orc, golden):
    g = golden("fp4")
    L = orc.lib()
    codes = np.array([L.orc_e2m1_code(float(v)) for v in g["e2m1_in"]], np.uint8)
    assert np.array_equal(codes, g["e2m1_codes"])
    vals = np.array([L.orc_e2m1_value(int(c)) for c in codes], np.float32)
    assert np.array_equal(vals, g["e2m1_values"])
    # the table of the reference's CPU-only test (tests/test_fp4gemm.py:263-268)
    v = [0.0, 0.25, 0.26, 0.74, 0.75, 1.25, 1.26, 1.75, 2.5, 2.51, 3.49, 3.5, 5.0, 5.01, 100.0,
         -0.75, -6.0]
    want = [0.0, 0.0, 0.5, 0.5, 1.0, 1.0, 1.5, 2.0, 2.0, 3.0, 3.0, 4.0, 4.0, 6.0, 6.0, -1.0, -6.0]
    assert [L.orc_e2m1_value(L.orc_e2m1_code(x)) for x in v] == want


def test_blocked_scale_layout(orc, golden):
    g = golden("fp4")
    sf, flat = g["blocked_in"], g["blocked_out"]
    rows, cols = sf.shape
    for r in (0, 5, 37, 127, 128, 199):
        for j in range(cols):
            assert flat[orc.fp4_sf_offset(r, j, cols)] == sf[r, j]
    # known answers (tests/test_fp4gemm.py:272-276)
    assert orc.fp4_sf_offset(37, 2, cols) == (37 % 32) * 16 + (37 // 32) * 4 + 2
    assert orc.fp4_sf_offset(5, 5, cols) == 512 + 5 * 16 + 1
    assert orc.fp4_scale_bytes(200, 12 * 16, "nvfp4") == flat.size
    assert orc.fp4_scale_bytes(1, 256, "nvfp4") == 128 * 16
    assert orc.fp4_scale_bytes(129, 256, "mxfp4") == 256 * 8


def test_fp4_quantize_bytes(orc, golden):
    g = golden("fp4")
    q, sf, s = orc.fp4_quantize(g["x"], "nvfp4")
    assert s == g["nv_s"][0]
    assert np.array_equal(q, g["nv_q"]) and np.array_equal(sf, g["nv_sf"])
    q, sf, _ = orc.fp4_quantize(g["x"], "nvfp4", scale=0.01)
    assert np.array_equal(q, g["nv001_q"]) and np.array_equal(sf, g["nv001_sf"])
    q, sf, s = orc.fp4_quantize(g["x"], "mxfp4")
    assert s is None
    assert np.array_equal(q, g["mx_q"]) and np.array_equal(sf, g["mx_sf"])


def test_fp4gemm_against_reference(orc, golden):
    g = golden("fp4")
    qa, sfa, sa = orc.fp4_quantize(g["ga"], "nvfp4")
    qb, sfb, sb = orc.fp4_quantize(g["gb"], "nvfp4")
    assert np.array_equal(orc.fp4_dequantize(qa, sfa, "nvfp4"), g["nvg_deq_a"])
    c = orc.fp4gemm(qa, qb, sfa, sfb, sa, sb, "nvfp4")
    # the sums of e2m1 x e4m3-scale products are exact in fp32 at this K, so the outputs are
    # the reference's bits up to the order of the final scale product
    np.testing.assert_allclose(orc.bf16_to_f32(c), orc.bf16_to_f32(g["nvg_c"]), rtol=2 ** -7, atol=1e-3)
    qa, sfa, _ = orc.fp4_quantize(g["ga"], "mxfp4")
    qb, sfb, _ = orc.fp4_quantize(g["gb"], "mxfp4")
    c = orc.fp4gemm(qa, qb, sfa, sfb, 1.0, 1.0, "mxfp4")
    assert np.array_equal(c, g["mxg_c"])
