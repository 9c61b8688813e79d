"""The decode kernels' launch rule (split-K from bytes in flight) on the named device shapes: pure
host arithmetic through the C ABI, no GPU. The expected values are the table the reference's
tests/test_launch_config.py:39-129 pins for its two devices, plus the B200 shape."""

import pytest

import spark_kernels._C as _C

HGEMM_CTA = 24576
W4_BLOCK = 12288
W1_BLOCK = 8192
MB = 1 << 20


def cdiv(a, b):
    return -(-a // b)


@pytest.mark.parametrize("per_cta, want", [(HGEMM_CTA, 64), (W4_BLOCK, 128), (W1_BLOCK, 192)])
def test_need_ctas_rtx5090(per_cta, want):
    assert _C.need_ctas(per_cta, "rtx5090") == want


@pytest.mark.parametrize("per_cta, want", [(HGEMM_CTA, 9), (W4_BLOCK, 18), (W1_BLOCK, 27)])
def test_need_ctas_gb10(per_cta, want):
    assert _C.need_ctas(per_cta, "gb10") == want == cdiv(273 * 800, per_cta)


@pytest.mark.parametrize("strips", [1, 4, 16, 36, 48, 64, 96, 448])
@pytest.mark.parametrize("kt", [8, 64, 224])
def test_split_k_rtx5090_bandwidth_line(strips, kt):
    assert _C.split_k_for(2 * 4096 * strips * 64, strips, kt, HGEMM_CTA, 340, "rtx5090") == min(kt, max(1, cdiv(64, strips)))


@pytest.mark.parametrize("tiles", [16, 64, 128, 144, 256, 384, 1792])
@pytest.mark.parametrize("groups", [4, 32, 112])
def test_split_k_rtx5090_w4_line(tiles, groups):
    assert _C.split_k_for(tiles * 16 * 4096 // 2, tiles, groups, W4_BLOCK, 2720, "rtx5090") == max(1, min(cdiv(128, tiles), groups))


@pytest.mark.parametrize("strips, want", [(1, 9), (4, 3), (8, 2), (9, 1), (16, 1), (36, 1), (64, 1)])
def test_split_k_gb10(strips, want):
    assert _C.split_k_for(2 * 4096 * strips * 64, strips, 64, HGEMM_CTA, 96, "gb10") == want


def test_split_k_clamps_and_wave_clause():
    assert _C.split_k_for(0, 1, 8, HGEMM_CTA, 340, "rtx5090") == 8
    assert _C.split_k_for(0, 1, 1, HGEMM_CTA, 96, "gb10") == 1
    assert _C.split_k_for(0, 1, 64, HGEMM_CTA, 96, "gb10") == 9
    assert _C.split_k_for(2 * 4096 * 1024, 16, 64, HGEMM_CTA, 340, "rtx5090") == 4
    assert _C.split_k_for(4096 * 1024 // 2, 64, 32, W4_BLOCK, 2720, "rtx5090") == 2
    assert _C.split_k_for(4096 * 1024 // 2, 64, 32, W4_BLOCK, 768, "gb10") == 1
    # the wave clause fires only when the bandwidth rule alone asks for more than one wave
    assert _C.need_ctas(1024, "gb10") == 214
    assert _C.split_k_for(0, 50, 64, 1024, 48, "gb10") == 6
    assert _C.split_k_for(0, 50, 64, 1024, 1000, "gb10") == 5


def test_forced_split_replaces_the_rule():
    try:
        _C.decode_force_split_k(3)
        assert _C.split_k_for(0, 64, 64, HGEMM_CTA, 340, "rtx5090") == 3
        assert _C.split_k_for(0, 64, 2, HGEMM_CTA, 340, "rtx5090") == 2
    finally:
        _C.decode_force_split_k(0)
    assert _C.split_k_for(0, 64, 64, HGEMM_CTA, 340, "rtx5090") == 1


@pytest.mark.parametrize("nbytes, fits", [(4096 * 4096 * 2, False), (4096 * 4096 // 2 + 32 * 4096 * 2, True),
                                          (4096 * 28672 // 2 + 32 * 28672 * 2, False), (18 * MB, True), (18 * MB + 1, False), (0, False)])
def test_fits_l2_gb10(nbytes, fits):
    assert _C.fits_l2(nbytes, "gb10") is fits


def test_fits_l2_other_shapes_and_errors():
    assert _C.fits_l2(72 * MB, "rtx5090") and not _C.fits_l2(72 * MB + 1, "rtx5090")
    # B200: the whole int4 gate|up weight (57.75 MB) stays L2 resident, the bf16 one does not
    assert _C.fits_l2(4096 * 28672 // 2 + 32 * 28672 * 2, "b200")
    assert not _C.fits_l2(4096 * 28672 * 2, "b200")
    assert _C.need_ctas(8192, "b200") == cdiv(10 * MB, 8192)   # 10 MiB in flight, measured with the stream probe
    with pytest.raises((ValueError, RuntimeError)):
        _C.fits_l2(1, "h100")


@pytest.mark.gpu
def test_device_shape_of_the_real_device(sk):
    import torch

    d = sk._C.device_shape()
    assert d["sm_count"] == torch.cuda.get_device_properties(0).multi_processor_count or d["forced"]
    assert d["l2_bytes"] > 0 and d["spec_gbps"] > 0 and d["bytes_in_flight"] > 0
