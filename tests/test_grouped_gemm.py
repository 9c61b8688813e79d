"""GPU parity of the grouped fp8 GEMM (one launch for all experts of a mixture-of-experts layer) against the oracle's
fp8 GEMM run expert by expert. Mirrors the reference's grouped-GEMM contract (include/spark/kernels.h:459-494):
device-side offsets, empty experts, ragged expert sizes, per-expert weight scales, the SwiGLU epilogue."""

import numpy as np
import pytest
import torch

from tests.parity import assert_bf16_close, t2n

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn


def _case(orc, sizes, N, K, seed):
    rng = np.random.default_rng(seed)
    T, E = int(sum(sizes)), len(sizes)
    a = rng.standard_normal((T, K)).astype(np.float32)
    w = rng.standard_normal((E, N, K)).astype(np.float32)
    qa, sa = orc.fp8_quantize_per_tensor(a)
    qw = np.empty((E, N, K), np.uint8)
    sw = np.empty(E, np.float32)
    for e in range(E):
        q, s = orc.fp8_quantize_per_tensor(np.ascontiguousarray(w[e]) * (1 + e % 3))
        qw[e], sw[e] = q, s[0]
    offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    return qa, sa, qw, sw, offsets


@pytest.mark.parametrize("sizes,N,K", [([5, 0, 130, 1, 64], 256, 256), ([128, 128], 128, 128), ([0, 0, 7], 384, 512),
                                        ([300, 17, 0, 129, 256, 3, 90, 1], 512, 384), ([200] * 16, 1024, 512)],
                         ids=["ragged", "exact", "leading-empty", "eight", "sixteen"])
def test_grouped_gemm_fp8_matches_oracle(sk, orc, sizes, N, K):
    qa, sa, qw, sw, off = _case(orc, sizes, N, K, len(sizes) + N)
    got = sk.grouped_gemm_fp8(torch.from_numpy(qa).cuda().view(E4M3), torch.from_numpy(qw).cuda().view(E4M3), torch.from_numpy(off).cuda(),
                              torch.from_numpy(sa).cuda(), torch.from_numpy(sw).cuda())
    assert got.shape == (sum(sizes), N) and sk._C.device_status() == 0
    for e in range(len(sizes)):
        r0, r1 = off[e], off[e + 1]
        if r1 > r0:
            assert_bf16_close(got[r0:r1], orc.fp8gemm(qa[r0:r1], qw[e], sa[0], sw[e]), f"grouped expert {e} of {sizes}")
    # the same bits every run
    again = sk.grouped_gemm_fp8(torch.from_numpy(qa).cuda().view(E4M3), torch.from_numpy(qw).cuda().view(E4M3), torch.from_numpy(off).cuda(),
                                torch.from_numpy(sa).cuda(), torch.from_numpy(sw).cuda())
    assert torch.equal(got, again)


def test_grouped_gemm_swiglu_fp8(sk, orc):
    sizes, N, K = [70, 0, 129, 33], 256, 256
    qa, sa, qw, sw, off = _case(orc, sizes, N, K, 99)
    got = sk.grouped_gemm_swiglu_fp8(torch.from_numpy(qa).cuda().view(E4M3), torch.from_numpy(qw).cuda().view(E4M3),
                                     torch.from_numpy(off).cuda(), torch.from_numpy(sa).cuda(), torch.from_numpy(sw).cuda())
    assert got.shape == (sum(sizes), N // 2)
    fa = orc.e4m3_to_f32(qa).astype(np.float64)
    for e in range(len(sizes)):
        r0, r1 = off[e], off[e + 1]
        if r1 == r0:
            continue
        c = fa[r0:r1] @ orc.e4m3_to_f32(qw[e]).astype(np.float64).T * float(sa[0]) * float(sw[e])
        g, u = c[:, 0::2], c[:, 1::2]
        assert_bf16_close(got[r0:r1], orc.bf16_bits((g / (1 + np.exp(-g)) * u).astype(np.float32)), f"grouped swiglu expert {e}")


def test_grouped_gemm_rejects_bad_input(sk):
    a = torch.zeros(8, 128, device="cuda").to(E4M3)
    w = torch.zeros(2, 128, 128, device="cuda").to(E4M3)
    off = torch.tensor([0, 4, 8], dtype=torch.int32, device="cuda")
    sk.grouped_gemm_fp8(a, w, off)
    with pytest.raises(RuntimeError):
        sk.grouped_gemm_fp8(a, w, off[:2].contiguous())
    with pytest.raises(ValueError):
        sk.grouped_gemm_fp8(a, torch.zeros(2, 64, 128, device="cuda").to(E4M3), off)   # N % 128
    assert sk._C._lib.spk_grouped_gemm_supports(8, 256, 256) == 1 and sk._C._lib.spk_grouped_gemm_supports(600, 256, 256) == 0
