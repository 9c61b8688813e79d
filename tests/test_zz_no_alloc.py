"""The allocation-free w4gemm entry point (spk_w4gemm_bf16_noalloc) against the CPU oracle.

Some users of the library cannot allocate device memory when they call a GEMM: an inference
engine whose own pool already holds all of HBM, a process that runs under a hard device-memory
cap, or a latency-critical loop that cannot take the device-wide synchronisation that comes with
cudaMalloc. For them the library has one entry point whose split-K scratch is a fixed array
inside the library image. This test calls it through the C ABI twice in a row (the second call
finds the array as the first one left it) and checks both results against the oracle and against
the regular entry point within the tolerance every GEMM test here uses, checks that the free
device memory does not move across the calls, and reads the entry point's own status word. It is
collected last so that a run that stops at the first failure has already run every other test."""

import pytest
import torch

from tests.parity import assert_bf16_close, seeded_acts, seeded_weight, t2n

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N,asym", [(1, 4096, 4096, False), (16, 1152, 256, True), (64, 4096, 6144, False)])
def test_noalloc_matches_the_oracle_twice(sk, orc, M, K, N, asym):
    ww = sk.W4Weight.quantize(seeded_weight(K, N, seed=3).cuda(), asym=asym)
    a = seeded_acts(M, K, seed=5).cuda()
    want = orc.w4gemm(t2n(a), t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    regular = t2n(sk.w4gemm(a, ww, variant=2))
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    a2 = seeded_acts(3, K, seed=6).cuda()
    out2 = torch.empty(3, N, dtype=torch.bfloat16, device="cuda")
    # The first call on a device resolves the fixed array's address (and, in a fresh process, makes the
    # driver load the library image that holds the array). After it nothing may move: every buffer the
    # checked calls touch exists already, and the comparisons (which allocate through torch) come last.
    sk._C.w4gemm_noalloc(a, ww.packed, ww.scales, ww.zeros, outs[2])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):
        sk._C.w4gemm_noalloc(a, ww.packed, ww.scales, ww.zeros, outs[call])
    # a different, smaller problem right after: it must not see what the previous one left behind
    sk._C.w4gemm_noalloc(a2, ww.packed, ww.scales, ww.zeros, out2)
    assert sk._C.w4gemm_noalloc_status() == 0
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry points changed the free device memory"
    for call in range(2):
        assert_bf16_close(outs[call], want, f"noalloc vs oracle, call {call} M={M} K={K} N={N}")
        assert_bf16_close(outs[call], regular, f"noalloc vs spk_w4gemm_bf16, call {call}")
    want2 = orc.w4gemm(t2n(a2), t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    assert_bf16_close(out2, want2, "noalloc after a larger call")


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(sk):
    K = 128
    a = torch.zeros(65, K, dtype=torch.bfloat16, device="cuda")
    packed = torch.zeros(256 // 16, 2 * K, dtype=torch.int32, device="cuda")
    scales = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="M <= 64"):
        sk._C.w4gemm_noalloc(a, packed, scales, None, torch.empty(65, 256, dtype=torch.bfloat16, device="cuda"))
    N = 32768 + 16
    a = torch.zeros(1, K, dtype=torch.bfloat16, device="cuda")
    packed = torch.zeros(N // 16, 2 * K, dtype=torch.int32, device="cuda")
    scales = torch.zeros(1, N, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="N <= 32768"):
        sk._C.w4gemm_noalloc(a, packed, scales, None, torch.empty(1, N, dtype=torch.bfloat16, device="cuda"))
