"""GPU parity of the W4A16 path (quantizer, repack, GEMM variants) against the CPU oracle and
the committed golden vectors. Mirrors the cases of the reference's tests/test_w4gemm.py."""

import numpy as np
import pytest
import torch

from tests.parity import assert_bf16_close, bf16_from_bits, seeded_acts, seeded_weight, t2n

pytestmark = pytest.mark.gpu

# (K, N): smallest legal, a single wide strip set, K with 3 and 9 groups (ragged ring), o-proj
WEIGHTS = [(128, 16), (256, 48), (384, 4096), (1152, 256), (4096, 4096)]
MS = [1, 3, 8, 9, 16, 17, 33, 64, 100, 256]


@pytest.mark.parametrize("asym", [False, True], ids=["sym", "asym"])
@pytest.mark.parametrize("shape", WEIGHTS, ids=lambda s: f"K{s[0]}_N{s[1]}")
def test_w4_quantize_matches_oracle(sk, orc, shape, asym):
    K, N = shape
    w = seeded_weight(K, N)
    w[:128, :16] = 0  # an all-zero group: scale 0, every code the zero point
    qweight, scales, zeros = sk.w4_quantize(w.cuda(), asym=asym)
    q_ref, s_ref, z_ref = orc.w4_quantize(t2n(w), asym=asym)
    assert qweight.shape == (K // 8, N) and qweight.dtype == torch.int32
    assert scales.shape == (K // 128, N) and scales.dtype == torch.bfloat16
    assert np.array_equal(t2n(qweight), q_ref)
    assert np.array_equal(t2n(scales), s_ref)
    if asym:
        assert np.array_equal(t2n(zeros), z_ref)
    else:
        assert zeros is None


@pytest.mark.parametrize("asym", [False, True], ids=["sym", "asym"])
def test_w4_quantize_ties_and_extreme_scales_match_oracle(sk, orc, asym):
    """The quantizer multiplies by the reciprocal of the scale and resolves exact ties itself instead of dividing:
    columns made of exact ties (w / s = k + 1/2 for every k), of values one bf16 step either side of a tie, of
    magnitudes from 1e-36 to 1e30, and random mantissas against every scale mantissa must give the oracle's codes."""
    K, N = 256, 256
    g = torch.Generator().manual_seed(5)
    w = torch.zeros(K, N)
    halves = torch.arange(-15, 16).float() * 0.5                      # -7.5 .. 7.5 in steps of 1/2: ties and integers
    for n in range(N):
        s0 = 2.0 ** ((n % 40) - 20) * (1 + (n % 7) / 8)               # scales with different mantissas and exponents
        col = halves[torch.randint(0, len(halves), (K,), generator=g)] * s0
        col[0], col[128] = 7 * s0, 7 * s0                             # |max| = 7 s0 in both groups: scale bf16(s0)
        if n % 3 == 1:                                                # one bf16 step off the ties
            bits = col.to(torch.bfloat16).view(torch.int16) + torch.randint(-1, 2, (K,), generator=g).to(torch.int16)
            col = bits.view(torch.bfloat16).float()
            col[0], col[128] = 7 * s0, 7 * s0
        w[:, n] = col
    w[:, 200:208] *= 1e-30                                            # scales whose reciprocal is huge
    w[:128, 208:216] *= 1e-37
    w[:, 216:224] *= 1e28
    w[:, 224:] = (torch.randn(K, 32, generator=g) * torch.logspace(-3, 3, 32)).float()
    w = w.to(torch.bfloat16)
    qweight, scales, zeros = sk.w4_quantize(w.cuda(), asym=asym)
    q_ref, s_ref, z_ref = orc.w4_quantize(t2n(w), asym=asym)
    assert np.array_equal(t2n(scales), s_ref)
    bad = np.argwhere(t2n(qweight) != q_ref)
    assert bad.size == 0, f"{len(bad)} words differ, first at {bad[:3].tolist()}"
    if asym:
        assert np.array_equal(t2n(zeros), z_ref)


@pytest.mark.parametrize("tag", ["sym", "asym"])
def test_w4_quantize_and_repack_golden(sk, golden, tag):
    g = golden("w4")
    w = bf16_from_bits(g["w"])
    qweight, scales, zeros = sk.w4_quantize(w, asym=tag == "asym")
    assert np.array_equal(t2n(qweight), g[f"{tag}_qweight"])
    assert np.array_equal(t2n(scales), g[f"{tag}_scales"])
    if tag == "asym":
        assert np.array_equal(t2n(zeros), g["asym_zeros"])
    assert np.array_equal(t2n(sk.w4_repack(qweight)), g[f"{tag}_packed"])


@pytest.mark.parametrize("shape", WEIGHTS, ids=lambda s: f"K{s[0]}_N{s[1]}")
def test_w4_repack_matches_oracle(sk, orc, shape):
    K, N = shape
    g = torch.Generator(device="cpu").manual_seed(K + N)
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8, generator=g)
    qweight = orc.w4_pack_gptq(q.numpy())
    packed = sk.w4_repack(torch.from_numpy(qweight).cuda())
    assert packed.shape == (N // 16, 2 * K) and packed.dtype == torch.int32
    assert np.array_equal(t2n(packed), orc.w4_repack(qweight))
    assert np.array_equal(orc.w4_unpack(t2n(packed)), q.numpy())


def _case(sk, orc, M, K, N, variant, asym=False, reps=1):
    w = seeded_weight(K, N, seed=K + N)
    a = seeded_acts(M, K, seed=M)
    ww = sk.W4Weight.quantize(w.cuda(), asym=asym)
    want = orc.w4gemm(t2n(a), t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    for _ in range(reps):
        got = sk.w4gemm(a.cuda(), ww, variant=variant)
        assert got.shape == (M, N) and got.dtype == torch.bfloat16
        assert_bf16_close(got, want, f"w4gemm v{variant} M={M} K={K} N={N}")


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
@pytest.mark.parametrize("M", MS)
@pytest.mark.parametrize("shape", WEIGHTS, ids=lambda s: f"K{s[0]}_N{s[1]}")
def test_w4gemm_matches_oracle(sk, orc, shape, M, variant):
    K, N = shape
    if variant == 0 and M * N * K > 2 ** 28:
        pytest.skip("the naive rung is only checked on the small shapes")
    if K * N >= 4096 * 4096 and M > 64:
        pytest.skip("oracle time: the large weight is covered at M <= 64 and by the Llama shapes")
    # three calls on variant 2: the split-K scratch and its counters are left zeroed
    _case(sk, orc, M, K, N, variant, reps=3 if variant == 2 else 1)


@pytest.mark.parametrize("M", [1, 16, 64, 100])
@pytest.mark.parametrize("variant", [0, 1, 2, 3])
def test_w4gemm_asymmetric(sk, orc, M, variant):
    _case(sk, orc, M, 1152, 256, variant, asym=True)
    if variant > 0 and M <= 64:
        _case(sk, orc, M, 4096, 4096, variant, asym=True)


LLAMA = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)]


@pytest.mark.parametrize("M", [1, 16, 64])
@pytest.mark.parametrize("shape", LLAMA, ids=lambda s: f"K{s[0]}_N{s[1]}")
def test_w4gemm_llama_shapes(sk, orc, shape, M):
    K, N = shape
    _case(sk, orc, M, K, N, -1, reps=2)


def test_w4gemm_weight_bits_are_the_oracle(sk, orc):
    """One-hot activations return the dequantized weight itself, bit for bit, on every variant."""
    K, N = 256, 64
    w = seeded_weight(K, N)
    ww = sk.W4Weight.quantize(w.cuda(), asym=True)
    deq = orc.w4_dequantize(t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    a = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    for v in range(sk.num_variants("w4gemm")):
        assert np.array_equal(t2n(sk.w4gemm(a, ww, variant=v)), deq), v


def test_w4gemm_golden(sk, golden):
    g = golden("w4")
    for tag in ("sym", "asym"):
        z = torch.from_numpy(g["asym_zeros"]).cuda() if tag == "asym" else None
        packed = torch.from_numpy(g[f"{tag}_packed"]).cuda()
        scales = bf16_from_bits(g[f"{tag}_scales"])
        a = bf16_from_bits(g["a"])
        for v in range(4):
            assert_bf16_close(sk.w4gemm(a, packed, scales, z, variant=v), g[f"{tag}_c"], f"golden {tag} v{v}")


def test_w4gemm_batch_invariant_rows(sk):
    """Variant 3: row i of C has the same bits whatever M is and wherever it sits in the batch."""
    K, N = 1152, 256
    ww = sk.W4Weight.quantize(seeded_weight(K, N).cuda())
    a = seeded_acts(513, K).cuda()
    full = sk.w4gemm(a, ww, variant=3)
    for M in (1, 3, 8, 9, 16, 17, 33, 64, 65, 129, 257, 512):  # the reference's list goes to 513
        assert torch.equal(sk.w4gemm(a[:M].contiguous(), ww, variant=3), full[:M]), M
    assert torch.equal(sk.w4gemm(a[5:6].contiguous(), ww, variant=3), full[5:6])


def test_w4gemm_rejects_bad_input(sk):
    w = seeded_weight(256, 64).cuda()
    ww = sk.W4Weight.quantize(w)
    a = torch.randn(4, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        sk.w4gemm(a[:, :128].contiguous(), ww)  # K mismatch
    with pytest.raises(RuntimeError):
        sk.w4gemm(a.float(), ww)  # not bf16
    with pytest.raises(RuntimeError):
        sk.w4_quantize(torch.randn(200, 64, device="cuda", dtype=torch.bfloat16))  # K % 128
    with pytest.raises(RuntimeError):
        sk.w4gemm(a, ww, variant=sk.num_variants("w4gemm"))
    assert ww.shape == (256, 64)


def test_w4gemm_in_a_cuda_graph(sk, orc):
    """The default variant captured in a CUDA graph replays correctly (scratch allocated before
    capture, left clean by every launch)."""
    K, N, M = 4096, 4096, 16
    ww = sk.W4Weight.quantize(seeded_weight(K, N).cuda())
    a = seeded_acts(M, K).cuda()
    sk._C.init()
    want = orc.w4gemm(t2n(a), t2n(ww.packed), t2n(ww.scales), None)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sk.w4gemm(a, ww, out=out)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sk.w4gemm(a, ww, out=out)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert_bf16_close(out, want, "graph replay")
    assert sk._C.device_status() == 0


@pytest.mark.parametrize("M", [1, 16, 48, 64])
def test_w4gemm_back_to_back_calls_chain_correctly(sk, orc, M):
    """Consecutive launches of the library overlap (the next GEMM's weight stream starts while the
    previous one finishes). A chain in which every GEMM reads the previous GEMM's output, enqueued
    without host synchronisation, must give what the same chain gives with a device synchronise
    between the calls."""
    K = N = 4096
    g = torch.Generator(device="cpu").manual_seed(5)
    # random codes, scales sized so that the chained activations stay O(1)
    ws = []
    for i in range(3):
        w = (torch.randn(K, N, generator=g) * (1.0 / K ** 0.5)).to(torch.bfloat16)
        ws.append(sk.W4Weight.quantize(w.cuda()))
    x0 = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()

    def chain(sync: bool):
        outs, x = [], x0
        for rep in range(4):
            for ww in ws:
                x = sk.w4gemm(x, ww, variant=2)
                if sync:
                    torch.cuda.synchronize()
                outs.append(x)
        torch.cuda.synchronize()
        return outs

    want = chain(True)
    for attempt in range(5):
        got = chain(False)
        for i, (a, b) in enumerate(zip(got, want)):
            # rounding differences of one call (split-K order) feed the next, so the comparison is against
            # the scale of the output; a launch that ran ahead of its input would be off by O(1)
            a32, b32 = a.float(), b.float()
            assert torch.isfinite(a32).all(), (attempt, i)
            assert (a32 - b32).abs().max().item() <= 0.03 * b32.abs().max().item(), (attempt, i, M)
    assert sk._C.device_status() == 0


def test_an_expired_wait_is_reported_and_the_scratch_is_clean_again(sk, orc):
    """A kernel whose bounded wait runs out sets the status word and may leave partial sums and strip
    counters behind. Reading the status reports it once, restores the scratch, and the next split-K
    GEMM matches the oracle. (The wait runs out in a test kernel that waits for a barrier phase nothing
    completes; nothing faults and the context stays usable.)"""
    K, N = 4096, 4096
    ww = sk.W4Weight.quantize(seeded_weight(K, N, seed=11).cuda())
    a = seeded_acts(1, K, seed=12).cuda()
    want = orc.w4gemm(t2n(a), t2n(ww.packed), t2n(ww.scales), None)
    assert sk._C.device_status() == 0
    sk._C.debug_expire_wait(4096)
    assert sk._C.device_status() == 3
    assert sk._C.device_status() == 0
    for M in (1, 64):  # the stream kernel's and the tensor-core kernel's split-K
        aa = seeded_acts(M, K, seed=12).cuda()
        assert_bf16_close(sk.w4gemm(aa, ww, variant=2), orc.w4gemm(t2n(aa), t2n(ww.packed), t2n(ww.scales), None),
                          f"after an expired wait, M={M}")
    assert_bf16_close(sk.w4gemm(a, ww, variant=2), want, "after an expired wait")
    assert sk._C.device_status() == 0


@pytest.mark.parametrize("asym", [False, True], ids=["sym", "asym"])
@pytest.mark.parametrize("M,K,N", [(256, 1152, 256), (300, 256, 192), (513, 512, 4096), (2048, 4096, 4096), (640, 256, 4160)])
def test_w4gemm_many_tokens_matches_oracle(sk, orc, M, K, N, asym):
    """From 256 tokens up the default variant dequantizes the weight once (bit-exact bf16((q - z) * s)) and runs
    a dense bf16 tensor-core GEMM. Checked on sampled rows over all columns at the large shape (a row of C
    depends on one row of A only), on everything below."""
    ww = sk.W4Weight.quantize(seeded_weight(K, N, seed=21).cuda(), asym=asym)
    a = seeded_acts(M, K, seed=22).cuda()
    got = sk.w4gemm(a, ww, variant=2)
    assert sk._C.device_status() == 0
    rows = np.arange(M) if M * N * K <= 2 ** 28 else np.unique(np.concatenate([[0, 127, 128, M - 1], np.random.default_rng(M).choice(M, 48, replace=False)]))
    want = orc.w4gemm(np.ascontiguousarray(t2n(a)[rows]), t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    assert_bf16_close(got[torch.from_numpy(rows).cuda()], want, f"w4gemm many tokens M={M} K={K} N={N}")


def test_w4gemm_many_tokens_weight_bits_are_the_oracle(sk, orc):
    """The dequantized weights of the many-token route, read back through one-hot activations, bit for bit."""
    K, N = 512, 128
    ww = sk.W4Weight.quantize(seeded_weight(K, N, seed=23).cuda(), asym=True)
    deq = orc.w4_dequantize(t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    K, N = 640, 4096                                          # 5 x 32 tiles: enough for the dense route
    ww = sk.W4Weight.quantize(seeded_weight(K, N, seed=23).cuda(), asym=True)
    deq = orc.w4_dequantize(t2n(ww.packed), t2n(ww.scales), t2n(ww.zeros))
    a = torch.eye(K, dtype=torch.bfloat16, device="cuda")   # 640 tokens
    assert np.array_equal(t2n(sk.w4gemm(a, ww, variant=2)), deq)
