"""Generates tests/golden/*.npz by running the reference's own torch restatement
(python/spark_kernels/reference.py, loaded by path from a checkout of the reference) on CPU.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The fixtures are committed; nothing at test time needs the checkout. Inputs are seeded
torch CPU generators, so the script is reproducible. bf16 tensors are stored as uint16 bit
patterns, e4m3 tensors as uint8 bytes.
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    path = os.path.join(root, "python", "spark_kernels", "reference.py")
    spec = importlib.util.spec_from_file_location("spark_reference_py", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy().copy()
    return t.contiguous().numpy().copy()


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def w4_fixtures(ref) -> dict:
    out = {}
    K, N = 384, 48
    w = (torch.randn(K, N, generator=gen(11)) / K ** 0.5).to(torch.bfloat16)
    w[:128, :16] = 0  # an all-zero group (tests/test_w4gemm.py:40)
    out["w"] = bits(w)
    for tag, asym in (("sym", False), ("asym", True)):
        q, s, z = ref.w4_quantize(w, asym=asym)
        out[f"{tag}_codes"] = bits(q)
        out[f"{tag}_scales"] = bits(s)
        if z is not None:
            out[f"{tag}_zeros"] = bits(z)
        qweight = ref.w4_pack_gptq(q)
        out[f"{tag}_qweight"] = bits(qweight)
        out[f"{tag}_packed"] = bits(ref.w4_repack(qweight))
        out[f"{tag}_deq"] = bits(ref.w4_dequantize(q, s, z))
        a = torch.randn(5, K, generator=gen(12)).to(torch.bfloat16)
        out["a"] = bits(a)
        out[f"{tag}_c"] = bits(ref.w4gemm(a, q, s, z))
    # random codes through pack / repack / unpack (tests/test_w4gemm.py:62-70)
    codes = torch.randint(0, 16, (256, 32), generator=gen(13), dtype=torch.uint8)
    qweight = ref.w4_pack_gptq(codes)
    packed = ref.w4_repack(qweight)
    assert torch.equal(ref.w4_unpack(packed), codes)
    out["rand_codes"] = bits(codes)
    out["rand_qweight"] = bits(qweight)
    out["rand_packed"] = bits(packed)
    return out


def fp8_fixtures(ref) -> dict:
    out = {}
    rows, K = 6, 256
    x = (torch.randn(rows, K, generator=gen(21)) * 3).to(torch.bfloat16)
    x[0, K // 2] = 900.0   # outlier (tests/test_fp8gemm.py:538-542)
    x[1] = 0               # all-zero row
    x[2] *= 1e-30          # tiny row
    out["x"] = bits(x)
    q, s = ref.quantize_fp8_pow2(x, per_row=False)
    out["tensor_q"], out["tensor_s"] = bits(q), bits(s)
    q, s = ref.quantize_fp8_pow2(x, per_row=True)
    out["row_q"], out["row_s"] = bits(q), bits(s)
    q, sf = ref.quantize_mx(x)
    out["mx_q"], out["mx_sf"] = bits(q), bits(sf)
    # exact powers of two and values straddling e4m3 rounding ties
    edge = torch.tensor([[448.0, 449.0, 464.0, 480.0, 1.0, 1.0625, 1.125, 1.1875,
                          2.0 ** -6, 2.0 ** -7, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 0.0, -0.0, -300.0,
                          17.0, 18.0, 19.0, 20.0, 21.0, 22.0, 23.0, 24.0,
                          0.3, 0.7, 1.3, 2.6, 5.2, 10.4, 20.8, 41.6]], dtype=torch.float32)
    out["edge_x"] = bits(edge)
    out["edge_q"] = bits(edge.clamp(-448, 448).to(torch.float8_e4m3fn))
    # GEMMs
    M, N, K = 8, 64, 256
    a = torch.randn(M, K, generator=gen(22))
    b = torch.randn(N, K, generator=gen(23))
    qa, sa = ref.quantize_per_tensor(a)
    qb, sb = ref.quantize_per_tensor(b)
    out["pt_a_f32"], out["pt_b_f32"] = bits(a), bits(b)
    out["pt_a"], out["pt_b"] = bits(qa), bits(qb)
    out["pt_sa"], out["pt_sb"] = bits(sa.reshape(1)), bits(sb.reshape(1))
    c = ((qa.float() @ qb.float().t()) * (sa * sb)).to(torch.bfloat16)
    out["pt_c"] = bits(c)
    ma, sfa = ref.quantize_mx(a.to(torch.bfloat16))
    mb, sfb = ref.quantize_mx(b.to(torch.bfloat16))
    out["mxg_a"], out["mxg_sfa"], out["mxg_b"], out["mxg_sfb"] = bits(ma), bits(sfa), bits(mb), bits(sfb)
    out["mxg_c"] = bits(ref.fp8gemm_mx(ma, sfa, mb, sfb))
    return out


def fp4_fixtures(ref) -> dict:
    out = {}
    rows, K = 130, 256
    x = (torch.randn(rows, K, generator=gen(31)) * 3).to(torch.bfloat16)
    x[0, :16] = 0       # an all-zero block (tests/test_fp4gemm.py:246-250)
    x[3, 40] = 500.0    # an outlier
    out["x"] = bits(x)
    q, sf, s = ref.quantize_nvfp4(x)
    out["nv_q"], out["nv_sf"], out["nv_s"] = bits(q), bits(sf), bits(s.reshape(1))
    q, sf, _ = ref.quantize_nvfp4(x, torch.tensor(0.01))
    out["nv001_q"], out["nv001_sf"] = bits(q), bits(sf)
    q, sf = ref.quantize_mxfp4(x)
    out["mx_q"], out["mx_sf"] = bits(q), bits(sf)
    # GEMMs: M = 5 rows of the same generator family, N = 64
    a = (torch.randn(5, K, generator=gen(32)) * 2).to(torch.bfloat16)
    b = (torch.randn(64, K, generator=gen(33)) * 2).to(torch.bfloat16)
    out["ga"], out["gb"] = bits(a), bits(b)
    qa, sfa, sa = ref.quantize_nvfp4(a)
    qb, sfb, sb = ref.quantize_nvfp4(b)
    out["nvg_c"] = bits(ref.fp4gemm(qa, sfa, qb, sfb, "nvfp4", sa, sb))
    out["nvg_deq_a"] = bits(ref.dequantize_fp4(qa, sfa, "nvfp4"))
    qa, sfa = ref.quantize_mxfp4(a)
    qb, sfb = ref.quantize_mxfp4(b)
    out["mxg_c"] = bits(ref.fp4gemm(qa, sfa, qb, sfb, "mxfp4"))
    # the e2m1 rounding table and the blocked layout
    v = torch.tensor([0.0, 0.25, 0.26, 0.74, 0.75, 1.25, 1.26, 1.75, 2.5, 2.51, 3.49, 3.5, 5.0,
                      5.01, 100.0, -0.75, -6.0, -0.1, -0.0])
    out["e2m1_in"] = bits(v)
    out["e2m1_codes"] = bits(ref.e2m1_codes(v))
    out["e2m1_values"] = bits(ref.e2m1_values(ref.e2m1_codes(v)))
    sfm = torch.randint(0, 255, (200, 12), generator=gen(34), dtype=torch.uint8)
    out["blocked_in"] = bits(sfm)
    out["blocked_out"] = bits(ref.to_blocked(sfm))
    return out


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    root = sys.argv[1]
    ref = load_reference(root)
    torch.set_num_threads(1)
    for name, fn in (("w4", w4_fixtures), ("fp8", fp8_fixtures), ("fp4", fp4_fixtures)):
        data = fn(ref)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **data)
        print(name, len(data), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
