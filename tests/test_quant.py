"""The quantized Linear classes (the reference's python/spark_kernels/quant.py surface): each
format at several batch sizes against (oracle-quantized activation) @ dequantized weight.
Mirrors reference tests/test_quant.py:53-68."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FORMATS = ("int4", "int4-asym", "fp8", "fp8-tok", "mxfp8", "nvfp4", "mxfp4")


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m", [1, 7, 64, 300])
def test_make_linear_against_dequantized_weight(sk, fmt, m):
    K, N = 512, 768
    g = torch.Generator(device="cpu").manual_seed(11)
    w = (torch.randn(K, N, generator=g) / K ** 0.5).to(torch.bfloat16).cuda()
    a = torch.randn(m, K, generator=g).to(torch.bfloat16).cuda()
    lin = sk.make_linear(w, fmt)
    got = lin(a).float()
    assert got.shape == (m, N)
    wd = lin.dequantize().float()
    assert wd.shape == (K, N)
    # the activation as the format sees it
    if fmt in ("int4", "int4-asym"):
        ad = a.float()
    elif fmt == "fp8":
        q, s = sk.fp8_quantize(a, "tensor")
        ad = q.float() * s
    elif fmt == "fp8-tok":
        q, s = sk.fp8_quantize(a, "row")
        ad = q.float() * s
    elif fmt == "mxfp8":
        q, sf = sk.fp8_quantize(a, "mx")
        ad = sk.formats.mx_dequantize(q, sf)
    else:
        q, sf, s = sk.fp4_quantize(a, fmt)
        ad = sk.formats.fp4_dequantize(q, sf, fmt, s)
    want = ad @ wd
    rel = ((got - want).norm() / want.norm()).item()
    assert rel < 1e-2, (fmt, m, rel)
    assert lin.nbytes() > 0


def test_batch_invariant_switch(sk):
    w = (torch.randn(512, 256, device="cuda") / 22).to(torch.bfloat16)
    a = torch.randn(40, 512, device="cuda", dtype=torch.bfloat16)
    for fmt in ("int4", "fp8-tok", "mxfp8"):
        lin = sk.make_linear(w, fmt)
        lin.set_batch_invariant(True)
        full = lin(a)
        assert torch.equal(lin(a[:7].contiguous()), full[:7]), fmt
    with pytest.raises(ValueError):
        sk.make_linear(w, "fp8").set_batch_invariant(True)
    with pytest.raises(ValueError):
        sk.make_linear(w, "nvfp4").set_batch_invariant(True)
    with pytest.raises(ValueError):
        sk.make_linear(w, "int3")
