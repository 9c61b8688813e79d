"""The GPTQ-checkpoint loader: zero-point packing and the group-order check on CPU, and on the GPU a layer built
from GPTQ tensors (written to a safetensors file and read back) against plain torch arithmetic on the same
tensors: weights bit for bit through one-hot activations, a GEMM within the bf16 tolerance."""

import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gptq_cpu():
    """gptq.py's pure-torch helpers without importing the package (which needs the CUDA library's device)."""
    pkg = os.path.join(ROOT, "5090-blackwell-kernels_b200", "python")
    if pkg not in sys.path:
        sys.path.insert(0, pkg)
    from spark_kernels import gptq

    return gptq


def test_qzeros_pack_unpack_and_conventions():
    gptq = _gptq_cpu()
    g = torch.Generator().manual_seed(3)
    zeros = torch.randint(1, 16, (5, 64), dtype=torch.uint8, generator=g)
    for off in (0, 1):
        packed = gptq.pack_qzeros(zeros, off)
        assert packed.dtype == torch.int32 and packed.shape == (5, 8)
        assert torch.equal(gptq.unpack_qzeros(packed, off), zeros)
    # nibble j of a word is column 8 c + j
    one = torch.zeros(1, 16, dtype=torch.uint8)
    one[0, 9] = 7
    assert gptq.pack_qzeros(one, 0)[0].tolist() == [0, 7 << 4]
    # the wrong convention shows as a zero point outside 0..15
    with pytest.raises(ValueError, match="convention"):
        gptq.unpack_qzeros(gptq.pack_qzeros(torch.full((1, 8), 15, dtype=torch.uint8), 0), 1)


def test_g_idx_must_be_trivial_and_reference_dequant():
    gptq = _gptq_cpu()
    gptq.check_g_idx(None, 256)
    gptq.check_g_idx(torch.arange(256, dtype=torch.int32) // 128, 256)
    with pytest.raises(ValueError, match="desc_act"):
        gptq.check_g_idx(torch.arange(256, dtype=torch.int32).flip(0) // 128, 256)
    # code i of word r is k = 8 r + i
    qweight = torch.zeros(16, 16, dtype=torch.int32)
    qweight[1, 3] = 0xA << 8                                  # k = 8 + 2, column 3, code 10
    zeros = torch.full((1, 16), 8, dtype=torch.uint8)
    scales = torch.full((1, 16), 0.5)
    w = gptq.dequantize_reference(qweight, zeros, scales)
    assert w.shape == (128, 16) and w[10, 3].item() == (10 - 8) * 0.5 and w[0, 0].item() == -4.0


@pytest.mark.gpu
@pytest.mark.parametrize("asym", [True, False], ids=["qzeros", "symmetric"])
def test_layer_from_gptq_tensors(sk, tmp_path, asym):
    from safetensors.torch import save_file

    from spark_kernels import gptq
    from tests.parity import assert_bf16_close  # noqa: F401  (bf16 tolerance of the repository)

    K, N, M = 512, 384, 5
    g = torch.Generator().manual_seed(11)
    qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), dtype=torch.int32, generator=g)
    scales = (torch.rand(K // 128, N, generator=g) * 0.02 + 0.001).to(torch.float16)
    zeros = torch.randint(1, 16, (K // 128, N), dtype=torch.uint8, generator=g) if asym else None
    tensors = {"model.layers.0.mlp.down_proj.qweight": qweight, "model.layers.0.mlp.down_proj.scales": scales,
               "model.layers.0.mlp.down_proj.g_idx": (torch.arange(K) // 128).to(torch.int32)}
    if asym:
        tensors["model.layers.0.mlp.down_proj.qzeros"] = gptq.pack_qzeros(zeros, 1)
    path = str(tmp_path / "layer.safetensors")
    save_file(tensors, path)
    lin = gptq.load_gptq_safetensors(path, "model.layers.0.mlp.down_proj", zero_offset=1)
    # the weight the kernels multiply by: bf16((q - z) * bf16(scale)), bit for bit, through one-hot activations
    z = zeros if asym else torch.full((K // 128, N), 8, dtype=torch.uint8)
    want = gptq.dequantize_reference(qweight, z, scales.to(torch.bfloat16)).to(torch.bfloat16)
    eye = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    got = torch.cat([lin(eye[i:i + 64]) for i in range(0, K, 64)])
    assert torch.equal(got.cpu(), want)
    # a GEMM against fp64 on those weights
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = (a.double() @ want.double()).float()
    out = lin(a.cuda()).float().cpu()
    err = (out - ref).abs()
    assert bool((err <= 1e-2 * ref.abs() + 2.0 ** -7 * ref.abs().max()).all())
    # what is rejected
    with pytest.raises(ValueError):
        gptq.from_gptq(qweight, None, scales, group_size=64)
    with pytest.raises(ValueError):
        gptq.from_gptq(qweight, None, scales[:, :-16])
