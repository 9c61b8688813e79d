"""A decode step through the quantized projections (python/spark_kernels/decode.py) against the same step
with bf16 torch matmuls on the dequantized weights, and its CUDA-graph replay against eager execution.
Mirrors the reference's whole-model checks (tests/test_quant.py:94-105,119-148): two layers, a few steps,
relative error of the hidden state per weight format (the comparison model does not quantize activations,
hence the wider bounds for the fp8 / fp4 formats)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {"int4": 2e-2, "int4-asym": 2e-2, "fp8-tok": 8e-2, "mxfp8": 8e-2, "nvfp4": 2.5e-1}


def _cfg(sk):
    from spark_kernels.decode import DecoderConfig

    return DecoderConfig(hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, layers=2)


@pytest.mark.parametrize("fmt", list(TOL))
@pytest.mark.parametrize("batch", [1, 4])
def test_decode_steps_match_dense_model(sk, fmt, batch):
    from spark_kernels import decode

    cfg = _cfg(sk)
    w = decode.random_weights(cfg, "cuda", seed=5)
    q = decode.QuantizedDecoder(cfg, w, fmt=fmt, batch=batch, max_len=8)
    ref = decode.TorchDecoder(cfg, q.dequantized_weights(), batch=batch, max_len=8)
    g = torch.Generator(device="cuda").manual_seed(6)
    for step in range(3):
        x = torch.randn(batch, cfg.hidden, device="cuda", generator=g).to(torch.bfloat16)
        pos = torch.full((batch,), step, dtype=torch.int64, device="cuda")
        got, want = q.decode(x, pos).float(), ref.decode(x, pos).float()
        rel = ((got - want).norm() / want.norm()).item()
        assert rel < TOL[fmt], (fmt, batch, step, rel)
    assert sk._C.device_status() == 0


def test_fused_swiglu_and_two_step_mlp_agree(sk):
    from spark_kernels import decode

    cfg = _cfg(sk)
    w = decode.random_weights(cfg, "cuda", seed=7)
    a = decode.QuantizedDecoder(cfg, w, fmt="int4", fuse_swiglu=True, batch=2, max_len=4)
    b = decode.QuantizedDecoder(cfg, w, fmt="int4", fuse_swiglu=False, batch=2, max_len=4)
    x = torch.randn(2, cfg.hidden, device="cuda").to(torch.bfloat16)
    pos = torch.zeros(2, dtype=torch.int64, device="cuda")
    ya, yb = a.decode(x, pos).float(), b.decode(x, pos).float()
    assert ((ya - yb).norm() / yb.norm()).item() < 1e-2


def test_graph_replay_equals_eager(sk):
    """The step captured once and replayed (fixed buffers, positions read on the device) gives the eager bits."""
    from spark_kernels import decode

    cfg = _cfg(sk)
    w = decode.random_weights(cfg, "cuda", seed=8)
    eager = decode.QuantizedDecoder(cfg, w, fmt="int4", batch=2, max_len=8)
    graphed = decode.QuantizedDecoder(cfg, w, fmt="int4", batch=2, max_len=8)
    graphed.capture(2)
    g = torch.Generator(device="cuda").manual_seed(9)
    for step in range(4):
        x = torch.randn(2, cfg.hidden, device="cuda", generator=g).to(torch.bfloat16)
        pos = torch.full((2,), step, dtype=torch.int64, device="cuda")
        assert torch.equal(graphed.replay(x, pos), eager.decode(x, pos)), step
