"""A decode step of a Llama-style decoder on the quantized projections of this library: the caller side
of the path, in the order the reference's engine runs it (python/spark_kernels/engine.py:441-456,
`_layers_quant`): per layer
    rmsnorm -> qkv projection -> rope + KV-cache append -> attention over the cache -> o projection ->
    residual add + rmsnorm -> gate|up projection -> SwiGLU -> down projection -> residual add
and its replay from a CUDA graph (engine.py:870-899). The four projections are `quant.make_linear`
objects (int4, fp8, mxfp8, nvfp4 ...), or, for int4 with `fuse_swiglu`, the fused gate|up + SwiGLU GEMM
of this library. The row operations between them (RMSNorm, RoPE, attention, residual adds) are outside
the quantized-GEMM path; plain torch stands in for the reference's row kernels here, so this module is
about the data flow through the projections (every GEMM consumes the previous one's output, unlike a
benchmark over fixed buffers), not about those kernels' speed.

`TorchDecoder` is the same arithmetic on the dequantized weights in bf16 torch matmuls, which is what the
reference checks its engine against (tests/test_quant.py:94-105).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops as sk
from . import quant


@dataclass(frozen=True)
class DecoderConfig:
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    layers: int = 32
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @property
    def qkv_cols(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


def random_weights(cfg: DecoderConfig, device, seed: int = 0) -> list[dict]:
    """bf16 weights of `cfg.layers` layers, [in, out] as the Linear classes take them: wqkv, wo, w_gate_up
    (gate columns first, then up), w_down, and the two norm gains."""
    g = torch.Generator(device=device).manual_seed(seed)
    h, inter = cfg.hidden, cfg.intermediate

    def w(k, n):
        return (torch.randn(k, n, device=device, generator=g) / k ** 0.5).to(torch.bfloat16)

    return [{"wqkv": w(h, cfg.qkv_cols), "wo": w(cfg.q_heads * cfg.head_dim, h), "w_gate_up": w(h, 2 * inter), "w_down": w(inter, h),
             "norm1": (1 + 0.1 * torch.randn(h, device=device, generator=g)).to(torch.bfloat16),
             "norm2": (1 + 0.1 * torch.randn(h, device=device, generator=g)).to(torch.bfloat16)} for _ in range(cfg.layers)]


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gain.float()).to(torch.bfloat16)


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, heads, d], pos [B]: rotate the two halves of every head by pos * theta^(-2 i / d)."""
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d)
    ang = pos.float()[:, None, None] * inv
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(torch.bfloat16)


class _Projections:
    """The four projections of one layer as callables."""

    def __init__(self, w: dict, fmt: str, fuse_swiglu: bool):
        self.qkv, self.o, self.down = (quant.make_linear(w[k], fmt) for k in ("wqkv", "wo", "w_down"))
        self.fused = fuse_swiglu and fmt in ("int4", "int4-asym")
        if self.fused:
            self.gate_up_w = sk.W4GateUpWeight.quantize(w["w_gate_up"], asym=fmt == "int4-asym")
        else:
            self.gate_up = quant.make_linear(w["w_gate_up"], fmt)

    def mlp_in(self, h: torch.Tensor) -> torch.Tensor:
        """silu(gate) * up of the gate|up projection: one fused launch, or GEMM + torch."""
        if self.fused:
            return sk.w4gemm_swiglu(h, self.gate_up_w)
        gu = self.gate_up(h)
        inter = gu.shape[1] // 2
        return (torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(torch.bfloat16)


class _Dense:
    """bf16 torch matmul on a given [K, N] weight (the comparison model's projections)."""

    def __init__(self, w: torch.Tensor):
        self.w = w

    def __call__(self, a: torch.Tensor) -> torch.Tensor:
        return a @ self.w


class QuantizedDecoder:
    """Decoder whose projections run on this library. `decode(x, pos)` advances every sequence of the batch by
    one token: x [B, hidden] bf16 are the embedded tokens, pos [B] int64 their positions; the KV cache holds
    `max_len` positions per sequence."""

    def __init__(self, cfg: DecoderConfig, weights: list[dict], fmt: str = "int4", fuse_swiglu: bool = True,
                 batch: int = 1, max_len: int = 64):
        self.cfg, self.fmt = cfg, fmt
        dev = weights[0]["wqkv"].device
        self.layers = [self._projections(w, fmt, fuse_swiglu) for w in weights]
        self.norms = [(w["norm1"], w["norm2"]) for w in weights]
        shape = (cfg.layers, batch, cfg.kv_heads, max_len, cfg.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.max_len = max_len
        self._graph = None

    def _projections(self, w, fmt, fuse_swiglu):
        return _Projections(w, fmt, fuse_swiglu)

    def dequantized_weights(self) -> list[dict]:
        """The weights the quantized projections really multiply by, for the comparison model."""
        out = []
        for lay, (n1, n2) in zip(self.layers, self.norms):
            if lay.fused:
                # undo the strip interleave: dequantize, then put gate strips first and up strips second
                full = quant.formats.w4_dequantize(lay.gate_up_w.packed, lay.gate_up_w.scales, lay.gate_up_w.zeros)
                strips = full.reshape(full.shape[0], -1, 16)
                gate_up = torch.cat([strips[:, 0::2].reshape(full.shape[0], -1), strips[:, 1::2].reshape(full.shape[0], -1)], 1)
            else:
                gate_up = lay.gate_up.dequantize()
            out.append({"wqkv": lay.qkv.dequantize(), "wo": lay.o.dequantize(), "w_gate_up": gate_up,
                        "w_down": lay.down.dequantize(), "norm1": n1, "norm2": n2})
        return out

    def decode(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B = x.shape[0]
        rows = torch.arange(B, device=x.device)
        # keys at positions <= pos are visible; the mask is computed from pos on the device (graph safe)
        visible = torch.arange(self.max_len, device=x.device)[None, :] <= pos[:, None]
        bias = torch.zeros(B, 1, 1, self.max_len, dtype=torch.float32, device=x.device).masked_fill(~visible[:, None, None, :], float("-inf"))
        for li, (lay, (n1, n2)) in enumerate(zip(self.layers, self.norms)):
            h = rmsnorm(x, n1, cfg.eps)
            qkv = lay.qkv(h)
            q, k, v = qkv.split([cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim], -1)
            q = rope(q.reshape(B, cfg.q_heads, cfg.head_dim), pos, cfg.rope_theta)
            k = rope(k.reshape(B, cfg.kv_heads, cfg.head_dim), pos, cfg.rope_theta)
            self.k_cache[li, rows, :, pos] = k
            self.v_cache[li, rows, :, pos] = v.reshape(B, cfg.kv_heads, cfg.head_dim)
            rep = cfg.q_heads // cfg.kv_heads
            keys = self.k_cache[li].repeat_interleave(rep, 1).float()   # [B, q_heads, L, d]
            vals = self.v_cache[li].repeat_interleave(rep, 1).float()
            att = torch.softmax((q.float()[:, :, None, :] @ keys.transpose(-1, -2)) / cfg.head_dim ** 0.5 + bias, -1) @ vals
            x = x + lay.o(att.reshape(B, -1).to(torch.bfloat16))
            x = x + lay.down(lay.mlp_in(rmsnorm(x, n2, cfg.eps)))
        return x

    # ---- CUDA-graph replay of the step (fixed buffers, as the reference's engine does) ----
    def capture(self, batch: int) -> None:
        dev = self.k_cache.device
        self._x = torch.zeros(batch, self.cfg.hidden, dtype=torch.bfloat16, device=dev)
        self._pos = torch.zeros(batch, dtype=torch.int64, device=dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm-up: every scratch of the library exists before capture
            self.decode(self._x, self._pos)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.k_cache.zero_()
        self.v_cache.zero_()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._y = self.decode(self._x, self._pos)

    def replay(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        self._x.copy_(x)
        self._pos.copy_(pos)
        self._graph.replay()
        return self._y


class TorchDecoder(QuantizedDecoder):
    """The comparison model: the same step with bf16 torch matmuls on given (dequantized) weights."""

    def __init__(self, cfg: DecoderConfig, weights: list[dict], batch: int = 1, max_len: int = 64):
        super().__init__(cfg, weights, fmt="dense", fuse_swiglu=False, batch=batch, max_len=max_len)

    def _projections(self, w, fmt, fuse_swiglu):
        class P:
            fused = False
            qkv, o, gate_up, down = _Dense(w["wqkv"]), _Dense(w["wo"]), _Dense(w["w_gate_up"]), _Dense(w["w_down"])
            mlp_in = _Projections.mlp_in
        return P()
