"""Host-side (torch) views of the quantized formats: what a stored weight stands for. Used by the
quantized Linear classes' `dequantize()`; the GEMMs never go through here."""

from __future__ import annotations

import torch

E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def w4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """packed int32 [N/16, 2K] (the w4gemm layout) -> codes uint8 [K, N]."""
    T, twoK = packed.shape
    K, N = twoK // 2, T * 16
    dev = packed.device
    words = (packed.to(torch.int64) & 0xFFFFFFFF).reshape(T, K // 64, 32, 4)
    p = torch.arange(8, device=dev)
    nib = (words[..., None] >> (4 * p)) & 15  # [T, U, lane, j, p]
    lane = torch.arange(32, device=dev)[:, None, None]
    j = torch.arange(4, device=dev)[None, :, None]
    pp = p[None, None, :]
    col = (lane >> 2) + 8 * (pp & 1) + 0 * j  # column inside the strip
    u = torch.arange(K // 64, device=dev)[:, None, None, None]
    step = 4 * (u & 1) + j[None]
    kin = 32 * (step >> 1) + 8 * (lane[None] & 3) + 4 * (step & 1) + 2 * ((pp[None] >> 1) & 1) + (pp[None] >> 2)
    k = 128 * (u >> 1) + kin  # [U, lane, j, p]
    out = torch.zeros(K, N, dtype=torch.uint8, device=dev)
    t = torch.arange(T, device=dev)[:, None, None, None, None]
    n = 16 * t + col[None, None].expand(T, K // 64, 32, 4, 8)
    out[k[None].expand_as(n).reshape(-1), n.reshape(-1)] = nib.reshape(-1).to(torch.uint8)
    return out


def w4_dequantize(packed, scales, zeros=None) -> torch.Tensor:
    """bf16 [K, N]: bf16((q - z) * s), z = 8 without zero points."""
    q = w4_unpack(packed).float()
    K, N = q.shape
    z = zeros.float() if zeros is not None else torch.full_like(scales, 8.0, dtype=torch.float32)
    w = (q.reshape(K // 128, 128, N) - z[:, None]) * scales.float()[:, None]
    return w.reshape(K, N).to(torch.bfloat16)


def from_blocked(flat: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    rp, cp = -(-rows // 128) * 128, -(-cols // 4) * 4
    t = flat.reshape(rp // 128, cp // 4, 32, 4, 4).transpose(2, 3).reshape(rp // 128, cp // 4, 128, 4)
    return t.permute(0, 2, 1, 3).reshape(rp, cp)[:rows, :cols]


def fp4_dequantize(q, sf, fmt: str = "nvfp4", scale=None) -> torch.Tensor:
    q = q.view(torch.uint8)
    rows, K = q.shape[0], 2 * q.shape[1]
    block = 16 if fmt == "nvfp4" else 32
    codes = torch.stack((q & 15, q >> 4), dim=-1).reshape(rows, K)
    mag = torch.tensor(E2M1, device=q.device)[(codes & 7).long()]
    vals = torch.where((codes & 8) != 0, -mag, mag)
    sfr = from_blocked(sf.view(torch.uint8), rows, K // block)
    bs = sfr.view(torch.float8_e4m3fn).float() if fmt == "nvfp4" else torch.exp2(sfr.float() - 127)
    out = vals * bs.repeat_interleave(block, dim=-1)
    return out * scale.float() if scale is not None else out


def mx_dequantize(q, sf) -> torch.Tensor:
    return q.float() * torch.exp2(sf.float() - 127).repeat_interleave(32, dim=-1)
