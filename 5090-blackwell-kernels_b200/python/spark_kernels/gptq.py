"""Loading GPTQ-style int4 checkpoints into the library's int4 projection.

The reference quantizes a bf16 checkpoint itself every time a model is built and has no loader for
already-quantized weights (python/spark_kernels/engine.py:328-342; docs/design/w4gemm.md:368 lists one as
missing). Its `w4gemm` takes exactly what such checkpoints hold, though: `qweight` int32 [K/8, N] with
eight 4-bit codes per word along K (code i of a word is k = 8 r + i), one scale and one zero point per
group of 128 k per column, every weight (q - z) * s (include/spark/kernels.h:375-416). The tensors of
one linear layer of an AutoGPTQ / GPTQ-for-LLaMa checkpoint are

    qweight  int32 [K/8, N]            as above
    qzeros   int32 [K/group, N/8]      eight 4-bit zero points per word along N; the classic writers
                                       store z - 1 (`zero_offset=1`), later ones z (`zero_offset=0`)
    scales   fp16  [K/group, N]
    g_idx    int32 [K]                 group of every k; only the trivial order k // group is supported
                                       (activation re-ordering, "desc_act", is not)

`from_gptq` turns them into an `Int4Linear` (repack on the GPU, zero points unpacked to the uint8
[K/128, N] the kernels read). Two things differ from the checkpoint's own arithmetic and are
stated, not hidden: the group size must be 128, and the scales become bf16 (the kernels multiply by
bf16 scales; an fp16 scale loses up to three mantissa bits, 2^-9 relative).
"""

from __future__ import annotations

import torch

from . import ops as sk
from . import quant

GROUP = sk.W4_GROUP


def unpack_qzeros(qzeros: torch.Tensor, zero_offset: int = 1) -> torch.Tensor:
    """int32 [G, N/8] (eight 4-bit zero points per word along N) -> uint8 [G, N], plus `zero_offset`."""
    if qzeros.dtype != torch.int32 or qzeros.dim() != 2:
        raise ValueError("qzeros must be int32 [groups, N / 8]")
    shifts = torch.arange(0, 32, 4, device=qzeros.device, dtype=torch.int32)
    z = (qzeros.unsqueeze(-1) >> shifts) & 0xF                      # [G, N/8, 8]; nibble j of a word is column 8 c + j
    z = z.reshape(qzeros.shape[0], -1) + int(zero_offset)
    if int(z.max()) > 15 or int(z.min()) < 0:
        raise ValueError(f"zero points outside 0..15 after adding zero_offset={zero_offset}: this checkpoint uses another convention")
    return z.to(torch.uint8)


def pack_qzeros(zeros: torch.Tensor, zero_offset: int = 1) -> torch.Tensor:
    """The inverse of `unpack_qzeros` (for writing test fixtures and exporting): uint8 [G, N] -> int32 [G, N/8]."""
    if zeros.dim() != 2 or zeros.shape[1] % 8 != 0:
        raise ValueError("zeros must be [groups, N] with N a multiple of 8")
    z = (zeros.to(torch.int64) - int(zero_offset)) & 0xF
    z = z.reshape(zeros.shape[0], -1, 8)
    word = torch.zeros(z.shape[:2], dtype=torch.int64, device=zeros.device)
    for j in range(8):
        word |= z[..., j] << (4 * j)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)  # the same 32 bits, as a signed word


def check_g_idx(g_idx: torch.Tensor | None, K: int, group: int = GROUP) -> None:
    """Only the trivial group order is supported: k belongs to group k // group."""
    if g_idx is None:
        return
    want = torch.arange(K, device=g_idx.device) // group
    if g_idx.numel() != K or not torch.equal(g_idx.to(want.dtype).reshape(-1), want):
        raise ValueError("g_idx is not k // group: activation-ordered (desc_act) checkpoints are not supported")


def dequantize_reference(qweight: torch.Tensor, zeros: torch.Tensor, scales: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """fp32 [K, N] = (q - z) * s with plain torch, from GPTQ-order codes, uint8 zeros and any float scales."""
    shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
    q = ((qweight.unsqueeze(1) >> shifts.view(1, 8, 1)) & 0xF).reshape(-1, qweight.shape[1])  # [K, N]: code i of word r is k = 8 r + i
    z = zeros.to(torch.int32).repeat_interleave(group, 0)
    s = scales.float().repeat_interleave(group, 0)
    return (q - z).float() * s


def from_gptq(qweight: torch.Tensor, qzeros: torch.Tensor | None, scales: torch.Tensor, g_idx: torch.Tensor | None = None,
              group_size: int = GROUP, zero_offset: int = 1, device=None) -> "quant.Int4Linear":
    """The tensors of one GPTQ linear layer -> `Int4Linear`. `qzeros=None` means symmetric codes (zero point 8)."""
    if group_size != GROUP:
        raise ValueError(f"group size {group_size}: the int4 kernels take groups of {GROUP}")
    if qweight.dtype != torch.int32 or qweight.dim() != 2:
        raise ValueError("qweight must be int32 [K / 8, N]")
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    if K % GROUP or N % 16:
        raise ValueError(f"K={K} must be a multiple of {GROUP} and N={N} of 16")
    if tuple(scales.shape) != (K // GROUP, N):
        raise ValueError(f"scales must be [{K // GROUP}, {N}], got {tuple(scales.shape)}")
    check_g_idx(g_idx, K)
    dev = torch.device(device) if device is not None else qweight.device
    zeros = None
    if qzeros is not None:
        if tuple(qzeros.shape) != (K // GROUP, N // 8):
            raise ValueError(f"qzeros must be [{K // GROUP}, {N // 8}], got {tuple(qzeros.shape)}")
        zeros = unpack_qzeros(qzeros, zero_offset).to(dev).contiguous()
    lin = quant.Int4Linear.__new__(quant.Int4Linear)
    lin.w4 = sk.W4Weight(sk.w4_repack(qweight.to(dev).contiguous()), scales.to(dev).to(torch.bfloat16).contiguous(), zeros)
    lin.variant = -1
    return lin


def load_gptq_safetensors(path: str, prefix: str, zero_offset: int = 1, device="cuda") -> "quant.Int4Linear":
    """Read `<prefix>.qweight`, `.qzeros`, `.scales` (and `.g_idx` if present) from a safetensors file."""
    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as f:
        keys = set(f.keys())

        def get(name, required=True):
            key = f"{prefix}.{name}"
            if key not in keys:
                if required:
                    raise KeyError(f"{key} is not in {path}")
                return None
            return f.get_tensor(key)

        return from_gptq(get("qweight"), get("qzeros", required=False), get("scales"), get("g_idx", required=False),
                         zero_offset=zero_offset, device=device)
