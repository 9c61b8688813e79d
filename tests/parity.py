"""Helpers shared by the GPU parity tests: tensor <-> oracle conversions and the output tolerance.

Tolerance for bf16 GEMM outputs (stated once, used everywhere): an element passes when it is
within 1e-2 relative of the oracle's value or within 2 bf16 ulps of it; on top of that an
absolute slack of 2^-14 of the largest |output| covers sums that cancel, where the fp32
summation order alone moves the result. Integer, byte and index outputs are compared for
equality, never through this.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as orc


def t2n(t):
    return orc.t2n(t)


def bf16_from_bits(a: np.ndarray, device="cuda") -> torch.Tensor:
    return orc.n2t(a, "bf16").to(device)


def assert_bf16_close(got: torch.Tensor, want_bits: np.ndarray, what: str = "") -> None:
    g = got.detach().float().cpu().numpy().astype(np.float64)
    w = orc.bf16_to_f32(want_bits).astype(np.float64)
    assert g.shape == w.shape, (g.shape, w.shape)
    err = np.abs(g - w)
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(w), 1e-38))) - 7)
    bound = np.maximum(1e-2 * np.abs(w), 2 * ulp) + 2.0 ** -14 * np.abs(w).max()
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} outside tolerance; worst at {i}: "
                             f"got {g[i]} want {w[i]} err {err[i]} bound {bound[i]}")


def seeded_weight(K: int, N: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(K, N, generator=g) / K ** 0.5).to(torch.bfloat16)


def seeded_acts(M: int, K: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(1000 + seed)
    return torch.randn(M, K, generator=g).to(torch.bfloat16)
