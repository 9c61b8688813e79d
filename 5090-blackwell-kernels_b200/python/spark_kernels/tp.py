"""Tensor-parallel sharding of the int4 projections of a Llama-style decoder layer, and the
full-depth projection stack that runs them (32 layers at 64 tokens). The reference is single GPU; this
is the one place the path shards: qkv and gate|up are split by columns (no communication), o and
down by rows (K), followed by one all-reduce of the [M, hidden] output.

Sharding is done on the GPTQ-order tensors (qweight [K/8, N], scales / zeros [K/128, N]) and each
rank repacks its own shard: a column slice of the repacked layout is a run of strips, but a K slice
is strided in it, so slicing before `w4_repack` is the simple exact way.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class LlamaShape:
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    layers: int = 32

    @property
    def qkv_cols(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


def column_indices(kind: str, shape: LlamaShape, rank: int, tp: int) -> torch.Tensor:
    """Output columns of projection `kind` ("qkv" or "gate_up") that rank `rank` of `tp` owns.
    qkv is fused [q | k | v] and is cut by heads; gate_up is fused [gate | up] and every rank takes
    the same slice of gate and of up."""
    if kind == "qkv":
        assert shape.q_heads % tp == 0 and shape.kv_heads % tp == 0, "heads must divide by tp"
        d, qh, kh = shape.head_dim, shape.q_heads // tp, shape.kv_heads // tp
        q0 = rank * qh * d
        k0 = shape.q_heads * d + rank * kh * d
        v0 = (shape.q_heads + shape.kv_heads) * d + rank * kh * d
        return torch.cat([torch.arange(q0, q0 + qh * d), torch.arange(k0, k0 + kh * d), torch.arange(v0, v0 + kh * d)])
    if kind == "gate_up":
        assert shape.intermediate % (16 * tp) == 0
        w = shape.intermediate // tp
        return torch.cat([torch.arange(rank * w, (rank + 1) * w), torch.arange(shape.intermediate + rank * w,
                                                                              shape.intermediate + (rank + 1) * w)])
    raise ValueError(f"{kind} is not a column-split projection")


def shard_columns(qweight, scales, zeros, cols: torch.Tensor):
    """Column shard of a GPTQ-order int4 weight: the same columns of codes, scales and zero points."""
    cols = cols.to(qweight.device)
    z = None if zeros is None else zeros.index_select(1, cols).contiguous()
    return qweight.index_select(1, cols).contiguous(), scales.index_select(1, cols).contiguous(), z


def shard_rows(qweight, scales, zeros, rank: int, tp: int):
    """K shard of a GPTQ-order int4 weight: K / tp consecutive k (a multiple of 128, so whole groups
    and whole packed words)."""
    K = qweight.shape[0] * 8
    assert K % (128 * tp) == 0, "K / tp must be a multiple of the group size"
    k0, k1 = rank * K // tp, (rank + 1) * K // tp
    z = None if zeros is None else zeros[k0 // 128:k1 // 128].contiguous()
    return qweight[k0 // 8:k1 // 8].contiguous(), scales[k0 // 128:k1 // 128].contiguous(), z


class ProjectionStack:
    """The int4 projections of `shape.layers` decoder layers on one rank of a tensor-parallel
    group, run back to back on a batch of M tokens: qkv (column split), o (row split + all-reduce),
    gate|up (column split), down (row split + all-reduce). Weights are synthetic random codes and
    scales of the sharded shapes (what each rank would hold after sharding and repacking); the glue
    between projections (attention, SwiGLU, norms) is outside the path, so every projection reads
    a fixed activation buffer of its input shape."""

    def __init__(self, sk, shape: LlamaShape, M: int, rank: int, tp: int, device, seed: int = 0):
        self.sk, self.shape, self.M, self.tp = sk, shape, M, tp
        g = torch.Generator(device=device).manual_seed(seed + rank)
        h, d = shape.hidden, shape.head_dim
        self.dims = {  # name -> (K, N) per rank
            "qkv": (h, shape.qkv_cols // tp),
            "o": (shape.q_heads * d // tp, h),
            "gate_up": (h, 2 * shape.intermediate // tp),
            "down": (shape.intermediate // tp, h),
        }
        self.weights = []
        for _ in range(shape.layers):
            layer = {}
            for name, (K, N) in self.dims.items():
                packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (N // 16, 2 * K), dtype=torch.int32, device=device, generator=g)
                scales = (torch.randn(K // 128, N, device=device, generator=g).abs() * 0.02).to(torch.bfloat16)
                layer[name] = (packed, scales)
            self.weights.append(layer)
        self.x = {n: torch.randn(M, K, device=device, generator=g).to(torch.bfloat16) for n, (K, _) in self.dims.items()}
        self.y = {n: torch.empty(M, N, device=device, dtype=torch.bfloat16) for n, (_, N) in self.dims.items()}
        self.launches_per_pass = 4 * shape.layers

    def bytes_per_pass(self) -> int:
        """Algorithmic bytes of one pass over all ranks (the full, unsharded weights)."""
        total = 0
        for name, (K, N) in self.dims.items():
            Kf = K * self.tp if name in ("o", "down") else K
            Nf = N * self.tp if name in ("qkv", "gate_up") else N
            total += 2 * self.M * Kf + Kf * Nf // 2 + 2 * (Kf // 128) * Nf + 2 * self.M * Nf
        return total * self.shape.layers

    def run(self, all_reduce=None) -> None:
        sk = self.sk
        for layer in self.weights:
            for name in ("qkv", "o", "gate_up", "down"):
                packed, scales = layer[name]
                sk.w4gemm(self.x[name], packed, scales, None, -1, self.y[name])
                if all_reduce is not None and name in ("o", "down"):
                    all_reduce(self.y[name])


class PushAllReduce:
    """All-reduce (sum) of small bf16 tensors over the ranks of a one-node process group by direct
    peer stores: every rank owns a buffer in device memory, the ranks exchange CUDA IPC handles of
    their buffers once through the process group, and each call is one kernel per rank that writes
    the local tensor into every peer's buffer, waits for the peers' writes to land in its own, and
    sums them in rank order (the same bits on all ranks). Safe to capture in a CUDA graph: the call
    counter lives on the device. All ranks must call it the same number of times with the same sizes.

        ar = PushAllReduce(sk, group=None, max_elems=64 * 4096, device=dev)
        ar(y)            # y: contiguous bf16, numel % 8 == 0, numel <= max_elems
        ar.close()
    """

    def __init__(self, sk, group, max_elems: int, device):
        import torch.distributed as dist

        self._C, self.group, self.slot_elems = sk._C, group, int(max_elems)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device(device)
        # Every rank takes part in both exchanges even if a local step failed, so that a failure (CUDA IPC
        # closed to the container, out of memory) raises on all ranks instead of leaving peers in a collective.
        self.local, self.ptrs, handle, err = 0, [], None, None
        with self._on_device():
            try:
                self.local = self._C.comm_alloc(self.world, self.slot_elems)
                handle = self._C.comm_export(self.local)
            except Exception as e:  # noqa: BLE001 - reported to every rank below
                err = f"rank {self.rank}: {e}"
            handles = [None] * self.world
            dist.all_gather_object(handles, (handle, err), group=group)
            errs = [e for (_, e) in handles if e]
            if not errs:
                try:
                    self.ptrs = [self.local if r == self.rank else self._C.comm_open(handles[r][0]) for r in range(self.world)]
                except Exception as e:  # noqa: BLE001
                    err = f"rank {self.rank}: {e}"
            opened = [None] * self.world
            dist.all_gather_object(opened, err, group=group)
            errs = errs or [e for e in opened if e]
            if errs:
                self._release()
                raise RuntimeError("push all-reduce unavailable: " + "; ".join(errs))
        dist.barrier(group)

    def _on_device(self):
        return torch.cuda.device(self.device) if self.device.type == "cuda" else contextlib.nullcontext()

    def _release(self) -> None:
        for ptr in self.ptrs:
            if ptr and ptr != self.local:
                try:
                    self._C.comm_close(ptr)
                except Exception:  # noqa: BLE001 - best effort on the failure path
                    pass
        if self.local:
            try:
                self._C.comm_free(self.local)
            except Exception:  # noqa: BLE001
                pass
        self.local, self.ptrs = 0, []

    def __call__(self, t: torch.Tensor, mode: int = 0) -> torch.Tensor:
        """mode 0: the library picks the form (one hop of flagged words up to four ranks, two phases of flagged words
        beyond); 1 one phase with arrival counters, 2 two phases with counters, 3 two phases of flagged words, 4 one
        hop of flagged words."""
        return self._C.allreduce_push(t, self.ptrs, self.rank, self.slot_elems, mode)

    def status(self) -> int:
        """0, or the status a bounded wait for a peer left behind (synchronizes the device)."""
        with self._on_device():
            return self._C.comm_status(self.local)

    def close(self) -> None:
        import torch.distributed as dist

        with self._on_device():
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            dist.barrier(self.group)  # nobody closes a buffer a peer may still be writing to
            for r, ptr in enumerate(self.ptrs):
                if r != self.rank:
                    self._C.comm_close(ptr)
            dist.barrier(self.group)
            self._C.comm_free(self.local)
        self.ptrs = []
