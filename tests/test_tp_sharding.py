"""Tensor-parallel sharding of the int4 projections, checked on CPU with two gloo ranks: each rank
shards the GPTQ-order weight, repacks its shard and multiplies with the oracle; column shards
gathered and row shards all-reduced must reproduce the unsharded product."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        from spark_kernels import tp

        shape = tp.LlamaShape(hidden=256, q_heads=4, kv_heads=2, head_dim=32, intermediate=256, layers=1)
        g = torch.Generator().manual_seed(5)  # same weights on every rank
        M = 5
        a = torch.randn(M, shape.hidden, generator=g).to(torch.bfloat16)
        results = {}
        for kind, N in (("qkv", shape.qkv_cols), ("gate_up", 2 * shape.intermediate)):
            w = (torch.randn(shape.hidden, N, generator=g) / 16).to(torch.bfloat16)
            qw, sc, zp = orc.w4_quantize(orc.t2n(w), asym=True)
            full = orc.bf16_to_f32(orc.w4gemm(orc.t2n(a), orc.w4_repack(qw), sc, zp))
            cols = tp.column_indices(kind, shape, rank, world)
            q_s, s_s, z_s = tp.shard_columns(torch.from_numpy(qw), torch.from_numpy(sc.view(np.int16)), torch.from_numpy(zp), cols)
            part = orc.bf16_to_f32(orc.w4gemm(orc.t2n(a), orc.w4_repack(q_s.numpy()), s_s.numpy().view(np.uint16), z_s.numpy()))
            # column split: this rank's outputs are exactly its columns of the full product
            results[kind] = bool(np.array_equal(part, full[:, cols.numpy()]))
            gathered = [torch.zeros(cols.numel(), dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, cols)
            results[kind + "_cover"] = sorted(torch.cat(gathered).tolist()) == list(range(N))
        # row split: partial products all-reduced
        K, N = shape.intermediate, shape.hidden
        h = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(K, N, generator=g) / 16).to(torch.bfloat16)
        qw, sc, _ = orc.w4_quantize(orc.t2n(w))
        full = orc.bf16_to_f32(orc.w4gemm(orc.t2n(h), orc.w4_repack(qw), sc, None))
        q_s, s_s, _ = tp.shard_rows(torch.from_numpy(qw), torch.from_numpy(sc.view(np.int16)), None, rank, world)
        k0, k1 = rank * K // world, (rank + 1) * K // world
        part = orc.bf16_to_f32(orc.w4gemm(orc.t2n(h[:, k0:k1].contiguous()), orc.w4_repack(q_s.numpy()),
                                          s_s.numpy().view(np.uint16), None))
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        # each partial was rounded to bf16 before the sum, so the match is to bf16 rounding
        results["down"] = bool(np.allclose(t.numpy(), full, rtol=2 ** -6, atol=2 ** -6))
        out[rank] = results
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_full_product():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        assert all(out[rank].values()), (rank, dict(out[rank]))


def test_column_indices_llama3_8b():
    from spark_kernels import tp

    s = tp.LlamaShape()
    for n in (2, 4, 8):
        assert tp.column_indices("qkv", s, 0, n).numel() == 6144 // n
        assert tp.column_indices("gate_up", s, n - 1, n).numel() == 28672 // n
        assert tp.column_indices("qkv", s, 0, n).numel() % 16 == 0
    with pytest.raises(ValueError):
        tp.column_indices("down", s, 0, 2)


class _FakeComm:
    """Stands in for the library's spk_comm_* entry points on CPU: buffers are ints, handles are the
    int as 64 bytes; rank `fail_export_on` cannot export, rank `fail_open_on` cannot open."""

    def __init__(self, rank, fail_export_on=-1, fail_open_on=-1):
        self.rank, self.fail_export_on, self.fail_open_on = rank, fail_export_on, fail_open_on
        self.freed, self.closed, self.calls = [], [], []

    def comm_alloc(self, world, slot_elems):
        return 1000 + self.rank

    def comm_export(self, ptr):
        if self.rank == self.fail_export_on:
            raise RuntimeError("ipc closed")
        return ptr.to_bytes(64, "little")

    def comm_open(self, handle):
        if self.rank == self.fail_open_on:
            raise RuntimeError("open refused")
        return int.from_bytes(handle, "little") + 5000  # a peer mapping has another address

    def comm_close(self, ptr):
        self.closed.append(ptr)

    def comm_free(self, ptr):
        self.freed.append(ptr)

    def comm_status(self, ptr):
        return 0

    def allreduce_push(self, t, ptrs, rank, slot_elems, mode=0):
        self.calls.append((tuple(ptrs), rank, slot_elems))
        return t


def _push_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from types import SimpleNamespace

        from spark_kernels import tp

        res = {}
        fake = _FakeComm(rank)
        ar = tp.PushAllReduce(SimpleNamespace(_C=fake), None, 4096, "cpu")
        # own buffer at index rank, the peers' mappings elsewhere, in rank order
        res["ptrs"] = ar.ptrs == [1000 + r if r == rank else 6000 + r for r in range(world)]
        ar(torch.zeros(8))
        res["call"] = fake.calls == [(tuple(ar.ptrs), rank, 4096)]
        ar.close()
        res["closed"] = fake.closed == [6000 + r for r in range(world) if r != rank] and fake.freed == [1000 + rank]
        # a rank that cannot export / open: every rank raises, nobody is left in a collective, buffers are released
        for kw in ({"fail_export_on": 1}, {"fail_open_on": 0}):
            fake = _FakeComm(rank, **kw)
            try:
                tp.PushAllReduce(SimpleNamespace(_C=fake), None, 4096, "cpu")
                res[str(kw)] = False
            except RuntimeError as e:
                res[str(kw)] = "push all-reduce unavailable" in str(e)
        dist.barrier()
        out[rank] = res
    finally:
        dist.destroy_process_group()


def test_push_allreduce_setup_agrees_across_ranks():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_push_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        assert all(out[rank].values()), (rank, dict(out[rank]))
