"""The push all-reduce on two GPUs of one node against an fp32 rank-order sum (bit for bit), eager
and replayed from a CUDA graph, and its bounded wait when a peer does not take part. Needs two GPUs; skipped otherwise. The ranks are child processes."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = r"""
import os, sys
sys.path.insert(0, os.environ["SPK_REPO"]); sys.path.insert(0, os.path.join(os.environ["SPK_REPO"], "5090-blackwell-kernels_b200", "python"))
import torch, torch.distributed as dist
import spark_kernels as sk
from spark_kernels import tp
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
ar = tp.PushAllReduce(sk, None, 64 * 4096, torch.device("cuda", rank))
g = torch.Generator(device="cuda").manual_seed(100 + rank)
for n in (8, 4096, 16 * 4096, 64 * 4096):
    for rep in range(3):
        x = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = torch.zeros(n, device="cuda")
        for p in parts:          # rank order, fp32, one rounding: the kernel's definition
            want += p.float()
        got = ar(x.clone())
        torch.cuda.synchronize()
        assert torch.equal(got, want.to(torch.bfloat16)), (n, rep)
        if n % (8 * world) == 0:   # the two-phase form (reduce-scatter + all-gather), forced, interleaved with the other
            for mode in (2, 3, 4, 1, 3, 4):
                got2 = ar(x.clone(), mode=mode)
                torch.cuda.synchronize()
                assert torch.equal(got2, want.to(torch.bfloat16)), ("mode", mode, n, rep)
# replayed from a CUDA graph: the call counter advances on the device
y = torch.randn(64 * 4096, device="cuda", generator=g).to(torch.bfloat16)
buf = y.clone()
side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(side):
    ar(buf)
torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize()
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph):
    ar(buf); ar(buf)
parts = [torch.empty_like(y) for _ in range(world)]
dist.all_gather(parts, y)
for rep in range(4):
    buf.copy_(y)
    graph.replay()
    torch.cuda.synchronize()
    s1 = torch.zeros_like(y, dtype=torch.float32)
    for p in parts: s1 += p.float()
    s1 = s1.to(torch.bfloat16)          # first sum; every rank then holds s1, the second sum is world * s1
    s2 = torch.zeros_like(y, dtype=torch.float32)
    for _ in range(world): s2 += s1.float()
    assert torch.equal(buf, s2.to(torch.bfloat16)), rep
assert ar.status() == 0
# a peer that never makes the call: the wait gives up after about a second and leaves a status word
# (no trap, the context stays usable); the data is left unsummed
dist.barrier()
if rank == 0:
    lone = torch.ones(8, device="cuda", dtype=torch.bfloat16)
    ar(lone)
    assert ar.status() == 3, "expected the bounded wait to report a timeout"
    assert torch.equal(lone, torch.ones_like(lone))
    assert torch.zeros(4, device="cuda").sum().item() == 0.0   # the device still answers
dist.barrier()
ar.close()
dist.barrier()
print("RANK_OK", rank, flush=True)
os._exit(0)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_push_allreduce_two_gpus(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, SPK_REPO=repo, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"RANK_OK {r}" in out, out[-3000:]
