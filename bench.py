"""Benchmark of the int4 W4A16 decode GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("llama3_8b_mlp_int4_decode"): the Llama-3-8B MLP projections with
int4 group-128 weights, gate|up fused (N = 28672, K = 4096) and down (N = 4096, K = 14336), at
M = 1, 16 and 64 tokens. One step runs both GEMMs of LAYERS distinct layers at each M, so the
weights streamed between two uses of the same layer (1.4 GB) far exceed the 126 MB L2: the
inputs are larger than L2, no flush is needed. The step is captured once in a CUDA graph and
replayed; timing is CUDA events around the K replays, max over ranks.

metric/value: algorithmic bytes moved per second (the reference's own traffic model:
2MK + KN/2 + 2(K/128)N + 2MN per GEMM), whole job. roofline: the same figure per launch of the
stream kernel against the measured HBM copy bandwidth. e2e: the same metric with, every step,
the activations copied from pinned host memory and the last layer's outputs read back.
cpu_baseline / --impl reference: the CPU restatement of the reference's arithmetic (the
reference has no CPU int4 GEMM of its own) timed on the host cores on a bounded sample.

With N > 1 the projections run tensor parallel: qkv / gate|up column-split (no communication),
o / down row-split followed by one all-reduce of the [M, 4096] output; total work is fixed, so
scaling is "strong". There the headline value is the full-depth projection stack (32 layers x qkv, o,
gate|up, down at 64 tokens, the workload the scaling target is stated on) and the MLP-only numbers
ride along under "mlp". Before anything is timed at N > 1 one layer is CHECKED: the gathered
column-split output and the all-reduced row-split output (push and NCCL) of real sharded weights
against the unsharded GEMM; the line carries "tp_check" and the run fails if it does not hold.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "5090-blackwell-kernels_b200", "python")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

HIDDEN, INTER = 4096, 14336
MS = (1, 16, 64)
LAYERS = 16
WORKLOAD = "llama3_8b_mlp_int4_decode"
STACK_WORKLOAD = "llama3_8b_projection_stack_int4_decode"
FALLBACK_HBM_GBS = 6650.0


def alg_bytes(M: int, N: int, K: int) -> int:
    """Traffic floor of one symmetric W4A16 GEMM (reference scripts/shape_utils.py:310-321)."""
    return 2 * M * K + K * N // 2 + 2 * (K // 128) * N + 2 * M * N


def kernel_for(m: int) -> str:
    """The kernel the default route launches for m tokens on the Llama MLP shapes (w4gemm.cu, w4gemm_tmem.cu)."""
    return "w4_tmem_kernel" if 16 <= m <= 64 else "w4_stream_kernel"


# DRAM bytes moved per algorithmic byte, from one ncu capture per kernel (dram__bytes_read.sum +
# dram__bytes_write.sum over the launch's algorithmic bytes; the captures are summarised under profiles/).
EXPERTS = 8   # experts of the grouped fp8 GEMM rows (--kind grouped)
NCU_TRAFFIC_RATIO = {"w4_tmem_kernel": 1.04, "w4_stream_kernel": 1.005}


def step_bytes(layers: int) -> int:
    return layers * sum(alg_bytes(m, 2 * INTER, HIDDEN) + alg_bytes(m, HIDDEN, INTER) for m in MS)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi in the background during the timed region: SM clock and throttle reasons."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU arm -------------------------------------------------------------------------------------

def cpu_sample(threads: int = 0):
    """One bounded sample of the workload on the host: one of the 16 layers, gate|up and down at
    every token count of the GPU arm (M = 1, 16, 64), all host threads.
    Returns (GB/s of algorithmic bytes, seconds, threads, description)."""
    import numpy as np

    from oracle import oracle as orc

    orc.lib()
    if threads <= 0:
        # every core this process may run on; a launcher's OMP_NUM_THREADS=1 default must not shrink it
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    ms = MS
    total, secs = 0, 0.0
    for (K, N) in ((HIDDEN, 2 * INTER), (INTER, HIDDEN)):
        packed = rng.integers(-2 ** 31, 2 ** 31 - 1, size=(N // 16, 2 * K), dtype=np.int64).astype(np.int32)
        scales = orc.bf16_bits(np.abs(rng.standard_normal((K // 128, N)).astype(np.float32)) * 0.02)
        for M in ms:
            a = orc.bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
            t0 = time.perf_counter()
            orc.w4gemm(a, packed, scales, None, threads=threads)
            secs += time.perf_counter() - t0
            total += alg_bytes(M, N, K)
    used = threads
    return total / secs / 1e9, secs, used, "1 of 16 layers: gate|up 28672x4096 and down 4096x14336 at M=1,16,64"


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        gbs, secs, used, sample = cpu_sample(0)
        if i >= args.warmup:
            vals.append((gbs, secs))
    value = sum(v for v, _ in vals) / len(vals)
    ms = 1e3 * sum(s for _, s in vals) / len(vals)
    line = {
        "impl": "reference", "metric": "int4_decode_gemm_gbps", "value": round(value, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16xint4->fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": LAYERS, "M": list(MS), "gate_up": [2 * INTER, HIDDEN],
                   "down": [HIDDEN, INTER], "group": 128},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm -------------------------------------------------------------------------------------

def tp_check(sk, dist, dev, rank, tp, reducers) -> dict:
    """One MLP layer with REAL sharded weights at 64 tokens, before anything is timed: every rank builds
    the same full GPTQ-order weight (same seed), takes its shard (columns of gate|up, rows of down),
    repacks it, runs its GEMM, and the gathered / all-reduced result is compared with the unsharded
    GEMM of the same weight on this rank. Tolerance: 2e-2 relative plus 2e-2 of the largest |output|
    (each rank's partial sum is rounded to bf16 before the all-reduce adds them)."""
    import torch

    from spark_kernels import tp as tpmod

    shape = tpmod.LlamaShape()
    M = 64
    g = torch.Generator(device=dev).manual_seed(4242)  # the same on every rank
    res = {}

    def full_weight(K, N):
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), dtype=torch.int32, device=dev, generator=g)
        sc = (torch.randn(K // 128, N, device=dev, generator=g).abs() * 0.02).to(torch.bfloat16)
        return qw, sc

    def close(got, want):
        got, want = got.float(), want.float()
        bound = 2e-2 * want.abs() + 2e-2 * want.abs().max()
        err = (got - want).abs()
        return bool((err <= bound).all().item()), float((err / want.abs().max()).max().item())

    # gate|up: column split, no communication
    qw, sc = full_weight(HIDDEN, 2 * INTER)
    x = torch.randn(M, HIDDEN, device=dev, generator=g).to(torch.bfloat16)
    want = sk.w4gemm(x, sk.w4_repack(qw), sc)
    cols = tpmod.column_indices("gate_up", shape, rank, tp)
    qs, ss, _ = tpmod.shard_columns(qw, sc, None, cols)
    part = sk.w4gemm(x, sk.w4_repack(qs), ss)
    parts = [torch.empty_like(part) for _ in range(tp)]
    dist.all_gather(parts, part)
    got = torch.empty_like(want)
    for r in range(tp):
        got[:, tpmod.column_indices("gate_up", shape, r, tp).to(dev)] = parts[r]
    ok, err = close(got, want)
    res["gate_up_gathered"] = {"ok": ok, "max_err_over_max": round(err, 5)}
    del qw, sc, qs, ss, parts, got, want
    # down: row split, all-reduce (every reducer the timed runs use)
    qw, sc = full_weight(INTER, HIDDEN)
    h = torch.randn(M, INTER, device=dev, generator=g).to(torch.bfloat16)
    want = sk.w4gemm(h, sk.w4_repack(qw), sc)
    qs, ss, _ = tpmod.shard_rows(qw, sc, None, rank, tp)
    k0, k1 = rank * INTER // tp, (rank + 1) * INTER // tp
    hs = h[:, k0:k1].contiguous()
    packed = sk.w4_repack(qs)
    for name, fn in reducers.items():
        y = sk.w4gemm(hs, packed, ss)
        fn(y)
        torch.cuda.synchronize()
        ok, err = close(y, want)
        res[f"down_allreduce_{name}"] = {"ok": ok, "max_err_over_max": round(err, 5)}
    flags = torch.tensor([1.0 if all(v["ok"] for v in res.values()) else 0.0,
                          1.0 if all(v["ok"] for k, v in res.items() if k != "down_allreduce_push") else 0.0], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    res["status"] = "ok" if flags[0].item() >= 1.0 else "FAILED"
    res["status_without_push"] = "ok" if flags[1].item() >= 1.0 else "FAILED"  # the same on every rank
    return res


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import spark_kernels as sk

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = world
    assert (2 * INTER) % (16 * tp) == 0 and INTER % (128 * tp) == 0
    sk._C.init()
    # the all-reduce after the row-split GEMMs: direct peer stores (one kernel per rank), or NCCL
    reduce, reduce_name = None, "none"
    if world > 1:
        reduce, reduce_name = (lambda t: dist.all_reduce(t)), "nccl"
        if args.allreduce == "push":
            try:
                from spark_kernels import tp as tpmod_

                pusher = tpmod_.PushAllReduce(sk, None, 64 * HIDDEN, dev)
                # One kernel per rank, peer stores over NVLink: one hop (every rank stores its tensor into every
                # peer) while the sum is latency bound, reduce-scatter + all-gather (two hops, 2 (world - 1) / world
                # of the tensor per rank) for large tensors on four ranks and more; the library picks.

                def reduce(t, _p=pusher):
                    return _p(t)

                reduce_name = "push (flagged peer stores over NVLink, one kernel per rank; one hop while (world - 1) x the doubled tensor is within 1 MiB, two phases beyond)"
            except Exception as e:  # CUDA IPC can be closed to a container; NCCL then carries the sum
                reduce_name = f"nccl (push unavailable: {type(e).__name__})"
            ok_all = torch.tensor([1.0 if reduce_name.startswith("push") else 0.0], device=dev)
            dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
            if ok_all.item() < 1.0 and reduce_name.startswith("push"):
                reduce, reduce_name = (lambda t: dist.all_reduce(t)), "nccl (push unavailable on a peer)"
    tp_res = None
    if world > 1:
        reducers = {"nccl": lambda t: dist.all_reduce(t)}
        if reduce_name.startswith("push"):
            reducers["push"] = lambda t, _p=pusher: _p(t)
        tp_res = tp_check(sk, dist, dev, rank, tp, reducers)
        if tp_res["status"] != "ok" and tp_res["status_without_push"] == "ok":
            # only the push all-reduce disagrees with the unsharded GEMM: time with NCCL (checked above) and say so
            reduce, reduce_name = (lambda t: dist.all_reduce(t)), "nccl (the push all-reduce failed the check against the unsharded GEMM)"
            tp_res["status"] = "ok"
            tp_res["note"] = "push all-reduce failed the check; NCCL is what is timed"
        if tp_res["status"] != "ok":
            if rank == 0:
                print(json.dumps({"metric": "int4_decode_gemm_gbps", "value": None, "n_gpus": world, "tp_check": tp_res}), flush=True)
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            os._exit(3)
        torch.cuda.empty_cache()

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def rand_weight(K, N):
        packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (N // 16, 2 * K), dtype=torch.int32, device=dev, generator=gen)
        scales = (torch.randn(K // 128, N, device=dev, generator=gen).abs() * 0.02).to(torch.bfloat16)
        return packed, scales

    # column split of gate|up (N / tp columns), row split of down (K / tp rows)
    gu = [rand_weight(HIDDEN, 2 * INTER // tp) for _ in range(LAYERS)]
    dn = [rand_weight(INTER // tp, HIDDEN) for _ in range(LAYERS)]
    x = {m: torch.randn(m, HIDDEN, device=dev, generator=gen).to(torch.bfloat16) for m in MS}
    h = {m: torch.randn(m, INTER // tp, device=dev, generator=gen).to(torch.bfloat16) for m in MS}
    y_gu = {m: torch.empty(m, 2 * INTER // tp, device=dev, dtype=torch.bfloat16) for m in MS}
    y_dn = {m: torch.empty(m, HIDDEN, device=dev, dtype=torch.bfloat16) for m in MS}
    launches_per_step = 0

    def step_m(m):
        n = 0
        for layer in range(LAYERS):
            sk.w4gemm(x[m], gu[layer][0], gu[layer][1], None, -1, y_gu[m])
            sk.w4gemm(h[m], dn[layer][0], dn[layer][1], None, -1, y_dn[m])
            n += 2
            if world > 1:
                reduce(y_dn[m])
        return n

    # eager warm-up on a side stream, then capture one graph per token count; a step replays all of them
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launches_per_step = sum(step_m(m) for m in MS)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graphs = {}
    for m in MS:
        graphs[m] = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graphs[m]):
            step_m(m)
    torch.cuda.synchronize()

    class _Step:
        @staticmethod
        def replay():
            for m in MS:
                graphs[m].replay()

    graph = _Step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        graph.replay()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)

    # the same launches timed per token count (the roofline of the dominant kernel comes from here)
    ms_by_m = {}
    for m in MS:
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(args.steps):
            graphs[m].replay()
        g1.record()
        barrier()
        ms_by_m[m] = g0.elapsed_time(g1) / args.steps

    # end to end: activations from pinned host memory every step, outputs read back every step
    pin_x = {m: torch.randn(m, HIDDEN).to(torch.bfloat16).pin_memory() for m in MS}
    pin_h = {m: torch.randn(m, INTER // tp).to(torch.bfloat16).pin_memory() for m in MS}
    out_gu = {m: torch.empty(m, 2 * INTER // tp, dtype=torch.bfloat16).pin_memory() for m in MS}
    out_dn = {m: torch.empty(m, HIDDEN, dtype=torch.bfloat16).pin_memory() for m in MS}
    h2d = sum(t.numel() * 2 for t in list(pin_x.values()) + list(pin_h.values()))
    d2h = sum(t.numel() * 2 for t in list(out_gu.values()) + list(out_dn.values()))

    def e2e_step():
        for m in MS:
            x[m].copy_(pin_x[m], non_blocking=True)
            h[m].copy_(pin_h[m], non_blocking=True)
        graph.replay()
        for m in MS:
            out_gu[m].copy_(y_gu[m], non_blocking=True)
            out_dn[m].copy_(y_dn[m], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None

    # the full-depth projection stack (qkv, o, gate|up, down of 32 layers) at 64 tokens
    del gu, dn
    torch.cuda.empty_cache()
    from spark_kernels import tp as tpmod

    stack = tpmod.ProjectionStack(sk, tpmod.LlamaShape(), 64, rank, tp, dev, seed=99)
    reduce_fn = reduce
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        stack.run(reduce_fn)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    sgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(sgraph):
        stack.run(reduce_fn)
    for _ in range(3):
        sgraph.replay()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        sgraph.replay()
    s1.record()
    barrier()
    ms_stack = s0.elapsed_time(s1)
    # the stack end to end: its four activation inputs from pinned host memory and its outputs back, every pass
    spin_x = {n: torch.randn(t.shape).to(torch.bfloat16).pin_memory() for n, t in stack.x.items()}
    spin_y = {n: torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for n, t in stack.y.items()}
    stack_h2d = sum(t.numel() * 2 for t in spin_x.values())
    stack_d2h = sum(t.numel() * 2 for t in spin_y.values())

    def stack_e2e():
        for n, t in spin_x.items():
            stack.x[n].copy_(t, non_blocking=True)
        sgraph.replay()
        for n, t in spin_y.items():
            t.copy_(stack.y[n], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        stack_e2e()
    barrier()
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    q0.record()
    for _ in range(args.steps):
        stack_e2e()
    q1.record()
    barrier()
    ms_stack_e2e = q0.elapsed_time(q1)
    # the same pass with the all-reduces left out: what the sums (and the gaps they open in the launch chain) cost
    ms_stack_gemms = ms_stack
    if world > 1:
        ngraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ngraph):
            stack.run(None)
        for _ in range(3):
            ngraph.replay()
        barrier()
        n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0.record()
        for _ in range(args.steps):
            ngraph.replay()
        n1.record()
        barrier()
        ms_stack_gemms = n0.elapsed_time(n1)
        del ngraph

    status = sk._C.device_status()
    launches_per_pass, stack_bytes = stack.launches_per_pass, stack.bytes_per_pass()
    if world > 1:
        t = torch.tensor([ms_total, ms_e2e, float(status), ms_stack, ms_stack_gemms, ms_stack_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e, status, ms_stack, ms_stack_gemms, ms_stack_e2e = (t[0].item(), t[1].item(), int(t[2].item()), t[3].item(),
                                                                           t[4].item(), t[5].item())
    assert status == 0, f"a kernel reported device status {status}"

    if rank == 0:
        total_bytes = step_bytes(LAYERS)  # whole job: the shards of all ranks add up to the full weights
        value = total_bytes * args.steps / (ms_total * 1e-3) / 1e9
        e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
        peak, which = measured_peak()
        # per token count: algorithmic bytes of this rank's launches over their measured time; the
        # dominant kernel is the one behind the token count with the largest share of the step
        by_m = {}
        for m in MS:
            b = LAYERS * (alg_bytes(m, 2 * INTER // tp, HIDDEN) + alg_bytes(m, HIDDEN, INTER // tp))
            by_m[m] = {"kernel": kernel_for(m), "launches": 2 * LAYERS, "us_per_launch": round(ms_by_m[m] * 1e3 / (2 * LAYERS), 2),
                       "gbps": round(b / (ms_by_m[m] * 1e-3) / 1e9, 1), "bytes_per_launch": b // (2 * LAYERS)}
        top = max(MS, key=lambda m: ms_by_m[m])
        achieved = by_m[top]["gbps"]
        traffic = NCU_TRAFFIC_RATIO.get(by_m[top]["kernel"])
        secondary = None
        if world == 1 and not args.no_cpu:
            del stack, sgraph
            torch.cuda.empty_cache()
            secondary = secondary_gemms()
            assert sk._C.device_status() == 0, "a kernel reported a device status in the secondary GEMMs"
        cpu = None
        if world == 1 and not args.no_cpu:
            gbs, secs, used, sample = cpu_sample(0)
            cpu = {"value": round(gbs, 4), "unit": "GB/s", "cores": used, "kind": "port", "sample": sample,
                   "seconds": round(secs, 2)}
        stack_value = stack_bytes * args.steps / (ms_stack * 1e-3) / 1e9
        stack_rank_bytes = stack_bytes // tp  # the shards of all ranks add up to the full weights
        mlp_cfg = {"workload": WORKLOAD, "layers": LAYERS, "M": list(MS), "gate_up": [2 * INTER, HIDDEN],
                   "down": [HIDDEN, INTER], "group": 128, "parallelism": f"tp{tp}", "allreduce": reduce_name,
                   "l2": "inputs larger than L2 (1.4 GB of weights per step)", "launch": "cuda graph"}
        mlp_roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": round(achieved / peak, 4), "peak_source": which,
                        "traffic": None if traffic is None or tp > 1 else int(traffic * by_m[top]["bytes_per_launch"]),
                        "kernel": by_m[top]["kernel"], "tokens": top, "bytes_per_launch": by_m[top]["bytes_per_launch"],
                        "share_of_step": round(ms_by_m[top] / sum(ms_by_m.values()), 3),
                        "by_tokens": {str(m): by_m[m] for m in MS}}
        tp_stack = {"workload": STACK_WORKLOAD + " (32 layers x qkv,o,gate_up,down; M=64)",
                    "value": round(stack_value, 2), "unit": "GB/s",
                    "ms_per_pass": round(ms_stack / args.steps, 4), "parallelism": f"tp{tp}",
                    "ms_per_pass_without_allreduce": round(ms_stack_gemms / args.steps, 4),
                    "e2e": round(stack_bytes * args.steps / (ms_stack_e2e * 1e-3) / 1e9, 2),
                    "allreduces_per_pass": 0 if world == 1 else 2 * 32, "launches_per_pass": launches_per_pass}
        # kernels of this library launched inside the timed regions (the tcgen05 int4 route is two launches per
        # GEMM: activation re-ordering + GEMM; every all-reduce by peer stores is one more)
        mlp_launches = sum(2 * LAYERS * (2 if kernel_for(m) == "w4_tmem_kernel" else 1) for m in MS)
        if world == 1:
            line = {
                "metric": "int4_decode_gemm_gbps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_total / args.steps, 4),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16xint4->fp32",
                "data": "synthetic", "config": mlp_cfg, "roofline": mlp_roofline, "cpu_baseline": cpu,
                "e2e": {"value": round(e2e, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "tp_stack": tp_stack, "secondary": secondary,
                "gpu_launches": (mlp_launches + 2 * launches_per_pass) * args.steps, "clocks": clocks,
            }
        else:
            # N > 1: the projection stack is the headline (the workload the scaling target is stated on); a "step"
            # is one pass; the MLP-only numbers ride along under "mlp"
            stack_achieved = stack_rank_bytes * args.steps / (ms_stack * 1e-3) / 1e9
            line = {
                "metric": "int4_decode_gemm_gbps", "value": round(stack_value, 2), "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_stack / args.steps, 4),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16xint4->fp32",
                "data": "synthetic",
                "config": {"workload": STACK_WORKLOAD, "layers": 32, "M": [64], "projections": ["qkv", "o", "gate_up", "down"],
                           "group": 128, "parallelism": f"tp{tp}", "allreduce": reduce_name,
                           "l2": "inputs larger than L2 (3.6 GB of weights per pass over all ranks)", "launch": "cuda graph"},
                "roofline": {"bound": "hbm", "achieved": round(stack_achieved, 1), "peak": peak, "unit": "GB/s",
                             "frac": round(stack_achieved / peak, 4), "peak_source": which, "traffic": None,
                             "kernel": "w4_tmem_kernel (+ all-reduce after o / down)", "tokens": 64,
                             "bytes_per_launch": stack_rank_bytes // launches_per_pass, "per": "rank, whole pass incl. all-reduces"},
                "cpu_baseline": None,
                "e2e": {"value": tp_stack["e2e"], "unit": "GB/s", "h2d_bytes_per_step": stack_h2d, "d2h_bytes_per_step": stack_d2h},
                "tp_check": tp_res, "tp_stack": tp_stack,
                "mlp": {"value": round(value, 2), "unit": "GB/s", "ms_per_step": round(ms_total / args.steps, 4),
                        "e2e": round(e2e, 2), "config": mlp_cfg, "roofline": mlp_roofline},
                "secondary": None,
                "gpu_launches": (2 * launches_per_pass + (2 * 32 if reduce_name.startswith("push") else 0)) * args.steps,
                "clocks": clocks,
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Captured graphs hold NCCL work; tearing the process group down with them alive was seen to
        # block forever on this software stack. Drop them, line the ranks up, and leave without the
        # interpreter's teardown.
        graphs.clear()
        del sgraph
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def time_one_gemm(kind: str, d0: int, d1: int, d2: int, steps: int, use_graph: bool) -> dict:
    """A small case for ncu and for the secondary rows: one shape through the public op, a few
    launches, timed with CUDA events. w4: K,N,M over 4 weight copies (larger than L2 together for the
    Llama shapes); w4swiglu: the same through the fused gate|up + SwiGLU launch (N = 2 x intermediate).
    fp8 / fp8block / mxfp8 / nvfp4 / mxfp4: M,N,K (weights rotated past L2 when M <= 64). grouped: T,N,K over
    EXPERTS equal experts. quant-w4: K,N of a bf16 weight; quant-fp8row / quant-fp8mx / quant-fp4: rows,K
    of a bf16 matrix (the third number is ignored), rate = bytes read + written."""
    import torch

    import spark_kernels as sk

    g = torch.Generator(device="cuda").manual_seed(0)
    stream_bytes = None
    if kind.startswith("quant-"):
        rows, cols = d0, d1
        x = (torch.randn(rows, cols, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        if kind == "quant-w4":      # [K, N] weight -> int4 codes (half a byte) + a bf16 scale per 128 k
            calls, out_bytes = [lambda: sk.w4_quantize(x)], rows * cols * (0.5 + 2 / 128)
        elif kind == "quant-fp8row":
            calls, out_bytes = [lambda: sk.fp8_quantize(x, "row")], rows * cols + 4 * rows
        elif kind == "quant-fp8mx":
            calls, out_bytes = [lambda: sk.fp8_quantize(x, "mx")], rows * cols * (1 + 1 / 32)
        else:
            sc = torch.tensor(0.01, device="cuda")
            calls, out_bytes = [lambda: sk.fp4_quantize(x, "nvfp4", sc)], rows * cols * (0.5 + 1 / 16)
        work, unit = 2 * rows * cols + out_bytes, "GB/s"
    elif kind == "grouped":
        T, N, K, E = d0, d1, d2, EXPERTS
        a = torch.randn(T, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
        w = (torch.randn(E, N, K, device="cuda", generator=g) * 0.05).to(torch.float8_e4m3fn)
        off = torch.tensor([T * e // E for e in range(E + 1)], dtype=torch.int32, device="cuda")
        sa, sb = torch.ones(1, device="cuda"), torch.ones(E, device="cuda")
        calls = [lambda: sk.grouped_gemm_fp8(a, w, off, sa, sb)]
        work, unit = 2 * T * N * K, "TFLOP/s"
        stream_bytes = T * K + E * N * K + 2 * T * N
    elif kind == "w4swiglu":
        K, N, M = d0, d1, d2
        ws = []
        for _ in range(4):
            wq = sk.W4GateUpWeight.quantize((torch.randn(K, N, device="cuda", generator=g) * 0.02).to(torch.bfloat16))
            ws.append(wq)
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        calls = [lambda i=i: sk.w4gemm_swiglu(a, ws[i], out) for i in range(4)]
        work, unit = alg_bytes(M, N, K) - M * N, "GB/s"   # half the output bytes of the plain GEMM
    elif kind == "w4":
        K, N, M = d0, d1, d2
        ws = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (N // 16, 2 * K), dtype=torch.int32, device="cuda", generator=g),
               (torch.rand(K // 128, N, device="cuda", generator=g) * 0.02).to(torch.bfloat16)) for _ in range(4)]
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        calls = [lambda i=i: sk.w4gemm(a, ws[i % 4][0], ws[i % 4][1], None, -1, out) for i in range(4)]
        work, unit = alg_bytes(M, N, K), "GB/s"
    else:
        M, N, K = d0, d1, d2
        a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        # decode shapes stream the weights: rotate over enough copies to exceed L2 (126 MB)
        copies = 1 if M > 64 else max(2, -(-(300 << 20) // (N * K)))
        bs = [torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(copies)]
        if kind == "fp8":
            qa, sa = sk.fp8_quantize(a, "tensor")
            qs = [sk.fp8_quantize(b, "tensor") for b in bs]
            calls = [lambda q=q: sk.fp8gemm(qa, q[0], sa, q[1]) for q in qs]
        elif kind == "fp8block":  # fp32 scales: 1 x 128 blocks of A, 128 x 128 blocks of B
            qa, sa = sk.fp8_quantize_block128(a.float(), 1)
            qs = [sk.fp8_quantize_block128(b.float(), 128) for b in bs]
            calls = [lambda q=q: sk.fp8gemm_block128(qa, q[0], sa, q[1]) for q in qs]
        elif kind == "mxfp8":
            qa, sfa = sk.fp8_quantize(a, "mx")
            qs = [sk.fp8_quantize(b, "mx") for b in bs]
            calls = [lambda q=q: sk.fp8gemm(qa, q[0], sfa=sfa, sfb=q[1]) for q in qs]
        else:
            qa, sfa, sa = sk.fp4_quantize(a, kind)
            qs = [sk.fp4_quantize(b, kind) for b in bs]
            if kind == "mxfp4":
                calls = [lambda q=q: sk.fp4gemm(qa, q[0], sfa, q[1], fmt="mxfp4") for q in qs]
            else:
                calls = [lambda q=q: sk.fp4gemm(qa, q[0], sfa, q[1], fmt="nvfp4", scale_a=sa.reshape(1), scale_b=q[2].reshape(1))
                         for q in qs]
        del bs
        work, unit = 2 * M * N * K, "TFLOP/s"
        # the reference's traffic model (scripts/shape_utils.py:342-345): operands + block scales + bf16 output
        per_elem = {"fp8": 1.0, "fp8block": 1.0, "mxfp8": 1.0 + 1 / 32, "nvfp4": 0.5 + 1 / 16, "mxfp4": 0.5 + 1 / 32}[kind]
        stream_bytes = (M * K + K * N) * per_elem + 2 * M * N
    for i in range(3):
        calls[i % len(calls)]()
    torch.cuda.synchronize()
    n = max(1, steps)
    timing = "eager launches, CUDA events"
    if use_graph:
        # the launches of one pass captured in a CUDA graph: what a decode engine replays
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(len(calls)):
                calls[i]()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                calls[i % len(calls)]()
        graph.replay()
        torch.cuda.synchronize()
        timing = "CUDA graph of the launches, CUDA events"
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if use_graph:
        graph.replay()
    else:
        for i in range(n):
            calls[i % len(calls)]()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    rate = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    extra = {} if stream_bytes is None else {"gbps": round(stream_bytes / (ms * 1e-3) / 1e9, 1)}
    return {"one_gemm": [d0, d1, d2], "kind": kind, "launches": 3 + n, "us_per_launch": round(ms * 1e3, 2),
                      "rate": round(rate, 1), "unit": unit, **extra, "timing": timing,
                      "status": sk._C.device_status()}


def run_one_gemm(args) -> None:
    import torch

    import spark_kernels as sk

    d0, d1, d2 = (int(v) for v in args.one_gemm.split(","))
    torch.cuda.set_device(0)
    sk._C.init()
    print(json.dumps(time_one_gemm(args.kind, d0, d1, d2, args.steps, args.graph)))


def secondary_gemms() -> list:
    """The fp8 / NVFP4 rows of the headline metric, measured in the same run: the 8192^3 GEMMs against the
    tensor peak (50 launches each, so the region is long enough to settle under the power cap; both the
    burst and the sustained measured bf16 rate are given as denominators: fp8 runs at twice, fp4 at four
    times the bf16 rate on this part) and the 16 x 4096 x 4096 decode GEMMs as weight streams."""
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        bf16, sustained, src = float(peaks["bf16_tflops"]), float(peaks.get("bf16_tflops_sustained", 0.0)) or None, "measured bf16 x"
    except Exception:
        bf16, sustained, src = 1590.0, 1400.0, "fallback bf16 x"
    hbm, _ = measured_peak()
    rows = []
    for kind, mult in (("fp8", 2), ("fp8block", 2), ("nvfp4", 4)):
        r = time_one_gemm(kind, 8192, 8192, 8192, 50, False)
        rows.append({"kind": kind, "shape": [8192, 8192, 8192], "us": r["us_per_launch"], "tflops": r["rate"], "launches": 50,
                     "frac": round(r["rate"] / (mult * bf16), 3), "peak": f"{src}{mult} (burst)",
                     "frac_sustained": None if sustained is None else round(r["rate"] / (mult * sustained), 3),
                     "timing": r["timing"]})
        r = time_one_gemm(kind, 16, 4096, 4096, 40, True)
        rows.append({"kind": kind, "shape": [16, 4096, 4096], "us": r["us_per_launch"], "gbps": r["gbps"],
                     "frac": round(r["gbps"] / hbm, 3), "peak": "hbm", "timing": r["timing"]})
    # int4 with many tokens (dequantize once + dense bf16 tcgen05 GEMM), against the bf16 peak
    K, N, M = 4096, 28672, 2048
    r = time_one_gemm("w4", K, N, M, 20, False)
    tf = 2.0 * M * N * K / (r["us_per_launch"] * 1e-6) / 1e12
    rows.append({"kind": "w4_prefill", "shape": [M, N, K], "us": r["us_per_launch"], "tflops": round(tf, 1), "launches": 20,
                 "frac": round(tf / bf16, 3), "peak": f"{src}1 (burst)",
                 "frac_sustained": None if sustained is None else round(tf / sustained, 3), "timing": r["timing"]})
    # the fused gate|up + SwiGLU launch at 64 tokens, as a weight stream
    r = time_one_gemm("w4swiglu", 4096, 28672, 64, 40, True)
    rows.append({"kind": "w4_gate_up_swiglu", "shape": [64, 28672, 4096], "us": r["us_per_launch"], "gbps": r["rate"],
                 "frac": round(r["rate"] / hbm, 3), "peak": "hbm", "timing": r["timing"]})
    # grouped fp8 GEMM: 8 experts x 512 tokens of a 4096 -> 28672 expert projection, one launch
    r = time_one_gemm("grouped", 4096, 28672, 4096, 20, False)
    rows.append({"kind": "grouped_fp8", "experts": EXPERTS, "shape": [4096, 28672, 4096], "us": r["us_per_launch"], "tflops": r["rate"],
                 "launches": 20, "frac": round(r["rate"] / (2 * bf16), 3), "peak": f"{src}2 (burst)",
                 "frac_sustained": None if sustained is None else round(r["rate"] / (2 * sustained), 3), "timing": r["timing"]})
    # quantizers and the packer's front end, as streams (bytes read + written)
    for kind, shape in (("quant-w4", (4096, 28672)), ("quant-fp8row", (8192, 8192)), ("quant-fp4", (8192, 8192))):
        r = time_one_gemm(kind, shape[0], shape[1], 0, 20, False)
        rows.append({"kind": kind, "shape": list(shape), "us": r["us_per_launch"], "gbps": r["rate"],
                     "frac": round(r["rate"] / hbm, 3), "peak": "hbm", "timing": r["timing"]})
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--allreduce", default="push", choices=["push", "nccl"],
                    help="N > 1: how the row-split GEMMs' outputs are summed")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline and the secondary (fp8 / fp4) legs")
    ap.add_argument("--one-gemm", default="", metavar="A,B,C",
                    help="profiling helper: run --steps launches of one GEMM shape through the public op and exit")
    ap.add_argument("--kind", default="w4", choices=["w4", "w4swiglu", "fp8", "fp8block", "mxfp8", "nvfp4", "mxfp4", "grouped",
                                                     "quant-w4", "quant-fp8row", "quant-fp8mx", "quant-fp4"],
                    help="with --one-gemm: which op (w4, w4swiglu take K,N,M; grouped T,N,K; quant-* rows,cols,0; the others M,N,K)")
    ap.add_argument("--graph", action="store_true", help="with --one-gemm: time the launches inside one CUDA graph")
    args = ap.parse_args()
    if args.one_gemm:
        run_one_gemm(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
