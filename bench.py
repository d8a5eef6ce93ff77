#!/usr/bin/env python
"""Benchmark of the matrix-multiplication path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload dense_tf32|dense_tf32x3|dense4000_tf32|dense4000_tf32x3|
                                linear_bwd|spgemm|spgemm_zipf|mlp]
                    [--per-gpu-batch B] [--no-extras] [--case NAME]

One JSON line on stdout (rank 0).  The headline workload is the large batched
dense GEMM, GLOBAL batch 8 of 4096^3 fp32-in / TF32, batch-sharded over the
ranks (rank r of N takes a contiguous range of the 8 batches: strong scaling,
no data-path collective).  A "step" is one pass of the path over that batch.
`value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the same
metric through the C ABI from pinned HOST buffers with the host<->device copies
inside the timed region.  `--per-gpu-batch B` instead gives every rank B
batches of its own (weak scaling; reported as such).

The other workloads shard the same way the path does: `linear_bwd` cuts the
8192 rows of dY / X into row blocks (dX rows final, dW / dB summed over the
ranks inside the timed region), `spgemm` cuts A into row blocks balanced by
scalar products with B replicated, `mlp` splits the batch of 64.

`--impl reference` times the reference's own CPU GEMM (oracle/_ref, compiled
from the reference tree; the oracle port when that build is absent) on a
bounded row slice of the same workload.

`--case NAME` runs one small, self-terminating case of a kernel for a profiler
capture (more than the 126 MB L2 touched, at most ~1.5 GB held, every kernel
launched a handful of times) and prints a one-line JSON summary; see
PROFILE_CASES.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes (read + written) of one launch, from ncu captures of small cases of the same
# kernels (`--case dense_tf32`, `--case spgemm`, `--case spgemm_zipf`); the bench
# scales them to its own launch
DENSE_TRAFFIC_4x2048 = 280.8e6
SPGEMM_TRAFFIC_PER_NNZC = {"poisson": 1762.4e6 / 136.1e6, "zipf": 671.3e6 / 53.3e6}

DENSE = {"dense_tf32": (4096, 0), "dense_tf32x3": (4096, 1), "dense4000_tf32": (4000, 0),
         "dense4000_tf32x3": (4000, 1)}
BATCH = 8
EXTRAS_DEADLINE_S = 300          # the extra workloads of the default run, all together


def dense_workload_text(n: int, per_gpu: int = 0) -> str:
    what = f"per GPU batch={per_gpu}" if per_gpu else f"global batch={BATCH}"
    return (f"dense batched GEMM y=a.b+c, {what} M=N=K={n}, fp32 in/out, "
            "a,b~N(0,1) c~U[-1,1)")


def spgemm_workload_text(dist_name: str) -> str:
    return f"csr spgemm 65536^2 0.1% {dist_name}"


def peaks():
    """Roofline denominators: measured on this pool when the file is present."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU during a timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.f,
                stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None
        # nvidia-smi needs a moment to start: wait for its first line
        t0 = time.time()
        while self.p is not None and self.lines() == 0 and time.time() - t0 < 5.0:
            time.sleep(0.05)

    def lines(self) -> int:
        try:
            return sum(1 for _ in open(self.f.name))
        except OSError:
            return 0

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------- reference arm

def cpu_gemm_sample(n: int, rows: int, repeats: int = 1):
    """Times the reference CPU GEMM on `rows` output rows of one n^3 batch.
    Returns (seconds per pass, kind, flops per pass)."""
    from oracle import oracle as O
    from sapphire_b200 import workloads as W
    kind = "reference" if O.have_ref() else "port"
    a = W.normal(0, "a", (rows, n), 1.0, 0)
    b = W.normal(0, "b", (n, n), 1.0, 0)
    c = W.uniform_pm1(0, "c", (rows, n), 0)
    fn = O.ref().ref_gemm if kind == "reference" else O.port().orc_gemm
    best = None
    for _ in range(repeats):
        y = c.copy()
        t = time.perf_counter()
        fn(y.size, y.reshape(-1), a.reshape(-1), b.reshape(-1), rows, n, n)
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    return best, kind, 2.0 * rows * n * n


def cpu_spgemm_sample(dist_name: str, rows: int):
    """Times the CPU sparse oracle (the reference ships no sparse GEMM to time) on
    the first `rows` rows of the benchmark's A against the full B.
    Returns (seconds, flops)."""
    from oracle import oracle as O
    from sapphire_b200 import workloads as W
    from sapphire_b200 import runner
    M = N = 65536
    rA, cA, vA = W.csr_random(0, M, N, 0.001, dist_name)
    rB, cB, vB = W.csr_random(1, N, N, 0.001, dist_name)
    rb, cb, vb = runner.csr_row_block(rA, cA, vA, range(0, rows))
    t = time.perf_counter()
    _, _, _, prods = O.spgemm(rb, cb, vb, rB, cB, vB, rows, N)
    return time.perf_counter() - t, 2.0 * prods



def run_reference_arm(args):
    """The reference's own CPU implementation of the path on this host: for the
    dense workloads Sapphire's Dense::Naive::Gemm (single-threaded: the reference
    has no threading), for the sparse workloads the CPU oracle (the reference
    declares its sparse GEMM without defining it)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    if args.workload in ("spgemm", "spgemm_zipf"):
        dist_name = "poisson" if args.workload == "spgemm" else "zipf"
        rows = 4096
        for i in range(args.warmup + args.steps):
            dt, flops = cpu_spgemm_sample(dist_name, rows)
            if i >= args.warmup:
                times.append(dt)
        sec = float(np.mean(times))
        value, unit, metric, kind = flops / sec / 1e9, "GFLOP/s", "CSR SpGEMM throughput", "port"
        workload = spgemm_workload_text(dist_name)
        sample = f"first {rows} rows of A against the full B per step, Gustavson CPU oracle"
    else:
        n, _ = DENSE.get(args.workload, (4096, 0))
        rows = 32
        kind = None
        for i in range(args.warmup + args.steps):
            dt, kind, flops = cpu_gemm_sample(n, rows)
            if i >= args.warmup:
                times.append(dt)
        sec = float(np.mean(times))
        value, unit, metric = flops / sec / 1e12, "TFLOP/s", "batched dense GEMM throughput"
        workload = dense_workload_text(n)
        sample = (f"{rows} output rows of one {n}x{n}x{n} batch per step "
                  f"(2*{rows}*{n}^2 FLOP); the rate extrapolates to the full workload")
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------- small profiler cases

def _case_dense(mode, ta=False, tb=False, n=2048, batch=4, k=0):
    """k: inner dimension when it differs from n (k = 32 is one k-block per tile:
    the kernel is then all epilogue)."""
    import torch
    from sapphire_b200 import ops
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    k = k or n
    a = torch.randn(batch, k, n, device=dev, generator=g) if ta else torch.randn(batch, n, k, device=dev, generator=g)
    b = torch.randn(batch, n, k, device=dev, generator=g) if tb else torch.randn(batch, k, n, device=dev, generator=g)
    c = torch.rand(batch, n, n, device=dev, generator=g)
    out = torch.empty_like(c)
    for _ in range(3):
        ops.gemm(ctx, a, b, c, out, mode=mode, trans_a=ta, trans_b=tb)
    torch.cuda.synchronize()
    ctx.check_device_status()
    return {"check": float(out[0, 0, 0]), "launches": ctx.launch_count()}


def _case_dense_small_batch(K=1536):
    """A wide Linear layer's forward pass at batch 64, y = relu(bias + x.W): few
    tiles and a long inner dimension, the k-slices kernel (the operands are small: this
    case is latency-bound, not a DRAM measurement)."""
    import torch
    from sapphire_b200 import ops
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    x = torch.randn(64, K, device=dev, generator=g)
    w = torch.randn(K, 512, device=dev, generator=g)
    bias = torch.randn(512, device=dev, generator=g)
    out = torch.empty(64, 512, device=dev)
    for _ in range(3):
        ops.gemm(ctx, x, w, None, out, bias=bias, relu=True)
    torch.cuda.synchronize()
    ctx.check_device_status()
    return {"check": float(out[0, 0]), "launches": ctx.launch_count()}


def _case_spgemm(dist_name, M=32768, N=65536):
    import torch
    from sapphire_b200 import ops
    from sapphire_b200 import workloads as W
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    rA, cA, vA = W.csr_random(0, M, N, 0.001, dist_name)
    rB, cB, vB = W.csr_random(1, N, N, 0.001, dist_name)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, dev)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, dev)
    for _ in range(2):
        Cm = ops.spgemm(ctx, A, B)
    torch.cuda.synchronize()
    return {"nnzC": Cm.nnz, "nnzA": int(cA.size), "nnzB": int(cB.size),
            "products": int(W.csr_products(rA, cA, rB).sum()), "launches": ctx.launch_count()}


def _case_im2col():
    """The bench's convolution: 32 x 64 x 56 x 56 input, 3 x 3 taps, padding 1
    (cols = 231 MB, larger than L2)."""
    import torch
    from sapphire_b200 import conv, ops
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    x = torch.randn(32, 64, 56, 56, device=dev, generator=g)
    for _ in range(3):
        cols = conv.im2col(ctx, x, 3, 3, (1, 1), (1, 1), (1, 1))
    torch.cuda.synchronize()
    return {"check": float(cols[0, 0, 0]), "launches": ctx.launch_count()}


def _case_mlp():
    """Three eager steps of the 784-512-256-10 MLP at batch 64."""
    import torch
    from sapphire_b200 import _lib as L
    from sapphire_b200 import mlp, ops
    from sapphire_b200 import workloads as W
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    Ws, bs = W.mlp_init(0)
    trainer = mlp.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32)
    x, onehot = W.mlp_batch(0)
    x, onehot = torch.from_numpy(x).to(dev), torch.from_numpy(onehot).to(dev)
    for _ in range(3):
        loss = trainer.step(x, onehot)
    torch.cuda.synchronize()
    return {"check": float(loss[0]), "launches": ctx.launch_count()}


def _case_gemm_rs():
    """dW = x^T.dy for 8192 x 4096 x 4096 twice: a plain GEMM with its fused column
    sum, then the reduce-scatter variant with eight owners that all live on this
    GPU (the epilogue is the same code whoever owns the buffers)."""
    import torch
    from sapphire_b200 import ops
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    x = torch.randn(8192, 4096, device=dev, generator=g) * 0.02
    dy = torch.randn(8192, 4096, device=dev, generator=g) * 0.02
    dw = torch.empty(4096, 4096, device=dev)
    db = torch.empty(4096, device=dev)
    owners = [torch.zeros(512, 4096, device=dev) for _ in range(8)]
    for _ in range(3):
        ops.gemm(ctx, x, dy, None, dw, trans_a=True, colsum_out=db, colsum_scale=1.0 / 8192)
    for _ in range(3):
        ops.gemm_reduce_scatter(ctx, x, dy, [t.data_ptr() for t in owners], 4096, trans_a=True,
                                colsum_out=db, colsum_scale=1.0 / 8192)
    torch.cuda.synchronize()
    return {"check": float(dw[0, 0]), "check_rs": float(owners[0][0, 0]) / 3,
            "launches": ctx.launch_count()}


PROFILE_CASES = {
    "dense_tf32": lambda: _case_dense(0),                       # 4 x 2048^3, NN, pair kernel
    "dense_tf32x3": lambda: _case_dense(1),
    "dense_tn": lambda: _case_dense(0, ta=True),
    "dense_nt": lambda: _case_dense(0, tb=True),
    "dense_epilogue": lambda: _case_dense(0, n=8192, batch=1, k=32),
    "dense_small_batch": _case_dense_small_batch,               # 64 x 512 x 1536, bias + ReLU: k-slices kernel
    "dense_single_4096": lambda: _case_dense(0, n=4096, batch=1),   # what one GPU of eight runs
    "spgemm": lambda: _case_spgemm("poisson"),                  # 32768 rows of the 65536^2 case
    "spgemm_zipf": lambda: _case_spgemm("zipf"),
    "im2col": _case_im2col,
    "mlp": _case_mlp,
    "gemm_rs": _case_gemm_rs,
}


def pin_to_gpu_numa_node(local: int):
    """Binds this process to the CPUs next to its GPU, so that pinned host buffers
    allocated afterwards (first touch) sit on that NUMA node.  Returns the node
    number or None when the platform does not say."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        base = f"/sys/bus/pci/devices/{bus}"
        node = int(open(base + "/numa_node").read().strip())
        cpus = set()
        for part in open(base + "/local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        if cpus:
            os.sched_setaffinity(0, cpus & os.sched_getaffinity(0) or cpus)
        return node
    except Exception:
        return None


# --------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_tf32")
    ap.add_argument("--per-gpu-batch", type=int, default=0,
                    help="dense workloads: every rank gets this many batches of its own (weak "
                         "scaling) instead of its share of the global batch of 8")
    ap.add_argument("--linear-bwd-comm", default="fused", choices=["fused", "fused_store", "nccl"],
                    help="how the linear_bwd workload sums dW over ranks (see bench_linear_bwd)")
    ap.add_argument("--mlp-comm", default="peer", choices=["peer", "nccl"],
                    help="how the mlp workload sums its gradients over ranks (see bench_mlp)")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None, help="run one small profiler case and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.case:
        if args.case not in PROFILE_CASES:
            raise SystemExit(f"unknown case {args.case}; one of {sorted(PROFILE_CASES)}")
        print(json.dumps({"case": args.case, **PROFILE_CASES[args.case]()}), flush=True)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return

    # NCCL and others print to stdout: keep fd 1 for the one JSON line only
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    from sapphire_b200 import _lib as L
    from sapphire_b200 import ops
    from sapphire_b200 import runner as R
    from sapphire_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa_node = pin_to_gpu_numa_node(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    ctx = ops.Context(local)
    pk = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def timed(fn, steps, warmup):
        """CUDA-event time per step on the current stream, max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        launches0 = ctx.launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        return max_over_ranks(ms), (ctx.launch_count() - launches0)

    # ---------------------------------------------------------------- dense
    def my_batches(per_gpu):
        """(number of batches this rank owns, global batch).  Strong scaling: a
        contiguous share of the global batch of 8 (a rank beyond the 8th gets none)."""
        if per_gpu:
            return per_gpu, per_gpu * world
        return len(R.contiguous_shard(BATCH, world, rank)), BATCH

    def dense_inputs(n, nb):
        # device-side generation keeps start-up short; the parity tests use the
        # numpy generators, the timing does not depend on the values
        g = torch.Generator(device=dev)
        g.manual_seed(1234 + rank)
        a = torch.randn(max(nb, 1), n, n, device=dev, generator=g)
        b = torch.randn(max(nb, 1), n, n, device=dev, generator=g)
        c = torch.rand(max(nb, 1), n, n, device=dev, generator=g) * 2 - 1
        return a, b, c

    def bench_dense(n, mode, steps, warmup, sample_clocks, per_gpu=0, yardstick=False):
        nb, global_batch = my_batches(per_gpu)
        a, b, c = dense_inputs(n, nb)
        out = torch.empty_like(c)
        if nb:
            fn = lambda: ops.gemm(ctx, a[:nb], b[:nb], c[:nb], out[:nb], mode=mode)
        else:
            fn = lambda: None
        sampler = ClockSampler(local) if sample_clocks and rank == 0 else None
        n0 = sampler.lines() if sampler else 0
        ms, launches = timed(fn, steps, warmup)
        clocks = None
        if sampler:
            # a short timed region may end between two samples: keep the same loop
            # running (untimed) until a few samples under this load exist
            t0 = time.time()
            while sampler.lines() - n0 < 8 and time.time() - t0 < 2.0:
                for _ in range(10):
                    fn()
                torch.cuda.synchronize()
            clocks = sampler.stop()
            clocks["window"] = "warm-up + timed steps + untimed continuation of the same loop"
        ctx.check_device_status()
        res = {"ms": ms, "tflops_total": 2.0 * global_batch * n ** 3 / ms / 1e9,
               "launches": launches, "clocks": clocks, "global_batch": global_batch,
               "local_batch": nb}
        if yardstick and nb and mode == 0:
            # the library call the reference makes (cuBLAS TF32 through torch), same inputs
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            yfn = lambda: torch.baddbmm(c[:nb], a[:nb], b[:nb], out=out[:nb])
            yms, _ = timed(yfn, steps, warmup)
            torch.backends.cuda.matmul.allow_tf32 = prev
            res["yardstick"] = {
                "what": "cuBLAS TF32 (torch.baddbmm, allow_tf32) on the same inputs and batch split; "
                        "a library call, NOT on the product path",
                "ms_per_step": yms, "tflops_total": 2.0 * global_batch * n ** 3 / yms / 1e9}
        del a, b, c, out
        return res

    def bench_dense_e2e(n, mode, steps, per_gpu=0):
        """Host pinned buffers -> H2D -> GEMM -> D2H, all inside the timed region."""
        nb, global_batch = my_batches(per_gpu)
        m = max(nb, 1)
        ha, hb, hc, hy = (torch.empty(m, n, n).pin_memory() for _ in range(4))
        for h in (ha, hb, hc):
            h.normal_()
        da, db, dc, dy = (torch.empty(m, n, n, device=dev) for _ in range(4))

        # per batch: H2D on one stream, GEMM on the compute stream, D2H on a third,
        # chained by events, so that the copies of batch i+1 overlap the GEMM of batch i.
        # Steps follow each other like the passes of a streaming job: the uploads of the
        # next step start while the last product of this one is still on its way back;
        # a device buffer is overwritten only after its last reader of the step before
        # (events per batch: product done, result copied out).
        h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(m)]
        ev_out = [torch.cuda.Event() for _ in range(m)]
        ev_back = [torch.cuda.Event() for _ in range(m)]
        h2d.wait_stream(torch.cuda.current_stream(dev))      # the buffers above are initialised
        d2h.wait_stream(torch.cuda.current_stream(dev))

        def step():
            main = torch.cuda.current_stream(dev)
            for i in range(nb):
                with torch.cuda.stream(h2d):
                    h2d.wait_event(ev_out[i])               # the product that read these buffers
                    da[i].copy_(ha[i], non_blocking=True)
                    db[i].copy_(hb[i], non_blocking=True)
                    dc[i].copy_(hc[i], non_blocking=True)
                    ev_in[i].record(h2d)
                main.wait_event(ev_in[i])
                main.wait_event(ev_back[i])                 # dy[i] of the step before is on the host
                ops.gemm(ctx, da[i], db[i], dc[i], dy[i], mode=mode)
                ev_out[i].record(main)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(ev_out[i])
                    hy[i].copy_(dy[i], non_blocking=True)
                    ev_back[i].record(d2h)
            main.wait_stream(d2h)                           # the step ends when its results are back

        ms, _ = timed(step, steps, 1)
        per_batch = n * n * 4
        h2d_total = sum_over_ranks(3.0 * nb * per_batch)
        d2h_total = sum_over_ranks(1.0 * nb * per_batch)
        return ms, 2.0 * global_batch * n ** 3 / ms / 1e9, int(h2d_total), int(d2h_total)

    # --------------------------------------------------------------- sparse
    def bench_spgemm(dist_name, steps, warmup):
        """One global A (seed 0) and B (seed 1); rank r multiplies its row block of A,
        the blocks balanced by scalar products, against the whole (replicated) B.
        No collective: C stays distributed by rows."""
        M = N = 65536
        rA, cA, vA = W.csr_random(0, M, N, 0.001, dist_name)
        rB, cB, vB = W.csr_random(1, N, N, 0.001, dist_name)
        work = W.csr_products(rA, cA, rB)
        rows = R.balanced_row_blocks(work, world)[rank]
        rb, cb, vb = R.csr_row_block(rA, cA, vA, rows)
        A = ops.CsrMatrix.from_numpy(rb, cb, vb, len(rows), N, dev)
        B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, dev)
        res = {}
        def fn():
            res["C"] = ops.spgemm(ctx, A, B)
        ms, launches = timed(fn, steps, warmup)
        nnzC_local = res["C"].nnz
        nnzC = int(sum_over_ranks(float(nnzC_local)))
        prods = int(work.sum())
        # what one GPU must move: its rows of A and C, and all of B
        local_bytes = 8 * (cb.size + cB.size + nnzC_local) + 4 * 3 * (len(rows) + 1)
        nbytes = sum_over_ranks(float(local_bytes)) / world
        # dram read + written by one call's kernels, from an ncu capture of the first
        # 32768 rows of the same product, scaled by the output entries of this launch
        traffic = SPGEMM_TRAFFIC_PER_NNZC.get(dist_name)
        traffic = traffic * nnzC / world if traffic else None
        return {"workload": spgemm_workload_text(dist_name), "ms_per_step": ms,
                "gflops_total": 2.0 * prods / ms / 1e6, "nnzC": nnzC, "products": prods,
                "rows_of_rank0": len(rows),
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6,
                             "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / pk["hbm_gbs"], "traffic": traffic,
                             "traffic_source": "ncu on the first 32768 rows, scaled by nnz(C)" if traffic else None,
                             "per": "GPU (mean over ranks of the bytes each must move / max time)",
                             "peak_source": pk["source"]},
                "gpu_launches": launches}

    def bench_linear_bwd(steps, warmup, comm_mode="fused"):
        """Backward GEMMs of one Linear layer, global dY / X of 8192 rows cut into row
        blocks over the ranks (boundaries at multiples of 128): dx = dy.W^T is final
        per rank; dW = x^T.dy and dB are partial sums, added up over the ranks inside
        the timed region:
          "fused"  the dW GEMM adds its tiles into the owning rank's window over
                   NVLink from its epilogue (GEMM + reduce-scatter in one kernel),
                   one tiny all-reduce as barrier, then every rank pulls the reduced
                   row blocks from the owners' windows with copy-engine transfers
                   while the dx GEMM runs (runner.FusedWeightGradient, route "add");
          "fused_store"  the tiles are stored into this rank's slot of the owner's
                   window instead, the owner adds its slots in fixed order (a
                   bit-reproducible sum), second barrier, same gather (route "store");
          "nccl"   plain GEMM, then an NCCL all-reduce of dW that overlaps the dx GEMM.
        With several ranks the fused dW is checked against the NCCL route once,
        outside the timed region."""
        total_rows, width = 8192, 4096
        mine = R.row_shard(total_rows, world, rank, 128)
        rows = max(len(mine), 1)
        g = torch.Generator(device=dev); g.manual_seed(7 + rank)
        dy = torch.randn(rows, width, device=dev, generator=g) * 0.02
        x = torch.randn(rows, width, device=dev, generator=g) * 0.02
        w = torch.randn(width, width, device=dev, generator=g) * 0.02
        dx = torch.empty(rows, width, device=dev)
        dw = torch.empty(width, width, device=dev)
        db = torch.empty(width, device=dev)
        comm = torch.cuda.Stream(dev) if world > 1 else None
        done = torch.cuda.Event() if world > 1 else None
        fused = world > 1 and comm_mode in ("fused", "fused_store") and width % (world * 128) == 0
        reducer = None
        if fused:
            reducer = R.FusedWeightGradient(ctx, width, width, rank, world,
                                            route="add" if comm_mode == "fused" else "store")
            if not reducer.ok:                           # agreed across ranks: all fall back together
                reducer.close()
                reducer, fused = None, False

        def nccl_route():
            main = torch.cuda.current_stream(dev)
            # dW first: its allreduce then travels while dX, which needs no exchange, computes
            ops.gemm(ctx, x, dy, None, dw, trans_a=True, colsum_out=db,     # dW = x^T.dy, dB
                     colsum_scale=1.0 / total_rows)
            if world > 1:
                done.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.all_reduce(dw)
                    dist.all_reduce(db)
            ops.gemm(ctx, dy, w, None, dx, trans_b=True)                    # dx = dy.W^T
            if world > 1:
                main.wait_stream(comm)

        def fused_route():
            reducer.start(x, dy, dw, db, total_rows=total_rows)
            ops.gemm(ctx, dy, w, None, dx, trans_b=True)
            reducer.wait()

        check = None
        if fused:
            nccl_route()
            torch.cuda.synchronize()
            want_dw, want_db = dw.clone(), db.clone()
            fused_route()
            torch.cuda.synchronize()
            err_w = float((dw - want_dw).norm() / want_dw.norm())
            err_b = float((db - want_db).norm() / want_db.norm())
            check = {"dw_rel_err_fused_vs_nccl": max_over_ranks(err_w),
                     "db_rel_err_fused_vs_nccl": max_over_ranks(err_b)}
        fn = fused_route if fused else nccl_route
        ms, launches = timed(fn, steps, warmup)
        if reducer is not None:
            reducer.close()
        flops = 2 * 2.0 * total_rows * width * width
        label = f"linear backward dY[8192x4096] X[8192x4096] W[4096x4096], rows sharded x{world}"
        if world > 1:
            label += ((", dW reduce-scatter fused into the GEMM epilogue (peer adds) + copy-engine gather"
                       if comm_mode == "fused" else
                       ", dW tiles stored into the owners' slots from the GEMM epilogue, slots summed in "
                       "fixed order, copy-engine gather")
                      if fused else ", dW/dB NCCL allreduce overlapped with the dx GEMM")
        out = {"workload": label, "ms_per_step": ms, "tflops_total": flops / ms / 1e9,
               "gpu_launches": launches}
        if check:
            out["check"] = check
        return out

    def bench_mlp(steps, warmup, comm="peer"):
        """The 784-512-256-10 MLP training step, global batch 64 split over the
        ranks (strong scaling).  The gradients are summed over the ranks inside the
        step: comm "peer" = the library's exchange over peer memory fused with the
        SGD update (two kernels), "nccl" = one all-reduce of the flat bucket + scale +
        SGD.  lr 1e-4: at 0.01 Sapphire's un-normalised gradients leave the finite
        range by step 3."""
        from sapphire_b200 import mlp as M
        Ws, bs = W.mlp_init(0)
        trainer = M.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32, world=world, comm=comm, rank=rank)
        how = ("gradient exchange over peer memory fused with SGD" if trainer.exchange is not None
               else "NCCL gradient allreduce inside" if world > 1 else "single rank")
        per = 64 // world
        x, onehot = W.mlp_batch(0)
        xs = torch.from_numpy(x[rank * per:(rank + 1) * per]).to(dev)
        ys = torch.from_numpy(onehot[rank * per:(rank + 1) * per]).to(dev)
        ms, launches = timed(lambda: trainer.step(xs, ys), steps, warmup)
        flops = 3 * 2.0 * 64 * sum(i * o for i, o in zip(W.MLP_WIDTHS[:-1], W.MLP_WIDTHS[1:]))
        out = {"workload": f"MLP 784-512-256-10 SGD step, global batch 64 over {world} rank(s), {how}",
               "ms_per_step": ms,
               "gflops_total": flops / ms / 1e6, "gpu_launches": launches,
               "kernels_per_step": launches // max(steps, 1)}
        try:
            trainer.capture(per)
            gms, _ = timed(lambda: trainer.step_graph(xs, ys), steps, warmup)
            out["ms_per_step_cuda_graph"] = gms
        except Exception as e:                       # capture is an optimisation, not the path
            out["cuda_graph_error"] = repr(e)[:200]
        ctx.check_device_status()
        trainer.close()
        return out

    def bench_conv(steps, warmup):
        """Conv2D forward as im2col + one batched GEMM with the filter matrix shared
        by every image (the host lowering of the reference, run on the device):
        32 x 64 x 56 x 56 input, 128 filters of 3 x 3, padding 1."""
        from sapphire_b200 import conv
        N, Cc, H, Wd, Cout, k = 32, 64, 56, 56, 128, 3
        g = torch.Generator(device=dev); g.manual_seed(11 + rank)
        x = torch.randn(N, Cc, H, Wd, device=dev, generator=g)
        f = torch.randn(Cout, Cc, k, k, device=dev, generator=g) * 0.05
        y = torch.zeros(N, Cout, H, Wd, device=dev)
        ms_cols, _ = timed(lambda: conv.im2col(ctx, x, k, k, (1, 1), (1, 1), (1, 1)), steps, warmup)
        ms_all, launches = timed(lambda: conv.conv2d_forward(ctx, y, x, f, (1, 1), (1, 1), (1, 1)),
                                 steps, warmup)
        P, rows = H * Wd, Cc * k * k
        col_bytes = 4.0 * N * (Cc * H * Wd + rows * P)            # x read once, cols written once
        flops = 2.0 * N * Cout * rows * P
        return {"workload": "conv2d forward 32x64x56x56, 128 filters 3x3 pad 1 (im2col + batched GEMM), "
                            "replicated per rank",
                "ms_per_step": ms_all, "tflops_per_gpu": flops / ms_all / 1e9,
                "im2col_ms": ms_cols,
                "im2col_roofline": {"bound": "hbm", "achieved": col_bytes / ms_cols / 1e6,
                                    "peak": pk["hbm_gbs"], "unit": "GB/s",
                                    "frac": col_bytes / ms_cols / 1e6 / pk["hbm_gbs"]},
                "gpu_launches": launches}

    # ------------------------------------------------------------- headline
    tf32_peak = pk["bf16_tflops"] / 2.0
    peak_note = f"{pk['source']}: cuBLAS bf16 burst / 2 (TF32 runs at half the bf16 rate)"
    if args.workload in DENSE:
        n, mode = DENSE[args.workload]
        r = bench_dense(n, mode, args.steps, args.warmup, True, args.per_gpu_batch, yardstick=True)
        ms = r["ms"]
        # the slowest rank bounds the step: its share of the global batch is what one GPU achieved
        busiest = args.per_gpu_batch or -(-BATCH // world)
        per_gpu = 2.0 * busiest * n ** 3 / ms / 1e9
        line = {
            "metric": "batched dense GEMM throughput", "value": r["tflops_total"], "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak" if args.per_gpu_batch else "strong",
            "vs_baseline": None,
            "dtype": "tf32" if mode == 0 else "3xtf32 (fp32-accurate)", "data": "synthetic",
            "config": {"workload": dense_workload_text(n, args.per_gpu_batch),
                       "global_batch": r["global_batch"],
                       "parallelism": f"batch-sharded x{world} ({busiest} batch(es) on the busiest GPU)",
                       "l2": "working set per step (4 x %d MiB on the busiest GPU) larger than the "
                             "126 MB L2" % (busiest * n * n * 4 >> 20)},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tf32_peak,
                         "unit": "TFLOP/s", "frac": per_gpu / tf32_peak,
                         # dram read + write of one launch: measured by ncu on the 4 x 2048^3
                         # case, scaled by the matrix bytes of this launch (the capture shows
                         # traffic == every matrix once)
                         "traffic": DENSE_TRAFFIC_4x2048 * (busiest * n * n) / (4 * 2048 * 2048),
                         "traffic_source": "ncu, scaled from the 4x2048^3 capture",
                         "per": "GPU (the busiest rank's FLOPs / max-over-ranks time)",
                         "peak_source": peak_note},
            "gpu_launches": r["launches"], "clocks": r["clocks"],
        }
        if "yardstick" in r:
            line["yardstick"] = r["yardstick"]
        e_ms, e_val, h2d, d2h = bench_dense_e2e(n, mode, max(2, min(args.steps, 5)), args.per_gpu_batch)
        line["e2e"] = {"value": e_val, "unit": "TFLOP/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "host_numa_node_of_rank0": numa_node,
                       "note": "pinned host buffers allocated after binding each rank to the CPUs "
                               "next to its GPU; PCIe / host-memory bound"}
    elif args.workload in ("spgemm", "spgemm_zipf"):
        r = bench_spgemm("poisson" if args.workload == "spgemm" else "zipf", args.steps,
                         args.warmup)
        line = {"metric": "CSR SpGEMM throughput", "value": r["gflops_total"],
                "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": r["workload"],
                           "parallelism": f"A row blocks x{world} balanced by scalar products, B replicated",
                           "nnzC": r["nnzC"], "products": r["products"]},
                "roofline": r["roofline"], "gpu_launches": r["gpu_launches"]}
    elif args.workload == "linear_bwd":
        r = bench_linear_bwd(args.steps, args.warmup, args.linear_bwd_comm)
        per_gpu = r["tflops_total"] / world
        line = {"metric": "Linear backward GEMM throughput", "value": r["tflops_total"],
                "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
                "config": {"workload": r["workload"], "check": r.get("check")},
                "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tf32_peak,
                             "unit": "TFLOP/s", "frac": per_gpu / tf32_peak, "traffic": None,
                             "per": "GPU", "peak_source": peak_note},
                "gpu_launches": r["gpu_launches"]}
    elif args.workload == "mlp":
        r = bench_mlp(args.steps, args.warmup, args.mlp_comm)
        best = min(r["ms_per_step"], r.get("ms_per_step_cuda_graph", r["ms_per_step"]))
        line = {"metric": "MLP training step time", "value": best, "unit": "ms/step",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
                "config": {"workload": r["workload"], "eager_ms_per_step": r["ms_per_step"],
                           "cuda_graph_ms_per_step": r.get("ms_per_step_cuda_graph"),
                           "cuda_graph_error": r.get("cuda_graph_error")},
                "gpu_launches": r["gpu_launches"]}
    else:
        raise SystemExit(f"unknown workload {args.workload}")

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if args.workload in ("spgemm", "spgemm_zipf"):
            dist_name = "poisson" if args.workload == "spgemm" else "zipf"
            sec, flops = cpu_spgemm_sample(dist_name, 8192)
            line["cpu_baseline"] = {
                "value": flops / sec / 1e9, "unit": "GFLOP/s", "cores": 1, "kind": "port",
                "sample": f"first 8192 rows of A against the full B, {sec:.1f} s; CPU Gustavson "
                          "oracle (the reference ships no sparse GEMM implementation)"}
        else:
            n = DENSE.get(args.workload, (4096, 0))[0]
            rows = 96
            sec, kind, flops = cpu_gemm_sample(n, rows)
            line["cpu_baseline"] = {
                "value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
                "sample": f"{rows} output rows of one {n}^3 batch, {sec:.1f} s; Sapphire's CPU GEMM "
                          "is a single-threaded scalar loop"}

    if not args.no_extras and args.workload == "dense_tf32" and not args.per_gpu_batch:
        extras = []
        line["other_workloads"] = extras

        # The headline above is measured; should one of the extra workloads below stall
        # (a rank that died, a collective that never completes) every rank leaves after
        # the deadline and rank 0 still prints the line with the extras finished so far.
        def give_up():
            if rank == 0:
                line["other_workloads_incomplete"] = (
                    f"stopped after {EXTRAS_DEADLINE_S} s with {len(extras)} extra workload(s) done")
                os.write(json_fd, (json.dumps(line) + "\n").encode())
            os._exit(0)

        watchdog = threading.Timer(EXTRAS_DEADLINE_S, give_up)
        watchdog.daemon = True
        watchdog.start()
        for name in ("dense_tf32x3", "dense4000_tf32"):
            n, mode = DENSE[name]
            r = bench_dense(n, mode, 5, 3, False)
            extras.append({"workload": f"{name} global batch={BATCH} n={n}, batch-sharded x{world}",
                           "scaling": "strong", "ms_per_step": r["ms"], "tflops_total": r["tflops_total"]})
        if world > 1:
            # every rank with 8 batches of its own: shows that the ranks do not disturb each other
            r = bench_dense(4096, 0, 5, 3, False, per_gpu=BATCH)
            extras.append({"workload": f"dense_tf32 per GPU batch={BATCH} n=4096", "scaling": "weak",
                           "ms_per_step": r["ms"], "tflops_total": r["tflops_total"]})
            extras.append(bench_linear_bwd(10, 3, "nccl"))
        extras.append(bench_linear_bwd(10, 3))
        extras.append(bench_spgemm("poisson", 5, 3))
        extras.append(bench_spgemm("zipf", 5, 3))
        extras.append(bench_mlp(50, 5))
        if world > 1:
            extras.append(bench_mlp(50, 5, "nccl"))
        extras.append(bench_conv(10, 3))
        watchdog.cancel()

    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())


if __name__ == "__main__":
    main()
