#!/usr/bin/env python
"""Benchmark of the matrix-multiplication path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload dense_tf32|dense_tf32x3|dense4000_tf32|linear_bwd|spgemm|spgemm_zipf|mlp]
                    [--no-extras]

One JSON line on stdout (rank 0).  The headline workload is the large batched
dense GEMM, 8 x 4096^3 fp32-in / TF32 per GPU (weak scaling: every rank owns 8
independent batches, no data-path collective).  A "step" is one pass of the
path over that batch.  `value` is whole-job TFLOP/s with inputs resident in
HBM; `e2e` is the same metric through the C ABI from pinned HOST buffers with
the host<->device copies inside the timed region.

`--impl reference` times the reference's own CPU GEMM (oracle/_ref, compiled
from the reference tree; the oracle port when that build is absent) on a
bounded row slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DENSE = {"dense_tf32": (4096, 0), "dense_tf32x3": (4096, 1), "dense4000_tf32": (4000, 0),
         "dense4000_tf32x3": (4000, 1)}
BATCH = 8


def dense_workload_text(n: int) -> str:
    return (f"dense batched GEMM y=a.b+c, per GPU batch={BATCH} M=N=K={n}, fp32 in/out, "
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


FUSED_RS_VALIDATED_WORLD = 8


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
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------- our arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_tf32")
    ap.add_argument("--linear-bwd-comm", default="fused", choices=["fused", "nccl"],
                    help="how the linear_bwd workload sums dW over ranks (see bench_linear_bwd)")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

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
    from sapphire_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
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
    def dense_inputs(n, on_device=True):
        # this rank's 8 batches of the global [8*world, n, n] tensors
        ids = list(range(rank * BATCH, (rank + 1) * BATCH))
        if on_device:
            # device-side generation keeps start-up short; the parity tests use the
            # numpy generators, the timing does not depend on the values
            g = torch.Generator(device=dev)
            g.manual_seed(1234 + rank)
            a = torch.randn(BATCH, n, n, device=dev, generator=g)
            b = torch.randn(BATCH, n, n, device=dev, generator=g)
            c = torch.rand(BATCH, n, n, device=dev, generator=g) * 2 - 1
            return a, b, c
        return W.dense_batched(0, ids, n, n, n, "normal")

    def bench_dense(n, mode, steps, warmup, sample_clocks):
        a, b, c = dense_inputs(n)
        out = torch.empty_like(c)
        fn = lambda: ops.gemm(ctx, a, b, c, out, mode=mode)
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
        flops = 2.0 * BATCH * n * n * n
        per_gpu = flops / ms / 1e9
        del a, b, c, out
        return ms, per_gpu, launches, clocks

    def bench_dense_e2e(n, mode, steps):
        """Host pinned buffers -> H2D -> GEMM -> D2H, all inside the timed region."""
        ha = torch.empty(BATCH, n, n).pin_memory()
        hb = torch.empty(BATCH, n, n).pin_memory()
        hc = torch.empty(BATCH, n, n).pin_memory()
        hy = torch.empty(BATCH, n, n).pin_memory()
        for h in (ha, hb, hc):
            h.normal_()
        da, db, dc = (torch.empty(BATCH, n, n, device=dev) for _ in range(3))
        dy = torch.empty(BATCH, n, n, device=dev)

        # per batch: H2D on one stream, GEMM on the compute stream, D2H on a third,
        # chained by events, so that the copies of batch i+1 overlap the GEMM of batch i
        h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(BATCH)]
        ev_out = [torch.cuda.Event() for _ in range(BATCH)]

        def step():
            main = torch.cuda.current_stream(dev)
            h2d.wait_stream(main)
            d2h.wait_stream(main)
            for i in range(BATCH):
                with torch.cuda.stream(h2d):
                    da[i].copy_(ha[i], non_blocking=True)
                    db[i].copy_(hb[i], non_blocking=True)
                    dc[i].copy_(hc[i], non_blocking=True)
                    ev_in[i].record(h2d)
                main.wait_event(ev_in[i])
                ops.gemm(ctx, da[i], db[i], dc[i], dy[i], mode=mode)
                ev_out[i].record(main)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(ev_out[i])
                    hy[i].copy_(dy[i], non_blocking=True)
            main.wait_stream(d2h)

        ms, _ = timed(step, steps, 1)
        nbytes = ha.numel() * 4
        return ms, 2.0 * BATCH * n ** 3 / ms / 1e9, 3 * nbytes, nbytes

    # --------------------------------------------------------------- sparse
    def bench_spgemm(dist_name, steps, warmup):
        M = N = 65536
        rA, cA, vA = W.csr_random(0 + 2 * rank, M, N, 0.001, dist_name)
        rB, cB, vB = W.csr_random(1, N, N, 0.001, dist_name)
        A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, dev)
        B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, dev)
        res = {}
        def fn():
            res["C"] = ops.spgemm(ctx, A, B)
        ms, launches = timed(fn, steps, warmup)
        nnzC = res["C"].nnz
        prods = int(W.csr_products(rA, cA, rB).sum())
        nbytes = 8 * (cA.size + cB.size + nnzC) + 4 * 3 * (M + 1)
        # dram read + written by the two row kernels of one call, from the ncu capture of the
        # half-size uniform case (profiles/spgemm_cta_rows_32768x65536.md: symbolic 41 + 217 MB,
        # numeric 652 + 1034 MB), scaled by the output size; no capture of the Zipf case
        traffic = (258.0e6 + 1686.0e6) * nnzC / 136.2e6 if dist_name == "poisson" else None
        return {"workload": spgemm_workload_text(dist_name), "ms_per_step": ms,
                "gflops_per_gpu": 2.0 * prods / ms / 1e6, "nnzC": nnzC, "products": prods,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6,
                             "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / pk["hbm_gbs"], "traffic": traffic,
                             "traffic_source": "ncu, scaled from the 32768-row capture" if traffic else None,
                             "peak_source": pk["source"]},
                "gpu_launches": launches}

    def bench_linear_bwd(steps, warmup, comm_mode="fused"):
        """dW = x^T.dy (+ dB) and dx = dy.W^T on this rank's 8192 rows.  With several
        ranks dW and dB are summed over the ranks inside the timed region:
          "fused"  the dW GEMM adds its tiles into the owning rank's window over
                   NVLink from its epilogue (GEMM + reduce-scatter in one kernel),
                   one tiny all-reduce as barrier, then every rank pulls the reduced
                   row blocks from the owners' windows with copy-engine transfers
                   while the dx GEMM runs (runner.FusedWeightGradient);
          "nccl"   plain GEMM, then an NCCL all-reduce of dW that overlaps the dx GEMM."""
        rows, width = 8192, 4096
        g = torch.Generator(device=dev); g.manual_seed(7 + rank)
        dy = torch.randn(rows, width, device=dev, generator=g) * 0.02
        x = torch.randn(rows, width, device=dev, generator=g) * 0.02
        w = torch.randn(width, width, device=dev, generator=g) * 0.02
        dx = torch.empty(rows, width, device=dev)
        dw = torch.empty(width, width, device=dev)
        db = torch.empty(width, device=dev)
        comm = torch.cuda.Stream(dev) if world > 1 else None
        done = torch.cuda.Event() if world > 1 else None
        fused = world > 1 and comm_mode == "fused" and width % (world * 128) == 0
        reducer = None
        if fused:
            from sapphire_b200 import runner as R
            reducer = R.FusedWeightGradient(ctx, width, width, rank, world)
            if not reducer.ok:                           # agreed across ranks: all fall back together
                reducer.close()
                reducer, fused = None, False

        def fn():
            main = torch.cuda.current_stream(dev)
            if fused:
                reducer.start(x, dy, dw, db)
            else:
                # dW first: its allreduce then travels while dX, which needs no exchange, computes
                ops.gemm(ctx, x, dy, None, dw, trans_a=True, colsum_out=db,     # dW = x^T.dy, dB
                         colsum_scale=1.0 / (rows * world))
                if world > 1:
                    done.record(main)
                    with torch.cuda.stream(comm):
                        comm.wait_event(done)
                        dist.all_reduce(dw)
                        dist.all_reduce(db)
            ops.gemm(ctx, dy, w, None, dx, trans_b=True)                    # dx = dy.W^T
            if fused:
                reducer.wait()
            elif world > 1:
                main.wait_stream(comm)
        ms, launches = timed(fn, steps, warmup)
        if reducer is not None:
            reducer.close()
        flops = 2 * 2.0 * rows * width * width
        label = "linear backward dY[8192x4096] X[8192x4096] W[4096x4096]"
        if world > 1:
            label += (" per GPU, dW reduce-scatter fused into the GEMM epilogue (peer adds) + "
                      "copy-engine gather" if fused else " per GPU, dW/dB NCCL allreduce overlapped with the dx GEMM")
        return {"workload": label, "ms_per_step": ms, "tflops_per_gpu": flops / ms / 1e9,
                "gpu_launches": launches}

    def bench_mlp(steps, warmup):
        """The 784-512-256-10 MLP training step, global batch 64 split over the
        ranks (strong scaling), one flat gradient allreduce per step.  lr 1e-4: at
        0.01 Sapphire's un-normalised gradients leave the finite range by step 3."""
        from sapphire_b200 import mlp as M
        Ws, bs = W.mlp_init(0)
        trainer = M.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32, world=world)
        per = 64 // world
        x, onehot = W.mlp_batch(0)
        xs = torch.from_numpy(x[rank * per:(rank + 1) * per]).to(dev)
        ys = torch.from_numpy(onehot[rank * per:(rank + 1) * per]).to(dev)
        ms, launches = timed(lambda: trainer.step(xs, ys), steps, warmup)
        flops = 3 * 2.0 * 64 * sum(i * o for i, o in zip(W.MLP_WIDTHS[:-1], W.MLP_WIDTHS[1:]))
        out = {"workload": f"MLP 784-512-256-10 SGD step, global batch 64 over {world} rank(s), "
                           "gradient allreduce inside", "ms_per_step": ms,
               "gflops_total": flops / ms / 1e6, "gpu_launches": launches,
               "kernels_per_step": launches // max(steps, 1)}
        try:
            trainer.capture(per)
            gms, _ = timed(lambda: trainer.step_graph(xs, ys), steps, warmup)
            out["ms_per_step_cuda_graph"] = gms
        except Exception as e:                       # capture is an optimisation, not the path
            out["cuda_graph_error"] = repr(e)[:200]
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
        return {"workload": "conv2d forward 32x64x56x56, 128 filters 3x3 pad 1 (im2col + batched GEMM)",
                "ms_per_step": ms_all, "tflops_per_gpu": flops / ms_all / 1e9,
                "im2col_ms": ms_cols,
                "im2col_roofline": {"bound": "hbm", "achieved": col_bytes / ms_cols / 1e6,
                                    "peak": pk["hbm_gbs"], "unit": "GB/s",
                                    "frac": col_bytes / ms_cols / 1e6 / pk["hbm_gbs"]},
                "gpu_launches": launches}

    # ------------------------------------------------------------- headline
    if args.workload in DENSE:
        n, mode = DENSE[args.workload]
        ms, per_gpu, launches, clocks = bench_dense(n, mode, args.steps, args.warmup, True)
        value = per_gpu * world
        tf32_peak = pk["bf16_tflops"] / 2.0
        line = {
            "metric": "batched dense GEMM throughput", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32" if mode == 0 else "3xtf32 (fp32-accurate)", "data": "synthetic",
            "config": {"workload": dense_workload_text(n),
                       "global_batch": BATCH * world, "parallelism": f"batch-sharded x{world}",
                       "l2": "inputs (3 x %d MiB) larger than the 126 MB L2" % (BATCH * n * n * 4 >> 20)},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tf32_peak,
                         "unit": "TFLOP/s", "frac": per_gpu / tf32_peak,
                         # dram read+write of one launch: 280.8 MB measured by ncu on the
                         # 4 x 2048^3 case (profiles/gemm_tcgen05_tf32_4x2048.md), scaled by
                         # the matrix bytes of this launch (traffic == every matrix once)
                         "traffic": 280.8e6 * (BATCH * n * n) / (4 * 2048 * 2048),
                         "traffic_source": "ncu, scaled from the 4x2048^3 capture",
                         "peak_source": f"{pk['source']}: cuBLAS bf16 burst / 2 (TF32 runs at half "
                                        "the bf16 rate)"},
            "gpu_launches": launches, "clocks": clocks,
        }
        e_ms, e_val, h2d, d2h = bench_dense_e2e(n, mode, max(2, min(args.steps, 5)))
        line["e2e"] = {"value": e_val * world, "unit": "TFLOP/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    elif args.workload in ("spgemm", "spgemm_zipf"):
        r = bench_spgemm("poisson" if args.workload == "spgemm" else "zipf", args.steps,
                         args.warmup)
        line = {"metric": "CSR SpGEMM throughput", "value": r["gflops_per_gpu"] * world,
                "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": r["workload"], "parallelism": f"A row blocks x{world}, B replicated"},
                "roofline": r["roofline"], "gpu_launches": r["gpu_launches"]}
    elif args.workload == "linear_bwd":
        r = bench_linear_bwd(args.steps, args.warmup, args.linear_bwd_comm)
        tf32_peak = pk["bf16_tflops"] / 2.0
        line = {"metric": "Linear backward GEMM throughput", "value": r["tflops_per_gpu"] * world,
                "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
                "config": {"workload": r["workload"]},
                "roofline": {"bound": "tensor", "achieved": r["tflops_per_gpu"], "peak": tf32_peak,
                             "unit": "TFLOP/s", "frac": r["tflops_per_gpu"] / tf32_peak,
                             "traffic": None},
                "gpu_launches": r["gpu_launches"]}
    elif args.workload == "mlp":
        r = bench_mlp(args.steps, args.warmup)
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

    if not args.no_extras and args.workload == "dense_tf32":
        extras = []
        for name in ("dense_tf32x3", "dense4000_tf32"):
            n, mode = DENSE[name]
            ms, per_gpu, _, _ = bench_dense(n, mode, 5, 3, False)
            extras.append({"workload": f"{name} batch={BATCH} n={n}", "ms_per_step": ms,
                           "tflops_per_gpu": per_gpu})
        # the fused GEMM + reduce-scatter route has been run on FUSED_RS_VALIDATED_WORLD ranks;
        # beyond that the default run keeps to the NCCL route (--workload linear_bwd
        # --linear-bwd-comm fused runs it on any rank count)
        if world > 1:
            extras.append(bench_linear_bwd(10, 3, "nccl"))
        if world <= FUSED_RS_VALIDATED_WORLD:
            extras.append(bench_linear_bwd(10, 3))
        extras.append(bench_spgemm("poisson", 5, 3))
        extras.append(bench_spgemm("zipf", 5, 3))
        extras.append(bench_mlp(50, 5))
        extras.append(bench_conv(10, 3))
        line["other_workloads"] = extras

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
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())


if __name__ == "__main__":
    main()
