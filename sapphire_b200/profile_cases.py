"""Small, self-terminating cases of each kernel for `ncu` captures.

    python -m sapphire_b200.profile_cases dense_tf32 | dense_tf32x3 | dense_tn | spgemm | spgemm_zipf
                                          | im2col | mlp | gemm_rs | dense_epilogue

Each case touches more than the 126 MB L2 but holds at most ~1.5 GB on the
device and launches every kernel a handful of times, so that a full-set
capture of one or two launches ends by itself within a couple of minutes.
"""
from __future__ import annotations

import sys

import torch

from . import _lib as L
from . import ops
from . import workloads as W


def dense(mode: int, ta: bool = False, tb: bool = False, n: int = 2048, batch: int = 4, k: int = 0) -> None:
    """k: inner dimension when it differs from n (k = 32 is one k-block per tile:
    the kernel is then all epilogue)."""
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
    print("dense case done", float(out[0, 0, 0]))


def spgemm(dist: str, M: int = 32768, N: int = 65536) -> None:
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    rA, cA, vA = W.csr_random(0, M, N, 0.001, dist)
    rB, cB, vB = W.csr_random(1, N, N, 0.001, dist)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, dev)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, dev)
    for _ in range(2):
        Cm = ops.spgemm(ctx, A, B)
    torch.cuda.synchronize()
    print("spgemm case done", Cm.nnz)


def im2col() -> None:
    """The bench's convolution: 32 x 64 x 56 x 56 input, 3 x 3 taps, padding 1
    (cols = 231 MB, larger than L2)."""
    from . import conv
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    x = torch.randn(32, 64, 56, 56, device=dev, generator=g)
    for _ in range(3):
        cols = conv.im2col(ctx, x, 3, 3, (1, 1), (1, 1), (1, 1))
    torch.cuda.synchronize()
    print("im2col case done", float(cols[0, 0, 0]))


def mlp_step() -> None:
    """Three eager steps of the 784-512-256-10 MLP at batch 64."""
    from . import mlp
    dev = torch.device("cuda:0")
    ctx = ops.Context(0)
    Ws, bs = W.mlp_init(0)
    trainer = mlp.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32)
    x, onehot = W.mlp_batch(0)
    x, onehot = torch.from_numpy(x).to(dev), torch.from_numpy(onehot).to(dev)
    for _ in range(3):
        loss = trainer.step(x, onehot)
    torch.cuda.synchronize()
    print("mlp case done", float(loss[0]))


def gemm_reduce_scatter() -> None:
    """dW = x^T.dy for 8192 x 4096 x 4096 twice: a plain GEMM with its fused column
    sum, then the reduce-scatter variant with eight owners that all live on this
    GPU (the epilogue is the same code whoever owns the buffers)."""
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
    print("gemm_rs case done", float(dw[0, 0]), float(owners[0][0, 0]) / 3)


def main() -> None:
    case = sys.argv[1] if len(sys.argv) > 1 else "dense_tf32"
    if case == "dense_tf32":
        dense(L.MODE_TF32)
    elif case == "dense_tf32x3":
        dense(L.MODE_TF32X3)
    elif case == "dense_tn":
        dense(L.MODE_TF32, ta=True)
    elif case == "dense_nt":
        dense(L.MODE_TF32, tb=True)
    elif case == "spgemm":
        spgemm("poisson")
    elif case == "spgemm_zipf":
        spgemm("zipf")
    elif case == "im2col":
        im2col()
    elif case == "mlp":
        mlp_step()
    elif case == "gemm_rs":
        gemm_reduce_scatter()
    elif case == "dense_epilogue":
        dense(L.MODE_TF32, n=8192, batch=1, k=32)
    else:
        raise SystemExit(f"unknown case {case}")


if __name__ == "__main__":
    main()
