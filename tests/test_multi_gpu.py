"""Two-rank runs of the data-parallel MLP step on two GPUs (skipped with fewer),
with the gradients summed by an NCCL all-reduce and by the library's own exchange
over peer memory: the weights after five steps (for the peer exchange the last two
are replays of the captured CUDA graph) must equal the single-process CPU oracle on
the full batch, which checks the dW SUM / dB MEAN rule end to end."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir, comm):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                      RANK=str(rank), LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from sapphire_b200 import _lib as L
    from sapphire_b200 import mlp, ops, runner
    from sapphire_b200 import workloads as W
    runner.init_distributed("nccl")
    dev = torch.device("cuda", rank)
    ctx = ops.Context(rank)
    Ws, bs = W.mlp_init(0)
    trainer = mlp.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32X3, world=world, comm=comm, rank=rank)
    assert (trainer.exchange is not None) == (comm == "peer")

    def shard(t):
        x, onehot = W.mlp_batch(t)
        mine = runner.contiguous_shard(x.shape[0], world, rank)
        return (torch.from_numpy(x[mine.start:mine.stop]).to(dev),
                torch.from_numpy(onehot[mine.start:mine.stop]).to(dev))

    for t in range(3):
        trainer.step(*shard(t))
    torch.cuda.synchronize()
    ctx.check_device_status()
    if comm == "peer":
        # the exchange keeps its step number on the device: the captured step replays
        trainer.capture(shard(0)[0].shape[0])
        for t in range(3, 5):
            trainer.step_graph(*shard(t))
    else:
        for t in range(3, 5):
            trainer.step(*shard(t))
    torch.cuda.synchronize()
    ctx.check_device_status()
    np.save(os.path.join(out_dir, f"params{rank}.npy"), trainer.params.compact().cpu().numpy())
    dist.barrier()
    trainer.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("comm", ["nccl", "peer"])
def test_dp_mlp_two_gpus_matches_single_process_oracle(tmp_path, comm):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    from sapphire_b200 import workloads as W
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path), comm), nprocs=2, join=True)
    got = [np.load(os.path.join(str(tmp_path), f"params{r}.npy")) for r in range(2)]
    Ws, bs = W.mlp_init(0)
    net = O.MlpOracle(Ws, bs, 1e-4)
    for t in range(5):
        net.step(*W.mlp_batch(t))
    want = np.concatenate([w.reshape(-1) for w in net.W] + [b.reshape(-1) for b in net.b])
    err = np.linalg.norm(got[0].astype(np.float64) - want) / np.linalg.norm(want)
    assert err <= 1e-5, err
    # every rank applied the same summed gradient: replicas stay bit-identical
    assert np.array_equal(got[0].view(np.uint32), got[1].view(np.uint32))


def _rs_worker(rank, world, port, out_dir, route):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                      RANK=str(rank), LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from sapphire_b200 import _lib as L
    from sapphire_b200 import ops, runner
    runner.init_distributed("nccl")
    dev = torch.device("cuda", rank)
    ctx = ops.Context(rank)
    rows, n_in, n_out = 512, 1024, 768                 # per-rank batch rows; dW is [n_in, n_out]
    g = torch.Generator(device=dev); g.manual_seed(100 + rank)
    reducer = runner.FusedWeightGradient(ctx, n_in, n_out, rank, world, route=route)
    assert reducer.ok
    dw = torch.empty(n_in, n_out, device=dev)
    db = torch.empty(n_out, device=dev)
    worst = 0.0
    for _ in range(5):                                  # the three windows come round again
        x = torch.randn(rows, n_in, device=dev, generator=g)
        dy = torch.randn(rows, n_out, device=dev, generator=g)
        reducer.start(x, dy, dw, db, mode=L.MODE_TF32X3)
        reducer.wait()
        # the unfused route: local product, NCCL all-reduce
        ref = ops.gemm(ctx, x, dy, trans_a=True, mode=L.MODE_TF32X3)
        dist.all_reduce(ref)
        worst = max(worst, float((dw - ref).norm() / ref.norm()))
    xs = [torch.empty_like(x) for _ in range(world)]
    dys = [torch.empty_like(dy) for _ in range(world)]
    dist.all_gather(xs, x); dist.all_gather(dys, dy)
    torch.cuda.synchronize()
    ctx.check_device_status()
    if rank == 0:
        X = torch.cat(xs).double().cpu().numpy(); DY = torch.cat(dys).double().cpu().numpy()
        np.savez(os.path.join(out_dir, "rs.npz"), dw=dw.cpu().numpy(), ref=ref.cpu().numpy(),
                 db=db.cpu().numpy(), exact_dw=X.T @ DY, exact_db=DY.mean(0), worst=worst)
    reducer.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("route", ["store", "add"])
def test_gemm_fused_with_reduce_scatter_over_peer_memory(tmp_path, route):
    """Each rank's dW tiles go from the GEMM epilogue to the owning rank's window over
    CUDA IPC peer mappings -- stored into the rank's own slot and summed by the owner in
    slot order ("store"), or added with system-scope fp32 reductions ("add"); after the
    copy-engine gather every rank holds the sum over ranks, equal to the all-reduce of
    the local products and to the fp64 product of the gathered operands."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_rs_worker, args=(2, port, str(tmp_path), route), nprocs=2, join=True)
    r = np.load(os.path.join(str(tmp_path), "rs.npz"))
    scale = np.linalg.norm(r["exact_dw"])
    assert np.linalg.norm(r["dw"] - r["exact_dw"]) / scale <= 1e-5
    assert np.linalg.norm(r["dw"].astype(np.float64) - r["ref"]) / scale <= 1e-6
    assert np.abs(r["db"] - r["exact_db"]).max() <= 1e-5
    assert float(r["worst"]) <= 1e-6                    # every one of the five steps
