"""Two-rank NCCL run of the data-parallel MLP step on two GPUs (skipped with
fewer): the weights after three steps must equal the single-process CPU oracle
on the full batch, which checks the dW SUM / dB MEAN rule end to end."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
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
    trainer = mlp.MlpTrainer(ctx, Ws, bs, 1e-4, mode=L.MODE_TF32X3, world=world)
    for t in range(3):
        x, onehot = W.mlp_batch(t)
        mine = runner.contiguous_shard(x.shape[0], world, rank)
        trainer.step(torch.from_numpy(x[mine.start:mine.stop]).to(dev),
                     torch.from_numpy(onehot[mine.start:mine.stop]).to(dev))
    torch.cuda.synchronize()
    ctx.check_device_status()
    if rank == 0:
        np.save(os.path.join(out_dir, "params.npy"), trainer.params.flat.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_dp_mlp_two_gpus_matches_single_process_oracle(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    from sapphire_b200 import workloads as W
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = np.load(os.path.join(str(tmp_path), "params.npy"))
    Ws, bs = W.mlp_init(0)
    net = O.MlpOracle(Ws, bs, 1e-4)
    for t in range(3):
        net.step(*W.mlp_batch(t))
    want = np.concatenate([w.reshape(-1) for w in net.W] + [b.reshape(-1) for b in net.b])
    err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
    assert err <= 1e-5, err
