"""CPU tests of the multi-GPU host logic: sharding helpers, and the gradient
reduction rule exercised by two real ranks over gloo."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sapphire_b200 import runner
from sapphire_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_contiguous_shard_covers_everything():
    for n in (0, 1, 7, 8, 13):
        for world in (1, 2, 4, 8):
            seen = []
            for r in range(world):
                seen += list(runner.contiguous_shard(n, world, r))
            assert seen == list(range(n))


def test_row_shard_alignment():
    blocks = [runner.row_shard(8192, 8, r, align=1024) for r in range(8)]
    assert [len(b) for b in blocks] == [1024] * 8
    blocks = [runner.row_shard(1000, 4, r, align=128) for r in range(4)]
    assert blocks[0].start == 0 and blocks[-1].stop == 1000
    assert all(b.start % 128 == 0 for b in blocks)
    assert sum(len(b) for b in blocks) == 1000


def test_balanced_row_blocks_balance_products():
    rA, cA, _ = W.csr_random(0, 4096, 4096, row_dist="zipf", zipf_cap=1024)
    rB, _, _ = W.csr_random(1, 4096, 4096, row_dist="zipf", zipf_cap=1024)
    work = W.csr_products(rA, cA, rB)
    blocks = runner.balanced_row_blocks(work, 8)
    assert blocks[0].start == 0 and blocks[-1].stop == 4096
    assert all(blocks[i].stop == blocks[i + 1].start for i in range(7))
    sums = np.array([work[b.start:b.stop].sum() for b in blocks])
    assert sums.sum() == work.sum()
    # no block exceeds the ideal share by more than the heaviest single row
    assert sums.max() <= work.sum() / 8 + work.max()


def test_csr_row_block_rebases_row_pointers():
    r, c, v = W.csr_random(3, 100, 50, 0.1)
    rb, cb, vb = runner.csr_row_block(r, c, v, range(20, 60))
    assert rb[0] == 0 and rb[-1] == cb.size == vb.size
    assert np.array_equal(np.diff(rb.astype(np.int64)), np.diff(r[20:61].astype(np.int64)))
    assert np.array_equal(cb, c[r[20]:r[60]])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _dp_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
                      RANK=str(rank), LOCAL_RANK=str(rank))
    from oracle import oracle as O
    w, r, _ = runner.init_distributed("gloo")
    assert (w, r) == (world, rank)
    Ws, bs = W.mlp_init(0)
    x, onehot = W.mlp_batch(0)
    mine = runner.contiguous_shard(x.shape[0], world, rank)
    net = O.MlpOracle(Ws, bs, 0.01)
    _, dW, dB = net.gradients(x[mine.start:mine.stop], onehot[mine.start:mine.stop])
    bucket = runner.GradBucket.create([w_.shape for w_ in Ws], "cpu")
    for dst, g in zip(bucket.dW, dW):
        dst.copy_(torch.from_numpy(g))
    for dst, g in zip(bucket.dB, dB):
        dst.copy_(torch.from_numpy(g))
    bucket.allreduce(world)
    if rank == 0:
        np.save(os.path.join(out_dir, "flat.npy"), bucket.compact().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_dp_gradient_reduction_rule_two_ranks(tmp_path):
    """dW SUM + dB MEAN over two half batches equals the single-process batch-64
    gradients of the CPU oracle."""
    from oracle import oracle as O
    world = 2
    mp.spawn(_dp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    flat = np.load(os.path.join(str(tmp_path), "flat.npy"))
    Ws, bs = W.mlp_init(0)
    x, onehot = W.mlp_batch(0)
    _, dW, dB = O.MlpOracle(Ws, bs, 0.01).gradients(x, onehot)
    want = np.concatenate([g.reshape(-1) for g in dW] + [g.reshape(-1) for g in dB])
    err = np.linalg.norm(flat - want) / np.linalg.norm(want)
    assert err <= 1e-6, err
