"""Multi-GPU runner: one process per GPU, torch.distributed for the plumbing.

Work is partitioned, not replicated:

* batched dense GEMM   contiguous batch ranges per rank, no collective;
* Linear backward      row blocks of dY / X per rank, W replicated; dX rows are
                       final, dW and dB partial sums need one allreduce;
* data-parallel MLP    the batch is split; all gradients travel in one flat
                       bucket, one allreduce per step;
* CSR sparse GEMM      row blocks of A balanced by scalar products, B
                       replicated, no collective (C stays distributed).

Reduction rule of the gradients.  Sapphire's Linear backward leaves dW as the
plain sum over the samples of the batch and scales dB by 1 / batch
(Sources/Sapphire/operations/Backward/LinearBackward.cpp:72-73, 93-97).  With the batch
split over R ranks the single-process result is therefore

    dW = SUM over ranks of dW_local          dB = MEAN over ranks of dB_local

(each local dB already carries 1 / local batch).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def env_world() -> Tuple[int, int, int]:
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_distributed(backend: str) -> Tuple[int, int, int]:
    world, rank, local = env_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return world, rank, local


# ------------------------------------------------------------------ sharding

def contiguous_shard(n_items: int, world: int, rank: int) -> range:
    """Items [lo, hi) of rank: the first n % world ranks take one extra."""
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def row_shard(rows: int, world: int, rank: int, align: int = 1) -> range:
    """Row block of rank with boundaries at multiples of `align`."""
    units = (rows + align - 1) // align
    r = contiguous_shard(units, world, rank)
    return range(min(r.start * align, rows), min(r.stop * align, rows))


def balanced_row_blocks(work: np.ndarray, world: int) -> List[range]:
    """Contiguous row blocks with near-equal total work (scalar products of the
    sparse GEMM): block r ends where the running sum passes (r+1)/world of the total."""
    work = np.asarray(work, dtype=np.int64)
    cs = np.concatenate([[0], np.cumsum(work)])
    total = int(cs[-1])
    cuts = [0]
    for r in range(1, world):
        target = total * r / world
        cut = int(np.searchsorted(cs, target, side="left"))
        cuts.append(max(cuts[-1], min(cut, work.size)))
    cuts.append(work.size)
    return [range(cuts[r], cuts[r + 1]) for r in range(world)]


def csr_row_block(row: np.ndarray, col: np.ndarray, val: np.ndarray, rows: range):
    """The CSR arrays of a block of rows (ROW rebased to start at 0)."""
    lo, hi = int(row[rows.start]), int(row[rows.stop])
    return ((row[rows.start:rows.stop + 1].astype(np.int64) - lo).astype(np.uint32),
            col[lo:hi], val[lo:hi])


# ------------------------------------------------------------ gradient bucket

@dataclass
class GradBucket:
    """All gradients (or parameters) of the MLP in one flat fp32 buffer: the dW
    blocks first, then the dB blocks, so that the mean scaling touches one
    contiguous tail.  Rows are padded to a multiple of four floats (the padding
    stays zero): a [256, 10] weight then has a 16-byte row pitch, which is what
    the tensor-core GEMM's TMA loads need -- unpadded it would fall to the
    CUDA-core kernel.  ``dW[l]`` / ``dB[l]`` are views of the logical shape;
    ``compact()`` returns the values without the padding."""
    flat: torch.Tensor
    dW: List[torch.Tensor]
    dB: List[torch.Tensor]
    n_weight: int

    @staticmethod
    def size(shapes: Sequence[Tuple[int, int]], pad: int = 4) -> int:
        """Floats in the flat buffer of these layer shapes."""
        ld = [(o + pad - 1) // pad * pad for _, o in shapes]
        return sum(i * l for (i, _), l in zip(shapes, ld)) + sum(ld)

    @staticmethod
    def create(shapes: Sequence[Tuple[int, int]], device, pad: int = 4,
               flat: "torch.Tensor | None" = None) -> "GradBucket":
        """``flat``: use this zeroed 1-D fp32 buffer (e.g. memory other ranks map)
        instead of allocating one."""
        ld = [(o + pad - 1) // pad * pad for _, o in shapes]
        nW = sum(i * l for (i, _), l in zip(shapes, ld))
        nB = sum(ld)
        if flat is None:
            flat = torch.zeros(nW + nB, dtype=torch.float32, device=device)
        elif flat.numel() != nW + nB or flat.dtype != torch.float32 or not flat.is_contiguous():
            raise ValueError("flat must be a contiguous fp32 buffer of GradBucket.size(shapes, pad) elements")
        dW, dB, off = [], [], 0
        for (i, o), l in zip(shapes, ld):
            dW.append(flat[off:off + i * l].view(i, l)[:, :o])
            off += i * l
        for (_, o), l in zip(shapes, ld):
            dB.append(flat[off:off + l][:o])
            off += l
        return GradBucket(flat, dW, dB, nW)

    def compact(self) -> torch.Tensor:
        """The dW blocks then the dB blocks, without row padding."""
        return torch.cat([w.reshape(-1) for w in self.dW] + [b.reshape(-1) for b in self.dB])

    def allreduce(self, world: int, scale_fn=None) -> None:
        """dW: SUM over ranks.  dB: MEAN over ranks."""
        if world <= 1:
            return
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM)
        tail = self.flat[self.n_weight:]
        if scale_fn is None:
            tail.mul_(1.0 / world)
        else:
            scale_fn(tail, 1.0 / world)


# ------------------------------------------------- gradient exchange, no NCCL

class PeerGradExchange:
    """The gradient sum of a data-parallel step over peer memory, fused with the SGD
    update (``sb200_dp_reduce`` + ``sb200_dp_update``): two kernels per step instead
    of an NCCL all-reduce, a scale and an SGD kernel.

    ``grads`` is this rank's flat gradient bucket (``count`` floats) in memory the
    other ranks map; build the ``GradBucket`` over it.  ``step(params, lr)`` enqueues
    the two kernels on the current stream; every rank must call it once per step.
    ``n_sum``: the first n_sum elements are summed over the ranks, the rest averaged
    (dW SUM, dB MEAN).  Construction and ``close`` are collective."""

    def __init__(self, ctx, count: int, n_sum: int, rank: int = 0, world: int = 1, group=None):
        import ctypes as C
        from . import _lib as L
        self.ctx, self.count, self.n_sum, self.rank, self.world = ctx, count, n_sum, rank, world
        self._L, self._C = L, C
        self._grads = PeerWindow(ctx, 1, count, rank, world, group)
        self._reduced = PeerWindow(ctx, 1, count, rank, world, group)
        self._flags = PeerWindow(ctx, 1, L.DP_FLAG_WORDS, rank, world, group)
        self.ok = self._grads.ok and self._reduced.ok and self._flags.ok
        self.grads = self._grads.mine.view(-1)
        self.grads.zero_()
        self._flags.mine.zero_()
        torch.cuda.synchronize(ctx.device)
        if world > 1:
            dist.barrier(group=group)                      # every rank's flag words are zero
        g = L.DpGroup()
        g.world, g.rank = world, rank
        for r in range(world):
            g.grads[r] = self._grads.pointers[r]
            g.reduced[r] = self._reduced.pointers[r]
            g.flags[r] = self._flags.pointers[r]
        self._group = g

    def step(self, params: torch.Tensor, lr: float) -> None:
        L, C = self._L, self._C
        st = torch.cuda.current_stream(torch.device("cuda", self.ctx.device)).cuda_stream
        L.check("sb200_dp_reduce", L.lib().sb200_dp_reduce(self.ctx.handle, C.byref(self._group),
                                                           self.count, st))
        L.check("sb200_dp_update", L.lib().sb200_dp_update(self.ctx.handle, C.byref(self._group),
                                                           params.data_ptr(), self.count, self.n_sum,
                                                           float(lr), st))

    def close(self, group=None) -> None:
        for w in (self._grads, self._reduced, self._flags):
            w.close(group)


# ------------------------------------------- GEMM fused with its reduce-scatter

class PeerWindow:
    """One [rows, cols] fp32 buffer per rank that every rank of the node can add
    into: the landing zone of ``ops.gemm_reduce_scatter``.  ``mine`` is this
    rank's buffer as a tensor; ``pointers[o]`` is rank o's buffer as seen from
    this process (a CUDA IPC mapping for o != rank).  Handles travel through
    ``all_gather_object``.  With ``world == 1`` no IPC is involved.

    Construction is collective and does not raise half-way: a rank whose
    mapping fails still takes part in the closing barrier and every rank then
    sees ``ok == False`` (agreed by an all-reduce), so that callers can fall
    back together instead of leaving some ranks inside a collective."""

    def __init__(self, ctx, rows: int, cols: int, rank: int = 0, world: int = 1, group=None):
        import ctypes as C
        from . import _lib as L
        self.ctx, self.rank, self.world, self.rows, self.cols = ctx, rank, world, rows, cols
        self._lib, self._C = L, C
        nbytes = rows * cols * 4
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        L.check("sb200_peer_alloc", L.lib().sb200_peer_alloc(ctx.handle, nbytes, C.byref(ptr), handle))
        self._own = ptr.value
        self.mine = _tensor_over(self._own, rows, cols, ctx.device, self)
        self.pointers: List[int] = [0] * world
        self.pointers[rank] = self._own
        self._opened: List[int] = []
        self.ok = True
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            for o in range(world):
                if o == rank:
                    continue
                p = C.c_void_p()
                if L.lib().sb200_peer_open(ctx.handle, handles[o], C.byref(p)) != 0 or not p.value:
                    self.ok = False
                    continue
                self.pointers[o] = p.value
                self._opened.append(p.value)
            # nobody frees before everybody has mapped, and everybody learns whether all could
            agreed = torch.tensor([1.0 if self.ok else 0.0], device=torch.device("cuda", ctx.device))
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            self.ok = bool(agreed.item() > 0.5)
        # every rank's buffer as a tensor of this process (peer mappings for the others):
        # sources of copy-engine transfers, never operands of library kernels
        self.views: List[torch.Tensor] = [
            self.mine if o == rank else
            (_tensor_over(self.pointers[o], rows, cols, ctx.device, self) if self.pointers[o] else None)
            for o in range(world)]

    def close(self, group=None) -> None:
        """Unmaps the peers' buffers, waits for every rank to have done so, frees
        this rank's buffer.  ``mine`` must not be used afterwards."""
        L = self._lib
        torch.cuda.synchronize(self.ctx.device)
        for p in self._opened:
            L.lib().sb200_peer_close(self.ctx.handle, p)
        self._opened = []
        if self.world > 1:
            dist.barrier(group=group)
        if self._own:
            L.lib().sb200_peer_free(self.ctx.handle, self._own)
            self._own = 0


def _tensor_over(ptr: int, rows: int, cols: int, device: int, keepalive) -> torch.Tensor:
    """A torch view of library-owned device memory (no copy, no ownership)."""
    class _Iface:
        pass
    holder = _Iface()
    holder.__cuda_array_interface__ = {"shape": (rows, cols), "typestr": "<f4", "data": (ptr, False),
                                       "version": 3, "strides": None}
    holder._keepalive = keepalive
    return torch.as_tensor(holder, device=torch.device("cuda", device))


class PeerBarrier:
    """A barrier between the ranks' streams without a collective library: every rank
    holds SB200_DP_FLAG_WORDS flag words that the others map, and ``sb200_peer_barrier``
    (a one-warp kernel) announces and waits.  ``ok`` as in ``PeerWindow``."""

    def __init__(self, ctx, rank: int = 0, world: int = 1, group=None):
        import ctypes as C
        from . import _lib as L
        self.ctx, self.rank, self.world = ctx, rank, world
        self.window = PeerWindow(ctx, 1, L.DP_FLAG_WORDS, rank, world, group)
        self.window.mine.zero_()
        torch.cuda.synchronize(ctx.device)
        self.ok = self.window.ok
        if world > 1:
            dist.barrier(group=group)                    # every rank's words are zero before the first use
        self._arr = (C.c_void_p * world)(*[int(p) for p in self.window.pointers])
        self._fn = L.lib().sb200_peer_barrier
        self._L = L

    def __call__(self) -> None:
        self._L.check("sb200_peer_barrier",
                      self._fn(self.ctx.handle, self._arr, self.world, self.rank,
                               torch.cuda.current_stream(self.ctx.device).cuda_stream))

    def close(self, group=None) -> None:
        self.window.close(group)


class FusedWeightGradient:
    """dW = sum over ranks of x_r^T . dy_r for a Linear layer whose batch rows are
    split over the ranks, with the scatter half of the reduce-scatter inside the
    GEMM kernel.  Two routes:

    "add" (default)  the tiles are ADDED into the owning rank's window over NVLink
             (``sb200_gemm_reduce_scatter``, fp32 reductions at system scope); one
             barrier, then every rank pulls the owners' reduced blocks into
             ``dw_full`` with copy-engine transfers.  Windows are zeroed ahead of
             their use.  Arrival-order sums.
    "store"  every rank's tiles are STORED from the epilogue into its own slot of
             the owning rank's window (``sb200_gemm_scatter``, plain 16-byte stores);
             after a barrier every owner adds its ``world`` slots in slot order
             (``sb200_sum_blocks``: a fixed order, the sum is bit-reproducible), a
             second barrier, the same gather.  Measured about level with "add" on 2 and 4
             GPUs and slower on 8 (8192 x 4096 x 4096: 0.331 against 0.309 ms on 4,
             0.728 against 0.392 ms on 8).

    start()  runs the route up to the gather, which goes to one stream per owner (with
             the all-reduce of the bias gradient on this rank's own);
    wait()   makes the current stream wait for those streams.

    Work that needs no exchange (the dx GEMM) goes between the two calls.  Three
    windows rotate: a window is written again (or zeroed) only after every peer has
    finished copying it out (each rank passed a barrier after its copies).  ``ok``
    is False on every rank when any rank could not map a peer's window (callers
    fall back together)."""

    def __init__(self, ctx, n_in: int, n_out: int, rank: int = 0, world: int = 1, group=None,
                 route: str = "add"):
        if route not in ("store", "add"):
            raise ValueError("route is 'store' or 'add'")
        self.ctx, self.rank, self.world, self.group, self.route = ctx, rank, world, group, route
        self.n_in, self.n_out = n_in, n_out
        self.block_rows = n_in // world
        slots = world if route == "store" else 1
        self.windows = [PeerWindow(ctx, slots * self.block_rows, n_out, rank, world, group) for _ in range(3)]
        # the barrier between the GEMM that writes into the peers' windows and the reads
        self.barrier = PeerBarrier(ctx, rank, world, group) if world > 1 else None
        self.ok = all(w.ok for w in self.windows) and (self.barrier is None or self.barrier.ok)
        dev = torch.device("cuda", ctx.device)
        # one stream per owner: a peer copy costs ~60 us whatever its size, so the
        # world - 1 pulls of a step run side by side, not one after the other
        self.sides = [torch.cuda.Stream(dev) for _ in range(max(world, 1))]
        self.side = self.sides[rank if world > 1 else 0]
        self.pulled = [torch.cuda.Event() for _ in range(max(world, 1))]
        self.done = torch.cuda.Event()
        self.tick = torch.zeros(1, device=dev)
        self.turn = 0
        for w in self.windows:
            w.mine.zero_()
        self._barrier()

    def _barrier(self) -> None:
        if self.barrier is not None and self.ok:
            self.barrier()
        elif self.world > 1:
            dist.all_reduce(self.tick, group=self.group)

    def start(self, x: torch.Tensor, dy: torch.Tensor, dw_full: torch.Tensor, db: torch.Tensor,
              mode: int = 0, total_rows: int = 0) -> None:
        """``total_rows``: rows of the global batch when the ranks' shares differ
        (0: every rank holds ``x.shape[0]`` rows)."""
        from . import ops
        # the gather below must stay a copy-engine transfer: torch turns copy_ into
        # cudaMemcpyAsync only between dense tensors of one dtype, anything else would
        # become an elementwise kernel reading a peer mapping
        if (dw_full.dtype != torch.float32 or not dw_full.is_contiguous()
                or tuple(dw_full.shape) != (self.n_in, self.n_out)):
            raise ValueError("dw_full must be a contiguous fp32 [n_in, n_out] tensor")
        cur, nxt = self.windows[self.turn % 3], self.windows[(self.turn + 1) % 3]
        self.turn += 1
        dev = torch.device("cuda", self.ctx.device)
        main = torch.cuda.current_stream(dev)
        rows = self.block_rows
        store = self.route == "store"
        # dB: 1 / (global batch), so that the SUM over ranks below is the mean over the batch
        scale = 1.0 / (total_rows or x.shape[0] * self.world)
        if store:
            # this rank's slot in every owner's window
            slot = self.rank * rows * self.n_out * 4
            ops.gemm_reduce_scatter(self.ctx, x, dy, [p + slot for p in cur.pointers], self.n_out,
                                    trans_a=True, mode=mode, colsum_out=db, colsum_scale=scale, store=True)
            self._barrier()                              # every rank's stores have landed
            blocks = cur.mine.view(self.world, rows, self.n_out)
            ops.sum_blocks(self.ctx, blocks[0], blocks)  # the reduced block, in slot 0
            self._barrier()                              # every owner's block is reduced
        else:
            nxt.mine.zero_()
            ops.gemm_reduce_scatter(self.ctx, x, dy, cur.pointers, self.n_out, trans_a=True, mode=mode,
                                    colsum_out=db, colsum_scale=scale)
            self._barrier()                              # all adds have landed
        self.done.record(main)
        for o in range(self.world):
            with torch.cuda.stream(self.sides[o]):
                self.sides[o].wait_event(self.done)
                dw_full[o * rows:(o + 1) * rows].copy_(cur.views[o][:rows], non_blocking=True)
                if o == self.rank and self.world > 1:       # the local copy is short: this stream
                    dist.all_reduce(db, group=self.group)   # also carries the bias gradient
                self.pulled[o].record(self.sides[o])

    def wait(self) -> None:
        main = torch.cuda.current_stream(torch.device("cuda", self.ctx.device))
        for o in range(self.world):
            main.wait_event(self.pulled[o])

    def close(self) -> None:
        for w in self.windows:
            w.close(self.group)
        if self.barrier is not None:
            self.barrier.close(self.group)
