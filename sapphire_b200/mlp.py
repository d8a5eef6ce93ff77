"""A Linear -> ReLU -> ... -> Linear -> SoftMax -> CrossEntropy training step on
the B200 kernels, with the semantics of Sapphire's units:

forward   y = bias + x.W, W stored [in, out]: one GEMM with the bias in its
          epilogue (the reference runs a rank-1 Gemm for the bias first,
          Sources/Sapphire/operations/Forward/Linear.cpp:134-136)
backward  dx = dy.W^T and dW = x^T.dy through descriptor transposes, dB as the
          fused column sum scaled by 1 / batch
          (Sources/Sapphire/operations/Backward/LinearBackward.cpp:27-99 materialises both
          transposes and runs a ones-Gemm for dB)
update    SGD z <- z - lr * dz (Sources/Sapphire/operations/optimizers/SGD.cpp:22-28), applied
          after the backward pass (and after the gradient allreduce when the batch
          is split over ranks); the reference updates inside backward, after dx
          of the same layer was formed with the old weight, which is the same
          arithmetic.

With ``fused=True`` (the default) the elementwise steps ride in the GEMM
epilogues: the forward ReLU (Sources/Sapphire/compute/dense/cuda/kernels/ActivationKernel.cu:11-22)
in the forward GEMM, the ReLU backward gate (ActivationBackwardKernel.cu:11-24)
in the dx GEMM, and SoftMax + CrossEntropy + their backward passes run as one
kernel: seven kernels fewer per step and no zero-filled temporaries, with
bit-identical results.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from . import _lib as L
from . import ops
from .runner import GradBucket, PeerGradExchange


class MlpTrainer:
    def __init__(self, ctx: ops.Context, weights: Sequence[np.ndarray], biases: Sequence[np.ndarray],
                 lr: float, mode: int = L.MODE_TF32, world: int = 1, fused: bool = True,
                 row_pad: int = 4, comm: str = "nccl", rank: int = 0):
        """``row_pad``: rows of the parameter / gradient buffers are padded to this
        many floats.  4 (16 bytes) puts the 10-column output layer on the
        tensor-core kernel; 1 keeps its rows dense, which sends that layer to the
        CUDA-core kernel (sequential fp32 sums, bit-identical to the reference).
        ``comm``: how the gradients are summed over ``world`` ranks: "nccl" (one
        all-reduce of the flat bucket, then the SGD kernel) or "peer" (the two
        kernels of ``PeerGradExchange``: sum over peer memory fused with the update;
        needs ``rank``)."""
        self.ctx, self.lr, self.mode, self.world = ctx, float(lr), mode, world
        self.fused, self.row_pad = fused, row_pad
        self._plan = None                      # prepared calls of the fused step, per batch size
        dev = torch.device("cuda", ctx.device)
        shapes = [w.shape for w in weights]
        # parameters share the gradient bucket's layout: one SGD kernel updates them all
        self.params = GradBucket.create(shapes, dev, row_pad)
        for dst, w in zip(self.params.dW, weights):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(w)))
        for dst, b in zip(self.params.dB, biases):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(b)))
        self.exchange = None
        if comm == "peer" and world > 1:
            self.exchange = PeerGradExchange(ctx, GradBucket.size(shapes, row_pad), 0, rank, world)
            if not self.exchange.ok:                       # agreed across ranks: all fall back together
                self.exchange.close()
                self.exchange = None
        if self.exchange is not None:
            self.grads = GradBucket.create(shapes, dev, row_pad, flat=self.exchange.grads)
            self.exchange.n_sum = self.grads.n_weight
        else:
            self.grads = GradBucket.create(shapes, dev, row_pad)
        self.W, self.b = self.params.dW, self.params.dB

    def forward_backward(self, x: torch.Tensor, onehot: torch.Tensor) -> torch.Tensor:
        """Fills the gradient bucket with this rank's gradients; returns the
        per-sample loss."""
        if self.fused:
            return self._forward_backward_fused(x, onehot)
        ctx, mode = self.ctx, self.mode
        nl = len(self.W)
        B = x.shape[0]
        acts: List[torch.Tensor] = [x]
        pre: List[torch.Tensor] = []
        for l in range(nl):
            y = ops.gemm(ctx, acts[-1], self.W[l], bias=self.b[l], mode=mode)
            pre.append(y)
            if l < nl - 1:
                acts.append(ops.relu(ctx, y))
        prob = ops.softmax(ctx, pre[-1])
        loss = ops.cross_entropy(ctx, prob, onehot)
        dprob = torch.zeros_like(prob)
        ops.cross_entropy_backward(ctx, dprob, prob, onehot)
        dy = torch.zeros_like(prob)
        ops.softmax_backward(ctx, dy, dprob, prob)
        if self.row_pad > 1 and dy.shape[1] % self.row_pad:
            # same row pitch as the fused path, so that both run the same GEMM kernels
            ld = (dy.shape[1] + self.row_pad - 1) // self.row_pad * self.row_pad
            padded = torch.empty((B, ld), dtype=torch.float32, device=dy.device)[:, :dy.shape[1]]
            padded.copy_(dy)
            dy = padded
        for l in reversed(range(nl)):
            dx = ops.gemm(ctx, dy, self.W[l], trans_b=True, mode=mode)
            ops.gemm(ctx, acts[l], dy, out=self.grads.dW[l], trans_a=True, mode=mode,
                     colsum_out=self.grads.dB[l], colsum_scale=1.0 / B)
            if l > 0:
                dpre = torch.zeros_like(pre[l - 1])
                ops.relu_backward(ctx, dpre, dx, pre[l - 1])
                dy = dpre
        return loss

    def _forward_backward_fused(self, x: torch.Tensor, onehot: torch.Tensor) -> torch.Tensor:
        ctx, mode = self.ctx, self.mode
        nl = len(self.W)
        B = x.shape[0]
        acts: List[torch.Tensor] = [x]              # acts[l] = input of layer l (ReLU output of l-1)
        for l in range(nl):
            acts.append(ops.gemm(ctx, acts[-1], self.W[l], bias=self.b[l], mode=mode, relu=l < nl - 1))
        _, loss, dy = ops.softmax_cross_entropy(ctx, acts[-1], onehot, row_pad=self.row_pad)
        for l in reversed(range(nl)):
            # dx first, like the reference; the first layer's dx is computed and dropped as there
            dx = ops.gemm(ctx, dy, self.W[l], trans_b=True, mode=mode,
                          relu_gate=acts[l] if l > 0 else None)
            ops.gemm(ctx, acts[l], dy, out=self.grads.dW[l], trans_a=True, mode=mode,
                     colsum_out=self.grads.dB[l], colsum_scale=1.0 / B)
            dy = dx
        return loss

    # ------------------------------------------------------- prepared step
    def _build_plan(self, x: torch.Tensor, onehot: torch.Tensor):
        """The fused step as a list of calls whose arguments are marshalled once:
        every buffer of the step is allocated here and reused, only the addresses
        of the step's input and label change from call to call.  A step launched
        eagerly then costs a dozen ctypes calls instead of a dozen trips through
        the shape-checking front end (which took 2-3 times the GPU time of the
        step); the kernels, their arguments and therefore the results are those
        of `_forward_backward_fused`."""
        import ctypes as C
        ctx, mode = self.ctx, self.mode
        nl = len(self.W)
        B = x.shape[0]
        dev = x.device
        calls, patch_x, acts = [], [], [x]
        for l in range(nl):
            out = torch.empty(B, self.W[l].shape[1], dtype=torch.float32, device=dev)
            calls.append(ops.prepare_gemm(ctx, acts[-1], self.W[l], out=out, bias=self.b[l], mode=mode,
                                          relu=l < nl - 1))
            if l == 0:
                patch_x.append(calls[-1])
            acts.append(out)
        unit = acts[-1].shape[1]
        ld = (unit + self.row_pad - 1) // self.row_pad * self.row_pad
        prob = torch.empty(B, unit, dtype=torch.float32, device=dev)
        loss = torch.empty(B, dtype=torch.float32, device=dev)
        dlogits = torch.empty((B, ld), dtype=torch.float32, device=dev)[:, :unit]
        ce = ops.PreparedCall("sb200_softmax_cross_entropy", L.lib().sb200_softmax_cross_entropy,
                              [ctx.handle, prob.data_ptr(), loss.data_ptr(), dlogits.data_ptr(),
                               dlogits.stride(0) if B > 1 else max(unit, dlogits.stride(0)),
                               acts[-1].data_ptr(), onehot.data_ptr(), B, unit],
                              ctx.device, [prob, loss, dlogits, acts[-1]], loss)
        calls.append(ce)
        dy = dlogits
        side = set()                                     # the weight-gradient GEMMs
        for l in reversed(range(nl)):
            dx = torch.empty(B, self.W[l].shape[0], dtype=torch.float32, device=dev)
            # dW_l needs only dy_l and the layer's input: nothing of the backward chain
            # waits for it, so it is listed before dx_l and may run beside it
            calls.append(ops.prepare_gemm(ctx, acts[l], dy, out=self.grads.dW[l], trans_a=True, mode=mode,
                                          colsum_out=self.grads.dB[l], colsum_scale=1.0 / B))
            side.add(len(calls) - 1)
            if l == 0:
                patch_x.append(calls[-1])
            calls.append(ops.prepare_gemm(ctx, dy, self.W[l], out=dx, trans_b=True, mode=mode,
                                          relu_gate=acts[l] if l > 0 else None))
            if l == 0:
                late = len(calls) - 1                    # the input's gradient: nobody reads it
            dy = dx
        for c in calls:
            c.args = list(c.args)
        return {"batch": B, "calls": calls, "side": side, "late": late, "patch_x": patch_x, "ce": ce, "loss": loss,
                "x_shape": tuple(x.shape), "y_shape": tuple(onehot.shape),
                "fork": [torch.cuda.Event() for _ in range(nl + 1)], "join": torch.cuda.Event(),
                "side_stream": torch.cuda.Stream(dev), "late_stream": torch.cuda.Stream(dev),
                "late_join": torch.cuda.Event(), "late_pending": False}

    def _run_plan(self, x: torch.Tensor, onehot: torch.Tensor) -> torch.Tensor:
        plan = self._plan
        if (plan is None or plan["x_shape"] != tuple(x.shape) or plan["y_shape"] != tuple(onehot.shape)):
            plan = self._plan = self._build_plan(x, onehot)
        if not (x.is_contiguous() and onehot.is_contiguous() and x.dtype == torch.float32
                and onehot.dtype == torch.float32):
            raise ValueError("the prepared step takes contiguous fp32 inputs")
        for c in plan["patch_x"]:
            c.args[8] = x.data_ptr()                       # operand A of the first layer's two GEMMs
        plan["ce"].args[6] = onehot.data_ptr()
        if not torch.cuda.is_current_stream_capturing():
            for c in plan["calls"]:
                c()
            return plan["loss"]
        # Under capture the three weight-gradient GEMMs go to a second stream: the
        # graph then has them beside the dx chain instead of inside it (8 kernels on
        # the critical path instead of 11).  The gradient of the network's input, which
        # nobody reads, goes to a third and is joined only at the end of the step, so
        # the gradient exchange / SGD does not wait for it.  Launched eagerly the step
        # is bound by the host, where the event calls would cost more than the overlap
        # gives.
        # (One context on three streams: allowed here because no two of these calls touch
        # the context's workspace at once -- in TF32 mode the dW GEMMs carry their column
        # sums inside the kernel, and the GEMMs that may be k-sliced (forward, dx) form one
        # chain, the input's gradient being its last link; in 3xTF32 mode only the column
        # sums of the dW calls use it, all on the one side stream, and nothing is k-sliced.)
        main = torch.cuda.current_stream(x.device)
        side, late, forks, k = plan["side_stream"], plan["late_stream"], plan["fork"], 0
        for i, c in enumerate(plan["calls"]):
            if i in plan["side"] or i == plan["late"]:
                branch = late if i == plan["late"] else side
                forks[k].record(main)                      # what the call reads is complete in stream order
                branch.wait_event(forks[k])
                k += 1
                with torch.cuda.stream(branch):
                    c()
            else:
                c()
        plan["join"].record(side)
        main.wait_event(plan["join"])                      # gradients complete before the exchange / SGD
        plan["late_join"].record(late)
        plan["late_pending"] = True                        # `step` joins it after the update
        return plan["loss"]

    def step(self, x: torch.Tensor, onehot: torch.Tensor) -> torch.Tensor:
        """One training step; returns the per-sample loss (with the fused path a
        buffer that the next step overwrites)."""
        loss = self._run_plan(x, onehot) if self.fused else self.forward_backward(x, onehot)
        if self.exchange is not None:
            self.exchange.step(self.params.flat, self.lr)
        else:
            self.grads.allreduce(self.world, lambda t, f: ops.scale(self.ctx, t, f))
            ops.sgd_update(self.ctx, self.params.flat, self.grads.flat, self.lr)
        plan = self._plan
        if self.fused and plan is not None and plan["late_pending"]:
            # the branch of the input's gradient rejoins: the step (a captured graph) ends
            # when it has, and the next step may overwrite what it read
            torch.cuda.current_stream(x.device).wait_event(plan["late_join"])
            plan["late_pending"] = False
        return loss

    def close(self) -> None:
        """Collective when the trainer exchanges gradients over peer memory."""
        if self.exchange is not None:
            self.exchange.close()
            self.exchange = None

    # ------------------------------------------------------------ CUDA graph
    def capture(self, batch: int) -> None:
        """Records one whole step (forward, backward, gradient allreduce, SGD) into
        a CUDA graph over static input buffers: the step is ~25 small kernels and
        launch-bound, a graph replays them with one launch.  Two eager steps run
        first so that every lazily created resource (kernel attributes, the
        column-sum scratch) exists before capture begins; the parameters are
        restored afterwards."""
        dev = self.params.flat.device
        n_in, n_out = self.W[0].shape[0], self.W[-1].shape[1]
        self._gx = torch.zeros(batch, n_in, device=dev)
        self._gy = torch.zeros(batch, n_out, device=dev)
        self._gy[:, 0] = 1.0
        saved = self.params.flat.clone()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.step(self._gx, self._gy)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.params.flat.copy_(saved)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._gloss = self.step(self._gx, self._gy)
        self.params.flat.copy_(saved)

    def step_graph(self, x: torch.Tensor, onehot: torch.Tensor) -> torch.Tensor:
        """One step through the captured graph; returns the per-sample loss buffer
        (overwritten by the next replay)."""
        self._gx.copy_(x, non_blocking=True)
        self._gy.copy_(onehot, non_blocking=True)
        self._graph.replay()
        return self._gloss
