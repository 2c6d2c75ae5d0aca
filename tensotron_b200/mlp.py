"""Data-parallel MLP training step on the GEMM engine.

The step is the reference's `Sequential(Linear, ReLU, ..., Linear)` + `CrossEntropy` +
`Adam` loop (examples/Tensotron.Examples/BenchExample.cs:630-699 shape of the loop;
src/Tensotron/Module.cs:82-112, src/Tensotron/TensorOps.Losses.cs:97-108,
src/Tensotron/Optimizers.cs:144-193), with every product going through the C-ABI library:

  forward   one fused launch per layer (GEMM + bias + ReLU)             tt_linear_fwd
  loss      softmax cross-entropy forward+backward, device labels       tt_softmax_cross_entropy
  backward  per layer: activation backward + fixed-order bias gradient,
            dX (NN GEMM), dW (TN GEMM)                                  tt_linear_bwd
  exchange  "nccl": one NCCL all-reduce (sum) per layer's gradient slice, issued as soon as
            the slice is final so it overlaps the rest of the backward pass, then
  update    one fused Adam over the flat parameter buffer                tt_adam_step
  exchange  "peer": the weight-gradient GEMM stores every finished tile into the memory of the
            rank that owns those rows (NVLink stores from the epilogue); the owner sums the
            ranks' copies in rank order, runs Adam on its rows and stores the new rows into
            every rank's parameters (peer.py)               tt_peer_linear_bwd / _push / _adam_step

Parameters, gradients and Adam moments live in flat buffers laid out layer by layer
(W_i then b_i), so a layer's gradients are one contiguous slice and Adam is one launch.
Data parallelism: each rank holds `global_batch / world` rows; the loss and its gradient are
scaled by 1/global_batch, so the summed gradients equal the single-GPU gradients up to
summation order.  torch.distributed is plumbing (process group, NCCL stream handling).
"""
import math

import torch

from .runtime import ACT, LOSS, TT_LOSS_CE, TT_MATH_FP32, TensorRuntime, TensotronGemmError


def shard_rows(total, world, rank):
    """Contiguous row block [start, end) of `total` rows owned by `rank` (same split as the
    reference's ParallelRows: ceil-sized blocks, src/Tensotron/CpuKernels.cs:461-472)."""
    from .runtime import shard_range
    start, count = shard_range(total, world, rank)     # the split lives behind the C ABI (tt_shard_range)
    return start, start + count


def layer_layout(dims):
    """Offsets (in floats) of W_i and b_i inside the flat buffers; W_i is (out, in)."""
    offs, cur = [], 0
    for i in range(len(dims) - 1):
        w = cur
        cur += dims[i + 1] * dims[i]
        b = cur
        cur += dims[i + 1]
        cur = (cur + 3) & ~3  # keep every layer 16-byte aligned for TMA / 128-bit accesses
        offs.append((w, b))
    return offs, cur


class MlpTrainer:
    """act: activation between the layers ("relu" as in benchmark config 4, "tanh" as in the
    reference's control / PPO networks); loss: "ce" (cross-entropy on int32 labels) or "mse"
    (mean squared error against a float target, examples/Tensotron.Examples/BenchExample.cs:171);
    max_grad_norm > 0 adds ClipGradNorm before the optimizer step (:174).  fused: True runs the
    whole step as one launch (tt_mlp_train_step, single GPU, small networks), "auto" does so when
    the network and the batch fit and otherwise runs it layer by layer, False never does."""

    def __init__(self, dims, rt=None, device=0, lr=1e-3, seed=2, process_group=None, math_mode=TT_MATH_FP32,
                 exchange="nccl", peer_group=None, act="relu", loss="ce", max_grad_norm=0.0, clip_eps=1e-6,
                 fused=False):
        self.dims = list(dims)
        self.act = ACT[act]
        self.loss_kind = LOSS[loss]
        self.max_grad_norm = float(max_grad_norm)
        self.clip_eps = float(clip_eps)
        self.fused = fused
        self.last_step_fused = False
        self.L = len(dims) - 1
        self.device = device
        self.rt = rt or TensorRuntime(device)
        self.lr = lr
        self.pg = process_group
        self.math_mode = math_mode
        self.offs, total = layer_layout(self.dims)
        dev = torch.device("cuda", device)
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.exchange = exchange
        self.peer = None
        if exchange == "peer" and self.max_grad_norm > 0:
            raise ValueError("gradient clipping needs the whole gradient on one rank: use exchange='nccl'")
        if exchange == "peer":
            from .peer import CHANNELS, PeerGroup, exchange_plan, merge_segments
            self.peer = peer_group or PeerGroup(self.rt, total, process_group)
            self.own_rows, owned, replicated = exchange_plan(self.dims, self.peer.world, self.offs)
            # One exchange channel per layer, so a layer's optimizer step and the transfer of its
            # updated rows overlap the backward pass of the layers below; networks with more
            # layers than channels exchange everything in one piece after the backward pass.
            self.pipelined = self.L <= CHANNELS
            if self.pipelined:
                self.owned, self.replicated = owned[self.peer.rank], replicated
            else:
                self.owned = [merge_segments([s for lay in owned[self.peer.rank] for s in lay])]
                self.replicated = [merge_segments([s for lay in replicated for s in lay])]
            self.params, self.grads = self.peer.params, self.peer.grads
            self.fused = [False] * self.L     # which layers' scatter ran in the GEMM epilogue (last step)
        else:
            self.params = torch.zeros(total, device=dev)
            self.grads = torch.zeros(total, device=dev)
        self.m = torch.zeros(total, device=dev)
        self.v = torch.zeros(total, device=dev)
        self.adv = torch.zeros(3, device=dev)
        self.loss = torch.zeros(1, device=dev)
        self.n_params = total
        gen = torch.Generator().manual_seed(seed)   # same weights on every rank
        for i, (wo, bo) in enumerate(self.offs):
            fan_in, fan_out = self.dims[i], self.dims[i + 1]
            bound = 1.0 / math.sqrt(fan_in)           # Kaiming-uniform a=sqrt(5) (src/Tensotron/Init.cs:54-58)
            w = (torch.rand(fan_out * fan_in, generator=gen) * 2 - 1) * bound
            b = (torch.rand(fan_out, generator=gen) * 2 - 1) * bound
            self.params[wo:wo + fan_out * fan_in].copy_(w)
            self.params[bo:bo + fan_out].copy_(b)
        self._acts = None
        self._batch = 0

    # ---- views ----
    def weight(self, i, buf=None):
        buf = self.params if buf is None else buf
        wo, _ = self.offs[i]
        return buf[wo:wo + self.dims[i + 1] * self.dims[i]].view(self.dims[i + 1], self.dims[i])

    def bias(self, i, buf=None):
        buf = self.params if buf is None else buf
        _, bo = self.offs[i]
        return buf[bo:bo + self.dims[i + 1]]

    def layer_slice(self, i, buf):
        wo, bo = self.offs[i]
        return buf[wo:bo + self.dims[i + 1]]

    def _ensure_buffers(self, batch):
        if self._batch == batch:
            return
        dev = self.params.device
        self._acts = [torch.empty((batch, d), device=dev) for d in self.dims[1:]]
        self._dacts = [torch.empty((batch, d), device=dev) for d in self.dims[1:]]
        self._batch = batch

    def forward(self, x, labels, global_batch=None):
        """Forward pass + softmax cross-entropy (loss and its gradient w.r.t. the logits)."""
        rt = self.rt
        rt.SetCuBlasMathMode(self.math_mode)
        rows = x.shape[0]
        gb = global_batch or rows
        self._ensure_buffers(rows)
        L = self.L
        inp = x
        for i in range(L):
            act = self.act if i < L - 1 else 0
            rt.LaunchLinearForward(inp, self.weight(i), self.bias(i), self._acts[i], rows,
                                   self.dims[i + 1], self.dims[i], act)
            inp = self._acts[i]
        if self.loss_kind == TT_LOSS_CE:
            rt.LaunchSoftmaxCrossEntropy(self._acts[L - 1], labels, self._dacts[L - 1], self.loss, rows,
                                         self.dims[L], 1.0 / gb)
        else:
            if gb != rows:
                raise ValueError("the MSE loss is single-GPU only (its mean runs over this rank's rows)")
            rt.LaunchMseLoss(self._acts[L - 1], labels, self._dacts[L - 1], self.loss, rows * self.dims[L])

    # ---- one training step ----
    def step(self, x, labels, global_batch=None, apply_update=True):
        """x: (rows, dims[0]) float32 CUDA, labels: (rows,) int32 CUDA.  Returns the device
        scalar holding this rank's share of the mean loss (sum over ranks = global mean)."""
        rt, L, rows = self.rt, self.L, x.shape[0]
        self.last_step_fused = False
        if self.fused and self.peer is None and self.pg is None and apply_update and (global_batch or rows) == rows:
            try:
                rt.SetCuBlasMathMode(self.math_mode)
                rt.LaunchMlpTrainStep(self.dims, self.act, self.loss_kind, self.params, self.m, self.v, self.adv,
                                      self.grads, x, labels, self.loss, rows, lr=self.lr,
                                      max_grad_norm=self.max_grad_norm, clip_eps=self.clip_eps)
                self.last_step_fused = True
                return self.loss
            except TensotronGemmError as e:
                if e.status != 3 or self.fused is True:
                    raise
        self.forward(x, labels, global_batch)
        if self.peer is not None:
            if not apply_update:
                raise ValueError("the peer exchange reduces inside the optimizer step: apply_update must be True")
            if self.pipelined:
                for i in reversed(range(L)):
                    self.peer_backward_layer(x, i)
                    self.peer_push(i)
                    if i + 1 < L:
                        self.peer_update(i + 1)      # one layer late: the other ranks have had time to finish it
                self.peer_update(0)
            else:
                for i in reversed(range(L)):
                    self.peer_backward_layer(x, i)
                self.peer_push(0)
                self.peer_update(0)
            self.peer_sync()
            return self.loss
        handles = []
        for i in reversed(range(L)):
            act = self.act if i < L - 1 else 0
            layer_in = x if i == 0 else self._acts[i - 1]
            dx = self._dacts[i - 1] if i > 0 else None
            rt.LaunchLinearBackward(layer_in, self.weight(i), self._acts[i], self._dacts[i], dx,
                                    self.weight(i, self.grads), self.bias(i, self.grads), rows,
                                    self.dims[i + 1], self.dims[i], act)
            if self.pg is not None:
                import torch.distributed as dist
                handles.append(dist.all_reduce(self.layer_slice(i, self.grads), group=self.pg, async_op=True))
        for h in handles:
            h.wait()
        if self.max_grad_norm > 0:
            rt.LaunchClipGradNorm(self.grads, self.n_params, self.max_grad_norm, self.clip_eps)
        if apply_update:
            rt.LaunchAdam(self.params, self.grads, self.m, self.v, self.adv, self.n_params, lr=self.lr)
        return self.loss

    # The peer exchange in its phases (step() issues them in the order above; a test that
    # emulates several ranks on one GPU issues each phase for all ranks before the next one, so
    # that every flag is set before the kernel that waits for it runs).  `ch` is the exchange
    # channel = the layer (0 when the exchange is not pipelined).
    def peer_backward_layer(self, x, i):
        L, pr, rows = self.L, self.peer, x.shape[0]
        act = self.act if i < L - 1 else 0
        layer_in = x if i == 0 else self._acts[i - 1]
        dx = self._dacts[i - 1] if i > 0 else None
        w_off, b_off = self.offs[i]
        self.fused[i] = pr.linear_bwd(layer_in, self.weight(i), self._acts[i], self._dacts[i], dx, w_off, b_off,
                                      rows, self.dims[i + 1], self.dims[i], act, self.own_rows[i])

    def _first_channel(self):
        return self.L - 1 if self.pipelined else 0     # the channel whose calls come first in a step

    def peer_push(self, ch):
        self.peer.push(self.replicated[ch], channel=ch, new_step=(ch == self._first_channel()))

    def peer_update(self, ch):
        self.peer.adam_step(self.owned[ch], self.replicated[ch], self.m, self.v, self.adv, channel=ch, lr=self.lr,
                            advance=(ch == self._first_channel()))

    def peer_sync(self):
        self.peer.sync(self.L if self.pipelined else 1)

    def close(self):
        if self.peer is not None:
            self.peer.close()
            self.peer = None
