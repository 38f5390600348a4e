"""Inter-layer (pipeline) parallel engine: message-driven microbatch scheduling.

Same algorithm and user contract as the reference's
``axonn/inter_layer.py:40-460`` (``AxoNN_Inter_Layer_Engine``): each stage
reacts to whichever message arrives — an activation from the previous stage
triggers a forward pass, an activation gradient from the next stage triggers a
backward pass — the first stage keeps at most ``G_inter`` microbatches in
flight, the last stage computes the loss and immediately runs backward.  The
stage module must provide ``get_input_shape()`` / ``get_output_shape()`` with
``-1`` for the microbatch dimension.

What is different:

* transport is ``torch.distributed`` ``isend/irecv`` (NCCL over NVLink on
  GPUs, gloo on CPU) on one communicator per neighbour and direction instead of
  CUDA-aware MPI.  Each direction is FIFO and every stage handles forward and
  backward messages in arrival order, so the k-th message of a direction always
  carries microbatch k: sequence counters replace MPI tags;
* ``MPI.Request.Waitany`` becomes a poll over the two outstanding receives with
  a deadline (a silent peer raises ``PipelineTimeout`` instead of hanging);
* a send only orders itself after the producing kernels on the stream; there is
  no device-wide synchronize per message (reference ``:115``);
* the loss is accumulated on the device and read back once per batch.
"""

import threading
import os
import time
from dataclasses import dataclass
from enum import Enum

import torch
import torch.distributed as dist

from . import axonn as ax
from .intra_layer import sync_gradients


class PipelineTimeout(RuntimeError):
    """A neighbouring pipeline stage did not deliver a message in time."""


@dataclass
class LossScaler:
    """Dynamic loss scale for fp16 training (same constants as the reference)."""

    loss_scale: float = 2.0 ** 16
    max_scale: float = 2.0 ** 24
    min_scale: float = 2.0 ** 10
    scaling_window: float = 200
    no_overflow_iters: float = 0


class Operation(Enum):
    FW = 0
    BW = 1


class _Request:
    """Completion test for a p2p ``Work`` that behaves the same on NCCL and gloo.

    NCCL work objects report completion through ``is_completed()`` (a CUDA event
    query).  Gloo's only make progress visible inside ``wait()``, so for CPU
    tensors a helper thread waits and raises a flag."""

    def __init__(self, work, on_gpu):
        self.work, self.on_gpu = work, on_gpu
        self.error = None
        if not on_gpu:
            self._flag = threading.Event()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def _run(self):
        try:
            self.work.wait()
        except Exception as e:  # surfaced by done()/wait()
            self.error = e
        self._flag.set()

    def done(self):
        if self.on_gpu:
            return self.work.is_completed()
        if self.error is not None:
            raise self.error
        return self._flag.is_set()

    def wait(self, timeout=None):
        if self.on_gpu:
            self.work.wait()
            return
        if not self._flag.wait(timeout):
            raise PipelineTimeout("p2p operation did not complete in time")
        if self.error is not None:
            raise self.error


class AxoNN_Inter_Layer_Engine:
    """Pipeline training step over ``G_inter`` stages (reference ``axonn/inter_layer.py:40-460``).

    ``model`` is this stage's part of the network with ``get_input_shape()`` / ``get_output_shape()`` (``-1`` for
    the microbatch dimension); ``forward_backward_optimizer(batch, labels, optimizer)`` splits the batch into
    microbatches of ``config.micro_batch_size``, runs them through the stages with activations and gradients
    travelling over point-to-point messages, reduces gradients over the data-parallel group, handles fp16 loss
    scaling and steps the optimizer.  A stage that hears nothing from a neighbour for ``timeout_s`` raises
    ``PipelineTimeout``."""

    def __init__(self, model, loss_fn, computation_dtype=torch.bfloat16, timeout_s: float = 600.0):
        assert ax.is_initialized, "call axonn_b200.axonn.init(...) before creating the engine"
        self.model, self.criterion = model, loss_fn
        self.computation_dtype = computation_dtype
        self.scaler = LossScaler()
        # AXONN_PIPELINE_TIMEOUT_S overrides the deadline after which a stage that hears nothing from its
        # neighbours raises PipelineTimeout (with the direction it was waiting for)
        self.timeout_s = float(os.environ.get("AXONN_PIPELINE_TIMEOUT_S", timeout_s))
        self.device = ax.comm_handle.device
        self.input_tensors_cache, self.output_tensors_cache = {}, {}
        self.transit_tensors = []          # (work, tensor) of sends not yet complete
        self.requests = {"fw": None, "bw": None}
        self._seq = {"fw": 0, "bw": 0}
        self._connect_neighbours()

    def _connect_neighbours(self):
        """Exchange one element with each neighbouring stage in both directions, pair by pair in stage order.

        NCCL sets up the connection of a point-to-point communicator inside the first send / receive call on it,
        and that call does not return before the peer has made the matching call.  The engine posts its receives
        for forward and backward messages before it has anything to send, so with more than two stages a middle
        stage would sit in its first backward receive - whose sender can only answer after getting forward data
        through this very stage.  Connecting every pair up front, in an order without cycles, removes that wait
        from the schedule."""
        G, rank = ax.config.G_inter, self._rank
        if G <= 1:
            return
        token = torch.zeros(1, device=self.device, dtype=torch.float32)
        for s in range(G - 1):
            if rank == s:
                ax.comm_handle.send(token, s + 1, async_op=False)
                ax.comm_handle.recv(token, s + 1, async_op=False)
            elif rank == s + 1:
                ax.comm_handle.recv(token, s, async_op=False)
                ax.comm_handle.send(token, s, async_op=False)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ helpers
    @property
    def _rank(self):
        return ax.config.inter_layer_parallel_rank

    def _get_subtensor(self, tensor, microbatch_no):
        m = ax.config.micro_batch_size
        return tensor[microbatch_no * m:(microbatch_no + 1) * m]

    def _fill_shape(self, shape):
        return [ax.config.micro_batch_size if x == -1 else x for x in shape]

    def _autocast(self):
        enabled = self.computation_dtype in (torch.float16, torch.bfloat16)
        return torch.autocast(device_type=self.device.type, dtype=self.computation_dtype, enabled=enabled)

    # ------------------------------------------------------------------ p2p
    def _send(self, tensor, destination, microbatch_no):
        if destination < 0 or destination >= ax.config.G_inter:
            return
        self._clear_transit_tensors()
        tensor = tensor.detach().contiguous().to(self.computation_dtype)
        work = _Request(ax.comm_handle.send(tensor, destination, microbatch_no), tensor.is_cuda)
        self.transit_tensors.append((work, tensor))

    def _clear_transit_tensors(self, clear_all=False):
        keep = []
        for work, tensor in self.transit_tensors:
            if clear_all:
                work.wait(self.timeout_s)
            elif not work.done():
                keep.append((work, tensor))
        self.transit_tensors = keep

    def _post_recv(self, kind):
        if self.requests[kind] is not None:
            return
        if kind == "fw":
            shape, src = self.model.get_input_shape(), self._rank - 1
        else:
            shape, src = self.model.get_output_shape(), self._rank + 1
        buf = torch.empty(self._fill_shape(shape), device=self.device, dtype=self.computation_dtype)
        if kind == "fw":
            buf.requires_grad = True
        self.requests[kind] = (buf, _Request(ax.comm_handle.recv(buf, src), buf.is_cuda), self._seq[kind])
        self._seq[kind] += 1

    def _wait_any(self):
        """Block until one of the posted receives has completed; backward messages
        win ties (frees activation memory first).  Returns (kind, tensor, microbatch)."""
        deadline = time.monotonic() + self.timeout_s
        spins = 0
        while True:
            for kind in ("bw", "fw"):
                req = self.requests[kind]
                if req is not None and req[1].done():
                    req[1].wait()  # orders the current stream after the receive
                    self.requests[kind] = None
                    return kind, req[0], req[2]
            spins += 1
            if spins > 200:
                time.sleep(0.00005)
            if time.monotonic() > deadline:
                raise PipelineTimeout(
                    f"stage {self._rank}: no message from a neighbouring stage within {self.timeout_s}s "
                    f"(waiting for {[k for k, v in self.requests.items() if v is not None]})")

    # ------------------------------------------------------------------ compute
    def _forward_pass(self, input_activation, microbatch_no, eval_mode):
        last = self._rank == ax.config.G_inter - 1
        with self._autocast():
            if eval_mode:
                with torch.no_grad():
                    out = self.model(input_activation)
                if last:
                    self.output_tensors_cache[microbatch_no] = out
            else:
                out = self.model(input_activation)
                self.input_tensors_cache[microbatch_no] = input_activation
                self.output_tensors_cache[microbatch_no] = out
        if not last:
            self._send(out, self._rank + 1, microbatch_no)

    def _calc_loss(self, microbatch_no, labels, mul_factor=1.0, eval_mode=False):
        loss = self.criterion(self.output_tensors_cache[microbatch_no].float(), labels)
        scale = self.scaler.loss_scale if self.computation_dtype == torch.float16 else 1.0
        self.output_tensors_cache[microbatch_no] = mul_factor * loss * scale
        if eval_mode:
            del self.output_tensors_cache[microbatch_no]
        return loss.detach()

    def _backward_pass(self, output_gradients, microbatch_no):
        out = self.output_tensors_cache.pop(microbatch_no)
        inp = self.input_tensors_cache.pop(microbatch_no)
        out.backward(output_gradients)
        if self._rank > 0:
            self._send(inp.grad, self._rank - 1, microbatch_no)

    # ------------------------------------------------------------------ the step
    def forward_backward_optimizer(self, batch, labels, optimizer, eval_mode=False, post_bw_hook=None):
        """Forward, backward and optimizer step over one batch; returns the mean
        microbatch loss on the last stage and 0 elsewhere."""
        rank, G = self._rank, ax.config.G_inter
        mbs = ax.config.micro_batch_size
        assert mbs, "call axonn_b200.axonn.create_dataloader (or set config.micro_batch_size) first"
        n = batch.shape[0] // mbs
        self.model.eval() if eval_mode else self.model.train()
        loss_sum = torch.zeros((), device=self.device)
        if batch.device != self.device:
            batch = batch.to(self.device, non_blocking=True)
        if labels is not None and labels.device != self.device:
            labels = labels.to(self.device, non_blocking=True)

        if G == 1:
            for mb in range(n):
                self._forward_pass(self._get_subtensor(batch, mb), mb, eval_mode)
                loss_sum += self._calc_loss(mb, self._get_subtensor(labels, mb), 1.0 / n, eval_mode)
                if not eval_mode:
                    self._backward_pass(None, mb)
        elif self._schedule() == "1f1b":
            self._run_one_forward_one_backward(batch, labels, n, eval_mode, loss_sum)
        else:
            first, last = rank == 0, rank == G - 1
            fw_left = 0 if first else n
            bw_left = 0 if (last or eval_mode) else n
            self._seq = {"fw": 0, "bw": 0}
            injected = 0
            if first:
                for _ in range(min(G, n)):
                    self._forward_pass(self._get_subtensor(batch, injected), injected, eval_mode)
                    injected += 1
            if fw_left:
                self._post_recv("fw")
            if bw_left:
                self._post_recv("bw")
            while fw_left + bw_left:
                kind, tensor, mb = self._wait_any()
                if kind == "fw":
                    fw_left -= 1
                    if fw_left:
                        self._post_recv("fw")  # next transfer overlaps this forward
                    self._forward_pass(tensor, mb, eval_mode)
                    if last:
                        loss_sum += self._calc_loss(mb, self._get_subtensor(labels, mb), 1.0 / n, eval_mode)
                        if not eval_mode:
                            self._backward_pass(None, mb)
                else:
                    bw_left -= 1
                    if bw_left:
                        self._post_recv("bw")
                    self._backward_pass(tensor, mb)
                if first and injected < n:
                    self._forward_pass(self._get_subtensor(batch, injected), injected, eval_mode)
                    injected += 1
            if eval_mode and first:
                while injected < n:
                    while len(self.transit_tensors) >= G:
                        self._clear_transit_tensors()
                    self._forward_pass(self._get_subtensor(batch, injected), injected, eval_mode)
                    injected += 1
            self._clear_transit_tensors(clear_all=True)

        if eval_mode:
            value = float(loss_sum.item()) / n
            self._check_device_status()
            return value
        if post_bw_hook is not None:
            post_bw_hook(self.model)
        sync_gradients(self.model, mean=True, expert_mode=True)
        if self.computation_dtype == torch.float16:
            if not self._unscale_gradients():
                optimizer.step()
        else:
            optimizer.step()
        value = float(loss_sum.item()) / n   # host synchronisation: the step's kernels have finished
        self._check_device_status()
        return value

    def _schedule(self) -> str:
        """``message``: every stage keeps a receive posted in each direction and works on whatever arrives (the
        reference's schedule).  ``1f1b``: the fixed order that schedule settles into for equal-cost microbatches -
        stage s runs ``G_inter - s`` forwards, then alternates one backward and one forward - with every receive
        posted only at the moment its message is due, so no receive ever waits behind another one.
        ``AXONN_PIPELINE_SCHEDULE`` selects one; by default NCCL stages use the fixed order when there are more
        than two of them (a middle stage with two receives pending on NCCL communicators stopped making progress
        there; two stages and CPU ranks run the message-driven form)."""
        mode = os.environ.get("AXONN_PIPELINE_SCHEDULE", "auto")
        if mode in ("message", "1f1b"):
            return mode
        return "1f1b" if (self.device.type == "cuda" and ax.config.G_inter > 2) else "message"

    def _recv_now(self, kind):
        shape, src = ((self.model.get_input_shape(), self._rank - 1) if kind == "fw"
                      else (self.model.get_output_shape(), self._rank + 1))
        buf = torch.empty(self._fill_shape(shape), device=self.device, dtype=self.computation_dtype)
        ax.comm_handle.recv(buf, src, async_op=False)
        if kind == "fw":
            buf.requires_grad = True
        return buf

    def _run_one_forward_one_backward(self, batch, labels, n, eval_mode, loss_sum):
        rank, G = self._rank, ax.config.G_inter
        first, last = rank == 0, rank == G - 1

        def forward(mb):
            x = self._get_subtensor(batch, mb) if first else self._recv_now("fw")
            self._forward_pass(x, mb, eval_mode)
            if last:
                loss_sum.add_(self._calc_loss(mb, self._get_subtensor(labels, mb), 1.0 / n, eval_mode))

        def backward(mb):
            self._backward_pass(None if last else self._recv_now("bw"), mb)

        if eval_mode:
            for mb in range(n):
                forward(mb)
        else:
            warm = min(G - rank, n)
            for mb in range(warm):
                forward(mb)
            nf = warm
            for nb in range(n):
                backward(nb)
                if nf < n:
                    forward(nf)
                    nf += 1
        self._clear_transit_tensors(clear_all=True)

    def _check_device_status(self):
        """Raise if a kernel of this step reported an expired device-side wait (read after the loss readback,
        which already synchronised the host with the device)."""
        if self.device.type == "cuda":
            from .ops import _lib

            _lib.check_status(self.device.index)

    # ------------------------------------------------------------------ fp16 loss scaling
    def _sync_scale(self, local_overflow: torch.Tensor) -> bool:
        flag = local_overflow.to(device=self.device, dtype=torch.float32).reshape(1).clone()
        dist.all_reduce(flag)
        s = self.scaler
        if flag.item() > 0:
            s.loss_scale = max(s.loss_scale / 2.0, s.min_scale)
            s.no_overflow_iters = 0
            if ax.comm_handle.world_rank == 0:
                print(f"overflow detected - reducing loss scale to {s.loss_scale}", flush=True)
            return True
        s.no_overflow_iters += 1
        if s.no_overflow_iters == s.scaling_window:
            s.loss_scale = min(s.loss_scale * 2.0, s.max_scale)
            s.no_overflow_iters = 0
            if ax.comm_handle.world_rank == 0:
                print(f"increasing loss scale to {s.loss_scale}", flush=True)
        return False

    @torch.no_grad()
    def _unscale_gradients(self) -> bool:
        from . import ops

        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        ops.multi_tensor_scale_(grads, 1.0 / self.scaler.loss_scale)
        norm_sq = ops.multi_tensor_l2norm_sq(grads) if grads else torch.zeros(())
        return self._sync_scale(~torch.isfinite(norm_sq))
