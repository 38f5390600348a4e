"""Optimizers: fused multi-tensor AdamW and a host-offloaded variant.

``FusedAdamW`` keeps fp32 master weights and moments for (possibly bf16) model
parameters and updates every parameter of a group in one kernel launch
(``csrc/optim.cu``): gradient unscale / clip factor, moment update, decoupled
weight decay, master update and the bf16 model copy are a single pass over
memory, and a device-side ``found_inf`` flag skips the step without a host
synchronisation.  It is the working replacement for the reference's stale
``axonn/optim.py`` (``CPUAdam``, which depends on attributes removed from
``axonn/axonn.py``).

``CPUAdam`` reproduces that class's intent — optimizer state in pinned host
memory, streamed through fixed-size GPU staging buckets — on top of the same
kernel, with the copies double-buffered on a side stream.
"""

import ctypes
from typing import Iterable, Optional

import torch

from . import ops
from .ops import _lib, multi_tensor as _mt


class FusedAdamW(torch.optim.Optimizer):
    """AdamW whose whole step is one multi-tensor kernel per parameter group: fp32 master weights (for 16-bit
    parameters; ``master_weights`` forces either way) and fp32 moments are updated and the 16-bit model copy is
    written in the same pass.  ``grad_scale`` / ``found_inf`` (0-d device tensors) unscale the gradients and skip
    the update without a host synchronisation.  On CPU the same arithmetic runs in PyTorch."""

    def __init__(self, params: Iterable, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 master_weights: Optional[bool] = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self._tables = {}
        self.grad_scale = None  # optional 0-d fp32 device tensor multiplied into every gradient
        self.found_inf = None   # optional 0-d fp32 device tensor; non-zero skips the update

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            use_master = self.master_weights if self.master_weights is not None else p.dtype != torch.float32
            st["master"] = p.detach().float().clone() if use_master else None
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        return st

    def load_state_dict(self, state_dict):
        """``torch.optim.Optimizer.load_state_dict`` casts every floating-point state tensor to the dtype of
        its parameter, which would turn the fp32 master weights and moments of bf16 parameters into bf16.
        The fp32 values are restored from the incoming state dict afterwards, and the cached pointer
        tables (which still name the old state tensors) are dropped."""
        super().load_state_dict(state_dict)
        saved = state_dict["state"]
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for i, p in zip(ids, params):
            src = saved.get(i)
            if src is None:
                continue
            st = self.state[p]
            for key in ("master", "exp_avg", "exp_avg_sq"):
                v = src.get(key)
                if torch.is_tensor(v):
                    st[key] = v.detach().to(device=p.device, dtype=torch.float32).clone()
        self._tables.clear()

    @torch.no_grad()
    def step(self, closure=None, grad_attr="grad"):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            params = [p for p in group["params"] if getattr(p, grad_attr, None) is not None]
            if not params:
                continue
            for p in params:
                self._init_state(p)["step"] += 1
            step = self.state[params[0]]["step"]
            b1, b2 = group["betas"]
            if params[0].is_cuda:
                grads = [getattr(p, grad_attr) for p in params]
                grads = [g if g.is_contiguous() else g.contiguous() for g in grads]
                key = (gi, grad_attr)
                tab = self._tables.get(key)
                ptrs = tuple(g.data_ptr() for g in grads)
                if tab is None or tab.grad_ptrs != ptrs or tab.n != len(params):
                    masters, models = [], []
                    for p in params:
                        st = self.state[p]
                        if st["master"] is not None:
                            masters.append(st["master"])
                            models.append(p.data)
                        else:
                            masters.append(p.data)
                            models.append(None)
                    tab = ops.AdamTable(masters, models, grads, [self.state[p]["exp_avg"] for p in params],
                                        [self.state[p]["exp_avg_sq"] for p in params])
                    self._tables[key] = tab
                ops.multi_tensor_adamw(tab, group["lr"], b1, b2, group["eps"], group["weight_decay"], step,
                                       self.grad_scale, self.found_inf)
            else:
                gs = float(self.grad_scale) if self.grad_scale is not None else 1.0
                if self.found_inf is not None and float(self.found_inf) != 0:
                    continue
                for p in params:
                    st = self.state[p]
                    tgt = st["master"] if st["master"] is not None else p.data
                    ops.adamw_reference_(tgt, getattr(p, grad_attr), st["exp_avg"], st["exp_avg_sq"], group["lr"],
                                         b1, b2, group["eps"], group["weight_decay"], st["step"], gs)
                    if st["master"] is not None:
                        p.data.copy_(tgt)
        return loss


class FusedSGD(torch.optim.Optimizer):
    """SGD with momentum and weight decay (``torch.optim.SGD`` semantics without dampening or Nesterov) as one
    multi-tensor kernel launch per parameter group (``csrc/optim.cu::multi_sgd_kernel``); parameters and gradients
    may be fp32, bf16 or fp16, the momentum buffers are fp32.  On CPU tensors it falls back to the plain update."""

    def __init__(self, params: Iterable, lr=1e-2, momentum=0.9, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay))
        self._tables = {}
        self.grad_scale = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            for p in params:
                if "momentum_buffer" not in self.state[p]:
                    self.state[p]["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
            if params[0].is_cuda:
                grads = [p.grad if p.grad.is_contiguous() else p.grad.contiguous() for p in params]
                ptrs = tuple(g.data_ptr() for g in grads)
                tab = self._tables.get(gi)
                if tab is None or tab[0] != ptrs:
                    rows, prefix = [], 0
                    for p, g in zip(params, grads):
                        assert p.is_contiguous()
                        rows.append((p.data_ptr(), g.data_ptr(), self.state[p]["momentum_buffer"].data_ptr(), p.numel(),
                                     _mt._DT_CODE[p.dtype], _mt._DT_CODE[g.dtype], prefix, 0))
                        prefix += (p.numel() + _mt._CHUNK - 1) // _mt._CHUNK
                    host = torch.tensor(rows, dtype=torch.int64).pin_memory()
                    tab = self._tables[gi] = (ptrs, host, host.to(params[0].device, non_blocking=True), len(rows), prefix)
                st = _lib.lib().axb_multi_sgd(_lib.ptr(tab[2]), ctypes.c_int(tab[3]), ctypes.c_longlong(tab[4]),
                                              ctypes.c_float(group["lr"]), ctypes.c_float(group["momentum"]),
                                              ctypes.c_float(group["weight_decay"]), _lib.ptr(self.grad_scale),
                                              _lib.stream_ptr())
                _lib.check(st, "axb_multi_sgd")
                _lib.add_launches(1)
            else:
                for p in params:
                    g = p.grad.float() + group["weight_decay"] * p.float()
                    buf = self.state[p]["momentum_buffer"]
                    buf.mul_(group["momentum"]).add_(g)
                    p.add_(buf.to(p.dtype), alpha=-group["lr"])
        return loss


class CPUAdam(torch.optim.Optimizer):
    """AdamW with master weights and moments in pinned host memory.

    Every step streams the state through two GPU staging buckets of
    ``bucket_size`` fp32 elements: while bucket i is updated by the fused kernel
    on the compute stream, bucket i+1 is copied in and bucket i-1 copied out on a
    side stream (reference intent: ``axonn/optim.py:12-196``)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, bucket_size=16_000_000):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.bucket_size = int(bucket_size)
        self._staging = None
        self._side = None
        self._steps = 0

    def _host_state(self, p):
        st = self.state[p]
        if not st:
            pin = torch.cuda.is_available()
            st["master"] = torch.empty(p.numel(), dtype=torch.float32, pin_memory=pin).copy_(p.detach().float().view(-1))
            st["exp_avg"] = torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin)
            st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin)
        return st

    def state_dict(self):
        """The step count lives on the optimizer (one count for all parameters), so it is added to the dict."""
        sd = super().state_dict()
        sd["steps"] = self._steps
        return sd

    def load_state_dict(self, state_dict):
        """``torch.optim.Optimizer.load_state_dict`` would move the state to the parameters' device and cast it
        to their dtype; this optimizer's state is flat fp32 in (pinned) host memory and stays there."""
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        if len(ids) != len(params):
            raise ValueError("loaded state dict names a different number of parameters")
        for group, saved in zip(self.param_groups, state_dict["param_groups"]):
            group.update({k: v for k, v in saved.items() if k != "params"})
        for i, p in zip(ids, params):
            src = state_dict["state"].get(i)
            if src is None:
                continue
            st = self._host_state(p)
            for key in ("master", "exp_avg", "exp_avg_sq"):
                st[key].copy_(src[key].detach().reshape(-1).float())
            p.data.copy_(st["master"].view_as(p))
        self._steps = int(state_dict.get("steps", self._steps))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._steps += 1
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._host_state(p)
                if not p.is_cuda:
                    ops.adamw_reference_(st["master"], p.grad.view(-1), st["exp_avg"], st["exp_avg_sq"],
                                         group["lr"], b1, b2, group["eps"], group["weight_decay"], self._steps)
                    p.data.copy_(st["master"].view_as(p))
                    continue
                self._step_cuda(p, st, group, b1, b2)
        return loss

    def _step_cuda(self, p, st, group, b1, b2):
        dev = p.device
        if self._staging is None:
            self._staging = [[torch.empty(self.bucket_size, dtype=torch.float32, device=dev) for _ in range(3)]
                             for _ in range(2)]
            self._side = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        n = p.numel()
        grad = p.grad.contiguous().view(-1)
        flat = p.data.view(-1)
        nb = (n + self.bucket_size - 1) // self.bucket_size
        ready = [None, None]
        done = [None, None]

        def load(i):
            a, b = i * self.bucket_size, min(n, (i + 1) * self.bucket_size)
            slot = self._staging[i % 2]
            with torch.cuda.stream(self._side):
                if done[i % 2] is not None:
                    self._side.wait_event(done[i % 2])
                for buf, key in zip(slot, ("master", "exp_avg", "exp_avg_sq")):
                    buf[: b - a].copy_(st[key][a:b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._side)
                ready[i % 2] = ev

        load(0)
        for i in range(nb):
            a, b = i * self.bucket_size, min(n, (i + 1) * self.bucket_size)
            if i + 1 < nb:
                load(i + 1)
            slot = self._staging[i % 2]
            main.wait_event(ready[i % 2])
            model = flat[a:b] if p.dtype == torch.bfloat16 else None
            tab = ops.AdamTable([slot[0][: b - a]], [model], [grad[a:b]], [slot[1][: b - a]], [slot[2][: b - a]])
            ops.multi_tensor_adamw(tab, group["lr"], b1, b2, group["eps"], group["weight_decay"], self._steps)
            if model is None:
                flat[a:b].copy_(slot[0][: b - a])
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(ev)
                for buf, key in zip(slot, ("master", "exp_avg", "exp_avg_sq")):
                    st[key][a:b].copy_(buf[: b - a], non_blocking=True)
                d = torch.cuda.Event()
                d.record(self._side)
                done[i % 2] = d
        main.wait_stream(self._side)
