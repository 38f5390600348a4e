"""3-D tensor-parallel ``Linear`` (row x column x depth).

Behavioural twin of the reference's ``axonn/intra_layer/fully_connected.py``
(``Linear`` ``:190-400``, ``AsyncLinear`` ``:96-187``):

* the ``[out, in]`` weight is block-sharded — ``in`` over the *inner* group,
  ``out`` over the *outer* group — the local block is flattened and its 1-D
  view is sharded over the *depth* group, so the ``nn.Parameter`` is a flat
  1-D tensor (this is also the checkpoint format);
* forward: depth all-gather -> ``X @ W^T`` -> all-reduce over inner;
* backward: ``dX = dY @ W`` -> all-reduce over outer, ``dW = dY^T @ X`` ->
  reduce-scatter over depth;
* ``transpose=True`` swaps inner and outer so that consecutive layers chain
  without re-layout; ``expert_mode=False`` adds the data-parallel <-> tensor-
  parallel layout switches around the layer.

On CUDA the three GEMMs run on this package's tcgen05 kernels and, when the
group's ranks share an NVLink peer-memory heap, on the variants that fuse the
collective with the GEMM (``axonn_b200.parallel.fused``); on CPU the same
autograd function runs on ``torch.matmul`` + ``torch.distributed``.
"""

import ctypes
import math
import os
from typing import Optional, Sequence

import torch
import torch.distributed as dist
from torch.autograd import Function

from .. import axonn as ax
from .. import ops
from ..ops import _lib
from ..parallel import fused
from ..utils import divide
from . import overlap_communication as oc
from .asym_communication import (
    Dropv,
    GatherBatchScatterChannels,
    GatherChannelsScatterBatch,
    Gatherv,
    gather_batch_sizes,
)
from .communication import Drop, GatherSumBackward, _drop, _gather, _reduce_scatter


@torch.no_grad()
def extract_local_params_from_full_params(params, out_features_group, in_features_group, depth_group):
    """``W[out, in]`` -> this rank's flat shard:
    rows of my outer chunk, columns of my inner chunk, flattened, my depth slice
    (the layout stated at reference ``fully_connected.py:62-70``)."""
    no, ni = dist.get_world_size(out_features_group), dist.get_world_size(in_features_group)
    ro, ci = dist.get_rank(out_features_group), dist.get_rank(in_features_group)
    out_l, in_l = params.shape[0] // no, params.shape[1] // ni
    block = params[ro * out_l:(ro + 1) * out_l, ci * in_l:(ci + 1) * in_l].contiguous().view(-1)
    nd, dz = dist.get_world_size(depth_group), dist.get_rank(depth_group)
    n = divide(block.numel(), nd)
    return block[dz * n:(dz + 1) * n].clone()


@torch.no_grad()
def default_init_method(weight):
    return torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))


@torch.no_grad()
def initialize_params(out_features, in_features, out_features_group, in_features_group, depth_group,
                      init_method, init_device=None, dtype=torch.float32):
    """Materialise the full matrix with the caller's RNG stream (identical on
    every rank when seeded identically), keep this rank's shard."""
    if init_device is None:
        init_device = ax.config.device
    params = torch.empty((out_features, in_features), device=init_device, dtype=dtype)
    init_method(params)
    return extract_local_params_from_full_params(params, out_features_group, in_features_group, depth_group)


def _gathered_weight(weight, depth_group, local_shape, cache):
    """Depth all-gather of the flat shard, shaped ``[out_l, in_l]``."""
    full = _gather(weight, dim=0, process_group=depth_group, cache=cache)
    return full.reshape(local_shape)


_side_streams = {}
_OVERLAP_WGRAD_DEFAULT = "0"


def _side_stream(device):
    st = _side_streams.get(device)
    if st is None:
        st = _side_streams[device] = torch.cuda.Stream(device=device)
    return st


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def _wgrad_overlap_ctas() -> int:
    """CTAs that the communication-bound input-gradient kernel gets when it runs beside the weight-gradient GEMM
    (``AXONN_OVERLAP_WGRAD``: 0 = off, the two kernels run one after the other; otherwise an even CTA count)."""
    try:
        n = int(os.environ.get("AXONN_OVERLAP_WGRAD", _OVERLAP_WGRAD_DEFAULT))
    except ValueError:
        return 0
    return max(0, n) // 2 * 2


class AsyncLinear(Function):
    """``y = act(x @ W^T + b)`` with the three collectives of 3-D tensor parallelism.

    ``bias`` and ``activation`` are optional; when the forward all-reduce group has
    one rank they are applied in the GEMM epilogue, otherwise after the all-reduce."""

    @staticmethod
    def forward(ctx, input_, weight, bias, activation, forward_all_reduce_group, backward_all_reduce_group,
                depth_parallel_group, local_weight_shape, cache_weights):
        cache = bool(cache_weights) or oc.CACHE_WEIGHTS
        w_shard = weight
        compute_dtype = input_.dtype
        if torch.is_autocast_enabled(input_.device.type):
            compute_dtype = torch.get_autocast_dtype(input_.device.type)
            input_ = input_.to(compute_dtype)
        x2 = input_.reshape(-1, input_.shape[-1])
        inner_n = dist.get_world_size(forward_all_reduce_group)
        depth_n = dist.get_world_size(depth_parallel_group)
        b = None if bias is None else bias.to(compute_dtype)
        pre_act = None
        if activation not in (None, "gelu"):
            raise ValueError(f"unsupported fused activation {activation!r}")
        epi = ops.EPI_NONE
        if activation == "gelu":
            epi = ops.EPI_BIAS_GELU if b is not None else ops.EPI_GELU
        elif b is not None:
            epi = ops.EPI_BIAS
        prefetched = id(w_shard) in oc.weights_cache
        out_l, in_l = local_weight_shape
        ar_ok = inner_n > 1 and fused.usable(forward_all_reduce_group, x2, N=out_l, K=in_l)
        if (depth_n > 1 and not prefetched and (inner_n == 1 or ar_ok)
                and fused.all_gather_usable(depth_parallel_group, x2, w_shard, local_weight_shape, 0)):
            # one kernel: pull the depth shards of W over NVLink while computing, multiply, (all-reduce), epilogue
            res = fused.all_gather_gemm(0, x2, w_shard, depth_parallel_group, local_weight_shape,
                                        ar_group=forward_all_reduce_group if inner_n > 1 else None,
                                        bias=b, epilogue=epi, want_aux=activation == "gelu")
            out, w = res[0], res[1]
            if activation == "gelu":
                pre_act = res[2]
            if cache:
                oc.weights_cache[id(w_shard)] = [w_shard, w.reshape(-1), None]
        else:
            w = _gathered_weight(w_shard, depth_parallel_group, local_weight_shape, cache)
            if w.dtype != compute_dtype:
                w = w.to(compute_dtype)
            if ar_ok:
                # GEMM whose epilogue all-reduces the output tiles over NVLink peer memory,
                # then applies bias / GELU to the reduced values
                if activation == "gelu":
                    out, pre_act = fused.gemm_all_reduce(0, x2, w, forward_all_reduce_group, bias=b, epilogue=epi,
                                                         want_aux=True)
                else:
                    out = fused.gemm_all_reduce(0, x2, w, forward_all_reduce_group, bias=b, epilogue=epi)
            elif inner_n == 1 and x2.is_cuda and epi != ops.EPI_NONE:
                if activation == "gelu":
                    pre_act = torch.empty((x2.shape[0], local_weight_shape[0]), dtype=compute_dtype,
                                          device=x2.device)
                out = ops.matmul_nt(x2, w, bias=b, epilogue=epi, aux=pre_act)
            else:
                out = ops.matmul_nt(x2, w)
                if inner_n > 1:
                    dist.all_reduce(out, group=forward_all_reduce_group)
                if b is not None:
                    out = out.add_(b)
                if activation == "gelu":
                    pre_act = out
                    out = ops.gelu(out.detach())
        ctx.save_for_backward(input_, w_shard, pre_act)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.backward_all_reduce_group = backward_all_reduce_group
        ctx.depth_parallel_group = depth_parallel_group
        ctx.shape = local_weight_shape
        ctx.compute_dtype = compute_dtype
        # a view created inside a custom Function may not be modified in place later (rotary embeddings are
        # applied in place to the projection output): return the tensor itself when no reshape is needed
        target = (*input_.shape[:-1], local_weight_shape[0])
        return out if tuple(out.shape) == target else out.reshape(target)

    @staticmethod
    def backward(ctx, grad_output):
        input_, w_shard, pre_act = ctx.saved_tensors
        grad_output = grad_output.to(ctx.compute_dtype)
        go2 = grad_output.reshape(-1, grad_output.shape[-1])
        bias_sum = None
        if pre_act is not None:
            if ctx.has_bias and ctx.needs_input_grad[2]:
                # bias gradient in the same pass
                go2, bias_sum = ops.gelu_backward_colsum(go2, pre_act, out_dtype=ctx.bias_dtype)
            else:
                go2 = ops.gelu_backward(go2, pre_act)
        x2 = input_.reshape(-1, input_.shape[-1])
        overlap_rs = oc.OVERLAP_REDUCE_SCATTER
        overlap_ar = oc.OVERLAP_ALL_REDUCE
        outer_n = dist.get_world_size(ctx.backward_all_reduce_group)
        depth_n = dist.get_world_size(ctx.depth_parallel_group)
        grad_input = grad_weight = grad_bias = None
        handle = None

        def wgrad():
            if depth_n > 1 and go2.dtype == w_shard.dtype and \
                    fused.reduce_scatter_usable(ctx.depth_parallel_group, go2, x2, ctx.shape[0]):
                # weight-gradient GEMM whose epilogue reduce-scatters the row blocks (= depth shards of the
                # flattened weight) over NVLink peer memory
                return fused.gemm_reduce_scatter(2, go2, x2, ctx.depth_parallel_group,
                                                 out_dtype=w_shard.dtype).reshape(-1)
            gw = ops.matmul_tn(go2, x2, out_dtype=w_shard.dtype).reshape(-1)
            if depth_n > 1:
                gw = _reduce_scatter(gw, 0, ctx.depth_parallel_group, overlap_comm=overlap_rs)
                if overlap_rs:
                    oc.accumulate_later(w_shard, gw)
                    return None
            return gw

        def dgrad():
            # the cached copy (if any) is consumed here; otherwise gather again
            w = _gathered_weight(w_shard, ctx.depth_parallel_group, ctx.shape, cache=False)
            if w.dtype != ctx.compute_dtype:
                w = w.to(ctx.compute_dtype)
            return ops.matmul_nn(go2, w)

        if outer_n > 1 or not overlap_rs:
            # dgrad first so that its all-reduce hides under the wgrad GEMM
            side = None
            if ctx.needs_input_grad[0]:
                ar_ok = outer_n > 1 and fused.usable(ctx.backward_all_reduce_group, go2, N=ctx.shape[1],
                                                     K=ctx.shape[0])
                split = _wgrad_overlap_ctas() if (ar_ok and go2.is_cuda and ctx.needs_input_grad[1]) else 0
                if split:
                    # The fused input-gradient GEMM + all-reduce is bound by NVLink, the weight-gradient GEMM by the
                    # tensor cores: run them side by side on disjoint sets of SMs (two streams, CTA caps that add up to
                    # the SM count, so that both persistent grids are resident together).  The streams are joined
                    # again before this function returns, which keeps every buffer and channel in stream order
                    # across layers.
                    main = torch.cuda.current_stream()
                    side = _side_stream(go2.device)
                    side.wait_stream(main)
                    L = _lib.lib()
                    L.axb_gemm_set_max_ctas(ctypes.c_int(_sm_count(go2.device) - split))
                    with torch.cuda.stream(side):
                        grad_weight = wgrad()
                        if ctx.has_bias and ctx.needs_input_grad[2]:
                            grad_bias = bias_sum if bias_sum is not None else ops.column_sum(go2, out_dtype=ctx.bias_dtype)
                    L.axb_gemm_set_max_ctas(ctypes.c_int(split))
                if (depth_n > 1 and id(w_shard) not in oc.weights_cache
                        and (outer_n == 1 or ar_ok)
                        and fused.all_gather_usable(ctx.depth_parallel_group, go2, w_shard, ctx.shape, 1)):
                    grad_input, _ = fused.all_gather_gemm(
                        1, go2.contiguous(), w_shard, ctx.depth_parallel_group, ctx.shape,
                        ar_group=ctx.backward_all_reduce_group if outer_n > 1 else None)
                elif ar_ok:
                    w = _gathered_weight(w_shard, ctx.depth_parallel_group, ctx.shape, cache=False)
                    if w.dtype != ctx.compute_dtype:
                        w = w.to(ctx.compute_dtype)
                    grad_input = fused.gemm_all_reduce(1, go2.contiguous(), w, ctx.backward_all_reduce_group)
                else:
                    grad_input = dgrad()
                    if outer_n > 1:
                        handle = dist.all_reduce(grad_input, group=ctx.backward_all_reduce_group,
                                                 async_op=overlap_ar)
            if side is not None:
                _lib.lib().axb_gemm_set_max_ctas(ctypes.c_int(0))
                torch.cuda.current_stream().wait_stream(side)
            else:
                if ctx.needs_input_grad[1]:
                    grad_weight = wgrad()
                if ctx.has_bias and ctx.needs_input_grad[2]:
                    grad_bias = bias_sum if bias_sum is not None else ops.column_sum(go2, out_dtype=ctx.bias_dtype)
            if handle is not None and overlap_ar:
                handle.wait()
        else:
            # no activation all-reduce: start the reduce-scatter first, hide it under dgrad
            if ctx.needs_input_grad[1]:
                grad_weight = wgrad()
            if ctx.needs_input_grad[0]:
                grad_input = dgrad()
            if ctx.has_bias and ctx.needs_input_grad[2]:
                grad_bias = bias_sum if bias_sum is not None else ops.column_sum(go2, out_dtype=ctx.bias_dtype)
        if grad_input is not None:
            grad_input = grad_input.reshape(input_.shape)
        return grad_input, grad_weight, grad_bias, None, None, None, None, None, None


class Linear(torch.nn.Module):
    """Drop-in ``nn.Linear`` whose weight is sharded over the 3-D grid.

    Arguments follow reference ``fully_connected.py:191-203``."""

    def __init__(self, in_features, out_features, *args, transpose=False, bias=True, skip_bias_add=False,
                 init_method=None, expert_mode=False, tensor_parallel_dims: Optional[Sequence[int]] = None,
                 **kwargs):
        super().__init__()
        assert ax.is_initialized, "call axonn_b200.axonn.init(...) first"
        for k in ("use_easy_api", "easy_api"):
            # spelled this way by the reference's HF patches; honoured here
            if k in kwargs:
                expert_mode = not kwargs.pop(k)
        ch = ax.comm_handle
        self.inner_group, self.outer_group, self.depth_group = ch.get_intra_layer_groups(tensor_parallel_dims)
        if transpose:
            self.inner_group, self.outer_group = self.outer_group, self.inner_group
        self.inner_group_size = dist.get_world_size(self.inner_group)
        self.outer_group_size = dist.get_world_size(self.outer_group)
        self.depth_group_size = dist.get_world_size(self.depth_group)
        self.in_features, self.out_features = in_features, out_features
        self.expert_mode = expert_mode
        self.transpose = transpose
        self.local_in_features = divide(in_features, self.inner_group_size)
        self.local_out_features = divide(out_features, self.outer_group_size)
        if init_method is None:
            init_method = default_init_method
        dtype = kwargs.get("dtype") or torch.get_default_dtype()
        initial = initialize_params(out_features, in_features, self.outer_group, self.inner_group,
                                    self.depth_group, init_method, dtype=dtype)
        self.weight = torch.nn.Parameter(initial, requires_grad=True)
        self.weight.is_tensor_parallel = True
        self.weight.needs_depth_parallel_gradient_sync = False
        self.weight.process_group_for_norm_reduction = ch.intra_layer_group
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(self.local_out_features, dtype=dtype,
                                                       device=initial.device))
            self.bias.is_tensor_parallel = True
            self.bias.needs_depth_parallel_gradient_sync = True
            # a bias shard is replicated over inner and depth, distinct over outer
            self.bias.process_group_for_norm_reduction = self.outer_group
        else:
            self.bias = None
        self.skip_bias_add = skip_bias_add

    @property
    def local_weight_shape(self):
        return (self.local_out_features, self.local_in_features)

    def extra_repr(self):
        return (f"in={self.in_features}, out={self.out_features}, local={self.local_weight_shape}, "
                f"grid(inner,outer,depth)=({self.inner_group_size},{self.outer_group_size},"
                f"{self.depth_group_size}), transpose={self.transpose}, expert_mode={self.expert_mode}")

    def forward(self, x, cache_weights_in_all_gather=False, activation=None):
        """``activation="gelu"`` fuses bias + GELU (tanh form) into the layer; only
        meaningful when the bias is added inside the layer (expert mode, no
        ``skip_bias_add``)."""
        lead_shape = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
        switch_layout = (not self.expert_mode) and self.inner_group_size * self.outer_group_size > 1
        if switch_layout:
            inner_sizes = gather_batch_sizes(x.shape[0], self.inner_group, device=x.device)
            x = GatherBatchScatterChannels.apply(x, inner_sizes, self.inner_group)
            outer_sizes = gather_batch_sizes(x.shape[0], self.outer_group, device=x.device)
            x = Gatherv.apply(x, outer_sizes, self.outer_group)
        fuse_bias = self.expert_mode and not self.skip_bias_add
        if activation is not None and not fuse_bias and self.bias is not None:
            raise ValueError("activation= needs the bias to be added inside the layer")
        x = AsyncLinear.apply(x, self.weight, self.bias if fuse_bias else None, activation, self.inner_group,
                              self.outer_group, self.depth_group, self.local_weight_shape,
                              cache_weights_in_all_gather)
        if switch_layout:
            x = GatherChannelsScatterBatch.apply(x, outer_sizes, self.outer_group)
            x = Dropv.apply(x, inner_sizes, self.inner_group)
        x = x.reshape(*lead_shape, x.shape[-1])
        if self.bias is None or fuse_bias:
            return x
        bias = self.bias
        if not self.expert_mode:
            bias = GatherSumBackward.apply(bias, self.outer_group, self.inner_group)
        if self.skip_bias_add:
            return x, bias
        return x + bias.to(x.dtype)

    # ---------------------------------------------------------------- state dict
    def _is_full_weight_matrix(self, w):
        return w.ndim == 2 and w.size(0) == self.out_features and w.size(1) == self.in_features

    def _is_sharded_weight_matrix(self, w):
        return w.ndim == 1 and w.size(0) == divide(
            self.local_out_features * self.local_in_features, self.depth_group_size)

    @torch.no_grad()
    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Accept either a full ``[out, in]`` matrix (e.g. from ``nn.Linear`` or a
        run on another grid) or this rank's flat shard; same for the bias."""
        w = state_dict.get(prefix + "weight")
        if w is not None:
            if self._is_full_weight_matrix(w):
                state_dict[prefix + "weight"] = extract_local_params_from_full_params(
                    w, self.outer_group, self.inner_group, self.depth_group)
            elif not self._is_sharded_weight_matrix(w):
                raise ValueError(f"{prefix}weight of shape {tuple(w.shape)} is neither the full "
                                 f"[{self.out_features},{self.in_features}] matrix nor this rank's shard")
        if self.bias is not None:
            b = state_dict.get(prefix + "bias")
            if b is not None:
                if b.size(0) == self.out_features and self.outer_group_size > 1:
                    state_dict[prefix + "bias"] = Drop.apply(b, self.outer_group).clone()
                elif b.size(0) != self.local_out_features:
                    raise ValueError(f"{prefix}bias of length {b.size(0)} matches neither the full nor the "
                                     f"local output width")
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    @torch.no_grad()
    def full_weight(self):
        """Reassemble the full ``[out, in]`` matrix on every rank (tests, export)."""
        return self.full_tensor("weight")

    @torch.no_grad()
    def full_tensor(self, name, t=None):
        """Grid-independent form of a tensor laid out like parameter ``name`` (``"weight"`` or ``"bias"``):
        the parameter itself, or an optimizer state tensor of the same shape.  Collective over the layer's
        three groups; every rank receives the result."""
        t = getattr(self, name).detach() if t is None else t
        if name == "bias":
            return _gather(t, 0, self.outer_group)
        w = _gather(t, 0, self.depth_group).reshape(self.local_weight_shape)
        w = _gather(w, 1, self.inner_group)
        return _gather(w, 0, self.outer_group)

    @torch.no_grad()
    def shard_tensor(self, name, full):
        """Inverse of :meth:`full_tensor`: this rank's piece of a full ``[out, in]`` matrix or ``[out]`` vector."""
        if name == "bias":
            return _drop(full, 0, self.outer_group).clone()
        return extract_local_params_from_full_params(full, self.outer_group, self.inner_group, self.depth_group)
