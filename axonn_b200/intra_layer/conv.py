"""Tensor-parallel ``Conv2d``.

Same sharding and dataflow as the reference's ``axonn/intra_layer/conv.py``
(``:48-182``): the ``[out_c, in_c, k, k]`` filter bank is split over the outer
group on dim 0 and the inner group on dim 1, flattened and depth-sharded.
Forward: depth gather of the weight, drop input channels (inner) and batch
(depth), convolution, all-reduce over inner, gather channels (outer) and batch
(depth).  The overlap flag for the depth reduce-scatter is read from
``overlap_communication`` (the reference reads a name that its package does
not export, ``conv.py:139``).  Full-shape state dicts are accepted like in
``Linear``.
"""

import math

import torch
import torch.distributed as dist

from .. import axonn as ax
from ..utils import divide
from . import overlap_communication as oc
from .communication import (
    BackwardAllReduce,
    Drop,
    ForwardAllReduce,
    ForwardGather_BackwardReduceScatter,
    Gather,
    _drop,
    _gather,
)


@torch.no_grad()
def extract_local_params_from_full_params(params, out_group, in_group, depth_group):
    no, ni = dist.get_world_size(out_group), dist.get_world_size(in_group)
    ro, ci = dist.get_rank(out_group), dist.get_rank(in_group)
    oc_l, ic_l = params.shape[0] // no, params.shape[1] // ni
    block = params[ro * oc_l:(ro + 1) * oc_l, ci * ic_l:(ci + 1) * ic_l].contiguous().view(-1)
    nd, dz = dist.get_world_size(depth_group), dist.get_rank(depth_group)
    n = divide(block.numel(), nd)
    return block[dz * n:(dz + 1) * n].clone()


@torch.no_grad()
def default_init_method(weight):
    return torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))


class Conv2d(torch.nn.Module):
    """Drop-in ``nn.Conv2d`` (square kernels) whose filter bank is sharded over the 3-D grid: output channels over
    the outer group, input channels over the inner group, the flattened block over the depth group.
    ``forward(x, scatter_input=True, gather_output=True)`` takes and returns full tensors by default."""

    def __init__(self, in_channels, out_channels, kernel_size, *args, transpose=False, bias=True,
                 skip_bias_add=False, init_method=None, stride=1, padding=0, dilation=1, groups=1,
                 dtype=None, **kwargs):
        super().__init__()
        assert ax.is_initialized
        ch = ax.comm_handle
        inner, outer = ch.inner_intra_layer_parallel_group, ch.outer_intra_layer_parallel_group
        if transpose:
            inner, outer = outer, inner
        self.inner_group, self.outer_group = inner, outer
        self.depth_group = ch.depth_intra_layer_parallel_group
        self.inner_group_size = dist.get_world_size(inner)
        self.outer_group_size = dist.get_world_size(outer)
        self.depth_group_size = dist.get_world_size(self.depth_group)
        self.in_channels, self.out_channels = in_channels, out_channels
        if isinstance(kernel_size, (tuple, list)):
            assert kernel_size[0] == kernel_size[1], "square kernels only"
            kernel_size = kernel_size[0]
        self.kernel_size = kernel_size
        self.local_in_channels = divide(in_channels, self.inner_group_size)
        self.local_out_channels = divide(out_channels, self.outer_group_size)
        if init_method is None:
            init_method = default_init_method
        dtype = dtype or torch.get_default_dtype()
        full = torch.empty((out_channels, in_channels // groups, kernel_size, kernel_size),
                           device=ax.config.device, dtype=dtype)
        init_method(full)
        self.weight = torch.nn.Parameter(
            extract_local_params_from_full_params(full, outer, inner, self.depth_group))
        del full
        self.weight.is_tensor_parallel = True
        self.weight.needs_depth_parallel_gradient_sync = False
        self.weight.process_group_for_norm_reduction = ch.intra_layer_group
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(self.local_out_channels, dtype=dtype,
                                                       device=self.weight.device))
            self.bias.is_tensor_parallel = True
            self.bias.needs_depth_parallel_gradient_sync = True
            self.bias.process_group_for_norm_reduction = outer
        else:
            self.bias = None
        self.skip_bias_add = skip_bias_add
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups

    @property
    def local_weight_shape(self):
        return (self.local_out_channels, self.local_in_channels // self.groups if self.groups > 1
                else self.local_in_channels, self.kernel_size, self.kernel_size)

    def forward(self, x, scatter_input=True, gather_output=True, cache_weights_in_all_gather=False):
        weight = ForwardGather_BackwardReduceScatter.apply(
            self.weight, self.depth_group, 0, oc.OVERLAP_REDUCE_SCATTER,
            cache_weights_in_all_gather or oc.CACHE_WEIGHTS,
        ).reshape(self.local_weight_shape)
        if scatter_input:
            x = Drop.apply(x, self.inner_group, 1)
            x = Drop.apply(x, self.depth_group, 0)
        x = BackwardAllReduce.apply(x, self.outer_group)
        if weight.dtype != x.dtype and not torch.is_autocast_enabled(x.device.type):
            weight = weight.to(x.dtype)
        h = torch.nn.functional.conv2d(x, weight, bias=None, stride=self.stride, padding=self.padding,
                                       dilation=self.dilation, groups=self.groups)
        h = ForwardAllReduce.apply(h, self.inner_group)
        if gather_output:
            h = Gather.apply(h, self.outer_group, 1)
            h = Gather.apply(h, self.depth_group, 0)
        if self.bias is None:
            return h
        bias = self.bias
        if gather_output:
            bias = Gather.apply(bias, self.outer_group, 0)
        if self.skip_bias_add:
            return h, bias
        return h + bias.view(1, -1, 1, 1).to(h.dtype)

    @torch.no_grad()
    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        w = state_dict.get(prefix + "weight")
        if w is not None and w.ndim == 4:
            state_dict[prefix + "weight"] = extract_local_params_from_full_params(
                w, self.outer_group, self.inner_group, self.depth_group)
        b = state_dict.get(prefix + "bias") if self.bias is not None else None
        if b is not None and b.size(0) == self.out_channels and self.outer_group_size > 1:
            state_dict[prefix + "bias"] = Drop.apply(b, self.outer_group).clone()
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    @torch.no_grad()
    def full_tensor(self, name, t=None):
        """Grid-independent form of a tensor laid out like parameter ``name`` (``"weight"``: the
        ``[out_c, in_c, k, k]`` filter bank; ``"bias"``: ``[out_c]``).  Collective over the layer's groups."""
        t = getattr(self, name).detach() if t is None else t
        if name == "bias":
            return _gather(t, 0, self.outer_group)
        w = _gather(t, 0, self.depth_group).reshape(self.local_weight_shape)
        w = _gather(w, 1, self.inner_group)
        return _gather(w, 0, self.outer_group)

    @torch.no_grad()
    def shard_tensor(self, name, full):
        if name == "bias":
            return _drop(full, 0, self.outer_group).clone()
        return extract_local_params_from_full_params(full, self.outer_group, self.inner_group, self.depth_group)
