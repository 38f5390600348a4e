"""Hugging Face Transformers integration.

The reference patches ``__init__`` of specific attention / MLP classes of OPT,
Llama, Mistral and Mixtral (``axonn/models/transformers/modify_*.py``).

``parallelize(model_id_or_config=None)``
    context manager.  For OPT / Llama / Mistral / Mixtral ``ForCausalLM`` the
    architecture's attention and MLP constructors are patched (``patches.py``):
    q/k/v and the first MLP projections shard their outputs - and with them
    the attention heads - over the row group, the closing projections are
    transposed layers, head counts are divided by ``G_intra_r`` where the
    forward needs them.  For any other architecture (or no argument) every
    ``torch.nn.Linear`` constructed inside becomes a tensor-parallel ``Linear``
    in easy mode (inputs/outputs keep their full feature dimension, the batch
    is what each rank holds).  Either way ``AutoModelForCausalLM.from_config``
    builds a sharded model without materialising full weights on one GPU.

``parallelize_model(model)``
    converts an already constructed model in place, moving the existing
    weights into the shards; projections that close a block
    (``o_proj``, ``down_proj``, ``fc2``, ``w2``, ``out_proj``, ``dense``) get
    ``transpose=True`` so consecutive layers alternate layouts as in the
    reference's patches.
"""

from contextlib import contextmanager

import torch
import torch.nn as nn

from ... import axonn as ax
from ...intra_layer import Linear
from ...intra_layer.automatic_parallelism import auto_parallelize, is_parallelizable_linear

SUPPORTED_ARCHITECTURES = ("OPTForCausalLM", "LlamaForCausalLM", "MistralForCausalLM", "MixtralForCausalLM")
TRANSPOSED_PROJECTIONS = ("o_proj", "down_proj", "fc2", "w2", "out_proj", "dense_4h_to_h", "c_proj")


def _architecture_of(model_id_or_config):
    if model_id_or_config is None:
        return None
    cfg = model_id_or_config
    if isinstance(cfg, str):
        from transformers import AutoConfig

        cfg = AutoConfig.from_pretrained(cfg)
    archs = getattr(cfg, "architectures", None) or []
    return archs[0] if archs else None


@contextmanager
def parallelize(model_id_or_config=None, strict=False):
    """Build Transformers models with tensor-parallel linear layers.

    ``strict=True`` reproduces the reference's check that the architecture is
    one of OPT / Llama / Mistral / Mixtral ``ForCausalLM``."""
    arch = _architecture_of(model_id_or_config)
    if strict and arch not in SUPPORTED_ARCHITECTURES:
        raise ValueError(f"{arch} has not been validated for tensor parallelism")
    if arch in SUPPORTED_ARCHITECTURES:
        from . import patches

        undo = patches.apply_patches(arch)
        try:
            yield None
        finally:
            patches.remove_patches(undo)
        return
    with auto_parallelize():
        yield None


@torch.no_grad()
def parallelize_model(model: nn.Module, transposed=TRANSPOSED_PROJECTIONS, expert_mode=False, skip=("lm_head",)):
    """Swap every eligible ``nn.Linear`` of ``model`` for a tensor-parallel layer
    holding the same weights.  Returns the number of converted layers."""
    assert ax.is_initialized
    converted = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if type(child) is not nn.Linear or name in skip:
                continue
            if not is_parallelizable_linear(child.in_features, child.out_features):
                continue
            new = Linear(child.in_features, child.out_features, bias=child.bias is not None,
                         transpose=name in transposed, expert_mode=expert_mode, dtype=child.weight.dtype)
            new.load_state_dict(child.state_dict())
            new.to(child.weight.device)
            setattr(parent, name, new)
            converted += 1
    return converted
