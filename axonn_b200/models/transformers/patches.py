"""Per-architecture constructors for Hugging Face models (OPT, Llama, Mistral, Mixtral).

Counterpart of the reference's ``axonn/models/transformers/modify_llama.py:12-107``,
``modify_mistral.py:16-107``, ``modify_mixtral.py:16-109`` and ``modify_opt.py:12-86``: inside
``parallelize(...)`` the attention and MLP classes of the architecture build their projections as
tensor-parallel ``Linear`` layers — query/key/value and the first MLP projections split their output
features (hence the attention heads) over the row group, the projections that close a block
(``o_proj`` / ``out_proj`` / ``down_proj`` / ``fc2``) are built with ``transpose=True`` and reduce over it —
and head counts are divided by ``G_intra_r`` where the model's forward needs them.

The reference rewrites the constructors of one Transformers release line by line.  Here the original
constructor runs unchanged while ``torch.nn.Linear`` is replaced by a placeholder that only records its
arguments; afterwards the placeholders are swapped for tensor-parallel layers according to their attribute
names.  No full-size weight is ever materialised, and the patch does not depend on the constructor's body.

Layout rule: with ``G_intra_c == 1`` the layers run in expert mode (activations between blocks carry the
full hidden dimension and are replicated over the row group, as Hugging Face's embeddings and norms expect);
otherwise they run in easy mode (every layer switches layouts itself), which is correct for any grid.
Mixtral's experts are 3-D parameter tensors in current Transformers releases, not ``nn.Linear`` modules:
they stay replicated; only its attention is sharded.
"""

import importlib

import torch.nn as nn

from ... import axonn as ax
from ...intra_layer import Linear


class _PendingLinear(nn.Module):
    """Stands in for ``nn.Linear`` while a patched constructor runs: records the arguments only."""

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.has_bias = in_features, out_features, bias
        self.device, self.dtype = device, dtype


def expert_mode_for_grid() -> bool:
    return ax.config.G_intra_c == 1


def _divide_heads(module, attrs):
    r = ax.config.G_intra_r
    for a in attrs:
        v = getattr(module, a, None)
        if isinstance(v, int):
            assert v % r == 0, f"{a}={v} is not divisible by G_intra_r={r}"
            setattr(module, a, v // r)


def _patched_init(cls, transposed_by_name, head_attrs=()):
    original = cls.__init__

    def init(self, *args, **kwargs):
        real_linear = nn.Linear
        nn.Linear = _PendingLinear
        try:
            original(self, *args, **kwargs)
        finally:
            nn.Linear = real_linear
        expert = expert_mode_for_grid()
        for name, child in list(self.named_children()):
            if not isinstance(child, _PendingLinear):
                continue
            if name in transposed_by_name:
                new = Linear(child.in_features, child.out_features, bias=child.has_bias,
                             transpose=transposed_by_name[name], expert_mode=expert,
                             **({"dtype": child.dtype} if child.dtype is not None else {}))
            else:
                new = real_linear(child.in_features, child.out_features, bias=child.has_bias, dtype=child.dtype)
            if child.device is not None and str(child.device) != "meta":
                new = new.to(child.device)
            setattr(self, name, new)
        if expert and head_attrs:
            _divide_heads(self, head_attrs)

    init._axonn_original = original
    return init


_ATTN = {"q_proj": False, "k_proj": False, "v_proj": False, "o_proj": True}
_MLP = {"gate_proj": False, "up_proj": False, "down_proj": True}

# architecture -> [(module path, class name, {attribute: transpose}, head-count attributes to divide)]
PATCH_TABLE = {
    "LlamaForCausalLM": [
        ("transformers.models.llama.modeling_llama", "LlamaAttention", _ATTN, ("num_heads", "num_key_value_heads")),
        ("transformers.models.llama.modeling_llama", "LlamaMLP", _MLP, ()),
    ],
    "MistralForCausalLM": [
        ("transformers.models.mistral.modeling_mistral", "MistralAttention", _ATTN, ("num_heads", "num_key_value_heads")),
        ("transformers.models.mistral.modeling_mistral", "MistralMLP", _MLP, ()),
    ],
    "MixtralForCausalLM": [
        ("transformers.models.mixtral.modeling_mixtral", "MixtralAttention", _ATTN, ("num_heads", "num_key_value_heads")),
        # older releases: one module per expert with w1 / w3 (in) and w2 (out)
        ("transformers.models.mixtral.modeling_mixtral", "MixtralBlockSparseTop2MLP",
         {"w1": False, "w3": False, "w2": True}, ()),
    ],
    "OPTForCausalLM": [
        ("transformers.models.opt.modeling_opt", "OPTAttention",
         {"q_proj": False, "k_proj": False, "v_proj": False, "out_proj": True}, ("num_heads",)),
        ("transformers.models.opt.modeling_opt", "OPTDecoderLayer", {"fc1": False, "fc2": True}, ()),
    ],
}


def apply_patches(architecture):
    """Patch the constructors of ``architecture``; returns the list needed by ``remove_patches``."""
    undo = []
    for module_path, cls_name, names, heads in PATCH_TABLE[architecture]:
        try:
            mod = importlib.import_module(module_path)
        except ImportError:
            continue
        cls = getattr(mod, cls_name, None)
        if cls is None:          # class does not exist in the installed release
            continue
        undo.append((cls, cls.__init__))
        cls.__init__ = _patched_init(cls, names, heads)
    return undo


def remove_patches(undo):
    for cls, original in undo:
        cls.__init__ = original
