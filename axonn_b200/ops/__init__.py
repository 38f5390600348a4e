"""Operators: hand-written sm_100a kernels on GPU, PyTorch on CPU.

Every function here has two implementations with identical semantics: a CUDA
kernel from ``axonn_b200/csrc`` reached through ``ops._lib`` and a plain
PyTorch composition used on CPU (and as the numerical oracle in the tests).
"""

from .activation import gelu_backward_colsum, gelu, gelu_backward, swiglu  # noqa: F401
from .attention import flash_attention, flash_attention_packed  # noqa: F401
from .gemm import (  # noqa: F401
    EPI_BIAS,
    EPI_BIAS_GELU,
    EPI_GELU,
    EPI_NONE,
    matmul_nn,
    matmul_nt,
    matmul_tn,
)
from .linear import linear, linear_batched  # noqa: F401
from .loss import cross_entropy  # noqa: F401
from .multi_tensor import (  # noqa: F401
    all_reduce_bucketed_,
    multi_tensor_l2norm_sq,
    multi_tensor_scale_,
)
from .norm import add_layer_norm, add_rms_norm, column_sum, layer_norm, rms_norm  # noqa: F401
from .optim_step import AdamTable, adamw_reference_, multi_tensor_adamw, prune_topk_  # noqa: F401
from .rope import apply_rope, rope_table  # noqa: F401
