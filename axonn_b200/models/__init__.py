"""Model zoo built on the tensor-parallel layers and sm_100a kernels."""

from .gpt import GPT, GPTConfig  # noqa: F401
from .llama import Llama, LlamaConfig  # noqa: F401
from .mlp import MLP  # noqa: F401
