"""Model zoo built on the tensor-parallel layers and sm_100a kernels."""

from .generate import greedy_generate, parallel_argmax  # noqa: F401
from .gpt import GPT, DistributedGPT, GPTConfig  # noqa: F401
from .llama import Llama, LlamaConfig  # noqa: F401
from .mixtral import Mixtral, MixtralConfig  # noqa: F401
from .mlp import MLP  # noqa: F401
from .vgg import DistributedVGG16  # noqa: F401
from .vit import DistributedViT  # noqa: F401
