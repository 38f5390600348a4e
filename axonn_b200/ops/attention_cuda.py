"""Bindings of the flash-attention kernels (``csrc/flash_attn.cu``)."""

from . import _lib


def available():
    return hasattr(_lib.lib(), "axb_flash_attn_fwd")


def flash_attention_packed_cuda(qkv, causal, scale):
    raise NotImplementedError
