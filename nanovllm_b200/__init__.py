"""B200-native (sm_100a) paged-KV attention path for nano-vllm.

Public surface mirrors the reference's attention layer:

    from nanovllm_b200 import Attention, store_kvcache
    from nanovllm_b200.utils.context import set_context, get_context, reset_context

and `nanovllm_b200.integration.install()` swaps the layer into an importable nano-vllm.
The kernels live in libb200attn.so (C ABI: include/b200_attn.h), built by nanovllm_b200.build.
"""
from .layers.attention import (Attention, decode_attention, prefill_attention,  # noqa: F401
                               store_kvcache)

__all__ = ["Attention", "store_kvcache", "decode_attention", "prefill_attention"]
