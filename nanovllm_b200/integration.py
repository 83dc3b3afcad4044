"""Installs the B200 attention layer into an importable nano-vllm, in place of
nanovllm/layers/attention.py's `Attention` and `store_kvcache`.

    import nanovllm_b200.integration as integ
    integ.install()            # before constructing nanovllm.LLM
    from nanovllm import LLM

After install(), `nanovllm.models.qwen3.Qwen3Attention` builds this package's Attention
(nanovllm/models/qwen3.py:60-65), the model runner binds the cache onto it
(nanovllm/engine/model_runner.py:113-117) and the layer reads the engine's own per-step record
(nanovllm/utils/context.py).  Tensor-parallel ranks are spawned processes that re-import
everything: see `nanovllm_b200.autoinstall` (environment variable B200_ATTN_INSTALL) for installing
the layer in them as well.
"""
from __future__ import annotations

import importlib
import sys


def install(fuse_qk_norm_rope: bool = False, fast_decode_metadata: bool = False, small_allreduce: bool = False):
    """fuse_qk_norm_rope=True additionally replaces the body of `Qwen3Attention.forward`
    (nanovllm/models/qwen3.py:68-82) by one that runs q_norm, k_norm, rotary_emb and the cache store as a
    single kernel (layers/qk_norm_rope.py); nano-vllm's model module is imported for that.
    fast_decode_metadata=True rebinds `ModelRunner.prepare_decode` and the graph branch of `ModelRunner.run_model`
    (nanovllm/engine/model_runner.py:163-179, :188-205) to the packed one-copy, one-launch form of
    engine/decode_metadata.py.
    small_allreduce=True rebinds `RowParallelLinear.forward` (nanovllm/layers/linear.py:149-153) so that bf16 messages
    of at most 512 KiB are summed by the one-shot peer-memory kernel of engine/small_allreduce.py instead of NCCL."""
    from .layers import attention as ours
    ref_attn = sys.modules.get("nanovllm.layers.attention")
    if ref_attn is None:
        # Register this package's module under the reference's name BEFORE nano-vllm is imported,
        # so that its own attention file (and with it Triton and flash_attn) is never executed.
        sys.modules["nanovllm.layers.attention"] = ours
    elif ref_attn is not ours:
        ref_attn.Attention = ours.Attention
        ref_attn.store_kvcache = ours.store_kvcache
    ref_ctx = importlib.import_module("nanovllm.utils.context")
    ours.set_context_getter(ref_ctx.get_context)
    layers_pkg = importlib.import_module("nanovllm.layers")
    if sys.modules["nanovllm.layers.attention"] is ours:
        setattr(layers_pkg, "attention", ours)
    qwen3 = sys.modules.get("nanovllm.models.qwen3")
    if qwen3 is not None:
        qwen3.Attention = ours.Attention
    if fuse_qk_norm_rope:
        from .layers.qk_norm_rope import fused_attention_forward
        qwen3 = importlib.import_module("nanovllm.models.qwen3")
        qwen3.Qwen3Attention.forward = fused_attention_forward
    if fast_decode_metadata:
        from .engine.decode_metadata import install_into
        runner = importlib.import_module("nanovllm.engine.model_runner")
        install_into(runner.ModelRunner, ref_ctx)
    if small_allreduce:
        from .engine.small_allreduce import install_into as install_allreduce
        install_allreduce(importlib.import_module("nanovllm.layers.linear"))
    return ours
