"""Installs the B200 attention layer at import time when the environment asks for it.

nano-vllm starts its tensor-parallel ranks as spawned processes (nanovllm/engine/llm_engine.py:24-28):
each re-imports everything, so an `integration.install()` made in the parent is not inherited.  Importing
this module in every process closes that gap:

    B200_ATTN_INSTALL=1        install the attention layer
    B200_ATTN_INSTALL=fused    also replace Qwen3Attention.forward by the fused producer
                               (QK-norm + RoPE + cache store in one kernel)
    B200_ATTN_INSTALL=full     also rebind the model runner's decode metadata preparation
                               (one packed host-to-device copy and one launch per step)
    B200_ATTN_INSTALL=full+ar  also the one-shot all-reduce for decode-sized messages after the output projection

Two ways to get it imported in the children: import it at the top of the script that creates the `LLM`
(spawn re-imports that script's module in every child), or put a one-line `.pth` file into site-packages,

    import nanovllm_b200.autoinstall

which Python executes at interpreter start.  With the variable unset the import does nothing.
"""
import os

_mode = os.environ.get("B200_ATTN_INSTALL", "")
installed = False
if _mode and _mode != "0":
    from . import integration as _integration
    _integration.install(fuse_qk_norm_rope=_mode in ("fused", "full", "full+ar"), fast_decode_metadata=_mode in ("full", "full+ar"),
                         small_allreduce=(_mode == "full+ar"))
    installed = True
