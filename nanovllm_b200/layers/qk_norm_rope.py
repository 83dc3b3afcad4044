"""Producer side of the attention layer as one CUDA launch: per-head RMSNorm of q and k, rotary
embedding, and the cache store -- the work nano-vllm does between its fused qkv projection and its
attention call (nanovllm/models/qwen3.py:75-79 plus the store at nanovllm/layers/attention.py:62-63).

`qk_norm_rope_store` is the operator; `fused_attention_forward` is a drop-in body for
`Qwen3Attention.forward` (nanovllm/models/qwen3.py:68-82) that uses it and then calls this package's
attention with the store already done.  Everything runs through libb200attn's C ABI; there is no
fallback.
"""
from __future__ import annotations

import torch

from .. import _lib
from . import attention as _attn


def qk_norm_rope_store(qkv: torch.Tensor, positions: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                       cos_sin_cache: torch.Tensor, eps: float, num_heads: int, num_kv_heads: int,
                       k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
                       slot_mapping: torch.Tensor | None = None):
    """qkv (N, (H + 2 Hkv) * 128) bf16 -> (q (N, H, 128), k (N, Hkv, 128), v view (N, Hkv, 128)).
    q and k are normalised and rotated exactly in the reference's order of operations; with caches
    given, k and v of token i are also written to flat cache row slot_mapping[i] (-1: skipped)."""
    _attn._require_cuda(qkv, positions, q_weight, k_weight, cos_sin_cache)
    head_dim = 128
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    assert qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1, "qkv must be (N, (H + 2 Hkv) * 128), rows contiguous"
    assert qkv.dtype == torch.bfloat16 and q_weight.dtype == torch.bfloat16 and k_weight.dtype == torch.bfloat16
    assert cos_sin_cache.dtype == torch.float32 and cos_sin_cache.is_contiguous() and cos_sin_cache.shape[-1] == head_dim
    assert positions.dtype == torch.int64 and positions.numel() == n and positions.is_contiguous()
    assert q_weight.numel() == head_dim and k_weight.numel() == head_dim
    q = torch.empty(n, num_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(n, num_kv_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    v = qkv[:, (num_heads + num_kv_heads) * head_dim:].view(n, num_kv_heads, head_dim)
    have_cache = k_cache is not None and v_cache is not None and k_cache.numel() and v_cache.numel()
    n_slots = 0
    if have_cache:
        row = num_kv_heads * head_dim
        assert k_cache.stride(-1) == 1 and k_cache.stride(-2) == head_dim and k_cache.stride(1) == row
        assert v_cache.stride(-1) == 1 and v_cache.stride(-2) == head_dim and v_cache.stride(1) == row
        assert slot_mapping is not None and slot_mapping.numel() == n and slot_mapping.dtype == torch.int32
        n_slots = k_cache.numel() // row
    lib = _lib.load()
    _lib.check(lib.b200_qk_norm_rope_store(
        qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(),
        cos_sin_cache.data_ptr(), cos_sin_cache.shape[0], float(eps), q.data_ptr(), k.data_ptr(),
        k_cache.data_ptr() if have_cache else None, v_cache.data_ptr() if have_cache else None,
        slot_mapping.data_ptr() if have_cache else None, n_slots, n, num_heads, num_kv_heads, head_dim,
        _attn._stream_ptr()))
    return q, k, v


def fused_attention_forward(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
    """Body for `Qwen3Attention.forward` (nanovllm/models/qwen3.py:68-82): same inputs, same output,
    with q_norm, k_norm, rotary_emb and the cache store done by one kernel."""
    qkv = self.qkv_proj(hidden_states)
    attn = self.attn
    context = _attn.get_context()
    q, k, v = qk_norm_rope_store(qkv, positions, self.q_norm.weight, self.k_norm.weight,
                                 self.rotary_emb.cos_sin_cache, self.q_norm.eps, self.num_heads, self.num_kv_heads,
                                 attn.k_cache, attn.v_cache, context.slot_mapping)
    o = attn.forward(q, k, v, already_stored=True)
    return self.o_proj(o.flatten(1, -1))
