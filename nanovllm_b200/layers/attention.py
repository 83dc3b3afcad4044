"""Drop-in replacement for nano-vllm's attention layer (nanovllm/layers/attention.py).

Same surface as the reference: `store_kvcache(key, value, k_cache, v_cache, slot_mapping)` and
`Attention(num_heads, head_dim, scale, num_kv_heads).forward(q, k, v)`, the per-step metadata
read from `get_context()` (nanovllm/utils/context.py), the cache bound by the model runner onto
`k_cache` / `v_cache` with layout (num_blocks, block_size, num_kv_heads, head_dim)
(nanovllm/engine/model_runner.py:107-117).  The arithmetic runs in hand-written sm_100a CUDA
behind the C ABI of include/b200_attn.h; there is no Triton, no flash_attn and no fallback.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _lib
from ..utils import context as _own_context

# The function the layer reads its metadata from.  nanovllm_b200.integration rebinds it to the
# reference engine's get_context when the layer is installed into nano-vllm.
_context_getter = _own_context.get_context

_DECODE_WS_BATCH = 512  # the library splits larger batches into launches of at most this many


def get_context():
    return _context_getter()


def set_context_getter(fn):
    global _context_getter
    _context_getter = fn


def _stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("nanovllm_b200 kernels take CUDA tensors only (there is no CPU path)")


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor):
    """Same contract and asserts as the reference wrapper (nanovllm/layers/attention.py:33-40)."""
    n, num_heads, head_dim = key.shape
    d = num_heads * head_dim
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == d and v_cache.stride(1) == d
    assert slot_mapping.numel() == n
    assert key.dtype == value.dtype == k_cache.dtype == v_cache.dtype
    assert slot_mapping.dtype == torch.int32
    _require_cuda(key, value, k_cache, v_cache, slot_mapping)
    if n == 0:
        return
    lib = _lib.load()
    _lib.check(lib.b200_store_kvcache(
        key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        slot_mapping.data_ptr(), n, d, key.element_size(), k_cache.numel() // d, _stream_ptr()))


_workspaces: dict = {}


def _decode_workspace(device, num_heads, num_kv_heads, head_dim):
    """One zero-initialised workspace per (device, query heads per kv head); layers run back to back
    on a stream and share it.  Allocated on first use (the engine's eager warm-up precedes graph
    capture)."""
    key = (device.index, num_heads // num_kv_heads)
    ws = _workspaces.get(key)
    if ws is None:
        lib = _lib.load()
        nbytes = lib.b200_decode_workspace_bytes(_DECODE_WS_BATCH, num_heads, num_kv_heads, head_dim)
        if nbytes < 0:
            _lib.check(int(nbytes))
        ws = torch.zeros(int(nbytes), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def decode_attention(q, k_cache, v_cache, context_lens, block_tables, scale, num_kv_heads):
    """q (B, H, D) -> (B, 1, H, D), the shape flash_attn_with_kvcache returns for the reference's
    call (nanovllm/layers/attention.py:72-74)."""
    b, h, d = q.shape
    _require_cuda(q, k_cache, v_cache, context_lens, block_tables)
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and q.stride(1) == d
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert context_lens.dtype == torch.int32 and block_tables.dtype == torch.int32
    assert block_tables.stride(1) == 1 and context_lens.stride(0) == 1
    out = torch.empty(b, 1, h, d, dtype=q.dtype, device=q.device)
    if b == 0:
        return out
    ws = _decode_workspace(q.device, h, num_kv_heads, d)
    lib = _lib.load()
    _lib.check(lib.b200_decode_attn(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0], k_cache.shape[1],
        block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1], context_lens.data_ptr(),
        out.data_ptr(), ws.data_ptr(), ws.numel(), b, h, num_kv_heads, d, float(scale), _stream_ptr()))
    return out


def prefill_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale, num_kv_heads,
                      block_tables=None, kernel_variant=0):
    """Varlen causal attention.  With block_tables, k and v are the paged caches
    (nanovllm/layers/attention.py:65-70); otherwise packed (total_k, Hkv, D) activations."""
    tq, h, d = q.shape
    _require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, block_tables)
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and q.stride(1) == d
    assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
    out = torch.empty(tq, h, d, dtype=q.dtype, device=q.device)
    batch = cu_seqlens_q.numel() - 1
    if tq == 0 or batch <= 0:
        return out
    lib = _lib.load()
    if block_tables is not None:
        assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1
        assert k.is_contiguous() and v.is_contiguous() and k.dim() == 4
        rc = lib.b200_prefill_attn(
            q.data_ptr(), q.stride(0), None, None, 0, 0, 0, k.data_ptr(), v.data_ptr(), k.shape[0], k.shape[1],
            block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1], cu_seqlens_q.data_ptr(),
            cu_seqlens_k.data_ptr(), batch, tq, int(max_seqlen_q), int(max_seqlen_k), out.data_ptr(), h,
            num_kv_heads, d, float(scale), kernel_variant, _stream_ptr())
    else:
        assert k.stride(-1) == 1 and v.stride(-1) == 1 and k.stride(1) == d and v.stride(1) == d
        rc = lib.b200_prefill_attn(
            q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), k.shape[0], None, None,
            0, 0, None, 0, 0, cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), batch, tq, int(max_seqlen_q),
            int(max_seqlen_k), out.data_ptr(), h, num_kv_heads, d, float(scale), kernel_variant, _stream_ptr())
    _lib.check(rc)
    return out


class Attention(nn.Module):
    """Constructor, attributes and forward of the reference module
    (nanovllm/layers/attention.py:43-75); the model runner finds the layer through its
    `k_cache` / `v_cache` attributes (nanovllm/engine/model_runner.py:113-117)."""

    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, already_stored: bool = False):
        """`already_stored` is not part of the reference's signature: the fused producer kernel
        (layers/qk_norm_rope.py) has written k and v to the cache and passes True."""
        context = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if not already_stored and k_cache.numel() and v_cache.numel():
            store_kvcache(k, v, k_cache, v_cache, context.slot_mapping)
        if context.is_prefill:
            if context.block_tables is not None:    # prefix cache: keys and values come from the cache
                k, v = k_cache, v_cache
            return prefill_attention(q, k, v, context.cu_seqlens_q, context.cu_seqlens_k, context.max_seqlen_q,
                                     context.max_seqlen_k, self.scale, self.num_kv_heads, context.block_tables)
        return decode_attention(q, k_cache, v_cache, context.context_lens, context.block_tables, self.scale,
                                self.num_kv_heads)
