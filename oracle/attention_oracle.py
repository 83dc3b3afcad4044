"""CPU restatement of nano-vllm's paged-KV attention path (TEST INFRASTRUCTURE ONLY).

This file is the checker, never the product: only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs may import it.  The product path (nanovllm_b200) calls
hand-written CUDA through a C-ABI library and fails loudly when that library is missing.

What is restated, and from where (paths are relative to the nano-vllm project root):

* store_kvcache            nanovllm/layers/attention.py:10-40  (Triton kernel + wrapper)
* Attention.forward        nanovllm/layers/attention.py:59-75  (dispatch store -> prefill | decode)
* cache layout             nanovllm/engine/model_runner.py:107-117
* -1 padded block tables   nanovllm/engine/model_runner.py:119-123
* slot / cu_seqlens rules  nanovllm/engine/model_runner.py:125-179

The attention arithmetic itself lives in the third-party `flash-attn` package, which the
reference declares un-pinned (pyproject.toml:18; 2.8.3 is installed in this image) and whose
source is not part of the reference tree.  Its published algorithm is restated here:
S = scale * q @ k^T in fp32, GQA mapping q head h -> kv head h // (H / Hkv), causal mask
aligned to the bottom-right corner (query row r of a sequence with Lq queries and Lk keys sees
keys 0 .. Lk - Lq + r), softmax in fp32, O = P @ V in fp32, cast to the input dtype; rows with
no visible key produce zeros; the paged cache has shape (num_blocks, block_size, Hkv, D) and
token t of sequence i lives in block block_tables[i, t // block_size] at offset t % block_size.

Pinning: the reference ships no tests or golden vectors for this path, so nothing of its own
pins it ("parity unpinned" at the reference-test level).  The oracle is instead pinned against
outputs of the reference module itself (flash_attn + Triton, executed on a B200) committed under
tests/golden/ together with the script that produced them (tests/golden/make_golden.py).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Context:
    """Field-for-field copy of nanovllm/utils/context.py:5-14."""
    is_prefill: bool = False
    cu_seqlens_q: torch.Tensor | None = None
    cu_seqlens_k: torch.Tensor | None = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: torch.Tensor | None = None
    context_lens: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None


def store_kvcache_ref(key, value, k_cache, v_cache, slot_mapping):
    """nanovllm/layers/attention.py:21-30: for token i, slot = slot_mapping[i]; -1 is skipped;
    otherwise row i of key/value (Hkv*D elements) is copied to flat cache row `slot`.
    Mutates k_cache / v_cache in place (pure bit copy, any dtype)."""
    n, hkv, d = key.shape
    row = hkv * d
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == d and value.stride(1) == d
    assert k_cache.stride(1) == row and v_cache.stride(1) == row
    assert slot_mapping.numel() == n
    kc = k_cache.view(-1, row)
    vc = v_cache.view(-1, row)
    slots = slot_mapping.to(torch.int64)
    # Later tokens win on duplicate slots in a sequential restatement; the reference's
    # parallel kernel leaves duplicates unordered (only the all-zero capture pass has them).
    for i in range(n):
        s = int(slots[i])
        if s == -1:
            continue
        kc[s] = key[i].reshape(row)
        vc[s] = value[i].reshape(row)


def _gather_paged(cache, block_table_row, length, block_size):
    """Tokens 0..length-1 of one sequence from a (NB, block_size, Hkv, D) cache."""
    nblk = (length + block_size - 1) // block_size
    idx = block_table_row[:nblk].to(torch.int64)
    return cache[idx].reshape(nblk * block_size, cache.shape[2], cache.shape[3])[:length]


def _attend(q, k, v, scale, causal_offset):
    """q (Lq,H,D), k/v (Lk,Hkv,D) -> (Lq,H,D) fp32.  Query row r sees keys <= r + causal_offset.
    The G = H / Hkv query heads of a kv head are a separate axis, so K and V are never replicated."""
    lq, h, d = q.shape
    lk, hkv, _ = k.shape
    g = h // hkv
    qf = q.float().view(lq, hkv, g, d)
    kf = k.float()
    vf = v.float()
    s = torch.einsum("qhgd,khd->hgqk", qf, kf) * scale
    rows = torch.arange(lq).unsqueeze(1) + causal_offset
    cols = torch.arange(lk).unsqueeze(0)
    mask = cols > rows
    if bool(mask.any()):
        s = s.masked_fill(mask.view(1, 1, lq, lk), float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    p = torch.where(l > 0, p / l.clamp_min(1e-38), torch.zeros_like(p))
    return torch.einsum("hgqk,khd->qhgd", p, vf).reshape(lq, h, d)


def decode_attn_ref(q, k_cache, v_cache, context_lens, block_tables, scale):
    """Single-token paged decode (nanovllm/layers/attention.py:71-74 ->
    flash_attn_with_kvcache).  q (B,H,D) -> (B,1,H,D) in q.dtype; context_lens[i] == 0 gives zeros."""
    b, h, d = q.shape
    bs = k_cache.shape[1]
    out = torch.zeros(b, 1, h, d, dtype=torch.float32)
    for i in range(b):
        n = int(context_lens[i])
        if n <= 0:
            continue
        k = _gather_paged(k_cache, block_tables[i], n, bs)
        v = _gather_paged(v_cache, block_tables[i], n, bs)
        out[i, 0] = _attend(q[i:i + 1], k, v, scale, n - 1)[0]
    return out.to(q.dtype)


def prefill_attn_ref(q, k, v, cu_seqlens_q, cu_seqlens_k, scale, block_tables=None):
    """Varlen causal prefill (nanovllm/layers/attention.py:64-70 -> flash_attn_varlen_func).
    block_tables is None: k, v are packed (total_k, Hkv, D).  Otherwise k, v are the paged
    caches (NB, block_size, Hkv, D) and keys 0..Lk-1 of sequence i come through block_tables[i].
    Causal mask is bottom-right aligned (Lq may be smaller than Lk with a cached prefix)."""
    tq, h, d = q.shape
    nseq = cu_seqlens_q.numel() - 1
    out = torch.zeros(tq, h, d, dtype=torch.float32)
    for i in range(nseq):
        q0, q1 = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        k0, k1 = int(cu_seqlens_k[i]), int(cu_seqlens_k[i + 1])
        lq, lk = q1 - q0, k1 - k0
        if lq == 0:
            continue
        if block_tables is None:
            ki, vi = k[k0:k1], v[k0:k1]
        else:
            bs = k.shape[1]
            ki = _gather_paged(k, block_tables[i], lk, bs)
            vi = _gather_paged(v, block_tables[i], lk, bs)
        out[q0:q1] = _attend(q[q0:q1], ki, vi, scale, lk - lq)
    return out.to(q.dtype)


class AttentionRef:
    """Restatement of the reference module's dispatch (nanovllm/layers/attention.py:43-75)."""

    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])

    def forward(self, q, k, v, context: Context):
        k_cache, v_cache = self.k_cache, self.v_cache
        if k_cache.numel() and v_cache.numel():
            store_kvcache_ref(k, v, k_cache, v_cache, context.slot_mapping)
        if context.is_prefill:
            if context.block_tables is not None:
                k, v = k_cache, v_cache
            return prefill_attn_ref(q, k, v, context.cu_seqlens_q, context.cu_seqlens_k,
                                    self.scale, context.block_tables)
        return decode_attn_ref(q, k_cache, v_cache, context.context_lens,
                               context.block_tables, self.scale)
