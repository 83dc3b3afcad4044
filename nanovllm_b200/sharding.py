"""Tensor-parallel partition of the attention path: by KV head, no exchange step.

The reference shards q heads and KV heads across ranks (nanovllm/models/qwen3.py:29-38) and
gives each rank a cache holding only its own KV heads (nanovllm/engine/model_runner.py:107-111);
every rank receives identical slot_mapping / context_lens / block_tables.  Attention therefore
needs no collective: rank r owns KV heads [r * Hkv / tp, (r + 1) * Hkv / tp) and the G = H / Hkv
query heads of each.  The o_proj all-reduce that follows stays NCCL and is outside this path.
"""
from __future__ import annotations


def local_heads(num_heads: int, num_kv_heads: int, tp_size: int):
    """(local q heads, local kv heads) on every rank, with the reference's divisibility rule
    (nanovllm/models/qwen3.py:31-35)."""
    if tp_size <= 0 or num_kv_heads % tp_size or num_heads % tp_size:
        raise ValueError(f"heads ({num_heads}, {num_kv_heads}) are not divisible by tp_size {tp_size}")
    return num_heads // tp_size, num_kv_heads // tp_size


def head_slices(num_heads: int, num_kv_heads: int, tp_size: int, rank: int):
    """(slice of q heads, slice of kv heads) owned by `rank`."""
    if not 0 <= rank < tp_size:
        raise ValueError(f"rank {rank} outside [0, {tp_size})")
    h, hkv = local_heads(num_heads, num_kv_heads, tp_size)
    return slice(rank * h, (rank + 1) * h), slice(rank * hkv, (rank + 1) * hkv)


def shard_heads(x, head_slice, head_dim_index: int):
    """The rank's heads of an activation or cache, contiguous like the rank's own allocation."""
    idx = [slice(None)] * x.dim()
    idx[head_dim_index] = head_slice
    return x[tuple(idx)].contiguous()
