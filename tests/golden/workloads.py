"""Seeded synthetic workloads of the paged-KV attention path and their algorithmic work.

Input generators only -- no attention arithmetic lives here.  Shared by the golden-case builders, the
parity tests, bench.py and __graft_entry__.smoke(), so that all of them see the same seeded block
tables, slots and lengths.  The shapes are those of BASELINE.json's configurations:

  decode_cfg2          16/8 heads, batch 256, context lengths uniform in [100, 2048]
  decode_cfg4          32/8 heads (Qwen3-8B), batch 512, lengths uniform in [512, 8192]
  prefill_cfg3         256 sequences, lengths uniform in [100, 1024], dense K/V
  prefill_cfg3_prefix  the same batch read through the paged cache, the second half of the
                       sequences with a cached prefix of a random whole number of blocks

Block tables follow the reference's conventions: rows padded with -1
(nanovllm/engine/model_runner.py:119-123), slots as at :146-152 and :172.
"""
from __future__ import annotations

import math

import torch

BLOCK = 256

WORKLOADS = {
    "decode_cfg2": dict(kind="decode", H=16, Hkv=8, D=128, batch=256, lo=100, hi=2048, seed=2, layers=8),
    "decode_cfg4": dict(kind="decode", H=32, Hkv=8, D=128, batch=512, lo=512, hi=8192, seed=4, layers=3),
    "prefill_cfg3": dict(kind="prefill", H=16, Hkv=8, D=128, batch=256, lo=100, hi=1024, seed=3),
    "prefill_cfg3_prefix": dict(kind="prefill", H=16, Hkv=8, D=128, batch=256, lo=100, hi=1024, seed=3, prefix=True),
    # the producer side of the layer (QK-norm + rotary embedding + cache store as one kernel) on the
    # engine's largest prefill batch and on a decode batch; steps rotate over projection buffers larger than L2
    "producer_prefill": dict(kind="producer", H=16, Hkv=8, D=128, tokens=16384, seed=5, buffers=4),
    "producer_decode": dict(kind="producer", H=16, Hkv=8, D=128, tokens=256, seed=6, buffers=64),
}


def seeded_lens(w):
    """Sequence lengths of a workload and the generator, positioned for what is drawn next."""
    g = torch.Generator().manual_seed(w["seed"])
    return torch.randint(w["lo"], w["hi"] + 1, (w["batch"],), generator=g, dtype=torch.int32), g


def cached_prefixes(lens, generator):
    """prefill_cfg3_prefix: no prefix on the first half of the batch, a random whole number of blocks
    (leaving at least one query token) on the second half."""
    n = len(lens)
    prefix = torch.zeros(n, dtype=torch.int32)
    for i in range(n // 2, n):
        mxb = (int(lens[i]) - 1) // BLOCK
        prefix[i] = BLOCK * int(torch.randint(0, mxb + 1, (1,), generator=generator)) if mxb > 0 else 0
    return prefix


def cu_seqlens(lens):
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.as_tensor(lens).to(torch.int64).cumsum(0)
    return cu

# ----------------------------------------------------------------------------------------------
# Algorithmic work (the numbers roofline fractions are computed from)
# ----------------------------------------------------------------------------------------------

def decode_algorithmic_bytes(context_lens, num_heads, num_kv_heads, head_dim, elem_bytes=2):
    """K and V of every context token once, plus q read and o written."""
    total = int(torch.as_tensor(context_lens).to(torch.int64).sum())
    b = len(context_lens)
    return total * num_kv_heads * head_dim * 2 * elem_bytes + 2 * b * num_heads * head_dim * elem_bytes


def prefill_algorithmic_flops(lens_q, lens_k, num_heads, head_dim):
    """4*D flops per visible (query, key) pair per head (2*D for QK^T and 2*D for PV)."""
    pairs = 0
    for lq, lk in zip(lens_q, lens_k):
        lq, lk = int(lq), int(lk)
        pairs += lq * (lk - lq) + lq * (lq + 1) // 2
    return 4 * head_dim * num_heads * pairs


# ----------------------------------------------------------------------------------------------
# Block tables and slots
# ----------------------------------------------------------------------------------------------

def make_block_tables(lens, block_size, generator, slack=8, num_blocks=None):
    """Scattered block tables: a seeded random permutation of block ids, rows padded with -1
    (nanovllm/engine/model_runner.py:119-123)."""
    lens = [int(x) for x in lens]
    nblk = [(n + block_size - 1) // block_size for n in lens]
    total = sum(nblk)
    nb = num_blocks if num_blocks is not None else total + slack
    assert nb >= total
    perm = torch.randperm(nb, generator=generator)[:total].to(torch.int32)
    width = max(max(nblk), 1)
    bt = torch.full((len(lens), width), -1, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblk):
        bt[i, :n] = perm[o:o + n]
        o += n
    return bt, nb


def decode_slots(lens, block_tables, block_size):
    """Slot of the token appended this step (nanovllm/engine/model_runner.py:172)."""
    out = []
    for i, n in enumerate(lens):
        n = int(n)
        out.append(int(block_tables[i, (n - 1) // block_size]) * block_size + (n - 1) % block_size)
    return torch.tensor(out, dtype=torch.int32)


def prefill_slots(lens_k, prefix, block_tables, block_size):
    """Slots of the uncached tokens of every sequence (nanovllm/engine/model_runner.py:146-152)."""
    out = []
    for i, (lk, p) in enumerate(zip(lens_k, prefix)):
        for t in range(int(p), int(lk)):
            out.append(int(block_tables[i, t // block_size]) * block_size + t % block_size)
    return torch.tensor(out, dtype=torch.int32)


def rope_table(head_dim: int, max_position: int, base: float) -> torch.Tensor:
    """The (max_position, 1, head_dim) fp32 cos | sin table the reference's RotaryEmbedding holds
    (nanovllm/layers/rotary_embedding.py:27-34); an input of the producer workloads."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_position, dtype=torch.float), inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).unsqueeze_(1)


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
