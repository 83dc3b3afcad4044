"""CPU/torch restatement of the sum all-reduce behind nano-vllm's row-parallel projection (TEST INFRASTRUCTURE
ONLY; only tests/ may import it).

Reference call site: `dist.all_reduce(y)` in RowParallelLinear.forward, nanovllm/layers/linear.py:149-153 (default
op: SUM over the tensor-parallel ranks, in place, every rank ends with the same tensor).  The reference delegates
the arithmetic to NCCL, whose order of additions and intermediate precision are not specified; this restatement
fixes them the way the kernel under test does -- fp32 accumulation in rank order, one rounding to the input dtype --
so that the comparison can be bit-exact, and the tests additionally compare with NCCL itself within bf16 tolerance.
Pinning: the reference has no test for this call; "parity unpinned" at the reference-test level.
"""
from __future__ import annotations

import torch


def all_reduce_sum_ref(per_rank):
    """per_rank: list of same-shaped tensors, index = rank.  Returns what every rank holds afterwards."""
    acc = torch.zeros_like(per_rank[0], dtype=torch.float32)
    for x in per_rank:
        acc = acc + x.float()
    return acc.to(per_rank[0].dtype)
