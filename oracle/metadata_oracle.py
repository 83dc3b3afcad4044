"""CPU restatement of how nano-vllm's model runner prepares a decode step (TEST INFRASTRUCTURE ONLY; only
tests/ may import it).

Restated, with the reference lines each function follows (paths relative to the nano-vllm project):

* prepare_block_tables      nanovllm/engine/model_runner.py:119-123   rows padded with -1 to the longest
* prepare_decode            nanovllm/engine/model_runner.py:163-179   last token, len - 1, len,
                                                                      last block id * block_size + last_block_num_tokens - 1
* the graph-buffer update   nanovllm/engine/model_runner.py:196-202   ids/positions rows [0, bs); slot_mapping
                                                                      filled with -1, context_lens zeroed, then rows
                                                                      [0, bs); block_tables[:bs, :width]

The reference builds the tensors with pin_memory=True and copies them to the GPU; here they stay on the CPU.
Pinning: the reference has no tests for this code.  The restatement is pinned in tests/test_decode_metadata.py
against the reference's own Scheduler, BlockManager and Sequence classes (imported from an install of the
reference when present) driving a seeded request trace: the values asserted there are read off those objects
with the reference's own accessors (`seq.last_token`, `len(seq)`, `seq.block_table`, `seq.last_block_num_tokens`).
"""
from __future__ import annotations

import torch


def prepare_block_tables_ref(seqs):
    max_len = max(len(seq.block_table) for seq in seqs)
    rows = [seq.block_table + [-1] * (max_len - len(seq.block_table)) for seq in seqs]
    return torch.tensor(rows, dtype=torch.int32)


def prepare_decode_ref(seqs, block_size):
    input_ids, positions, slot_mapping, context_lens = [], [], [], []
    for seq in seqs:
        input_ids.append(seq.last_token)
        positions.append(len(seq) - 1)
        context_lens.append(len(seq))
        slot_mapping.append(seq.block_table[-1] * block_size + seq.last_block_num_tokens - 1)
    return (torch.tensor(input_ids, dtype=torch.int64), torch.tensor(positions, dtype=torch.int64),
            torch.tensor(slot_mapping, dtype=torch.int32), torch.tensor(context_lens, dtype=torch.int32),
            prepare_block_tables_ref(seqs))


def update_graph_buffers_ref(graph_vars, input_ids, positions, slot_mapping, context_lens, block_tables):
    """In place, on tensors shaped like the reference's graph_vars."""
    bs = input_ids.size(0)
    graph_vars["input_ids"][:bs] = input_ids
    graph_vars["positions"][:bs] = positions
    graph_vars["slot_mapping"].fill_(-1)
    graph_vars["slot_mapping"][:bs] = slot_mapping
    graph_vars["context_lens"].zero_()
    graph_vars["context_lens"][:bs] = context_lens
    graph_vars["block_tables"][:bs, :block_tables.size(1)] = block_tables
