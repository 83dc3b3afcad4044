"""Caller side of the decode path: a step's metadata from the scheduler's sequences into the buffers
the attention kernels (and the engine's CUDA graphs) read, with one host-to-device copy and one launch.

What it replaces in nano-vllm's model runner, per decode step:

* `ModelRunner.prepare_decode` + `prepare_block_tables` (nanovllm/engine/model_runner.py:163-179, :119-123):
  four Python lists and a list of padded lists, five freshly allocated pinned tensors, five
  host-to-device copies;
* the graph branch of `ModelRunner.run_model` (:193-203): seven device operations that move those
  tensors into the graph's static buffers.

Here the step is packed with numpy into ONE persistent pinned record (layout: include/b200_attn.h,
b200_unpack_decode_metadata), copied once, and scattered into the graph buffers by one kernel.  The
values are the reference's, bit for bit: input_ids = last tokens, positions = len - 1,
context_lens = len, slot = last block id * block_size + tokens in the last block - 1, block-table rows
padded with -1 to the longest row of the step.

`install_into(ModelRunner)` rebinds the two methods; the eager branch (batch > 512, enforce_eager)
keeps the reference's own run_model and reads views of the copied record.
"""
from __future__ import annotations

from itertools import chain

import numpy as np
import torch

from .. import _lib


class DecodeMetadataStager:
    """Two alternating pinned records and device records (a step's copy may still be in flight when the
    next step is packed; the engine's per-step read-back of the sampled tokens bounds the overlap to one)."""

    def __init__(self, max_batch: int, max_blocks: int, block_size: int, device=None):
        self.max_batch, self.max_blocks, self.block_size = int(max_batch), int(max_blocks), int(block_size)
        words = 6 * self.max_batch + self.max_batch * self.max_blocks
        self.device = torch.device(device) if device is not None else None
        pin = self.device is not None and self.device.type == "cuda"
        self._host = [torch.empty(words, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._np = [h.numpy() for h in self._host]
        self._dev = [torch.empty(words, dtype=torch.int32, device=self.device) for _ in range(2)] if pin else [None, None]
        self._turn = 0
        self.batch = 0
        self.width = 0

    # ---- host side (no GPU needed) ---------------------------------------------------------------------
    def pack(self, seqs) -> np.ndarray:
        """Fills the next pinned record from the scheduler's sequences; returns it as int32 words."""
        bs = len(seqs)
        if bs > self.max_batch:
            raise ValueError(f"decode batch {bs} exceeds the stager's capacity {self.max_batch}")
        self._turn ^= 1
        rec = self._np[self._turn]
        tables = [s.block_table for s in seqs]
        nblk = np.fromiter(map(len, tables), dtype=np.int64, count=bs)
        w = int(nblk.max()) if bs else 0
        if w > self.max_blocks:
            raise ValueError(f"block table of {w} blocks exceeds the stager's capacity {self.max_blocks}")
        total = int(nblk.sum())
        flat = np.fromiter(chain.from_iterable(tables), dtype=np.int32, count=total)
        ntok = np.fromiter(map(len, seqs), dtype=np.int64, count=bs)
        ids64 = rec[:2 * bs].view(np.int64)
        pos64 = rec[2 * bs:4 * bs].view(np.int64)
        ids64[:] = np.fromiter((s.last_token for s in seqs), dtype=np.int64, count=bs)
        pos64[:] = ntok - 1
        ends = np.cumsum(nblk)
        # Sequence.last_block_num_tokens (nanovllm/engine/sequence.py:60-62) with num_blocks = ceil(len / block_size)
        last_tokens = ntok - ((ntok + self.block_size - 1) // self.block_size - 1) * self.block_size
        rec[4 * bs:5 * bs] = flat[ends - 1].astype(np.int64) * self.block_size + last_tokens - 1
        rec[5 * bs:6 * bs] = ntok
        bt = rec[6 * bs:6 * bs + bs * w].reshape(bs, w)
        bt.fill(-1)
        rows = np.repeat(np.arange(bs), nblk)
        cols = np.arange(total) - np.repeat(ends - nblk, nblk)
        bt[rows, cols] = flat
        self.batch, self.width = bs, w
        return rec[:6 * bs + bs * w]

    def record_views(self, rec):
        """(input_ids, positions, slot_mapping, context_lens, block_tables) as views of a packed record
        (numpy array or torch tensor of int32 words) of the current batch and width."""
        bs, w = self.batch, self.width
        as64 = (lambda x: x.view(np.int64)) if isinstance(rec, np.ndarray) else (lambda x: x.view(torch.int64))
        return (as64(rec[:2 * bs]), as64(rec[2 * bs:4 * bs]), rec[4 * bs:5 * bs], rec[5 * bs:6 * bs],
                rec[6 * bs:6 * bs + bs * w].reshape(bs, w))

    # ---- device side -----------------------------------------------------------------------------------
    def to_device(self) -> torch.Tensor:
        """One host-to-device copy of the record packed last; returns the device record."""
        n = 6 * self.batch + self.batch * self.width
        dev = self._dev[self._turn]
        dev[:n].copy_(self._host[self._turn][:n], non_blocking=True)
        return dev[:n]

    def unpack_into(self, dev_record, input_ids, positions, slot_mapping, context_lens, block_tables):
        """One launch: the device record into the graph's static buffers, with the reference's effect
        (nanovllm/engine/model_runner.py:196-202)."""
        assert block_tables.stride(1) == 1 and input_ids.dtype == torch.int64 and positions.dtype == torch.int64
        assert slot_mapping.numel() == context_lens.numel() and input_ids.numel() >= self.batch
        lib = _lib.load()
        _lib.check(lib.b200_unpack_decode_metadata(
            dev_record.data_ptr(), self.batch, self.width, slot_mapping.numel(), block_tables.stride(0),
            input_ids.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr(), context_lens.data_ptr(),
            block_tables.data_ptr(), torch.cuda.current_stream().cuda_stream))


def install_into(model_runner_cls, context_module):
    """Rebinds `prepare_decode` and the graph branch of `run_model` of nano-vllm's ModelRunner
    (nanovllm/engine/model_runner.py:163-179, :188-205).  Everything else of the class is untouched."""
    orig_run_model = model_runner_cls.run_model

    def _stager(self):
        st = getattr(self, "_b200_decode_stager", None)
        if st is None:
            cfg = self.config
            max_blocks = (cfg.max_model_len + self.block_size - 1) // self.block_size
            st = DecodeMetadataStager(max(cfg.max_num_seqs, 512), max_blocks, self.block_size, torch.device("cuda"))
            self._b200_decode_stager = st
        return st

    def prepare_decode(self, seqs):
        st = _stager(self)
        st.pack(seqs)
        rec = st.to_device()
        self._b200_decode_record = rec
        input_ids, positions, slot_mapping, context_lens, block_tables = st.record_views(rec)
        context_module.set_context(False, slot_mapping=slot_mapping, context_lens=context_lens, block_tables=block_tables)
        return input_ids, positions

    @torch.inference_mode()
    def run_model(self, input_ids, positions, is_prefill):
        rec = getattr(self, "_b200_decode_record", None)
        if is_prefill or self.enforce_eager or input_ids.size(0) > 512 or rec is None:
            self._b200_decode_record = None
            return orig_run_model(self, input_ids, positions, is_prefill)
        self._b200_decode_record = None
        bs = input_ids.size(0)
        graph = self.graphs[next(x for x in self.graph_bs if x >= bs)]
        gv = self.graph_vars
        _stager(self).unpack_into(rec, gv["input_ids"], gv["positions"], gv["slot_mapping"], gv["context_lens"],
                                  gv["block_tables"])
        graph.replay()
        return self.model.compute_logits(gv["outputs"][:bs])

    model_runner_cls.prepare_decode = prepare_decode
    model_runner_cls.run_model = run_model
    return model_runner_cls
