"""Several host tensors as ONE pinned record and ONE host-to-device copy.

A decode step hands the attention layer three activations and three pieces of metadata; copied one by one
(as nanovllm/engine/model_runner.py:163-179 does with freshly pinned tensors) the per-copy latency dominates a
step of a fraction of a millisecond.  `PackedBuffers` lays the tensors out back to back (16-byte aligned) in one
persistent pinned buffer with a device twin; `upload()` is a single copy, and `host[name]` / `dev[name]` are views
with the requested shapes and dtypes.
"""
from __future__ import annotations

import torch


class PackedBuffers:
    def __init__(self, spec: dict, device):
        """spec: name -> (shape, dtype)."""
        self.device = torch.device(device)
        offsets, off = {}, 0
        for name, (shape, dtype) in spec.items():
            n = 1
            for s in shape:
                n *= int(s)
            nbytes = n * torch.empty(0, dtype=dtype).element_size()
            offsets[name] = (off, nbytes, tuple(int(s) for s in shape), dtype)
            off = (off + nbytes + 15) // 16 * 16
        self.nbytes = off
        pin = self.device.type == "cuda"
        self._host = torch.empty(off, dtype=torch.uint8, pin_memory=pin)
        self._dev = torch.empty(off, dtype=torch.uint8, device=self.device)
        view = lambda buf, o, nb, shape, dtype: buf[o:o + nb].view(dtype).view(shape)
        self.host = {k: view(self._host, *v) for k, v in offsets.items()}
        self.dev = {k: view(self._dev, *v) for k, v in offsets.items()}

    def upload(self):
        """One asynchronous copy of the whole record on the current stream."""
        self._dev.copy_(self._host, non_blocking=True)
        return self.dev
