"""The all-reduce behind the attention layer's output projection, for decode-sized messages.

nano-vllm's `RowParallelLinear.forward` ends in `dist.all_reduce(y)` (nanovllm/layers/linear.py:149-153): NCCL, 56
times per decode step of a 28-layer model, on messages of at most batch x hidden x 2 bytes.  At those sizes a
collective is pure latency.  `SmallAllReduce` does the sum in one kernel over plain peer loads and stores
(b200_small_allreduce in include/b200_attn.h): every rank owns an exchange buffer that all ranks of the node have
mapped through CUDA IPC.  Messages above the limit, non-bf16 or non-contiguous tensors go to `dist.all_reduce`
as before.

`install_into(linear_module)` rebinds `RowParallelLinear.forward`; the buffers are set up on the first small
message (a collective step: every rank reaches it at the same point, during the engine's eager warm-up before it
captures its CUDA graphs).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _lib


class SmallAllReduce:
    instances: list = []       # every communicator of this process (diagnostics: their status after a run)

    def __init__(self, group=None, wait_limit_seconds: float = 1.0):
        """Collective: every rank of `group` (default: the world) must construct it at the same point.
        All ranks must be processes on one node, one GPU each, current device already set."""
        lib = _lib.load()
        self.lib = lib
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.wait_limit = float(wait_limit_seconds)
        self.max_bytes = int(lib.b200_small_allreduce_max_bytes())
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.buffer = torch.zeros(int(lib.b200_small_allreduce_buffer_bytes()), dtype=torch.uint8, device=dev)
        self.state = torch.zeros(int(lib.b200_small_allreduce_state_bytes()), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize(dev)
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_int64(0)
        _lib.check(lib.b200_ipc_export(self.buffer.data_ptr(), handle, ctypes.byref(offset)))
        mine = (bytes(handle.raw), int(offset.value))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        ptrs = (ctypes.c_void_p * self.world)()
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                ptrs[r] = self.buffer.data_ptr()
                continue
            out = ctypes.c_void_p(0)
            _lib.check(lib.b200_ipc_open(ctypes.create_string_buffer(h, 64), off, ctypes.byref(out)))
            ptrs[r] = out.value
        self._ptrs = ptrs          # host array handed to every call (the library copies it into the launch)
        dist.barrier(group=group)  # nobody signals into a buffer that is not mapped and zeroed yet
        self.calls = 0
        SmallAllReduce.instances.append(self)

    def usable(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() % 8 == 0
                and 0 < t.numel() * 2 <= self.max_bytes and t.data_ptr() % 16 == 0)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """In place: t <- sum over ranks (fp32 accumulation in rank order, one rounding to bf16)."""
        _lib.check(self.lib.b200_small_allreduce(self._ptrs, self.rank, self.world, self.state.data_ptr(), t.data_ptr(),
                                                 t.numel(), self.wait_limit, torch.cuda.current_stream().cuda_stream))
        self.calls += 1
        return t

    def status(self) -> int:
        """0, or the library's timeout code if a rank's peers did not arrive within the wait limit."""
        return int(self.lib.b200_small_allreduce_status(self.state.data_ptr()))

    def reset(self):
        """Collective: after a timeout every rank zeroes its flags, epochs and status together."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.buffer.zero_()
        self.state.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)


def install_into(linear_module):
    """Rebinds `RowParallelLinear.forward` of nanovllm/layers/linear.py (:149-153): small bf16 messages take the
    one-shot kernel, everything else `dist.all_reduce` as before."""
    import torch.nn.functional as F
    cls = linear_module.RowParallelLinear
    holder = {"comm": None}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.linear(x, self.weight, self.bias if self.tp_rank == 0 else None)
        if self.tp_size > 1:
            comm = holder["comm"]
            small = (y.is_cuda and y.dtype == torch.bfloat16 and y.is_contiguous() and 0 < y.numel() * 2 <= 512 * 1024
                     and y.numel() % 8 == 0)
            if small and comm is None and not torch.cuda.is_current_stream_capturing():
                comm = holder["comm"] = SmallAllReduce()
            if small and comm is not None and comm.usable(y):
                comm.all_reduce_(y)
            else:
                dist.all_reduce(y)
        return y

    cls.forward = forward
    return cls
