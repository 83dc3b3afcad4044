"""Behind the path: the one-shot all-reduce for decode-sized messages (b200_small_allreduce) against the
restated sum (oracle/allreduce_oracle.py, bit-exact) and against NCCL (bf16 tolerance), as child processes on
two GPUs of one node -- eager, through CUDA-graph replay, and with a rank that does not show up (the bounded
wait runs out and reports; nothing faults or hangs).  Skipped where fewer than two GPUs are visible.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _child(rank, world, port, out_dir):
    import sys
    for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    from nanovllm_b200.engine.small_allreduce import SmallAllReduce
    from oracle.allreduce_oracle import all_reduce_sum_ref
    comm = SmallAllReduce(wait_limit_seconds=5.0)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    log = []

    def gathered(x):
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        return parts

    # eager: sizes from one vector to the limit, odd slice boundaries, many calls in a row
    for n in (8, 1024, 33 * 1024 + 8, 256 * 1024):
        for it in range(12):
            x = torch.randn(n, device=dev, dtype=torch.bfloat16, generator=g)
            parts = gathered(x)
            want = all_reduce_sum_ref(parts)
            nccl = x.clone()
            dist.all_reduce(nccl)
            got = comm.all_reduce_(x.clone())
            torch.cuda.synchronize()
            assert torch.equal(got, want), (n, it)
            # NCCL adds in bf16 in an order of its own: every one of its world - 1 additions rounds a partial sum that
            # is at most sum |x_r| in size (2^-8 relative each), whatever cancels in the end; ours rounds once
            bound = 2.0 ** -8 * world * torch.stack([p_.float().abs() for p_ in parts]).sum(0) + 1e-6
            assert bool(((got.float() - nccl.float()).abs() <= bound).all()), (n, it)
    log.append("eager ok")
    # the shape the engine sends: (batch, hidden) rows, inside a captured graph, replayed with fresh data
    static = torch.zeros(64, 1024, device=dev, dtype=torch.bfloat16)
    comm.all_reduce_(static)                       # warm-up outside capture
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(3):                         # three layers' worth
            comm.all_reduce_(static)
    for it in range(4):
        x = torch.randn(64, 1024, device=dev, dtype=torch.bfloat16, generator=g) * 0.1
        parts = gathered(x)
        want = parts
        for _ in range(3):                         # each replayed call sums what every rank holds at that point
            s = all_reduce_sum_ref(want)
            want = [s for _ in range(world)]
        static.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static, want[0]), it
    log.append("graph ok")
    assert comm.status() == 0
    # a rank that does not show up: the other one's wait runs out, its message is left as it was
    dist.barrier()
    comm.wait_limit = 0.3
    x = torch.randn(4096, device=dev, dtype=torch.bfloat16, generator=g)
    if rank == 0:
        y = comm.all_reduce_(x.clone())
        assert comm.status() == -8
        assert torch.equal(y, x)
    comm.reset()
    comm.wait_limit = 5.0
    assert comm.status() == 0
    x = torch.randn(4096, device=dev, dtype=torch.bfloat16, generator=g)
    want = all_reduce_sum_ref(gathered(x))
    assert torch.equal(comm.all_reduce_(x.clone()), want)
    log.append("timeout and recovery ok")
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        with open(os.path.join(out_dir, "ok.txt"), "w") as f:
            f.write("; ".join(log))
    dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs on one node")
def test_small_allreduce_ranks(tmp_path):
    """Two ranks, or B200_AR_TEST_WORLD of them (up to 8) where that many GPUs are visible."""
    world = min(int(os.environ.get("B200_AR_TEST_WORLD", "2")), torch.cuda.device_count(), 8)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_child, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert "timeout and recovery ok" in open(os.path.join(str(tmp_path), "ok.txt")).read()


def test_small_allreduce_argument_errors():
    from nanovllm_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda:0")
    import ctypes
    ptrs = (ctypes.c_void_p * 2)(x.data_ptr(), x.data_ptr())
    assert lib.b200_small_allreduce(ptrs, 0, 9, x.data_ptr(), x.data_ptr(), 64, 1.0, None) == -2      # too many ranks
    assert lib.b200_small_allreduce(ptrs, 0, 2, x.data_ptr(), x.data_ptr(), 60, 1.0, None) == -2      # not a multiple of 8
    assert lib.b200_small_allreduce(ptrs, 0, 2, x.data_ptr(), x.data_ptr(), 1 << 20, 1.0, None) == -2  # above the limit
    assert lib.b200_small_allreduce(ptrs, 0, 2, x.data_ptr(), None, 64, 1.0, None) == -1
    assert lib.b200_small_allreduce(ptrs, 0, 2, x.data_ptr(), x.data_ptr(), 0, 1.0, None) == 0        # empty: no-op
