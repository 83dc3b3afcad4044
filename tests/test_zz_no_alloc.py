"""GPU: the decode entry point that allocates nothing (b200_decode_attn_static).

Some users of the library cannot hand it a workspace: their engine has already spent all free
device memory on the KV cache, or their plugin contract forbids allocation inside a call.  For them
the library carries its own fixed scratch array.  This test calls that entry point through the C
ABI, several times in a row on different inputs (the array keeps the previous call's leftovers),
and checks each result against the ordinary entry point, which gets a fresh zeroed workspace from
torch, and against the CPU oracle.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  It needs nothing from the other tests and also passes alone.
"""
import pytest
import torch

from oracle.attention_oracle import decode_attn_ref
from workloads import default_scale, make_block_tables

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-2, 1e-2
DEV = "cuda:0"


def _problem(seed, lens, h, hkv):
    """Host tensors (for the oracle); the callers move them to the GPU."""
    g = torch.Generator().manual_seed(seed)
    bt, nb = make_block_tables(lens, 256, g)
    kc = (torch.randn(nb, 256, hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nb, 256, hkv, 128, generator=g) * 0.5).to(torch.bfloat16)
    q = (torch.randn(len(lens), h, 128, generator=g) * 0.5).to(torch.bfloat16)
    return q, kc, vc, torch.tensor(lens, dtype=torch.int32), bt


def _static(lib, q, kc, vc, cl, bt, hkv):
    out = torch.full((q.shape[0], 1, q.shape[1], 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = lib.b200_decode_attn_static(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), kc.shape[0], kc.shape[1],
                                     bt.data_ptr(), bt.stride(0), bt.shape[1], cl.data_ptr(), out.data_ptr(),
                                     q.shape[0], q.shape[1], hkv, 128, default_scale(128),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.b200_last_error()
    return out


def _with_workspace(lib, q, kc, vc, cl, bt, hkv):
    ws = torch.zeros(lib.b200_decode_workspace_bytes(1024, q.shape[1], hkv, 128), dtype=torch.uint8, device=DEV)
    out = torch.full((q.shape[0], 1, q.shape[1], 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = lib.b200_decode_attn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), kc.shape[0], kc.shape[1],
                              bt.data_ptr(), bt.stride(0), bt.shape[1], cl.data_ptr(), out.data_ptr(), ws.data_ptr(),
                              ws.numel(), q.shape[0], q.shape[1], hkv, 128, default_scale(128),
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.b200_last_error()
    return out


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    from nanovllm_b200 import _lib
    lib = _lib.load()
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    assert 0 < lib.b200_decode_static_scratch_bytes() < 16 << 20
    # Different problems back to back; all cut many (sequence, head) pairs across CTAs, so the scratch
    # (partials and arrival counters) is really exercised and really reused.  4 query heads per kv head
    # first, then 2: the slots of the partials are laid out differently, so the second call reads nothing
    # where the first one left it.  The third has more sequences than one launch takes (two launches, the
    # arrival counters of the first reused by the second).
    g = torch.Generator().manual_seed(3)
    many = torch.randint(1, 700, (600,), generator=g).tolist()
    problems = [(_problem(2, [9000, 64, 5, 0, 2049], 4, 1), 1),
                (_problem(1, [3000, 17, 700, 1, 4096, 255, 0, 1999], 16, 8), 8),
                (_problem(4, many, 4, 2), 2)]
    for host, hkv in problems:
        q, kc, vc, cl, bt = (x.to(DEV) for x in host)
        got = _static(lib, q, kc, vc, cl, bt, hkv)
        want = _with_workspace(lib, q, kc, vc, cl, bt, hkv)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), atol=ATOL, rtol=RTOL)
        oracle = decode_attn_ref(*host, default_scale(128))
        torch.testing.assert_close(got.float().cpu(), oracle.float(), atol=ATOL, rtol=RTOL)
    _lib.check(lib.b200_device_status())


def test_static_scratch_entry_point_rejects_oversize():
    from nanovllm_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    x = torch.zeros(64, dtype=torch.uint8, device=DEV)
    p = x.data_ptr()
    # 16 query heads per kv head x 2 CTAs per SM is more than the built-in scratch holds
    rc = lib.b200_decode_attn_static(p, 16 * 128, p, p, 1, 256, p, 1, 1, p, p, 8, 16, 1, 128, 0.1, None)
    assert rc == -4
    assert b"exceeds" in lib.b200_last_error()
