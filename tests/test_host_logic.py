"""CPU: the host-side mirror of the reference interface (module attributes, context record,
installation into nano-vllm) and the KV-head sharding rules, including a two-rank gloo run."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.attention_oracle import decode_attn_ref
from workloads import default_scale, make_block_tables

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def test_module_surface_matches_reference():
    from nanovllm_b200 import Attention
    att = Attention(16, 128, 0.0884, 8)
    assert (att.num_heads, att.head_dim, att.scale, att.num_kv_heads) == (16, 128, 0.0884, 8)
    # the model runner discovers the layer through these two attributes and rebinds them
    assert hasattr(att, "k_cache") and hasattr(att, "v_cache")
    assert att.k_cache.numel() == 0 and att.v_cache.numel() == 0
    assert list(dict(att.named_parameters())) == [] and list(att.state_dict()) == []


def test_context_record_matches_reference_fields():
    from nanovllm_b200.utils import context as c
    c.set_context(True, 1, 2, 3, 4, 5, 6, 7)
    got = c.get_context()
    assert (got.is_prefill, got.cu_seqlens_q, got.cu_seqlens_k, got.max_seqlen_q, got.max_seqlen_k,
            got.slot_mapping, got.context_lens, got.block_tables) == (True, 1, 2, 3, 4, 5, 6, 7)
    c.reset_context()
    assert c.get_context() == c.Context()
    if os.path.isdir(os.path.join(REF, "nanovllm")):
        import dataclasses
        import importlib.util
        spec = importlib.util.spec_from_file_location("_ref_context", os.path.join(REF, "nanovllm", "utils", "context.py"))
        ref = importlib.util.module_from_spec(spec)
        sys.modules["_ref_context"] = ref
        spec.loader.exec_module(ref)
        assert [f.name for f in dataclasses.fields(ref.Context)] == [f.name for f in dataclasses.fields(c.Context)]


def test_sharding_rules():
    from nanovllm_b200.sharding import head_slices, local_heads
    assert local_heads(32, 8, 4) == (8, 2)
    assert head_slices(32, 8, 8, 3) == (slice(12, 16), slice(3, 4))
    with pytest.raises(ValueError):
        local_heads(16, 8, 3)
    with pytest.raises(ValueError):
        head_slices(16, 8, 2, 2)


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from nanovllm_b200.sharding import head_slices, shard_heads
    g = torch.Generator().manual_seed(9)          # every rank builds the same global problem
    h, hkv, d = 8, 4, 128
    lens = [70, 300, 257]
    bt, nb = make_block_tables(lens, 256, g)
    kc = torch.randn(nb, 256, hkv, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, 256, hkv, d, generator=g).to(torch.bfloat16)
    q = torch.randn(len(lens), h, d, generator=g).to(torch.bfloat16)
    cl = torch.tensor(lens, dtype=torch.int32)
    qs, ks = head_slices(h, hkv, world, rank)
    local = decode_attn_ref(shard_heads(q, qs, 1), shard_heads(kc, ks, 2), shard_heads(vc, ks, 2), cl, bt,
                            default_scale(d))
    # no collective is part of the path; the gather below only lets rank 0 check the partition
    parts = [torch.empty_like(local.float()) for _ in range(world)] if rank == 0 else None
    dist.gather(local.float(), parts, dst=0)
    if rank == 0:
        full = decode_attn_ref(q, kc, vc, cl, bt, default_scale(d)).float()
        torch.save({"ok": torch.equal(torch.cat(parts, dim=2), full)}, os.path.join(out_dir, "r.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_kv_head_sharding_two_ranks_gloo(tmp_path):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert torch.load(os.path.join(str(tmp_path), "r.pt"))["ok"]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanovllm")), reason="reference install (baseline/_ref) not present")
def test_install_into_reference_engine():
    import subprocess
    code = f"""
import sys
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {REF!r})
import nanovllm_b200.integration as integ
ours = integ.install()
import nanovllm.layers.attention as ra
from nanovllm.models.qwen3 import Qwen3Attention
import nanovllm.models.qwen3 as q3
assert ra.Attention is ours.Attention and q3.Attention is ours.Attention
from nanovllm.utils.context import set_context, get_context
set_context(False, slot_mapping=1)
assert ours.get_context().slot_mapping == 1 and ours.get_context() is get_context()
assert ra is ours   # the reference's attention file (Triton + flash_attn imports) never ran
print('ok')
"""
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanovllm")), reason="reference install (baseline/_ref) not present")
@pytest.mark.parametrize("mode,expect", [("1", True), ("", False)])
def test_autoinstall_in_a_spawned_child(mode, expect):
    """What a spawned tensor-parallel rank does: a fresh interpreter that only imports the autoinstall module
    (as a `.pth` line or the top of the launching script would) ends up with this package's layer under the
    reference's module name -- and with nothing changed when the variable is unset."""
    import subprocess
    code = f"""
import sys
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {REF!r})
import nanovllm_b200.autoinstall as auto
import nanovllm_b200.layers.attention as ours
print(auto.installed, sys.modules.get('nanovllm.layers.attention') is ours)
"""
    env = dict(os.environ, B200_ATTN_INSTALL=mode)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.split() == [str(expect), str(expect)]


def _row_parallel_rank(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    import nanovllm.layers.linear as linear
    from nanovllm_b200.engine.small_allreduce import install_into
    g = torch.Generator().manual_seed(3)
    w = torch.randn(16, 8 * world, generator=g)
    x = torch.randn(5, 8 * world, generator=g)
    layer = linear.RowParallelLinear(8 * world, 16)
    layer.weight.data.copy_(w[:, rank * 8:(rank + 1) * 8])
    want = layer(x[:, rank * 8:(rank + 1) * 8])             # the reference's forward: F.linear + dist.all_reduce
    install_into(linear)
    got = layer(x[:, rank * 8:(rank + 1) * 8])              # rebound forward; CPU tensors take the same collective
    ok = torch.equal(got, want) and torch.allclose(got, x @ w.t(), atol=1e-5)
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        torch.save({"ok": all(flags)}, os.path.join(out_dir, "rp.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanovllm")), reason="reference install (baseline/_ref) not present")
def test_row_parallel_forward_hook_keeps_the_collective_for_other_tensors(tmp_path):
    """The rebound RowParallelLinear.forward (small bf16 CUDA messages go to the one-shot kernel) must leave every
    other tensor on `dist.all_reduce`: two gloo ranks on the CPU, result equal to the reference's own forward."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_row_parallel_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert torch.load(os.path.join(str(tmp_path), "rp.pt"))["ok"]


def test_packed_buffers_layout_and_views():
    """engine.packed_copy: several tensors as one record, views with the requested shapes and dtypes, 16-byte aligned."""
    from nanovllm_b200.engine.packed_copy import PackedBuffers
    spec = {"q": ((3, 2, 128), torch.bfloat16), "slots": ((3,), torch.int32), "ids": ((3,), torch.int64),
            "bt": ((3, 5), torch.int32)}
    pb = PackedBuffers(spec, "cpu")
    assert pb.nbytes % 16 == 0 and pb.nbytes >= 3 * 2 * 128 * 2 + 12 + 24 + 60
    for name, (shape, dtype) in spec.items():
        assert tuple(pb.host[name].shape) == shape and pb.host[name].dtype == dtype
        assert pb.host[name].data_ptr() % 16 == 0
    pb.host["ids"].copy_(torch.tensor([7, 8, 9]))
    pb.host["bt"].fill_(-1)
    dev = pb.upload()
    assert torch.equal(dev["ids"], torch.tensor([7, 8, 9])) and bool((dev["bt"] == -1).all())
    assert not dev["slots"].data_ptr() == pb.host["slots"].data_ptr()
