"""Caller side of the decode path: the packed one-copy / one-launch metadata preparation against a CPU
restatement of the reference's prepare_decode and graph-buffer update (oracle/metadata_oracle.py).

CPU: the packed record equals the reference's five tensors bit for bit, on synthetic sequences and on a seeded
request trace driven through the reference's own Scheduler / BlockManager / Sequence (when an install of the
reference is present).  GPU: the unpack kernel has the reference's effect on graph-style static buffers, and a
captured decode-attention graph replayed after it gives the oracle's attention output.
"""
import os
import random
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle.attention_oracle import decode_attn_ref, store_kvcache_ref
from oracle.metadata_oracle import prepare_decode_ref, update_graph_buffers_ref
from workloads import default_scale

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
DEV = "cuda:0"


class FakeSeq:
    """The attributes of nanovllm/engine/sequence.py that prepare_decode reads."""
    block_size = 256

    def __init__(self, num_tokens, block_table, last_token):
        self.num_tokens, self.block_table, self.last_token = num_tokens, block_table, last_token

    def __len__(self):
        return self.num_tokens

    @property
    def num_blocks(self):
        return (self.num_tokens + self.block_size - 1) // self.block_size

    @property
    def last_block_num_tokens(self):
        return self.num_tokens - (self.num_blocks - 1) * self.block_size


def _fake_batch(rng, bs, max_len=4096, num_blocks=5000):
    free = list(range(num_blocks))
    rng.shuffle(free)
    seqs = []
    for _ in range(bs):
        n = rng.choice([1, 255, 256, 257, 512, 513, rng.randint(1, max_len)])
        nb = (n + 255) // 256
        seqs.append(FakeSeq(n, [free.pop() for _ in range(nb)], rng.randint(0, 151935)))
    return seqs


def _assert_record_equals_reference(stager, rec, seqs):
    want = prepare_decode_ref(seqs, 256)
    got = stager.record_views(rec)
    for g, w in zip(got, want):
        g = torch.from_numpy(np.ascontiguousarray(g))
        assert g.dtype == w.dtype and g.shape == w.shape
        assert torch.equal(g, w)


@pytest.mark.parametrize("bs", [1, 2, 17, 256, 512])
def test_packed_record_equals_prepare_decode(bs):
    from nanovllm_b200.engine.decode_metadata import DecodeMetadataStager
    rng = random.Random(bs)
    stager = DecodeMetadataStager(512, 16, 256)
    for _ in range(3):                                   # the two records alternate
        seqs = _fake_batch(rng, bs)
        _assert_record_equals_reference(stager, stager.pack(seqs), seqs)
    with pytest.raises(ValueError):
        stager.pack(_fake_batch(rng, 513))
    with pytest.raises(ValueError):
        stager.pack([FakeSeq(5000, list(range(20)), 1)])


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanovllm")), reason="reference install (baseline/_ref) not present")
def test_packed_record_on_a_seeded_scheduler_trace():
    """The reference's own scheduler, block manager (prefix caching, preemption) and sequences produce the
    decode batches; every decode step's record must equal what the reference's prepare_decode would build."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from nanovllm.engine.scheduler import Scheduler
    from nanovllm.engine.sequence import Sequence
    from nanovllm.sampling_params import SamplingParams
    from nanovllm_b200.engine.decode_metadata import DecodeMetadataStager
    rng = random.Random(0)
    cfg = SimpleNamespace(max_num_seqs=64, max_num_batched_tokens=16384, eos=-1, num_kvcache_blocks=120,
                          kvcache_block_size=256)          # few blocks: the trace includes preemptions
    sched = Scheduler(cfg)
    shared = [rng.randint(0, 9999) for _ in range(300)]     # a common prefix: prefix-cache hits
    for i in range(96):
        prompt = (shared if i % 3 == 0 else []) + [rng.randint(0, 9999) for _ in range(rng.randint(100, 700))]
        sched.add(Sequence(prompt, SamplingParams(temperature=0.6, max_tokens=rng.randint(5, 120), ignore_eos=True)))
    stager = DecodeMetadataStager(64, 16, 256)
    decode_steps = 0
    while not sched.is_finished():
        seqs, is_prefill = sched.schedule()
        if not is_prefill:
            _assert_record_equals_reference(stager, stager.pack(seqs), seqs)
            decode_steps += 1
        sched.postprocess(seqs, [rng.randint(0, 9999) for _ in seqs])
    assert decode_steps > 100


@pytest.mark.gpu
def test_unpack_kernel_matches_the_graph_buffer_update():
    from nanovllm_b200.engine.decode_metadata import DecodeMetadataStager
    rng = random.Random(7)
    max_bs, cols = 512, 16
    stager = DecodeMetadataStager(max_bs, cols, 256, DEV)
    g = torch.Generator().manual_seed(1)
    mk = lambda: dict(input_ids=torch.randint(0, 1000, (max_bs,), generator=g),
                      positions=torch.randint(0, 1000, (max_bs,), generator=g),
                      slot_mapping=torch.randint(0, 1000, (max_bs,), generator=g, dtype=torch.int32),
                      context_lens=torch.randint(0, 1000, (max_bs,), generator=g, dtype=torch.int32),
                      block_tables=torch.randint(0, 1000, (max_bs, cols), generator=g, dtype=torch.int32))
    want = mk()                                          # stale contents, as after earlier steps
    got = {k: v.to(DEV) for k, v in want.items()}
    for bs in (300, 1, 512, 33):
        seqs = _fake_batch(rng, bs)
        update_graph_buffers_ref(want, *prepare_decode_ref(seqs, 256))
        stager.pack(seqs)
        stager.unpack_into(stager.to_device(), got["input_ids"], got["positions"], got["slot_mapping"],
                           got["context_lens"], got["block_tables"])
        torch.cuda.synchronize()
        for k in want:
            assert torch.equal(got[k].cpu(), want[k]), k


@pytest.mark.gpu
def test_staged_metadata_through_graph_replay():
    """The engine's decode form (nanovllm/engine/model_runner.py:215-250): a graph captured on all-zero static
    buffers, every step staged by one copy and one launch, then replayed."""
    import nanovllm_b200
    from nanovllm_b200.engine.decode_metadata import DecodeMetadataStager
    from nanovllm_b200.utils import context as ctxmod
    h, hkv, d, bucket, cols, nb = 16, 8, 128, 32, 16, 80
    g = torch.Generator().manual_seed(5)
    kc = (torch.randn(nb, 256, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nb, 256, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
    att = nanovllm_b200.Attention(h, d, default_scale(d), hkv)
    att.k_cache, att.v_cache = kc.to(DEV), vc.to(DEV)
    gv = dict(input_ids=torch.zeros(bucket, dtype=torch.int64, device=DEV), positions=torch.zeros(bucket, dtype=torch.int64, device=DEV),
              slot_mapping=torch.zeros(bucket, dtype=torch.int32, device=DEV), context_lens=torch.zeros(bucket, dtype=torch.int32, device=DEV),
              block_tables=torch.zeros(bucket, cols, dtype=torch.int32, device=DEV))
    s_q = torch.zeros(bucket, h, d, dtype=torch.bfloat16, device=DEV)
    s_k = torch.zeros(bucket, hkv, d, dtype=torch.bfloat16, device=DEV)
    s_v = torch.zeros(bucket, hkv, d, dtype=torch.bfloat16, device=DEV)
    s_out = torch.zeros(bucket, 1, h, d, dtype=torch.bfloat16, device=DEV)
    slot0 = (att.k_cache.view(-1, hkv * d)[0].clone(), att.v_cache.view(-1, hkv * d)[0].clone())
    ctxmod.set_context(False, slot_mapping=gv["slot_mapping"], context_lens=gv["context_lens"], block_tables=gv["block_tables"])
    with torch.inference_mode():
        s_out.copy_(att(s_q, s_k, s_v))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            s_out.copy_(att(s_q, s_k, s_v))
    torch.cuda.synchronize()
    att.k_cache.view(-1, hkv * d)[0] = slot0[0]          # capture stored zero rows into slot 0: put it back
    att.v_cache.view(-1, hkv * d)[0] = slot0[1]
    stager = DecodeMetadataStager(bucket, cols, 256, DEV)
    rng = random.Random(3)
    for bs in (20, 32, 3):
        seqs = _fake_batch(rng, bs, max_len=3000, num_blocks=nb)
        q = (torch.randn(bs, h, d, generator=g) * 0.5).to(torch.bfloat16)
        k = (torch.randn(bs, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
        v = (torch.randn(bs, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
        s_q[:bs], s_k[:bs], s_v[:bs] = q.to(DEV), k.to(DEV), v.to(DEV)
        stager.pack(seqs)
        stager.unpack_into(stager.to_device(), gv["input_ids"], gv["positions"], gv["slot_mapping"], gv["context_lens"],
                           gv["block_tables"])
        graph.replay()
        torch.cuda.synchronize()
        _, _, slots, lens, bt = prepare_decode_ref(seqs, 256)
        store_kvcache_ref(k, v, kc, vc, slots)
        want = decode_attn_ref(q, kc, vc, lens, bt, default_scale(d))
        torch.testing.assert_close(s_out[:bs].float().cpu(), want.float(), atol=2e-2, rtol=1e-2)
        assert not s_out[bs:].any()                      # padded rows: slot -1, length 0
        assert torch.equal(att.k_cache.cpu().view(torch.int16), kc.view(torch.int16))
    ctxmod.reset_context()
