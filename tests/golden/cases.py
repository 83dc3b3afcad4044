"""Seeded input builders for the golden parity cases.

Every case is rebuilt from its seed on the CPU (torch CPU generators are deterministic for a
given torch build), so only the reference's OUTPUTS are committed (tests/golden/golden.pt),
next to a SHA-256 of the inputs that detects generator drift.  The same builders feed
make_golden.py (runs the reference module on a GPU), the CPU oracle tests and the GPU parity tests.

Shapes and conventions follow the reference's caller: q/k/v are slices of one fused qkv
activation (nanovllm/models/qwen3.py:75-78: k and q become contiguous after RoPE, v stays a
strided view), block tables are padded with -1 (nanovllm/engine/model_runner.py:119-123).
"""
from __future__ import annotations

import hashlib
import os
import sys

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from oracle.attention_oracle import Context  # noqa: E402
from workloads import decode_slots, default_scale, make_block_tables, prefill_slots  # noqa: E402

BLOCK = 256
DT = torch.bfloat16

# name -> spec
CASES = {
    # BASELINE config 1 geometry (16/8/128, 64 blocks x 256, lens 100/257/513/1024) in bf16
    "dec_cfg1": dict(kind="decode", H=16, Hkv=8, D=128, NB=64, lens=[100, 257, 513, 1024], seed=101),
    # one KV head per GPU (Qwen3-8B at TP8: 4 q heads on 1 kv head); block-boundary lengths
    "dec_tp8": dict(kind="decode", H=4, Hkv=1, D=128, NB=24, lens=[1, 255, 256, 257, 2048, 700], seed=102),
    # G = 1 and G = 2 small
    "dec_g1": dict(kind="decode", H=2, Hkv=2, D=128, NB=12, lens=[64, 65, 1000], seed=103),
    "dec_tp4": dict(kind="decode", H=4, Hkv=2, D=128, NB=20, lens=[3, 129, 1500, 511, 512], seed=104),
    "pre_dense_small": dict(kind="prefill", H=4, Hkv=2, D=128, lens=[1, 17, 100, 256, 300], prefix=None, seed=201),
    "pre_dense_cfg": dict(kind="prefill", H=16, Hkv=8, D=128, lens=[64, 130], prefix=None, seed=202),
    "pre_dense_g4": dict(kind="prefill", H=4, Hkv=1, D=128, lens=[129, 5, 383], prefix=None, seed=203),
    # prefix-cache hits: K/V for the whole key range come from the paged cache
    "pre_paged": dict(kind="prefill", H=4, Hkv=2, D=128, lens=[300, 600, 513, 256, 700],
                      prefix=[0, 256, 512, 0, 512], NB=16, seed=301),
    "pre_paged_g4": dict(kind="prefill", H=4, Hkv=1, D=128, lens=[257, 1024, 90],
                         prefix=[256, 768, 0], NB=12, seed=302),
}


def _qkv(n, h, hkv, d, gen, scale=1.0):
    """q, k contiguous; v a strided view into a fused buffer, as the reference's caller passes them."""
    fused = (torch.randn(n, (h + 2 * hkv) * d, generator=gen) * scale).to(DT)
    q, k, v = fused.split([h * d, hkv * d, hkv * d], dim=-1)
    q = q.reshape(n, h, d).contiguous()
    k = k.reshape(n, hkv, d).contiguous()
    v = v.view(n, hkv, d)  # row stride (h + 2*hkv) * d
    return q, k, v


def build_case(name):
    """Returns (spec, tensors dict on CPU, Context on CPU)."""
    spec = CASES[name]
    gen = torch.Generator().manual_seed(spec["seed"])
    h, hkv, d = spec["H"], spec["Hkv"], spec["D"]
    t = {}
    if spec["kind"] == "decode":
        lens = spec["lens"]
        bt, nb = make_block_tables(lens, BLOCK, gen, num_blocks=spec["NB"])
        t["k_cache"] = (torch.randn(nb, BLOCK, hkv, d, generator=gen) * 0.5).to(DT)
        t["v_cache"] = (torch.randn(nb, BLOCK, hkv, d, generator=gen) * 0.5).to(DT)
        t["q"], t["k"], t["v"] = _qkv(len(lens), h, hkv, d, gen, 0.5)
        ctx = Context(is_prefill=False, slot_mapping=decode_slots(lens, bt, BLOCK),
                      context_lens=torch.tensor(lens, dtype=torch.int32), block_tables=bt)
    else:
        lens = spec["lens"]
        prefix = spec["prefix"] or [0] * len(lens)
        lq = [a - b for a, b in zip(lens, prefix)]
        cu_q = torch.tensor([0] + lq, dtype=torch.int32).cumsum(0).to(torch.int32)
        cu_k = torch.tensor([0] + lens, dtype=torch.int32).cumsum(0).to(torch.int32)
        t["q"], t["k"], t["v"] = _qkv(int(cu_q[-1]), h, hkv, d, gen)
        if spec["prefix"] is None:
            bt = None
            slots = None
        else:
            bt, nb = make_block_tables(lens, BLOCK, gen, num_blocks=spec["NB"])
            t["k_cache"] = torch.randn(nb, BLOCK, hkv, d, generator=gen).to(DT)
            t["v_cache"] = torch.randn(nb, BLOCK, hkv, d, generator=gen).to(DT)
            slots = prefill_slots(lens, prefix, bt, BLOCK)
        ctx = Context(is_prefill=True, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=max(lq),
                      max_seqlen_k=max(lens), slot_mapping=slots, block_tables=bt)
    return spec, t, ctx


def tensor_sha(*tensors):
    h = hashlib.sha256()
    for x in tensors:
        if x is None:
            h.update(b"none")
            continue
        x = x.detach().cpu().contiguous()
        h.update(str(tuple(x.shape)).encode())
        h.update(x.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def inputs_sha(t, ctx):
    return tensor_sha(t["q"], t["k"], t["v"].contiguous(), t.get("k_cache"), t.get("v_cache"),
                      ctx.slot_mapping, ctx.context_lens, ctx.block_tables, ctx.cu_seqlens_q, ctx.cu_seqlens_k)


def scale_of(spec):
    return default_scale(spec["D"])
