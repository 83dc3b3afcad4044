"""QK-norm + rotary embedding + cache store (the producer side of the attention layer).

CPU: the oracle (oracle/qk_norm_rope_oracle.py) against outputs of the reference's own RMSNorm and
RotaryEmbedding modules (tests/golden/qk_norm_rope_golden.pt).  GPU: the fused kernel through the
C ABI against the oracle and the golden outputs; the cache against the store oracle.
Tolerance for q and k: the arithmetic is fp32 with the reference's rounding points, only the order
of the 128-term sum of squares differs, so at most a few elements may land on the neighbouring bf16
value: |ours - ref| <= 2^-6 * |(ref_i, ref_{i +- 64})| + 1e-6 (one bf16 step of a rotated pair) everywhere,
and at least 99.5 % of the elements bit-equal.
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import qk_cases  # noqa: E402
from oracle.attention_oracle import store_kvcache_ref  # noqa: E402
from oracle.qk_norm_rope_oracle import qk_norm_rope_ref, rope_cos_sin_cache  # noqa: E402

GOLD = torch.load(os.path.join(HERE, "golden", "qk_norm_rope_golden.pt"), weights_only=True)


@pytest.fixture(scope="module")
def b200():
    import nanovllm_b200
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return nanovllm_b200, None


def _one_step(a, b):
    """A rotated element is x1 * cos -+ x2 * sin of two bf16 values; if one of them sits on the
    neighbouring bf16 value the result moves by at most 2^-7 * (|x1| + |x2|) <= 2^-6.5 * |(x1, x2)|,
    and the rotation keeps |(x1, x2)| = |(y_i, y_{i +- 64})|."""
    a, b = a.float(), b.float()
    pair = torch.sqrt(b * b + torch.roll(b, 64, dims=-1) ** 2)
    assert bool(((a - b).abs() <= pair * 2.0 ** -6 + 1e-6).all())
    same = (a == b).float().mean().item()
    assert same >= 0.995, f"only {same:.4f} of the elements are bit-equal"


@pytest.mark.parametrize("name", list(qk_cases.CASES))
def test_oracle_matches_reference_modules(name):
    spec, t = qk_cases.build(name)
    assert qk_cases.inputs_sha(t) == GOLD[name]["inputs_sha"], "seeded inputs drifted from the golden file"
    cache = rope_cos_sin_cache(spec["D"], spec["max_position"], spec["base"])
    q, k, v = qk_norm_rope_ref(t["qkv"], t["positions"], t["q_weight"], t["k_weight"], cache, spec["eps"],
                               spec["H"], spec["Hkv"], spec["D"])
    assert torch.equal(q, GOLD[name]["q"]) and torch.equal(k, GOLD[name]["k"])
    assert v.data_ptr() == t["qkv"][:, (spec["H"] + spec["Hkv"]) * spec["D"]:].data_ptr()    # still a view


@pytest.mark.gpu
@pytest.mark.parametrize("with_cache", [True, False])
@pytest.mark.parametrize("name", list(qk_cases.CASES))
def test_fused_kernel_matches_golden(b200, name, with_cache):
    pkg, _ = b200
    from nanovllm_b200.layers.qk_norm_rope import qk_norm_rope_store
    dev = torch.device("cuda:0")
    spec, t = qk_cases.build(name)
    H, Hkv, D, n = spec["H"], spec["Hkv"], spec["D"], spec["n"]
    cache = rope_cos_sin_cache(D, spec["max_position"], spec["base"])
    g = torch.Generator().manual_seed(spec["seed"] + 100)
    kc = vc = slots = None
    if with_cache:
        nb, bs = 6, 256
        kc = torch.randn(nb, bs, Hkv, D, generator=g).to(torch.bfloat16)
        vc = torch.randn(nb, bs, Hkv, D, generator=g).to(torch.bfloat16)
        slots = torch.randperm(nb * bs, generator=g)[:n].to(torch.int32)
        slots[::7] = -1                                         # padded rows of a captured graph
    q, k, v = qk_norm_rope_store(t["qkv"].to(dev), t["positions"].to(dev), t["q_weight"].to(dev), t["k_weight"].to(dev),
                                 cache.to(dev), spec["eps"], H, Hkv,
                                 None if kc is None else (kcd := kc.to(dev)), None if vc is None else (vcd := vc.to(dev)),
                                 None if slots is None else slots.to(dev))
    torch.cuda.synchronize()
    _one_step(q.cpu(), GOLD[name]["q"])
    _one_step(k.cpu(), GOLD[name]["k"])
    assert torch.equal(v.cpu(), t["qkv"][:, (H + Hkv) * D:].view(n, Hkv, D))
    if with_cache:
        # the cache must hold exactly the k the kernel returned and the v bits of qkv, nothing else touched
        want_k, want_v = kc.clone(), vc.clone()
        store_kvcache_ref(k.cpu(), t["qkv"][:, (H + Hkv) * D:].view(n, Hkv, D), want_k, want_v, slots)
        assert torch.equal(kcd.cpu(), want_k) and torch.equal(vcd.cpu(), want_v)
    assert _status(pkg) == 0


def _status(pkg):
    from nanovllm_b200 import _lib
    return _lib.load().b200_device_status()


@pytest.mark.gpu
def test_fused_kernel_argument_errors(b200):
    from nanovllm_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    x = torch.zeros(4, 4 * 128, dtype=torch.bfloat16, device=dev)
    pos = torch.zeros(4, dtype=torch.int64, device=dev)
    w = torch.ones(128, dtype=torch.bfloat16, device=dev)
    cs = torch.zeros(16, 128, dtype=torch.float32, device=dev)
    q = torch.empty(4, 2, 128, dtype=torch.bfloat16, device=dev)
    k = torch.empty(4, 1, 128, dtype=torch.bfloat16, device=dev)
    call = lambda **kw: lib.b200_qk_norm_rope_store(
        kw.get("qkv", x.data_ptr()), kw.get("stride", x.stride(0)), pos.data_ptr(), w.data_ptr(), w.data_ptr(), cs.data_ptr(), 16,
        1e-6, q.data_ptr(), k.data_ptr(), kw.get("kc"), None, None, 0, 4, 2, 1, kw.get("d", 128), None)
    assert call() == 0
    assert call(qkv=None) == -1            # null pointer
    assert call(d=64) == -2                # head_dim other than 128
    assert call(stride=100) == -3          # row stride shorter than the row
    assert call(kc=x.data_ptr()) == -1     # k_cache without v_cache
    torch.cuda.synchronize()
