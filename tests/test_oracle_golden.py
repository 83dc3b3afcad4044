"""CPU: the oracle (oracle/attention_oracle.py) against outputs of the reference module itself
(tests/golden/golden.pt, produced on a B200 by tests/golden/make_golden.py)."""
import os

import pytest
import torch

import cases
from oracle.attention_oracle import AttentionRef

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.pt")
ATOL, RTOL = 2e-2, 1e-2   # BASELINE tolerance for bf16 attention outputs


@pytest.fixture(scope="module")
def gold():
    return torch.load(GOLD, weights_only=True)


def test_golden_meta(gold):
    meta = gold["_meta"]
    assert meta["flash_attn"].startswith("2.")
    assert set(cases.CASES) <= set(gold)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_oracle_matches_reference(gold, name):
    spec, t, ctx = cases.build_case(name)
    g = gold[name]
    if cases.inputs_sha(t, ctx) != g["inputs_sha"]:
        pytest.skip("seeded inputs differ from the ones the golden file was made with (torch build drift)")
    att = AttentionRef(spec["H"], spec["D"], cases.scale_of(spec), spec["Hkv"])
    if "k_cache" in t:
        att.k_cache, att.v_cache = t["k_cache"], t["v_cache"]
    out = att.forward(t["q"], t["k"], t["v"], ctx)
    ref = g["out"]
    assert out.shape == ref.shape and out.dtype == ref.dtype
    if spec["kind"] == "decode":
        keep = torch.tensor(spec["lens"]) > 0
        out, ref = out[keep], ref[keep]
    torch.testing.assert_close(out.float(), ref.float(), atol=ATOL, rtol=RTOL)
    # the oracle's fp32 math sits well inside the band: what is left is bf16 rounding
    assert (out.float() - ref.float()).abs().mean() < 1e-3
    if "k_cache" in t:
        # cache after store_kvcache: bit-exact, including untouched slots
        assert cases.tensor_sha(t["k_cache"]) == g["k_cache_sha"]
        assert cases.tensor_sha(t["v_cache"]) == g["v_cache_sha"]
