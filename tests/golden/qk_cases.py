"""Seeded inputs of the QK-norm + RoPE parity cases (shared by the golden generator and the tests)."""
import hashlib

import torch

CASES = {
    # Qwen3-0.6B geometry, a decode-sized and a prefill-sized batch
    "qwen3_0p6b_decode": dict(H=16, Hkv=8, D=128, n=37, eps=1e-6, base=1e6, max_position=4096, seed=11),
    "qwen3_0p6b_prefill": dict(H=16, Hkv=8, D=128, n=300, eps=1e-6, base=1e6, max_position=4096, seed=12),
    # tensor-parallel shard of 8 (2 query heads, 1 kv head) and the 8B head ratio
    "tp8_shard": dict(H=2, Hkv=1, D=128, n=65, eps=1e-6, base=1e6, max_position=2048, seed=13),
    "qwen3_8b": dict(H=32, Hkv=8, D=128, n=19, eps=1e-6, base=1e6, max_position=8192, seed=14),
}


def build(name):
    spec = CASES[name]
    g = torch.Generator().manual_seed(spec["seed"])
    H, Hkv, D, n = spec["H"], spec["Hkv"], spec["D"], spec["n"]
    t = {
        "qkv": (torch.randn(n, (H + 2 * Hkv) * D, generator=g) * 1.5).to(torch.bfloat16),
        "positions": torch.randint(0, spec["max_position"], (n,), generator=g, dtype=torch.int64),
        "q_weight": (1.0 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16),
        "k_weight": (1.0 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16),
    }
    return spec, t


def inputs_sha(t):
    h = hashlib.sha256()
    for k in sorted(t):
        v = t[k].contiguous()
        h.update(k.encode())
        h.update(v.view(torch.uint8).numpy().tobytes() if v.dtype != torch.bfloat16 else v.view(torch.int16).numpy().tobytes())
    return h.hexdigest()
