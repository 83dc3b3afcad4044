"""CPU restatement of what nano-vllm does to q and k right before its attention layer
(TEST INFRASTRUCTURE ONLY; only tests/, __graft_entry__.smoke() and bench code may import it).

Restated, with the reference lines each step follows (paths relative to the nano-vllm project):

* split of the fused projection     nanovllm/models/qwen3.py:74-78   (q | k | v along the last dim;
                                                                      v stays a strided view)
* per-head RMSNorm of q and k       nanovllm/layers/layernorm.py:16-26
      x = x.float(); var = mean(x^2); x *= rsqrt(var + eps); x = x.to(bf16) * weight
* rotary embedding                  nanovllm/layers/rotary_embedding.py:6-14 and :37-48
      cos_sin = cache[positions]; x1, x2 = halves of x.float();
      y = cat(x1 * cos - x2 * sin, x2 * cos + x1 * sin).to(bf16)
* the cos/sin table                 nanovllm/layers/rotary_embedding.py:27-34
* store of k and v into the cache   nanovllm/layers/attention.py:21-30 (restated in attention_oracle.py)

Pinning: the reference has no tests for these layers.  The oracle is pinned against the reference's
own RMSNorm and RotaryEmbedding modules executed on the CPU (with TORCHDYNAMO_DISABLE=1, i.e. the
Python bodies under their @torch.compile decorators) on seeded inputs; the outputs are committed as
tests/golden/qk_norm_rope_golden.pt together with the script that made them
(tests/golden/make_qk_norm_rope_golden.py).
"""
from __future__ import annotations

import torch


def rope_cos_sin_cache(head_dim: int, max_position: int, base: float) -> torch.Tensor:
    """(max_position, 1, head_dim) fp32: cos of the head_dim/2 frequencies, then sin.
    nanovllm/layers/rotary_embedding.py:27-34."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).unsqueeze_(1)


def rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """nanovllm/layers/layernorm.py:16-26 (no residual): fp32 normalisation, cast, then the weight."""
    orig = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(orig) * weight


def rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """nanovllm/layers/rotary_embedding.py:6-14."""
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def qk_norm_rope_ref(qkv, positions, q_weight, k_weight, cos_sin_cache, eps, num_heads, num_kv_heads, head_dim):
    """qkv (N, (H + 2 Hkv) * D) -> q (N, H, D), k (N, Hkv, D) normalised and rotated, v (N, Hkv, D) a view.
    nanovllm/models/qwen3.py:74-79."""
    qs, ks = num_heads * head_dim, num_kv_heads * head_dim
    q, k, v = qkv.split([qs, ks, ks], dim=-1)
    q = rms_norm_ref(q.view(-1, num_heads, head_dim), q_weight, eps)
    k = rms_norm_ref(k.view(-1, num_kv_heads, head_dim), k_weight, eps)
    v = v.view(-1, num_kv_heads, head_dim)
    cos, sin = cos_sin_cache[positions].chunk(2, dim=-1)
    return rope_ref(q, cos, sin), rope_ref(k, cos, sin), v
