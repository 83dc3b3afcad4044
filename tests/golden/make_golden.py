"""Generates tests/golden/golden.pt by running the UNMODIFIED reference module on a CUDA GPU.

    python tests/golden/make_golden.py [--ref baseline/_ref] [--out tests/golden/golden.pt]

The reference (`nanovllm.layers.attention.Attention`: Triton store_kvcache + flash_attn) is
imported from --ref, a pip --target install of the reference tree.  For every case in
cases.CASES the seeded CPU inputs are moved to the GPU, the reference's Context is set exactly
as its ModelRunner would, `Attention.forward(q, k, v)` is called once, and the output plus a
SHA-256 of the resulting caches are stored.  Inputs are not stored: cases.build_case() rebuilds
them from the seed and `inputs_sha` guards against generator drift.
"""
import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.path.join(ROOT, "baseline", "_ref"))
    ap.add_argument("--out", default=os.path.join(HERE, "golden.pt"))
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    from nanovllm.layers.attention import Attention
    from nanovllm.utils.context import reset_context, set_context
    import flash_attn
    import triton

    dev = torch.device("cuda:0")
    gold = {"_meta": {"flash_attn": flash_attn.__version__, "triton": triton.__version__,
                      "torch": str(torch.__version__), "gpu": torch.cuda.get_device_name(0)}}
    for name in cases.CASES:
        spec, t, ctx = cases.build_case(name)
        d = {k: v.to(dev) for k, v in t.items()}
        att = Attention(spec["H"], spec["D"], cases.scale_of(spec), spec["Hkv"])
        if "k_cache" in d:
            att.k_cache, att.v_cache = d["k_cache"], d["v_cache"]
        mv = lambda x: None if x is None else x.to(dev)
        set_context(ctx.is_prefill, mv(ctx.cu_seqlens_q), mv(ctx.cu_seqlens_k), ctx.max_seqlen_q,
                    ctx.max_seqlen_k, mv(ctx.slot_mapping), mv(ctx.context_lens), mv(ctx.block_tables))
        with torch.inference_mode():
            o = att(d["q"], d["k"], d["v"])
        torch.cuda.synchronize()
        reset_context()
        gold[name] = {
            "out": o.cpu().clone(),
            "inputs_sha": cases.inputs_sha(t, ctx),
            "k_cache_sha": cases.tensor_sha(d["k_cache"]) if "k_cache" in d else None,
            "v_cache_sha": cases.tensor_sha(d["v_cache"]) if "v_cache" in d else None,
        }
        print(name, tuple(o.shape), o.dtype, "finite" if torch.isfinite(o.float()).all() else "NON-FINITE")
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    torch.save(gold, args.out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
