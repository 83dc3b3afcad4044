"""Generates tests/golden/qk_norm_rope_golden.pt from the reference's own RMSNorm and
RotaryEmbedding modules, executed on the CPU.

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_qk_norm_rope_golden.py --ref /path/to/nano-vllm

Both modules are plain torch under a @torch.compile decorator; with TORCHDYNAMO_DISABLE=1 their
Python bodies run as written.  The inputs are rebuilt from the seed by qk_cases.build(); only the
reference's outputs are stored.
"""
import argparse
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import qk_cases  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of a nano-vllm source tree")
    ap.add_argument("--out", default=os.path.join(HERE, "qk_norm_rope_golden.pt"))
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    from nanovllm.layers.layernorm import RMSNorm
    from nanovllm.layers.rotary_embedding import RotaryEmbedding
    gold = {"_meta": {"torch": str(torch.__version__), "dynamo_disabled": os.environ.get("TORCHDYNAMO_DISABLE")}}
    for name in qk_cases.CASES:
        spec, t = qk_cases.build(name)
        H, Hkv, D = spec["H"], spec["Hkv"], spec["D"]
        qn, kn = RMSNorm(D, eps=spec["eps"]), RMSNorm(D, eps=spec["eps"])
        qn.weight.data = t["q_weight"].clone()
        kn.weight.data = t["k_weight"].clone()
        rope = RotaryEmbedding(D, D, spec["max_position"], spec["base"])
        with torch.inference_mode():
            q, k, v = t["qkv"].split([H * D, Hkv * D, Hkv * D], dim=-1)
            q = qn(q.view(-1, H, D))
            k = kn(k.view(-1, Hkv, D))
            q, k = rope(t["positions"], q, k)
        gold[name] = {"q": q.clone(), "k": k.clone(), "inputs_sha": qk_cases.inputs_sha(t)}
        print(name, tuple(q.shape), tuple(k.shape), q.dtype)
    torch.save(gold, args.out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
