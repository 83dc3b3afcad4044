#!/usr/bin/env python
"""End-to-end output tokens/s of the nano-vllm engine with either attention layer
(BASELINE config 5: the workload of the reference's own bench.py).

    python bench_e2e.py --attn ours|reference [--fuse-producer] [--fast-metadata] [--tp 1] [--num-seqs 256] [--out FILE]

The ENGINE is the unmodified reference (scheduler, block manager, model runner, Qwen3 model,
CUDA graphs, sampler) imported from --ref (default baseline/_ref, a pip --target install of the
reference tree).  `--attn reference` leaves it untouched (Triton store_kvcache + flash_attn);
`--attn ours` installs nanovllm_b200's layer in its place before the engine is imported.
Everything else is identical between the two arms.

There are no checkpoints or tokenizer files on the box, so the model is a random-init
Qwen3-0.6B-architecture checkpoint (28 layers, hidden 1024, 16/8 heads, head_dim 128, MLP 3072,
vocab 151936, tied embeddings, bf16; N(0, 0.02) weights, unit norms) written once as safetensors
with the Hugging Face parameter names the reference's loader expects, plus a word-level
tokenizer of the same vocabulary size.  The workload follows the reference's bench.py: seed 0,
256 prompts of 100..1024 random token ids, max_tokens 100..1024, temperature 0.6, ignore_eos,
CUDA graphs on, max_model_len 4096.  Sampling is stochastic, so throughput is compared, not text.

One compatibility shim is applied to BOTH arms: transformers 5.x reports `rope_scaling` as a dict
for Qwen3, which the reference's get_rope() rejects; the loaded config gets `rope_scaling = None`
(rope theta then falls back to the reference's default 1e6, Qwen3's value).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from random import randint, seed

ROOT = os.path.dirname(os.path.abspath(__file__))
_REF = os.environ.get("B200_E2E_REF", os.path.join(ROOT, "baseline", "_ref"))
for _p in (ROOT, _REF):
    if _p not in sys.path:
        sys.path.insert(0, _p)

# Tensor-parallel ranks are spawned processes that re-import this file before they unpickle the
# model runner, so the layer is installed here, at import time, in every process of the `ours` arm
# (B200_ATTN_INSTALL set by main() below; unset = the reference's own layer).
import nanovllm_b200.autoinstall  # noqa: E402,F401


def make_model_dir(path: str):
    """Random-init Qwen3-0.6B-architecture checkpoint + tokenizer, written once."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast, Qwen3Config
    if os.path.exists(os.path.join(path, "model.safetensors")):
        return
    os.makedirs(path, exist_ok=True)
    cfg = Qwen3Config(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                      num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True, dtype="bfloat16",
                      eos_token_id=1, bos_token_id=2)
    cfg.save_pretrained(path)
    g = torch.Generator().manual_seed(0)
    w = {}

    def lin(name, out_f, in_f):
        w[name] = (torch.randn(out_f, in_f, generator=g) * 0.02).to(torch.bfloat16)

    w["model.embed_tokens.weight"] = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02).to(torch.bfloat16)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        lin(p + "self_attn.q_proj.weight", cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size)
        lin(p + "self_attn.k_proj.weight", cfg.num_key_value_heads * cfg.head_dim, cfg.hidden_size)
        lin(p + "self_attn.v_proj.weight", cfg.num_key_value_heads * cfg.head_dim, cfg.hidden_size)
        lin(p + "self_attn.o_proj.weight", cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim)
        w[p + "self_attn.q_norm.weight"] = torch.ones(cfg.head_dim, dtype=torch.bfloat16)
        w[p + "self_attn.k_norm.weight"] = torch.ones(cfg.head_dim, dtype=torch.bfloat16)
        lin(p + "mlp.gate_proj.weight", cfg.intermediate_size, cfg.hidden_size)
        lin(p + "mlp.up_proj.weight", cfg.intermediate_size, cfg.hidden_size)
        lin(p + "mlp.down_proj.weight", cfg.hidden_size, cfg.intermediate_size)
        w[p + "input_layernorm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
        w[p + "post_attention_layernorm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
    w["model.norm.weight"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
    save_file(w, os.path.join(path, "model.safetensors"))
    vocab = {f"t{i}": i for i in range(cfg.vocab_size)}
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="t0", eos_token="t1", bos_token="t2", pad_token="t3")
    fast.save_pretrained(path)


def install_rope_shim():
    import nanovllm.config as ncfg
    orig = ncfg.AutoConfig.from_pretrained

    def patched(*a, **k):
        c = orig(*a, **k)
        if isinstance(getattr(c, "rope_scaling", None), dict):
            c.rope_scaling = None
        return c

    ncfg.AutoConfig = type("AutoConfigShim", (), {"from_pretrained": staticmethod(patched)})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--attn", choices=["ours", "reference"], required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--num-seqs", type=int, default=256)
    ap.add_argument("--model-dir", default="/tmp/b200_e2e_qwen3_0p6b_random")
    ap.add_argument("--out", default="")
    ap.add_argument("--fuse-producer", action="store_true",
                    help="with --attn ours: q_norm + k_norm + rotary_emb + cache store as one kernel")
    ap.add_argument("--small-allreduce", action="store_true",
                    help="with --attn ours: also the one-shot all-reduce for decode-sized messages (implies --fast-metadata)")
    ap.add_argument("--fast-metadata", action="store_true",
                    help="with --attn ours: also the packed one-copy / one-launch decode metadata preparation "
                         "(implies --fuse-producer)")
    args = ap.parse_args()
    want_ar = args.small_allreduce and args.attn == "ours"
    want_fast = (args.fast_metadata or want_ar) and args.attn == "ours"
    want_fuse = "1" if ((args.fuse_producer or want_fast) and args.attn == "ours") else "0"
    want_env = "" if args.attn == "reference" else ("full+ar" if want_ar else ("full" if want_fast else ("fused" if want_fuse == "1" else "1")))
    if os.environ.get("B200_ATTN_INSTALL", "") != want_env:
        # set before anything of the engine is imported (and for spawned ranks), then start over
        os.environ["B200_ATTN_INSTALL"] = want_env
        os.execv(sys.executable, [sys.executable] + sys.argv)

    import torch
    make_model_dir(args.model_dir)
    from nanovllm import LLM, SamplingParams
    import nanovllm.layers.attention as attn_mod
    install_rope_shim()

    seed(0)
    max_in, max_out = 1024, 1024
    t_init = time.time()
    llm = LLM(args.model_dir, enforce_eager=False, max_model_len=4096, tensor_parallel_size=args.tp)
    t_init = time.time() - t_init
    prompts = [[randint(0, 10000) for _ in range(randint(100, max_in))] for _ in range(args.num_seqs)]
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=randint(100, max_out)) for _ in range(args.num_seqs)]
    llm.generate([[5, 6, 7, 8]], SamplingParams(max_tokens=8, ignore_eos=True), use_tqdm=False)   # warm-up
    lib_launches0 = None
    if args.attn == "ours":
        from nanovllm_b200 import _lib
        lib_launches0 = _lib.load().b200_launch_count()
    torch.cuda.synchronize()
    t = time.time()
    outs = llm.generate(prompts, sps, use_tqdm=False)
    torch.cuda.synchronize()
    t = time.time() - t
    total = sum(sp.max_tokens for sp in sps)
    produced = sum(len(o["token_ids"]) for o in outs)
    res = {
        "metric": "e2e_output_tok_per_s", "value": round(total / t, 2), "unit": "tok/s", "attn": args.attn,
        "fused_producer": want_fuse == "1", "fast_decode_metadata": bool(want_fast), "small_allreduce": bool(want_ar),
        "attention_module": attn_mod.__name__ + " from " + os.path.relpath(attn_mod.__file__, ROOT),
        "tp": args.tp, "num_seqs": args.num_seqs, "output_tokens": total, "produced_tokens": produced,
        "input_tokens": sum(len(p) for p in prompts), "seconds": round(t, 3), "engine_init_s": round(t_init, 1),
        "model": "random-init Qwen3-0.6B architecture (bf16)", "gpu": torch.cuda.get_device_name(0),
        "kv_blocks": llm.model_runner.config.num_kvcache_blocks,
    }
    if lib_launches0 is not None:
        from nanovllm_b200 import _lib
        res["lib_launches_rank0_eager"] = int(_lib.load().b200_launch_count() - lib_launches0)
        _lib.check(_lib.load().b200_device_status())
        if want_ar:
            from nanovllm_b200.engine.small_allreduce import SmallAllReduce
            res["small_allreduce_rank0"] = [{"status": c.status(), "host_calls": c.calls} for c in SmallAllReduce.instances]
    line = json.dumps(res)
    print(line, flush=True)
    if args.out:
        with open(args.out, "w") as f:
            f.write(line + "\n")


if __name__ == "__main__":
    main()
