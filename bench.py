#!/usr/bin/env python
"""Benchmark of the paged-KV attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  Default workload `decode_cfg2` is the configuration the headline metric
(paged decode-attention HBM GB/s) is quoted on: Qwen3-0.6B attention geometry (16 q heads, 8 kv
heads, head_dim 128), batch 256, context lengths uniform in [100, 2048], block size 256,
scattered random block tables, bf16.  One step = store_kvcache of one new token per sequence
followed by paged decode attention, on one layer's cache; consecutive steps walk over several
layers' caches (several GB in total), so no step finds its K/V in L2.

With N > 1 the path is sharded exactly as the reference's tensor parallelism does it -- by KV
head, identical metadata on every rank, no collective in the data path -- and `value` is the
bytes all ranks processed divided by the slowest rank's device time ("strong" scaling: the
global problem is fixed).

Besides the contract's keys the line carries
  roofline          the decode kernel alone (CUDA events around every launch) against the measured copy rate
  e2e               the same steps through Attention.forward with pinned host inputs and a host result
  hold              the K steps repeated for --hold-seconds, so that the nvidia-smi clock samples of `clocks`
                    fall inside a loaded region; `ms_x_sm_mhz` = step time x median SM clock
  cpu_baseline      the CPU restatement (oracle/) on the host cores, same sample as `--impl reference` takes
  library_baseline  (N = 1) what the reference's own GPU path achieves on the same box in the same run:
                    flash_attn_with_kvcache / flash_attn_varlen_func / the Triton store_kvcache, called with the
                    argument pattern of nanovllm/layers/attention.py:33-74 on the same tensors
  secondary         prefill TFLOP/s on BASELINE config 3 (dense); `secondaries` adds its prefix-cache form and,
                    at every N, decode on BASELINE config 4 (Qwen3-8B geometry, per-GPU and aggregate GB/s)

`--impl reference` times the reference's algorithm on the host cores (the CPU restatement under
oracle/, torch with all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import workloads as wl  # noqa: E402  (seeded input generators; no attention arithmetic)

WORKLOADS = wl.WORKLOADS
BLOCK = wl.BLOCK
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture of the
# library this file ships with (small case of the same kernel, scaled by the tiles a full launch streams)
TRAFFIC = {"decode_cfg2": 1143866100}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), bf16=float(p["bf16_tflops"]),
                    bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons (read-only query) sampled while the measured regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def count(self):
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def stop(self, skip=0):
        """Summary of the samples taken after the first `skip` lines."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                c = [x.strip() for x in line.split(",")]
                if len(c) >= 9:
                    rows.append(c)
            os.unlink(self.path)
        except Exception:
            pass
        rows = rows[skip:]
        if not rows:
            return out
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        pw = [float(r[3]) for r in rows if r[3].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(r[5 + j].lower().startswith("active") for r in rows)]
        out.update(sm_mhz=statistics.median(sm) if sm else None, sm_min_mhz=min(sm) if sm else None,
                   sm_max_mhz=max(mx) if mx else None, power_w_max=max(pw) if pw else None,
                   reasons=reasons, samples=len(rows))
        return out


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


class Ranks:
    """Barrier and max-over-ranks for one process per GPU (NCCL only for these two; none in the data path)."""

    def __init__(self, world, dev):
        self.world, self.dev = world, dev

    def barrier(self):
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max(self, x):
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())


# --------------------------------------------------------------------------------------------
# decode workloads (ours)
# --------------------------------------------------------------------------------------------
class DecodeProblem:
    """One decode workload on this rank: seeded metadata (identical on every rank), this rank's kv heads of
    `layers` caches, device-resident and pinned-host step inputs."""

    def __init__(self, w, rank, world, dev, layers):
        from nanovllm_b200.sharding import local_heads
        self.w, self.dev, self.layers = w, dev, layers
        self.h, self.hkv = local_heads(w["H"], w["Hkv"], world)
        self.d, self.b = w["D"], w["batch"]
        self.scale = self.d ** -0.5
        self.lens, g = wl.seeded_lens(w)
        self.bt, self.nb = wl.make_block_tables(self.lens.tolist(), BLOCK, g)
        self.slots = wl.decode_slots(self.lens.tolist(), self.bt, BLOCK)
        gd = torch.Generator(device=dev).manual_seed(1000 + rank)
        self.caches = []
        for _ in range(layers):
            kc = torch.randn(self.nb, BLOCK, self.hkv, self.d, device=dev, dtype=torch.bfloat16, generator=gd) * 0.5
            vc = torch.randn(self.nb, BLOCK, self.hkv, self.d, device=dev, dtype=torch.bfloat16, generator=gd) * 0.5
            self.caches.append((kc, vc))
        mk = lambda heads: (torch.randn(self.b, heads, self.d, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
        self.hq, self.hk, self.hv = mk(self.h), mk(self.hkv), mk(self.hkv)
        self.h_slots, self.h_lens, self.h_bt = self.slots.pin_memory(), self.lens.pin_memory(), self.bt.pin_memory()
        self.dq, self.dk, self.dv = self.hq.to(dev), self.hk.to(dev), self.hv.to(dev)
        self.d_slots, self.d_lens, self.d_bt = self.h_slots.to(dev), self.h_lens.to(dev), self.h_bt.to(dev)
        self.h_out = torch.empty(self.b, 1, self.h, self.d, dtype=torch.bfloat16).pin_memory()
        self.dec_bytes = wl.decode_algorithmic_bytes(self.lens, self.h, self.hkv, self.d)
        self.store_bytes = 2 * (2 * self.b * self.hkv * self.d * 2) + 4 * self.b   # K, V rows read + written, slots read
        self.step_bytes = self.dec_bytes + self.store_bytes

    def cache_gb(self):
        return self.layers * 2 * self.nb * BLOCK * self.hkv * self.d * 2 / 1e9

    def step(self, i, ev=None):
        import nanovllm_b200
        kc, vc = self.caches[i % self.layers]
        nanovllm_b200.store_kvcache(self.dk, self.dv, kc, vc, self.d_slots)
        if ev is not None:
            ev[0].record()
        o = nanovllm_b200.decode_attention(self.dq, kc, vc, self.d_lens, self.d_bt, self.scale, self.hkv)
        if ev is not None:
            ev[1].record()
        return o


def capture_steps(prob, steps, first):
    """The `steps` steps as one CUDA graph (the way the engine runs decode: nanovllm/engine/model_runner.py:215-250),
    so that the timed region holds the kernels and not the host's launch calls."""
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(steps):
                prob.step(first + i)
    torch.cuda.synchronize()
    return graph


def time_steps(prob, ranks, steps, first, graph=None):
    """EXACTLY `steps` steps between barrier + synchronize on both sides; device time, max over ranks (ms).
    With `graph` (capture_steps of the same steps) the steps are one graph replay, else eager launches."""
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ranks.barrier()
    t0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(steps):
            prob.step(first + i)
    t1.record()
    ranks.barrier()
    return ranks.max(t0.elapsed_time(t1))


def time_decode_launches(prob, ranks, steps, first):
    """The same steps once more with an event pair around every decode launch (kept out of the timed region:
    an event between the two kernels of a step serialises their programmatic overlap).  Mean ms, max over ranks."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    ranks.barrier()
    for i in range(steps):
        prob.step(first + i, evs[i])
    ranks.barrier()
    return ranks.max(statistics.mean(a.elapsed_time(b) for a, b in evs))


def run_decode(args, w, rank, world, local):
    import torch.distributed as dist
    import nanovllm_b200
    from nanovllm_b200 import _lib
    from nanovllm_b200.utils.context import reset_context, set_context

    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ranks = Ranks(world, dev)
    lib = _lib.load()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()            # nvidia-smi needs a moment before its first line: start it before the set-up
    prob = DecodeProblem(w, rank, world, dev, args.layers or w["layers"])
    att = nanovllm_b200.Attention(prob.h, prob.d, prob.scale, prob.hkv)

    # End to end: every step's q, k, v and metadata start in pinned host memory and its output ends there.  The
    # inputs travel as one packed record (one copy), two records alternate, and the copies run on a second
    # stream, so step i+1's inputs arrive while step i computes -- what an engine that overlaps its host
    # work with the GPU does; every step's copies are inside the timed region.
    from nanovllm_b200.engine.packed_copy import PackedBuffers
    spec = {"q": (prob.hq.shape, torch.bfloat16), "k": (prob.hk.shape, torch.bfloat16), "v": (prob.hv.shape, torch.bfloat16),
            "slots": (prob.h_slots.shape, torch.int32), "lens": (prob.h_lens.shape, torch.int32),
            "bt": (prob.h_bt.shape, torch.int32)}
    packs = [PackedBuffers(spec, dev) for _ in range(2)]
    for pk_ in packs:
        for name, src in (("q", prob.hq), ("k", prob.hk), ("v", prob.hv), ("slots", prob.h_slots), ("lens", prob.h_lens),
                          ("bt", prob.h_bt)):
            pk_.host[name].copy_(src)
    h_outs = [torch.empty_like(prob.h_out).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ev_done[i % 2])        # the step that last read this record has finished
            packs[i % 2].upload()
            ev_in[i % 2].record(copy_stream)

    def step_e2e(i, last):
        if not last:
            upload(i + 1)
        d_ = packs[i % 2].dev
        torch.cuda.current_stream().wait_event(ev_in[i % 2])
        att.k_cache, att.v_cache = prob.caches[i % prob.layers]
        set_context(False, slot_mapping=d_["slots"], context_lens=d_["lens"], block_tables=d_["bt"])
        o = att(d_["q"], d_["k"], d_["v"])
        ev_done[i % 2].record()
        reset_context()
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ev_done[i % 2])
            h_outs[i % 2].copy_(o, non_blocking=True)
            o.record_stream(copy_stream)

    def run_e2e(n):
        upload(0)
        for i in range(n):
            step_e2e(i, i == n - 1)
        torch.cuda.current_stream().wait_stream(copy_stream)

    for i in range(args.warmup):
        prob.step(i)
    ranks.barrier()
    # ---- timed region: K steps, inputs resident in HBM ----
    launches0 = lib.b200_launch_count()
    graph = None if args.eager else capture_steps(prob, args.steps, args.warmup)    # 2 kernel nodes per step
    if graph is not None:
        time_steps(prob, ranks, args.steps, args.warmup, graph)                    # first replay: untimed
        launches = lib.b200_launch_count() - launches0
        ms_total = time_steps(prob, ranks, args.steps, args.warmup, graph)
    else:
        launches0 = lib.b200_launch_count()
        ms_total = time_steps(prob, ranks, args.steps, args.warmup)
        launches = lib.b200_launch_count() - launches0
    eager_ms = time_steps(prob, ranks, args.steps, args.warmup) / args.steps
    dec_ms = time_decode_launches(prob, ranks, args.steps, args.warmup)
    # ---- end to end through the layer's forward, host buffers in, host result out ----
    run_e2e(max(3, args.warmup))
    ranks.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    e0.record()
    run_e2e(args.steps)
    e1.record()
    ranks.barrier()
    wall_ms = (time.perf_counter() - wall0) * 1e3
    e2e_ms = ranks.max(max(e0.elapsed_time(e1), wall_ms))
    # ---- hold: the K steps repeated until the clock sampler has a loaded region to look at ----
    skip = sampler.count() if rank == 0 else 0
    hold_ms, hold_steps, t_hold = [], 0, time.perf_counter()
    while True:
        hold_ms.append(time_steps(prob, ranks, args.steps, args.warmup, graph) / args.steps)
        hold_steps += args.steps
        flag = torch.tensor([1.0 if time.perf_counter() - t_hold < args.hold_seconds else 0.0], device=dev)
        if world > 1:
            dist.broadcast(flag, 0)
        if flag.item() == 0.0:
            break
    clocks = sampler.stop(skip) if rank == 0 else None
    _lib.check(lib.b200_device_status())

    ms_per_step = ms_total / args.steps
    value = world * prob.step_bytes / (ms_per_step * 1e-3) / 1e9
    pk = peaks()
    achieved = prob.dec_bytes / (dec_ms * 1e-3) / 1e9
    hold_med = statistics.median(hold_ms)
    out = {
        "metric": "paged_decode_attn_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "num_heads": w["H"], "num_kv_heads": w["Hkv"], "head_dim": prob.d,
                   "batch": prob.b, "context_lens": f"uniform[{w['lo']},{w['hi']}] seed {w['seed']}",
                   "sum_context": int(prob.lens.sum()), "block_size": BLOCK, "num_blocks": prob.nb,
                   "parallelism": f"tp{world} by kv head ({prob.hkv} kv heads per GPU), no collective",
                   "step": "store_kvcache(1 token/seq) + paged decode attention, one layer",
                   "timed_region": "eager launches" if args.eager else "one CUDA graph of the K steps (2 kernel nodes per step)",
                   "l2": f"inputs larger than L2: steps rotate over {prob.layers} layer caches "
                         f"({prob.cache_gb():.2f} GB per GPU)",
                   "bytes_per_step_per_gpu": prob.step_bytes},
        "roofline": {"bound": "hbm", "kernel": "decode_attn_kernel", "achieved": round(achieved, 1),
                     "peak": pk["hbm"], "unit": "GB/s", "frac": round(achieved / pk["hbm"], 4),
                     "peak_source": pk["source"], "frac_of_spec_8000": round(achieved / 8000.0, 4),
                     "algorithmic_bytes_per_launch": prob.dec_bytes, "avg_launch_ms": round(dec_ms, 5),
                     "traffic": TRAFFIC.get(args.workload) if world == 1 else None},
        "e2e": {"value": round(world * prob.step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9, 1), "unit": "GB/s",
                "ms_per_step": round(e2e_ms / args.steps, 5),
                "h2d_bytes_per_step": int(packs[0].nbytes), "d2h_bytes_per_step": int(prob.h_out.nbytes),
                "api": "nanovllm_b200.Attention.forward with set_context; pinned host q/k/v/metadata in as one packed "
                       "record (engine.packed_copy), host output out; copies on a second stream, two records alternating"},
        "gpu_launches": int(launches), "eager_ms_per_step": round(eager_ms, 5),
        "hold": {"seconds": args.hold_seconds, "steps": hold_steps, "ms_per_step": round(hold_med, 5),
                 "value": round(world * prob.step_bytes / (hold_med * 1e-3) / 1e9, 1)},
        "clocks": clocks,
    }
    if rank == 0 and clocks and clocks.get("sm_mhz"):
        out["hold"]["ms_x_sm_mhz"] = round(hold_med * clocks["sm_mhz"], 2)
    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_decode_baseline(w, sample=cpu_sample_size(w, args.steps))
    if not args.no_secondary:
        if world == 1:
            out["library_baseline"] = library_baseline(dev, prob)
        del prob, att
        torch.cuda.empty_cache()
        secondaries = []
        if world == 1:
            out["secondary"] = secondary_prefill(dev)
            secondaries.append(secondary_prefill(dev, workload="prefill_cfg3_prefix"))
        if args.workload != "decode_cfg4":
            secondaries.append(secondary_decode(args, "decode_cfg4", rank, world, dev, ranks))
        out["secondaries"] = secondaries
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else None


def secondary_decode(args, name, rank, world, dev, ranks, steps=30):
    """Another decode configuration, sharded the same way: per-GPU and aggregate GB/s, kernel roofline."""
    w = WORKLOADS[name]
    prob = DecodeProblem(w, rank, world, dev, w["layers"])
    for i in range(3):
        prob.step(i)
    graph = None if args.eager else capture_steps(prob, steps, 3)
    if graph is not None:
        time_steps(prob, ranks, steps, 3, graph)
    ms = time_steps(prob, ranks, steps, 3, graph) / steps
    dec_ms = time_decode_launches(prob, ranks, steps, 3)
    pk = peaks()
    per_gpu = prob.step_bytes / (ms * 1e-3) / 1e9
    kern = prob.dec_bytes / (dec_ms * 1e-3) / 1e9
    out = {"metric": "paged_decode_attn_hbm_gbs", "workload": name, "n_gpus": world, "steps": steps,
           "num_heads": w["H"], "num_kv_heads": w["Hkv"], "batch": w["batch"],
           "context_lens": f"uniform[{w['lo']},{w['hi']}] seed {w['seed']}",
           "parallelism": f"tp{world} by kv head ({prob.hkv} kv heads per GPU), no collective",
           "value": round(world * per_gpu, 1), "per_gpu": round(per_gpu, 1), "unit": "GB/s", "ms_per_step": round(ms, 5),
           "kernel_gbs": round(kern, 1), "kernel_ms": round(dec_ms, 5), "frac": round(kern / pk["hbm"], 4),
           "peak": pk["hbm"], "peak_source": pk["source"], "frac_of_spec_8000": round(kern / 8000.0, 4),
           "cache_gb_per_gpu": round(prob.cache_gb(), 2)}
    del prob
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------
# the reference's own GPU path on the same box (harness only: flash_attn and Triton never enter the product)
# --------------------------------------------------------------------------------------------
def _event_ms(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def library_baseline(dev, prob, iters=20):
    """flash_attn_with_kvcache, flash_attn_varlen_func and the Triton store_kvcache with the argument pattern of
    nanovllm/layers/attention.py:33-74, on the tensors of this run (decode: rotating over the same layer caches)."""
    out = {"what": "the reference's GPU path (flash_attn + Triton) on this box, same tensors, CUDA events"}
    try:
        import flash_attn
        from flash_attn import flash_attn_varlen_func, flash_attn_with_kvcache
        out["flash_attn"] = flash_attn.__version__
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"flash_attn does not import here: {e!r}"[:200]}
    try:
        state = {"i": 0}

        def dec():
            kc, vc = prob.caches[state["i"] % prob.layers]
            state["i"] += 1
            return flash_attn_with_kvcache(prob.dq.unsqueeze(1), kc, vc, cache_seqlens=prob.d_lens, block_table=prob.d_bt,
                                           softmax_scale=prob.scale, causal=True)
        ms = _event_ms(dec, iters)
        out["decode_ms"] = round(ms, 5)
        out["decode_gbs"] = round(prob.dec_bytes / (ms * 1e-3) / 1e9, 1)
    except Exception as e:  # noqa: BLE001
        out["decode_error"] = repr(e)[:200]
    try:
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        from nanovllm.layers.attention import store_kvcache as ref_store   # the reference's Triton kernel, unmodified
        state2 = {"i": 0}

        def st():
            kc, vc = prob.caches[state2["i"] % prob.layers]
            state2["i"] += 1
            ref_store(prob.dk, prob.dv, kc, vc, prob.d_slots)
        out["store_us"] = round(_event_ms(st, iters) * 1e3, 2)
        import nanovllm_b200
        state3 = {"i": 0}

        def st_ours():
            kc, vc = prob.caches[state3["i"] % prob.layers]
            state3["i"] += 1
            nanovllm_b200.store_kvcache(prob.dk, prob.dv, kc, vc, prob.d_slots)
        out["store_us_ours"] = round(_event_ms(st_ours, iters) * 1e3, 2)
    except Exception as e:  # noqa: BLE001
        out["store_error"] = repr(e)[:200]
    try:
        w, lens, cu, q, k, v = prefill_inputs(dev)
        mx = int(lens.max())
        flops = wl.prefill_algorithmic_flops(lens.tolist(), lens.tolist(), w["H"], w["D"])
        ms = _event_ms(lambda: flash_attn_varlen_func(q, k, v, max_seqlen_q=mx, cu_seqlens_q=cu, max_seqlen_k=mx,
                                                      cu_seqlens_k=cu, softmax_scale=w["D"] ** -0.5, causal=True,
                                                      block_table=None), 10)
        out["prefill_ms"] = round(ms, 4)
        out["prefill_tflops"] = round(flops / (ms * 1e-3) / 1e12, 1)
        del q, k, v
        lq, lens, cu_q, cu_k, bt, q, kc, vc = prefill_prefix_inputs(dev, WORKLOADS["prefill_cfg3_prefix"])
        flops = wl.prefill_algorithmic_flops(lq.tolist(), lens.tolist(), w["H"], w["D"])
        ms = _event_ms(lambda: flash_attn_varlen_func(q, kc, vc, max_seqlen_q=int(lq.max()), cu_seqlens_q=cu_q,
                                                      max_seqlen_k=int(lens.max()), cu_seqlens_k=cu_k,
                                                      softmax_scale=w["D"] ** -0.5, causal=True, block_table=bt), 10)
        out["prefill_prefix_ms"] = round(ms, 4)
        out["prefill_prefix_tflops"] = round(flops / (ms * 1e-3) / 1e12, 1)
    except Exception as e:  # noqa: BLE001
        out["prefill_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------
# CPU legs: the oracle timed on the host cores
# --------------------------------------------------------------------------------------------
def cpu_decode_baseline(w, sample, repeats=1):
    from oracle.attention_oracle import decode_attn_ref
    torch.set_num_threads(os.cpu_count() or 1)
    lens, g = wl.seeded_lens(w)
    lens = lens[:sample]
    bt, nb = wl.make_block_tables(lens.tolist(), BLOCK, g)
    hkv, h, d = w["Hkv"], w["H"], w["D"]
    kc = (torch.randn(nb, BLOCK, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nb, BLOCK, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
    q = (torch.randn(len(lens), h, d, generator=g) * 0.5).to(torch.bfloat16)
    decode_attn_ref(q[:4], kc, vc, lens[:4], bt[:4], d ** -0.5)
    t0 = time.perf_counter()
    for _ in range(repeats):
        decode_attn_ref(q, kc, vc, lens, bt, d ** -0.5)
    dt = (time.perf_counter() - t0) / repeats
    nbytes = wl.decode_algorithmic_bytes(lens, h, hkv, d)
    return {"value": round(nbytes / dt / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {len(lens)} of {w['batch']} sequences of the workload, fp32 math on bf16 data, "
                      f"{dt:.2f} s per pass", "seconds_per_pass": dt, "bytes_per_pass": nbytes}


_cpu_sample_cache = {}


def cpu_sample_size(w, steps):
    """Sequences per CPU pass, the same rule for the `ours` arm's cpu_baseline and for `--impl reference`: the
    whole batch if `steps` passes of it take under about a minute on this host, else as many as do."""
    key = (w["seed"], steps)
    if key not in _cpu_sample_cache:
        per_seq = cpu_decode_baseline(w, sample=8)["seconds_per_pass"] / 8
        _cpu_sample_cache[key] = int(max(2, min(w["batch"], 60.0 / max(steps, 1) / max(per_seq, 1e-6))))
    return _cpu_sample_cache[key]


def run_reference(args, w, rank, world):
    if rank != 0:
        return None
    if w["kind"] != "decode":
        raise SystemExit("--impl reference supports the decode workloads")
    # a step = the decode attention of the first `sample` sequences of the workload on the host cores
    sample = cpu_sample_size(w, args.steps)
    for _ in range(min(args.warmup, 2)):
        cpu_decode_baseline(w, sample=min(sample, 8))
    res = cpu_decode_baseline(w, sample=sample, repeats=args.steps)
    ms = res["seconds_per_pass"] * 1e3
    return {
        "impl": "reference", "metric": "paged_decode_attn_hbm_gbs", "value": res["value"], "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "num_heads": w["H"], "num_kv_heads": w["Hkv"], "head_dim": w["D"],
                   "batch": w["batch"], "step": f"decode attention of a {sample}-sequence sample on the host cores "
                                                 "(the reference has no CPU path of its own; this is the oracle port)"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# --------------------------------------------------------------------------------------------
# prefill (secondary metric; also a workload of its own)
# --------------------------------------------------------------------------------------------
def prefill_inputs(dev, w=None):
    w = w or WORKLOADS["prefill_cfg3"]
    lens, g = wl.seeded_lens(w)
    cu = wl.cu_seqlens(lens)
    t = int(cu[-1])
    gd = torch.Generator(device=dev).manual_seed(77)
    q = torch.randn(t, w["H"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    k = torch.randn(t, w["Hkv"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    v = torch.randn(t, w["Hkv"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    return w, lens, cu.to(dev), q, k, v


def prefill_prefix_inputs(dev, w):
    """Paged form: every key comes from the cache; the second half of the batch has a cached prefix."""
    lens, g = wl.seeded_lens(w)
    prefix = wl.cached_prefixes(lens, g)
    lq = lens - prefix
    cu_q, cu_k = wl.cu_seqlens(lq), wl.cu_seqlens(lens)
    bt, nb = wl.make_block_tables(lens.tolist(), BLOCK, g)
    gd = torch.Generator(device=dev).manual_seed(78)
    q = torch.randn(int(cu_q[-1]), w["H"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    kc = torch.randn(nb, BLOCK, w["Hkv"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    vc = torch.randn(nb, BLOCK, w["Hkv"], w["D"], device=dev, dtype=torch.bfloat16, generator=gd)
    return lq, lens, cu_q.to(dev), cu_k.to(dev), bt.to(dev), q, kc, vc


def secondary_prefill(dev, iters=10, workload="prefill_cfg3"):
    import nanovllm_b200
    w = WORKLOADS[workload]
    if w.get("prefix"):
        lq, lens, cu_q, cu_k, bt, q, kc, vc = prefill_prefix_inputs(dev, w)
        flops = wl.prefill_algorithmic_flops(lq.tolist(), lens.tolist(), w["H"], w["D"])
        f = lambda: nanovllm_b200.prefill_attention(q, kc, vc, cu_q, cu_k, int(lq.max()), int(lens.max()), w["D"] ** -0.5,
                                                    w["Hkv"], block_tables=bt)
        label = "prefill_cfg3_prefix (256 seqs, len uniform[100,1024], second half with a cached whole-block prefix, paged K/V)"
    else:
        w, lens, cu, q, k, v = prefill_inputs(dev, w)
        flops = wl.prefill_algorithmic_flops(lens.tolist(), lens.tolist(), w["H"], w["D"])
        mx = int(lens.max())
        f = lambda: nanovllm_b200.prefill_attention(q, k, v, cu, cu, mx, mx, w["D"] ** -0.5, w["Hkv"])
        label = "prefill_cfg3 (256 seqs, len uniform[100,1024], dense K/V, causal)"
    ms = _event_ms(f, iters)
    pk = peaks()
    tf = flops / (ms * 1e-3) / 1e12
    # a timed region of a few launches runs at burst clocks; a long one settles under the power cap,
    # where the cuBLAS figure to compare with is the sustained one
    kind = "sustained" if ms * iters > 250.0 else "burst"
    peak = pk["bf16_sustained"] if kind == "sustained" else pk["bf16"]
    return {"metric": "prefill_attn_tflops", "workload": label,
            "value": round(tf, 1), "unit": "TFLOP/s", "ms": round(ms, 4), "flops": flops,
            "frac_of_bf16_peak": round(tf / peak, 4), "peak": peak, "peak_source": pk["source"], "peak_kind": kind,
            "timed_ms": round(ms * iters, 1), "frac_of_spec_2250": round(tf / 2250.0, 4)}


def run_prefill(args, w, rank, world, local):
    if world != 1:
        raise SystemExit("the prefill workloads are single-GPU workloads")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    s = secondary_prefill(dev, iters=args.steps, workload=args.workload)
    return {"metric": s["metric"], "value": s["value"], "unit": s["unit"], "n_gpus": 1, "steps": args.steps,
            "warmup": 3, "ms_per_step": s["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": s["workload"]},
            "roofline": {"bound": "tensor", "achieved": s["value"], "peak": s["peak"], "unit": "TFLOP/s",
                         "frac": s["frac_of_bf16_peak"], "peak_source": s["peak_source"], "peak_kind": s["peak_kind"],
                         "timed_ms": s["timed_ms"], "traffic": None}}


def run_producer(args, w, rank, world, local):
    """QK-norm + RoPE + store: HBM GB/s over the algorithmic bytes (projection row read, q and k written,
    k and v written to the cache)."""
    if world != 1:
        raise SystemExit("the producer workloads are single-GPU workloads")
    from nanovllm_b200.layers.qk_norm_rope import qk_norm_rope_store
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    H, Hkv, D, n = w["H"], w["Hkv"], w["D"], w["tokens"]
    g = torch.Generator().manual_seed(w["seed"])
    nb = max(64, 2 * ((n + BLOCK - 1) // BLOCK))
    qkvs = [torch.randn(n, (H + 2 * Hkv) * D, generator=g).to(torch.bfloat16).to(dev) for _ in range(w["buffers"])]
    caches = [(torch.zeros(nb, BLOCK, Hkv, D, dtype=torch.bfloat16, device=dev),
               torch.zeros(nb, BLOCK, Hkv, D, dtype=torch.bfloat16, device=dev)) for _ in range(w["buffers"])]
    pos = torch.randint(0, 4096, (n,), generator=g, dtype=torch.int64).to(dev)
    slots = torch.randperm(nb * BLOCK, generator=g)[:n].to(torch.int32).to(dev)
    qw = (1.0 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(dev)
    kw = (1.0 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(dev)
    cs = wl.rope_table(D, 4096, 1e6).to(dev)
    lib = __import__("nanovllm_b200._lib", fromlist=["load"]).load()

    def step(i):
        kc, vc = caches[i % len(caches)]
        return qk_norm_rope_store(qkvs[i % len(qkvs)], pos, qw, kw, cs, 1e-6, H, Hkv, kc, vc, slots)

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    l0 = lib.b200_launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    a.record()
    for i in range(args.steps):
        step(i)
    b.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = a.elapsed_time(b) / args.steps
    nbytes = n * ((H + 2 * Hkv) * D * 2 + H * D * 2 + Hkv * D * 2 + 2 * Hkv * D * 2)
    pk = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"metric": "qk_norm_rope_store_hbm_gbs", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tokens": n, "num_heads": H, "num_kv_heads": Hkv, "head_dim": D,
                       "l2": "steps rotate over %d projection buffers and caches" % w["buffers"],
                       "bytes_per_step": nbytes},
            "roofline": {"bound": "hbm", "kernel": "qk_norm_rope_store_kernel", "achieved": round(gbs, 1), "peak": pk["hbm"],
                         "unit": "GB/s", "frac": round(gbs / pk["hbm"], 4), "peak_source": pk["source"], "traffic": None},
            "gpu_launches": int(lib.b200_launch_count() - l0), "clocks": clocks}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_cfg2", choices=list(WORKLOADS))
    ap.add_argument("--no-secondary", action="store_true", help="skip the library baseline and the secondary workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", type=int, default=0, help="layer caches the steps rotate over (0 = workload default)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of one CUDA graph of the K steps")
    ap.add_argument("--hold-seconds", type=float, default=2.0,
                    help="how long the steps are repeated after the timed region for the clock samples")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world, local = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        res = run_reference(args, w, rank, world)
    elif w["kind"] == "decode":
        res = run_decode(args, w, rank, world, local)
    elif w["kind"] == "producer":
        res = run_producer(args, w, rank, world, local)
    else:
        res = run_prefill(args, w, rank, world, local)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
