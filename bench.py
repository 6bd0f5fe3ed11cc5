#!/usr/bin/env python
"""Benchmark of the attention hot path: Qwen3-8B-shaped continuous-batch decode attention.

Workload (one "step" = one decode step's attention over all layers for the whole batch):
    64 sequences, context lengths uniform in [512, 32768] (seeded), 36 layers x (32 query heads, 8 KV heads,
    head_dim 128), f16 KV cache in the reference's 16-position tiles, fp32 queries ~N(0,1), device-filled ~N(0,1) caches.
    The batch is sharded by sequence over the ranks (longest first onto the least loaded rank), no data-path collective.
Metric: decode rows/s = sequences x steps / time (a row = one sequence's attention through all 36 layers).

    python bench.py [--gpus N] [--steps K] [--warmup W]            this library (librq_cuda.so through the C ABI)
    python bench.py --impl reference ...                            the reference's own CPU attention on the host cores

N > 1 is launched by torchrun (one rank per GPU); torch.distributed is used for the barrier and the max over ranks
only.  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_SEQ, N_LAYERS, N_HEADS, N_KV, HD = 64, 36, 32, 8, 128
CTX_LO, CTX_HI, CTX_SEED = 512, 32768, 20250
KV_BYTES_PER_POS = 2 * N_KV * HD * 2           # f16 K + V of one position of one layer: 4096 B (the algorithmic bytes)
METRIC = "Qwen3-8B attn: decode rows/s (B=64 ragged ctx)"
TRAFFIC_RATIO = (189.70 + 4.27) / 189.25  # measured DRAM bytes (read + written) over algorithmic K+V bytes, ncu capture of --small


def _synth():
    """gwenedeg_b200/synth.py (numpy only) loaded by path: the reference arm needs the workload's seeded context lengths
    without importing the package, whose import loads the CUDA library."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("rq_bench_synth", os.path.join(ROOT, "gwenedeg_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def contexts():
    return _synth().ragged_contexts(CTX_SEED, N_SEQ, CTX_LO, CTX_HI)


def workload_config(ctx_all, small=False):
    """The `config` object of the headline line: the workload only, the same in both arms."""
    return {"workload": "qwen3-8b-decode-small-profile-case" if small else "qwen3-8b-decode-b64-ragged",
            "sequences": N_SEQ, "layers": N_LAYERS, "heads": N_HEADS, "kv_heads": N_KV, "head_dim": HD, "kv_type": "f16",
            "ctx": f"U[{CTX_LO},{CTX_HI}] seed {CTX_SEED}", "positions_total": int(np.sum(ctx_all)),
            "l2": "inputs larger than L2: a layer pass streams 4,096 B per cached position, "
                  f"{int(np.sum(ctx_all)) * KV_BYTES_PER_POS / 1e9:.2f} GB over the batch"}


def shard(ctx, world):
    """Longest-first greedy packing of sequences onto ranks by context length."""
    load = [0] * world
    owner = [None] * len(ctx)
    for i in sorted(range(len(ctx)), key=lambda i: -int(ctx[i])):
        r = min(range(world), key=lambda r: load[r])
        owner[i] = r
        load[r] += int(ctx[i])
    return [[i for i in range(len(ctx)) if owner[i] == r] for r in range(world)]


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.p = None
        self.path = os.path.join("/tmp", f"rq_clocks_{os.getpid()}.csv")
        try:
            self.f = open(self.path, "w")
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                       "-i", str(gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.p:
            return out
        time.sleep(0.25)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def cpu_leg(ctx_all, reps, sample_every):
    """The reference's own CPU attention (oracle/_ref; else the plain-C restatement) on a bounded sample of the
    workload: every `sample_every`-th sequence, one layer, the reference's work items on its thread pool with all host
    cores.  Returns (rows/s scaled to the full batch and all layers, dict describing the run)."""
    from oracle import gwo
    orc = gwo.best()
    cores = orc.threads(os.cpu_count() or 1)
    idx = list(range(0, N_SEQ, sample_every))
    ctx = [int(ctx_all[i]) for i in idx]
    rng = np.random.default_rng(1)
    # one random 256-position block of all heads, tiled over a sequence's blocks (as the reference's own synthetic
    # fill does: forward.c:2385-2416): the bandwidth and arithmetic are those of distinct data
    blk_bytes = 16 * N_KV * orc.tile_bytes(2, HD, 0)
    blk = orc.f32_f16(rng.standard_normal(blk_bytes // 2).astype(np.float32)).view(np.uint8)
    caches = []
    for n in ctx:
        nb = (n + 255) // 256
        kl = np.tile(blk, nb)
        vl = np.tile(blk[::-1].copy(), nb)
        caches.append((kl, vl))
    q = rng.standard_normal((len(idx), N_HEADS, HD)).astype(np.float32)
    scale = float(1.0 / np.sqrt(np.float32(HD)))
    orc.bench_decode(2, N_KV, N_HEADS, HD, caches, ctx, q, scale, 1)  # warm-up (page faults, pool start)
    tot, best, _ = orc.bench_decode(2, N_KV, N_HEADS, HD, caches, ctx, q, scale, reps)
    t_layer_sample = tot / reps
    # linear in positions: scale the sample's layer time to the full batch, all layers
    t_step_full = t_layer_sample * (float(np.sum(ctx_all)) / float(sum(ctx))) * N_LAYERS
    info = {"value": N_SEQ / t_step_full, "unit": "rows/s", "cores": cores, "kind": "reference" if orc.kind == "ref" else "port",
            "isa": orc.isa, "library": orc.library,
            "sample": f"{len(idx)} of {N_SEQ} sequences (every {sample_every}th), 1 of {N_LAYERS} layers, {reps} reps, "
                      f"mean {t_layer_sample * 1e3:.1f} ms per layer pass (best {best * 1e3:.1f}), "
                      f"{sum(ctx) * KV_BYTES_PER_POS / t_layer_sample / 1e9:.1f} GB/s of KV; scaled by positions and layers"}
    return info


PF_LAYERS, PF_HEADS, PF_KV, PF_ROWS, PF_PREFIX = 28, 16, 8, 512, 3584


def prefill_leg(device, steps, layers=None, warm=3, kv="f16", exact=False):
    """Qwen3-0.6B-shaped chunked prefill attention (512 new rows over a 3584-position prefix, 28 layers, one
    sequence): TFLOP/s of the tensor-core prefill path, flops = 4 x head_dim per causal (query, key) pair per query head.
    kv: the cache type (quantised caches are expanded to f16 tiles once per layer call, inside the timed step; `roofline`
    times the tensor-core kernel alone); exact: quantised caches row by row through the bit-exact decode kernels instead."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    PF_LAYERS = layers or globals()["PF_LAYERS"]
    c = g.Context(device, n_attn=PF_LAYERS, n_heads=PF_HEADS, n_kv_heads=PF_KV, head_dim=HD, max_rows=PF_ROWS)
    s = c.new_seq(PF_PREFIX + PF_ROWS, {"f16": g.KV_F16, "q8": g.KV_Q8, "q4": g.KV_Q4, "q4k4": g.KV_Q4K4}[kv])
    s.fill_synthetic(PF_PREFIX + PF_ROWS, 77)
    c.set_exact(bool(exact))
    qn = PF_ROWS * PF_HEADS * HD
    q_host = c.pinned((PF_LAYERS, PF_ROWS, PF_HEADS, HD))
    q_host[:] = synth.normal(5, (PF_LAYERS, PF_ROWS, PF_HEADS, HD))
    q_dev, out_dev = c.malloc(q_host.nbytes), c.malloc(q_host.nbytes)
    c.h2d(q_dev, q_host)
    c.sync()

    def step():
        c.pass_begin([(s, PF_PREFIX, PF_ROWS)])
        for l in range(PF_LAYERS):
            c.attn_prefill_dev(l, q_dev + l * qn * 4, out_dev + l * qn * 4)
        c.pass_end(commit=False)

    for _ in range(warm):
        step()
    c.sync()
    c.timer_start()  # the whole path first, nothing between its launches
    for _ in range(steps):
        step()
    ms = c.timer_stop()
    c.profile_begin(steps * PF_LAYERS)  # then the same steps with CUDA events around each launch of the tensor-core kernel
    for _ in range(steps):
        step()
    c.sync()
    kern_ms, kern_n = c.profile_end()
    pairs = sum(p + 1 for p in range(PF_PREFIX, PF_PREFIX + PF_ROWS))
    flops_layer = 4.0 * HD * pairs * PF_HEADS
    c.close()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, how = float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        peak, how = 1590.0, "fallback"
    tf_step = flops_layer * PF_LAYERS * steps / (ms * 1e-3) / 1e12
    tf_kern = flops_layer * kern_n / (kern_ms * 1e-3) / 1e12
    if kv != "f16":
        return {"workload": f"qwen3-0.6b-prefill-512-over-3584-{kv}", "tflops": tf_step, "ms_per_chunk_all_layers": ms / steps,
                "kernels": "row by row through the bit-exact decode kernels" if exact else "f16 expansion + tensor-core prefill",
                "roofline": {"bound": "tensor", "achieved": tf_kern, "peak": peak, "unit": "TFLOP/s", "frac": tf_kern / peak, "traffic": None,
                             "peak_source": how, "kernel": "attn_part_kernel" if exact else "attn_prefill_kernel",
                             "flops_per_launch": flops_layer, "launches_timed": kern_n}}
    return {"workload": "qwen3-0.6b-prefill-512-over-3584", "tflops": tf_step, "ms_per_chunk_all_layers": ms / steps,
            "roofline": {"bound": "tensor", "achieved": tf_kern, "peak": peak, "unit": "TFLOP/s", "frac": tf_kern / peak, "traffic": None,
                         "peak_source": how, "kernel": "attn_prefill_kernel", "flops_per_launch": flops_layer, "launches_timed": kern_n}}


GA_LAYERS, GA_HEADS, GA_KV, GA_HD, GA_SEQ, GA_TOKENS, GA_CHUNK = 6, 16, 4, 256, 4, 8192, 512


def prefill_hd256_leg(device, steps, small=False):
    """The gated attention layers of the Qwen3.5-style hybrid stack as a prompt pass: 6 layers x (16 query / 4 KV heads,
    head_dim 256, sigmoid output gate), 4 sequences x 8,192 tokens in chunks of 512 rows per sequence over the f16 cache
    (the K / V rows of a chunk are in the cache when its attention runs).  TFLOP/s with 4 x head_dim flops per causal
    (query, key) pair per query head; `roofline` times the tensor-core kernel alone with events around its launches."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    layers, tokens = (2, 2048) if small else (GA_LAYERS, GA_TOKENS)
    c = g.Context(device, n_attn=layers, n_heads=GA_HEADS, n_kv_heads=GA_KV, head_dim=GA_HD, gated=True, max_rows=GA_SEQ * GA_CHUNK)
    seqs = []
    for i in range(GA_SEQ):
        s = c.new_seq(tokens, g.KV_F16)
        s.fill_synthetic(tokens, 900 + i)
        seqs.append(s)
    q = synth.normal(15, (GA_SEQ * GA_CHUNK, GA_HEADS, 2 * GA_HD))
    q_dev, out_dev = c.to_device(q), c.malloc(q.nbytes // 2)
    c.reserve(GA_SEQ * GA_CHUNK, GA_SEQ * GA_CHUNK * tokens, tokens)

    def prompt():
        for p0 in range(0, tokens, GA_CHUNK):
            c.pass_begin([(s, p0, GA_CHUNK) for s in seqs])
            for l in range(layers):
                c.attn_prefill_dev(l, q_dev, out_dev)
            c.pass_end(commit=False)

    prompt()
    c.sync()
    c.timer_start()
    for _ in range(steps):
        prompt()
    ms = c.timer_stop()
    c.profile_begin(steps * layers * (tokens // GA_CHUNK))
    for _ in range(steps):
        prompt()
    c.sync()
    kern_ms, kern_n = c.profile_end()
    c.close()
    pairs = tokens * (tokens + 1) // 2
    flops_prompt = 4.0 * GA_HD * GA_HEADS * GA_SEQ * pairs * layers
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, how = float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        peak, how = 1590.0, "fallback"
    tf_all = flops_prompt * steps / (ms * 1e-3) / 1e12
    tf_kern = flops_prompt * steps / (kern_ms * 1e-3) / 1e12
    return {"workload": "qwen3.5-gated-attention-prefill-4x8192-chunks-of-512", "layers": layers, "tokens": tokens, "tflops": tf_all,
            "ms_per_prompt_all_layers": ms / steps, "tokens_per_s": GA_SEQ * tokens * steps / (ms * 1e-3),
            "roofline": {"bound": "tensor", "achieved": tf_kern, "peak": peak, "unit": "TFLOP/s", "frac": tf_kern / peak, "traffic": None,
                         "peak_source": how, "kernel": "attn_prefill_hd256_kernel", "flops_per_prompt": flops_prompt, "launches_timed": kern_n}}


Q8_SEQ, Q8_CTX = 32, 40960
# bytes of K + V per position per layer: 8-bit half = int8 levels + a bf16 scale per 32 dims, 4-bit half = nibbles + the same
# scales; q8 = both halves 8-bit (2,176 B), q4 = K 8-bit, V 4-bit (1,664 B), q4k4 = both 4-bit (1,152 B)
_H8, _H4 = N_KV * (HD + HD // 32 * 2), N_KV * (HD // 2 + HD // 32 * 2)
Q_BYTES_PER_POS = {"q8": 2 * _H8, "q4": _H8 + _H4, "q4k4": 2 * _H4}


def q8_leg(args, rank, local_rank, world, kv="q8", dist=None, steps=None, warmup=None):
    """Qwen3-8B-shaped quantised-KV decode: 32 sequences at context 40,960, K and V as int8 (q8), 4-bit V (q4) or 4-bit K and V
    (q4k4) levels in blocks of 32 dims with bf16 scales (the reference's tile format).  q8 runs on the integer tensor cores (the
    cached levels are the MMA operands; --exact: the bit-exact CUDA-core kernels), the 4-bit types on the CUDA-core kernels.  With
    N > 1 every rank holds a group of KV heads of every sequence and the outputs are all-gathered (NCCL): returned beside the
    rows/s are the share of the step spent outside the attention kernels (gather + slicing copies) and whether a small pass
    gathered over the ranks equals the same pass on one GPU bit for bit.  Returns the JSON object of the leg (rank 0; else None)."""
    import hashlib
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from gwenedeg_b200.sharded import HeadShardedContext
    import torch
    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    own_group = False
    if world > 1 and dist is None:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        own_group = True
    layers = 2 if args.small else N_LAYERS
    nseq = 4 if args.small else Q8_SEQ
    kvt = {"q8": g.KV_Q8, "q4": g.KV_Q4, "q4k4": g.KV_Q4K4}[kv]
    sh = HeadShardedContext(local_rank, rank, world, n_attn=layers, n_heads=N_HEADS, n_kv_heads=N_KV, head_dim=HD, max_rows=nseq)
    c = sh.ctx
    c.set_exact(bool(args.exact))
    seqs = []
    for i in range(nseq):
        s = c.new_seq(Q8_CTX, kvt)
        s.fill_synthetic(Q8_CTX, 500 + i)
        seqs.append(s)
    c.sync()
    q = torch.from_numpy(synth.normal(11, (layers, nseq, N_HEADS, HD))).cuda()
    segs = [(s, Q8_CTX - 1, 1) for s in seqs]
    ql = [sh.local_q(q[l]) for l in range(layers)]
    out_l = torch.empty((nseq, sh.heads_local, HD), dtype=torch.float32, device="cuda")

    def step(gather=None):
        c.pass_begin(segs)
        outs = [sh.attn_decode(l, q[l], gather=gather) for l in range(layers)]
        c.pass_end(commit=False)
        return outs

    def step_local():  # the attention kernels alone: no gather, no slicing copies
        c.pass_begin(segs)
        with torch.cuda.stream(sh.stream):
            for l in range(layers):
                c.attn_decode_dev(l, ql[l].data_ptr(), out_l.data_ptr())
        c.pass_end(commit=False)

    def timed(fn, n):
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(sh.stream):
            e0.record()
        for _ in range(n):
            fn()
        with torch.cuda.stream(sh.stream):
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(warmup):
        step()
    ms = timed(step, steps)
    ms_local = timed(step_local, steps) if world > 1 else ms
    ms_nccl = timed(lambda: step("nccl"), steps) if world > 1 else None  # the same step with NCCL's all-gather + a transpose instead
    c.profile_begin(steps * layers)  # the kernel time of the roofline: a second pass with events around each launch
    for _ in range(steps):
        step_local()
    torch.cuda.synchronize()
    kern_ms, kern_n = c.profile_end()
    sh.close()

    # a small pass whose gathered rows must be the one-GPU rows: 2 sequences, one layer, rows written through kv_store
    digest_equal = None
    if world > 1:
        n = 1500
        k, v = synth.normal(1, (n, N_KV, HD)), synth.normal(2, (n, N_KV, HD))
        qv = synth.normal(3, (2, N_HEADS, HD))
        sv = HeadShardedContext(local_rank, rank, world, n_attn=1, n_heads=N_HEADS, n_kv_heads=N_KV, head_dim=HD)
        sv.ctx.set_exact(bool(args.exact))

        def fill(ctx, kk, vv):
            a = ctx.new_seq(n, kvt)
            for lo in range(0, n, 512):
                hi = min(n, lo + 512)
                ctx.pass_begin([(a, lo, hi - lo)])
                ctx.kv_store(0, np.ascontiguousarray(kk[lo:hi]), np.ascontiguousarray(vv[lo:hi]))
                ctx.pass_end()
            b = ctx.new_seq(n, kvt)
            b.copy_from(a, n)
            return a, b

        a, b = fill(sv.ctx, sv.local_kv(k), sv.local_kv(v))
        sv.ctx.pass_begin([(a, n - 1, 1), (b, 700, 1)])
        got = sv.attn_decode(0, torch.from_numpy(qv).cuda())
        torch.cuda.synchronize()
        got = got.cpu().numpy().copy()  # (the rows live in the context's own buffer: taken before it is closed)
        sv.ctx.pass_end(commit=False)
        sv.close()
        if rank == 0:
            full = g.Context(local_rank, n_attn=1, n_heads=N_HEADS, n_kv_heads=N_KV, head_dim=HD)
            full.set_exact(bool(args.exact))
            a, b = fill(full, k, v)
            full.pass_begin([(a, n - 1, 1), (b, 700, 1)])
            want = full.attn_decode(0, qv)
            full.pass_end(commit=False)
            full.close()
            digest_equal = hashlib.sha256(got.tobytes()).hexdigest() == hashlib.sha256(want.tobytes()).hexdigest()
        dist.barrier()
    if own_group:
        dist.destroy_process_group()
    if rank != 0:
        return None
    peak, how = peaks()
    bytes_launch = nseq * Q8_CTX * Q_BYTES_PER_POS[kv] / world
    achieved = bytes_launch / (kern_ms / max(kern_n, 1) * 1e-3) / 1e9
    tc = not args.exact
    return {"metric": f"Qwen3-8B attn: {kv} KV decode rows/s (B=32, ctx 40960)", "value": nseq * steps / (ms * 1e-3),
            "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
            "higher_is_better": True, "scaling": "strong", "dtype": "int8 x int8 -> int32, scales in f32" if tc else "f32", "data": "synthetic",
            "config": {"workload": f"qwen3-8b-decode-{kv}-b32-ctx40960", "layers": layers, "sequences": nseq},
            "run": {"parallelism": f"kv-head-sharded x{world}, gather fused into the merge kernel (peer stores over NVLink)" if world > 1 else "one GPU",
                    "kernels": "int8 tensor cores" if tc else "bit-exact CUDA cores",
                    "value_with_nccl_all_gather": nseq * steps / (ms_nccl * 1e-3) if ms_nccl else None},
            "outside_attention_kernels_share": max(0.0, 1.0 - ms_local / ms) if world > 1 else 0.0,
            "digest_equal_1gpu": digest_equal,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": bytes_launch * 1.0347 if tc and kv == "q8" else None,
                         "traffic_source": "ncu dram read + write of the small case of the same kernel (368.9 MB for 356.5 MB of K / V), scaled by "
                                           "positions" if tc and kv == "q8" else None,
                         "peak_source": how, "kernel": "attn_part_tc_kernel<4>" if tc else f"attn_part_kernel<{kv},128,4>",
                         "algorithmic_bytes_per_launch_rank0": bytes_launch, "launches_timed": kern_n}}


DN_LAYERS, DN_SEQ, DN_TOKENS, DN_HEADS, DN_DK = 18, 4, 8192, 16, 128


def deltanet_leg(local_rank, steps, small=False, rank=0, world=1):
    """Qwen3.5-style Gated DeltaNet: 18 linear layers, 4 sequences x 8,192 tokens, 16 heads, d_k = d_v = 128, post-prep rows
    resident on the device, prompt passes of 512 rows per sequence.  Reported: the chunked tensor-core form (the prefill
    path) as `value`, and the exact token recurrence (the decode path, bit-identical to the CPU code) beside it.
    flops = 8 d_k d_v per (token, head).  On N GPUs (N = 2 or 4) the sequences are dealt to the ranks (the state is per
    sequence: no collective on the data path), the time is the slowest rank's and the value the whole job's."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        if DN_SEQ % world:
            raise SystemExit(f"the DeltaNet workload has {DN_SEQ} sequences: run it on 1, 2 or 4 GPUs")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nseq = DN_SEQ // world
    layers = 2 if small else DN_LAYERS
    tokens = 1024 if small else DN_TOKENS
    chunk = 512  # rows per sequence per pass
    c = g.Context(local_rank, n_lin=layers, dn_nk=DN_HEADS, dn_nv=DN_HEADS, dn_dk=DN_DK, dn_dv=DN_DK, max_rows=nseq * chunk)
    seqs = [c.new_seq(tokens, g.KV_F16) for _ in range(nseq)]
    rows = synth.deltanet_rows(3 + rank, nseq * chunk, DN_HEADS, DN_HEADS, DN_DK, DN_DK)  # one pass worth of rows, reused
    rows_dev = c.to_device(rows)
    out_dev = c.malloc(nseq * chunk * DN_HEADS * DN_DK * 4)

    def run(fn):
        for pos in range(0, tokens, chunk):
            c.pass_begin([(s, pos, chunk) for s in seqs])
            for l in range(layers):
                fn(l, rows_dev, out_dev)
            c.pass_end()
        for s in seqs:
            s.truncate(0)

    res = {}
    for name, fn, nst in (("chunked", c.dn_chunk_dev, steps), ("exact", c.dn_rec_dev, max(1, min(steps, 2)))):
        run(fn)
        c.sync()
        if dist is not None:
            dist.barrier()
        n0 = c.launch_count()
        c.timer_start()
        for _ in range(nst):
            run(fn)
        ms = c.timer_stop()
        nl = c.launch_count() - n0
        if dist is not None:
            import torch
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the slowest rank's time
            ms = float(t[0].item())
            t2 = torch.tensor([float(nl)], dtype=torch.float64, device="cuda")
            dist.all_reduce(t2, op=dist.ReduceOp.SUM)
            nl = int(t2.item())
        res[name] = (DN_SEQ * tokens * nst / (ms * 1e-3), ms / nst, nl // nst)
    tok_s, ms_step, launches = res["chunked"]
    flops_tok = 8.0 * DN_DK * DN_DK * DN_HEADS * layers
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, how = float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        peak, how = 1590.0, "fallback"
    tf = flops_tok * tok_s / 1e12
    c.close()
    if dist is not None:
        dist.destroy_process_group()
    return {"metric": "Qwen3.5 Gated DeltaNet: tokens/s (all linear layers, prompt passes)", "value": tok_s, "unit": "tokens/s",
                      "n_gpus": world, "scaling": "strong", "steps": steps, "warmup": 1, "ms_per_step": ms_step, "higher_is_better": True, "dtype": "f16 operands, f32 state",
                      "data": "synthetic", "gpu_launches": launches,
                      "config": {"workload": "qwen3.5-deltanet-4x8192", "layers": layers, "tokens": tokens, "heads": DN_HEADS, "rows_per_pass": nseq * chunk,
                                 "parallelism": f"sequence-sharded x{world}"},
                      "form": "chunked (64-token WY / UT) on tcgen05", "tflops": tf,
                      "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peak, "unit": "TFLOP/s", "frac": tf / world / peak, "traffic": None,
                                   "peak_source": how, "kernel": "dn_chunk_kernel", "flops": "8 dk dv per (token, head): the recurrence's count"},
                      "exact_recurrence": {"tokens_per_s": res["exact"][0], "ms_per_step": res["exact"][1], "tflops": flops_tok * res["exact"][0] / 1e12,
                                           "form": "token by token, bit-identical to the CPU code"}}


def run_reference(args, rank, world):
    if rank != 0:
        return
    ctx_all = contexts()
    reps = max(1, args.steps)
    t0 = time.time()
    info = cpu_leg(ctx_all, reps, sample_every=2)
    line = {"metric": METRIC, "value": info["value"], "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * N_SEQ / info["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": workload_config(ctx_all),
            "cpu_baseline": info,
            "e2e": {"value": info["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.time() - t0}
    print(json.dumps(line), flush=True)


def run_ours(args, rank, local_rank, world):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            import torch
            torch.cuda.synchronize()
            dist.barrier()

    def reduce_max(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    ctx_all = contexts()
    mine = shard(ctx_all, args.shard_of)[0] if args.shard_of > 1 else shard(ctx_all, world)[rank]
    my_ctx = [int(ctx_all[i]) for i in mine]
    my_pos = sum(my_ctx)

    # distinct layer caches that fit: every layer of a rank's shard is my_pos x 4096 B (>> the 126 MB L2), so cycling
    # fewer than 36 distinct ones changes nothing for the memory system; all 36 are distinct whenever they fit
    probe = g.Context(local_rank, n_attn=1, n_heads=N_HEADS, n_kv_heads=N_KV, head_dim=HD, max_rows=N_SEQ)
    free, total = probe.mem_info()
    probe.close()
    per_layer = sum((n + 255) // 256 * 256 for n in my_ctx) * KV_BYTES_PER_POS
    n_distinct = int(max(1, min(N_LAYERS, (free * 0.80 - (2 << 30)) // per_layer)))
    c = g.Context(local_rank, n_attn=n_distinct, n_heads=N_HEADS, n_kv_heads=N_KV, head_dim=HD, max_rows=N_SEQ)
    seqs = []
    for j, (i, n) in enumerate(zip(mine, my_ctx)):
        s = c.new_seq(n, g.KV_F16)
        s.fill_synthetic(n, 1000 + i)
        seqs.append(s)
    c.sync()
    rows = len(seqs)
    segs = [(s, n - 1, 1) for s, n in zip(seqs, my_ctx)]
    qn = rows * N_HEADS * HD
    # resident inputs: the queries of every layer, and an output buffer per layer
    q_host = c.pinned((N_LAYERS, rows, N_HEADS, HD))
    q_host[:] = synth.normal(7 + rank, (N_LAYERS, rows, N_HEADS, HD))
    out_host = c.pinned((N_LAYERS, rows, N_HEADS, HD))
    q_dev = c.malloc(q_host.nbytes)
    out_dev = c.malloc(q_host.nbytes)
    c.h2d(q_dev, q_host)
    c.sync()

    def step_resident():
        c.pass_begin(segs)
        for l in range(N_LAYERS):
            c.attn_decode_dev(l % n_distinct, q_dev + l * qn * 4, out_dev + l * qn * 4)
        c.pass_end(commit=False)

    def step_e2e():
        c.pass_begin(segs)
        for l in range(N_LAYERS):
            c.check(c.L.rq_cuda_attn_decode(c.h, l % n_distinct, q_host[l].ctypes.data, out_host[l].ctypes.data))
        c.pass_end(commit=False)

    warm = args.warmup if args.small else max(args.warmup, 3)
    for _ in range(warm):
        step_resident()
    c.sync()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    l0 = c.launch_count()
    c.timer_start()  # the timed region: exactly `steps` steps, nothing but the library's launches on the stream
    for _ in range(args.steps):
        step_resident()
    ms = c.timer_stop()
    c.sync()
    barrier()
    launches = c.launch_count() - l0
    # the roofline's kernel time: the same steps again with CUDA events around each launch of the dominant kernel
    c.profile_begin(args.steps * N_LAYERS)
    for _ in range(args.steps):
        step_resident()
    c.sync()
    part_ms, part_n = c.profile_end()
    barrier()
    clocks = sampler.stop() if sampler else None
    ms_max = reduce_max(ms)
    launches = int(reduce_sum(launches))

    # end to end through the host-buffer entry point: pinned host q -> device, attention, result -> host, per layer
    if args.small:
        ms_e2e = float("nan")
    else:
        step_e2e()
        c.sync()
        out_host[:] = 0  # (the timed steps have to write every result again: checked below)
        barrier()
        t0 = time.perf_counter()
        c.timer_start()
        for _ in range(args.steps):
            step_e2e()
        ms_e2e = c.timer_stop()
        wall_e2e = (time.perf_counter() - t0) * 1e3
        resident = np.empty_like(out_host)  # the same layers through the resident path: equal bit for bit
        c.d2h(resident, out_dev)
        c.sync()
        if not np.array_equal(resident, out_host):
            raise RuntimeError("end-to-end results differ from the resident path's")
        barrier()
        ms_e2e = reduce_max(max(ms_e2e, wall_e2e))

    peak, how = peaks()
    bytes_per_launch = my_pos * KV_BYTES_PER_POS
    achieved = bytes_per_launch / (part_ms / max(part_n, 1) * 1e-3) / 1e9
    achieved = reduce_sum(achieved) / world  # mean over ranks of the per-GPU figure

    c.close()
    prefill = prefill_q8 = prefill_hd256 = deltanet = decode_q8 = decode_q8_sharded = None
    if not args.small:
        # the quantised-cache configuration (32 sequences at context 40,960, q8): on one GPU the whole batch; on N GPUs split by
        # KV-head group over the same process group, outputs all-gathered
        try:
            obj = q8_leg(args, rank, local_rank, world, kv="q8", dist=dist, steps=max(2, min(args.steps, 5)), warmup=3)
            if world == 1:
                decode_q8 = obj
            else:
                decode_q8_sharded = obj
        except Exception as e:
            decode_q8 = {"error": repr(e)}
    if world == 1 and not args.small:  # the other workloads ride on the one-GPU line only (each has its own --workload for N > 1)
        try:
            prefill = prefill_leg(local_rank, max(2, min(args.steps, 5)))
        except Exception as e:
            prefill = {"error": repr(e)}
        try:
            prefill_q8 = prefill_leg(local_rank, 2, kv="q8")
        except Exception as e:
            prefill_q8 = {"error": repr(e)}
        try:
            prefill_hd256 = prefill_hd256_leg(local_rank, 2)
        except Exception as e:
            prefill_hd256 = {"error": repr(e)}
        try:
            d = deltanet_leg(local_rank, 1)
            deltanet = {k: d[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "form", "tflops", "roofline", "exact_recurrence")}
        except Exception as e:
            deltanet = {"error": repr(e)}
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            try:
                cpu = cpu_leg(ctx_all, reps=50, sample_every=2)
            except Exception as e:  # the baseline is reported, never required
                cpu = {"value": None, "unit": "rows/s", "cores": 0, "kind": "unavailable", "sample": repr(e)}
        value = (len(mine) if args.shard_of > 1 else N_SEQ) * args.steps / (ms_max * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(ctx_all, args.small),
            "run": {"parallelism": f"sequence-sharded x{world}", "distinct_layer_caches_rank0": n_distinct,
                    "bytes_streamed_per_layer_pass_rank0": per_layer},
            "layer_rows_per_s": value * N_LAYERS,
            "e2e": {"value": N_SEQ * args.steps / (ms_e2e * 1e-3), "unit": "rows/s",
                    "h2d_bytes_per_step": N_LAYERS * N_SEQ * N_HEADS * HD * 4, "d2h_bytes_per_step": N_LAYERS * N_SEQ * N_HEADS * HD * 4},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": bytes_per_launch * TRAFFIC_RATIO, "traffic_source": "ncu dram read + write of the small case of the same kernel, scaled by positions", "peak_source": how, "kernel": "attn_part_kernel<f16,128,4>",
                         "algorithmic_bytes_per_launch_rank0": bytes_per_launch, "launches_timed": part_n},
            "cpu_baseline": cpu,
            "decode_q8": decode_q8,
            "decode_q8_head_sharded": decode_q8_sharded,
            "prefill": prefill,
            "prefill_q8": prefill_q8,
            "prefill_hd256": prefill_hd256,
            "deltanet": deltanet,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    # the JSON line is the only thing on standard output: what libraries write to file descriptor 1 (NCCL's version banner at the
    # first communicator) goes to standard error instead
    real = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    sys.stdout = real
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--exact", action="store_true", help="quantised-cache workloads: the bit-exact CUDA-core kernels instead of the "
                    "int8 tensor-core ones")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "prefill-q8", "prefill-q4", "prefill-q4k4", "prefill-hd256", "decode-q8", "decode-q4", "decode-q4k4", "deltanet"],
                    help="decode: the headline batched-decode benchmark (default); prefill: only the chunked-prefill leg "
                         "(512 rows over a 3584-position prefix), printed as its own line")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="profiling aid (one GPU): run only the sequences rank 0 of a W-rank job would own, to look at the "
                         "per-GPU workload of a multi-GPU run under ncu")
    ap.add_argument("--small", action="store_true",
                    help="profiling case for ncu captures: 8 sequences of 4096..8192 positions, 2 layers (about 0.4 GB of "
                         "KV per layer: larger than the L2, small enough for a multi-pass capture), no CPU / end-to-end legs")
    args = ap.parse_args()
    if args.small:
        global N_SEQ, N_LAYERS, CTX_LO, CTX_HI
        N_SEQ, N_LAYERS, CTX_LO, CTX_HI = 8, 2, 4096, 8192
        args.no_cpu = True
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload in ("decode-q8", "decode-q4", "decode-q4k4"):
        line = q8_leg(args, rank, local_rank, world, kv=args.workload[7:])
        if rank == 0:
            print(json.dumps(line), flush=True)
        return
    if args.workload == "deltanet":
        line = deltanet_leg(local_rank, args.steps, small=args.small, rank=rank, world=world)
        if rank == 0:
            print(json.dumps(line), flush=True)
        return
    if args.workload == "prefill-hd256":
        if rank == 0:
            r = prefill_hd256_leg(local_rank, args.steps, small=args.small)
            print(json.dumps({"metric": "Qwen3.5 gated attn (head_dim 256): prefill TFLOP/s (4 x 8192 in chunks of 512)", "value": r["tflops"],
                              "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": 1, "higher_is_better": True, "dtype": "f16",
                              "data": "synthetic", "config": {"workload": r["workload"], "layers": r["layers"], "tokens": r["tokens"]},
                              "ms_per_step": r["ms_per_prompt_all_layers"], "tokens_per_s": r["tokens_per_s"], "roofline": r["roofline"]}), flush=True)
        return
    if args.workload.startswith("prefill"):
        if rank == 0:
            kv = args.workload[8:] or "f16"
            r = prefill_leg(local_rank, args.steps, layers=2 if args.small else None, warm=args.warmup, kv=kv, exact=args.exact)
            print(json.dumps({"metric": f"Qwen3-0.6B attn: prefill TFLOP/s (512 rows over 3584, {kv} cache)", "value": r["tflops"], "unit": "TFLOP/s",
                              "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "f16",
                              "data": "synthetic", "config": {"workload": r["workload"], "layers": 2 if args.small else PF_LAYERS},
                              "ms_per_step": r["ms_per_chunk_all_layers"], "kernels": r.get("kernels"), "roofline": r["roofline"]}), flush=True)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        # started without torchrun: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr",
               "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__), "--gpus", str(args.gpus), "--steps", str(args.steps),
               "--warmup", str(args.warmup)] + (["--no-cpu"] if args.no_cpu else [])
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
