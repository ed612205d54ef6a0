#!/usr/bin/env python
"""Benchmark of the packed-INT4-KV decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--scale F] [--shard heads|context]

A step is one decode-attention pass over one batch: ``knlp_b200_decode_attention``, the
balanced one-launch kernel (plus its small merge launch when one sequence is spread over
the whole machine).  Default workload: Llama-3-8B shape (32 q / 8 kv heads, d 128), batch
32, every sequence at 131 072 tokens of asymmetric INT4 KV (group 32, fp16 scale and zero),
bf16 queries, paged cache with 16-token pages: 5.37 GB of packed KV per step, far larger
than L2, so no flush is needed between steps.  The step is captured once in a CUDA graph
and replayed (the library's calls neither allocate nor synchronise); CUDA events bracket
the K timed replays and each of them.

With N > 1 (launched under torchrun, one rank per GPU) the kv heads are sharded across
ranks: rank r owns heads [r*8/N, (r+1)*8/N) of the same seeded cache and their q heads;
attention needs no exchange under a head shard, each rank keeps its output slice.  Total
work is fixed (strong scaling).  ``--shard context`` splits every sequence into contiguous
token segments instead; each rank emits one packed softmax partial per (sequence, q head),
ONE NCCL all-gather moves them, every rank merges.

Prints ONE JSON line on rank 0.  ``value`` is whole-job algorithmic HBM throughput with
inputs resident; ``e2e`` is the same through the operator API with host buffers (pinned h2d
of the step's query, new K/V token, slots and lengths; quantize-append; decode; d2h of the
output).  ``secondary`` lists the other benchmark configurations measured the same way in
the same process.  ``--impl reference`` times the CPU restatement of the reference's
dequantize-then-attend path (PyTorch eager, fp32, all host cores) on a bounded sample of
the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "int4_kv_decode_attn_achieved_hbm"
UNIT = "TB/s"
PAGE = 16

# name -> (q heads, kv heads, head_dim, batch, context or (lo, hi), K mode, V mode, q dtype)
SHAPES = {
    "gpt2_mha_1k": (12, 12, 64, 1, 1024, "int4_asym", "int4_asym", "f32"),
    "llama8b_b32_8k": (32, 8, 128, 32, 8192, "int4_asym", "int4_asym", "bf16"),
    "llama8b_b32_128k": (32, 8, 128, 32, 131072, "int4_asym", "int4_asym", "bf16"),
    "llama8b_b1_384k": (32, 8, 128, 1, 393216, "int4_asym", "int4_asym", "bf16"),
    "llama70b_ragged": (64, 8, 128, 64, (1024, 32768), "int4_asym", "int4_asym", "bf16"),
    "mixed_k8v4": (32, 8, 128, 128, (512, 4096), "int8", "int4_asym", "bf16"),
    "k8v8": (32, 8, 128, 128, (512, 4096), "int8", "int8", "bf16"),
}


def shape_of(workload: str):
    import re
    if workload in SHAPES:
        return SHAPES[workload]
    m = re.fullmatch(r"llama8b_b(\d+)_(\d+)k", workload)
    if m:
        return (32, 8, 128, int(m.group(1)), int(m.group(2)) * 1024, "int4_asym", "int4_asym", "bf16")
    raise SystemExit(f"bench.py: no shape known for workload {workload!r}")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))]


# ------------------------------------------------------------------ clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v == "Active":
                    reasons.add(n)
        sm.sort()
        pw.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_mhz_min": sm[0] if sm else None, "power_w_median": pw[len(pw) // 2] if pw else None,
                "power_w_max": pw[-1] if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def job_config(workload: str, scale: float, world: int, shard: str) -> dict:
    """The benchmark configuration, identical for both arms of a run."""
    hq, hkv, d, batch, ctx, km, vm, qd = shape_of(workload)
    if isinstance(ctx, tuple):
        context = f"uniform in [{int(ctx[0] * scale)}, {int(ctx[1] * scale)}]"
    else:
        context = int(ctx * scale)
    if world == 1:
        par = "single GPU"
    elif shard == "context":
        par = f"context shard x{world} (+1 NCCL all-gather of partials)"
    else:
        par = f"kv-head shard x{world}"
    return {"workload": workload, "scale": scale, "n_seqs": batch, "q_heads": hq, "kv_heads": hkv,
            "head_dim": d, "context": context, "kv": f"K {km} / V {vm}, group 32", "page": PAGE,
            "q_dtype": qd, "parallelism": par}


# ------------------------------------------------------------------ CPU leg
def kv_bytes_per_token_head(km: str, vm: str, d: int) -> int:
    ng = d // 32
    side = lambda m: d + 2 * ng if m == "int8" else d // 2 + (4 * ng if m == "int4_asym" else 2 * ng)
    return side(km) + side(vm)


def cpu_sample(workload: str, scale: float, max_tokens: int, repeats: int, warmup: int) -> dict:
    """Time the CPU restatement of the reference's dequantize-then-attend path
    (oracle/torch_eager.py: PyTorch eager, fp32, torch's intra-op pool on every host core)
    on a bounded sample of the workload: ONE sequence, all kv heads, up to ``max_tokens``
    tokens of the workload's value distribution, quantized on the CPU by the oracle's own
    quantizer.  The time of a whole step is extrapolated linearly in the tokens."""
    import numpy as np
    import torch
    from oracle import kv_oracle as O
    from oracle import torch_eager as TE

    hq, hkv, d, batch, ctx, km, vm, qd = shape_of(workload)
    mean_ctx = (ctx[0] + ctx[1]) / 2 if isinstance(ctx, tuple) else ctx
    step_tokens = batch * mean_ctx * scale
    T = max(1, min(int(mean_ctx * scale), max_tokens))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rng = np.random.default_rng(2000)
    chs = np.where(rng.random((hkv, d)) < 0.01, 10.0, 1.0).astype(np.float32)
    nb = (T + PAGE - 1) // PAGE
    k8 = km == "int8"
    kc = np.zeros((nb, PAGE, hkv, d if k8 else d // 2), np.int8 if k8 else np.uint8)
    vc = np.zeros((nb, PAGE, hkv, d // 2), np.uint8)
    ks = np.zeros((nb, PAGE, hkv, d // 32), np.float16)
    vs, kz, vz = np.zeros_like(ks), np.zeros_like(ks), np.zeros_like(ks)
    for t0 in range(0, T, 8192):  # quantize in chunks: the fp32 K/V never exist whole
        n = min(8192, T - t0)
        k = rng.standard_normal((n, hkv, d), dtype=np.float32) * chs
        v = rng.standard_normal((n, hkv, d), dtype=np.float32) * chs
        slots = np.arange(t0, t0 + n)
        if k8:
            O.reshape_and_cache_k_int8(k, kc, ks, slots)
            O.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
        else:
            O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
    q = rng.standard_normal((1, hq, d), dtype=np.float32)
    t = torch.from_numpy
    args = (t(q), t(kc), t(vc), t(ks), t(vs), t(np.arange(nb, dtype=np.int32)[None]),
            t(np.array([T], np.int32)), hkv, d)
    kw = dict(k_zeros=None if k8 else t(kz), v_zeros=t(vz), k_int8=k8)
    secs = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        TE.decode(*args, **kw)
        if i >= warmup:
            secs.append(time.perf_counter() - t0)
    nbytes = T * hkv * kv_bytes_per_token_head(km, vm, d) + q.size * 4 * 2 + 4 * nb
    med = pct(secs, 0.5)
    frac = T / step_tokens
    return {"value": nbytes / med / 1e12, "seconds_median": med, "seconds_p10": pct(secs, 0.1),
            "seconds_p90": pct(secs, 0.9), "cores": cores, "fraction_of_step": frac,
            "ms_per_step_extrapolated": med / frac * 1e3, "cpu_extrapolated": frac < 1.0,
            "sample": (f"1 sequence x {hkv} kv heads x {T} tokens of the workload's distribution "
                       f"= {frac:.3g} of a step; PyTorch eager fp32 dequantize -> SDPA, "
                       f"{cores} threads; median of {repeats} after {warmup} warm-up")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    full = args.workload == "gpt2_mha_1k"
    s = cpu_sample(args.workload, args.scale, 1024 if full else 32768,
                   repeats=max(args.steps, 1), warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": s["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": s["ms_per_step_extrapolated"], "cpu_extrapolated": s["cpu_extrapolated"],
        "ms_per_sample": s["seconds_median"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u8 codes + f16 scales -> f32", "data": "synthetic",
        "config": job_config(args.workload, args.scale, world, args.shard),
        "cpu_baseline": {"value": s["value"], "unit": UNIT, "cores": s["cores"], "kind": "port",
                         "sample": s["sample"]},
        "e2e": {"value": s["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
class Timed:
    """K replays of a captured step, timed with CUDA events (all of them and each)."""

    def __init__(self, torch, dev, need_flush: bool):
        self.torch, self.dev = torch, dev
        # L2 is 126 MB.  A working set of at least twice that is streamed without help; a
        # smaller one gets L2 flushed by writing a 256 MB buffer between the timed steps.
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if need_flush else None

    def run(self, replay, K: int, barrier):
        torch = self.torch
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(K)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(K):
            if self.flush is not None:
                self.flush.fill_(i & 0xFF)
            ev[i][0].record()
            replay()
            ev[i][1].record()
        e1.record()
        barrier()
        each = [a.elapsed_time(b) for a, b in ev]
        total = sum(each) if self.flush is not None else e0.elapsed_time(e1)
        return total, each


GRAPHS = []  # every captured graph, so that teardown can release them all


def capture(torch, fn, warm: int = 3):
    """fn() captured in a CUDA graph (after ``warm`` eager calls, which also size the library's
    workspace); falls back to the eager calls if capture is refused."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    try:
        # thread-local: CUDA calls of other threads (a process group's watchdog) are theirs
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            fn()
    except RuntimeError as exc:
        torch.cuda.synchronize()
        return fn, f"eager calls (graph capture failed: {str(exc)[:80]})"
    GRAPHS.append(graph)
    return graph.replay, "captured in one CUDA graph, replayed"


def measure_decode(torch, ops, w, K: int, W: int, barrier, ctx_mode: bool, shardlib):
    """Device-resident decode step of workload ``w``: returns timing dict and the replay fn."""
    dev = w.query.device
    kp, vp = w.planes()
    S, Hq, d = w.query.shape
    nblocks = w.key_cache.shape[0]
    out = torch.empty((S, Hq, d), dtype=w.query.dtype, device=dev)
    packed = torch.empty((S, Hq, d + 2), dtype=torch.float32, device=dev) if ctx_mode else None

    def step():
        if ctx_mode:
            # context shard: the rank's packed partial straight from the decode launch, ONE
            # NCCL all-gather, the merge of the ranks' partials
            ops.decode_attention(w.query, kp, vp, nblocks, w.block_table, w.seq_lens, w.n_kv_heads,
                                 d, PAGE, max_seq_len=w.max_seq_len, emit_partial=True, out=packed)
            gathered = shardlib.all_gather_packed(packed)
            return ops.combine_packed(gathered, out_dtype=w.query.dtype)
        return ops.decode_attention(w.query, kp, vp, nblocks, w.block_table, w.seq_lens,
                                    w.n_kv_heads, d, PAGE, max_seq_len=w.max_seq_len, out=out)

    replay, mode = capture(torch, step)
    for _ in range(W):
        replay()
    timed = Timed(torch, dev, need_flush=w.algorithmic_bytes() < 2 * 126e6)
    total_ms, each = timed.run(replay, K, barrier)
    return {"total_ms": total_ms, "each_ms": each, "mode": mode,
            "l2": ("L2 flushed (256 MB write) between timed steps" if timed.flush is not None
                   else "inputs larger than L2 (no flush needed)")}, replay


def ctx_breakdown(torch, ops, w, shardlib, barrier, n=30):
    """Where a context-sharded step spends its time: CUDA events around the three pieces of
    an EAGER step (decode launch that emits the rank's packed partial; NCCL all-gather;
    merge of the ranks' partials), median over ``n`` steps, plus the whole eager step."""
    dev = w.query.device
    kp, vp = w.planes()
    S, Hq, d = w.query.shape
    packed = torch.empty((S, Hq, d + 2), dtype=torch.float32, device=dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n)]
    for i in range(-3, n):
        e = ev[max(i, 0)]
        barrier()
        e[0].record()
        ops.decode_attention(w.query, kp, vp, w.key_cache.shape[0], w.block_table, w.seq_lens,
                             w.n_kv_heads, d, PAGE, max_seq_len=w.max_seq_len, emit_partial=True,
                             out=packed)
        e[1].record()
        gathered = shardlib.all_gather_packed(packed)
        e[2].record()
        ops.combine_packed(gathered, out_dtype=w.query.dtype)
        e[3].record()
    torch.cuda.synchronize()
    med = lambda a, b: pct([e[a].elapsed_time(e[b]) * 1e3 for e in ev], 0.5)
    return {"decode_emit_partial_us": med(0, 1), "all_gather_us": med(1, 2),
            "merge_ranks_us": med(2, 3), "eager_step_us": med(0, 3),
            "note": "eager calls, rank 0's events; launch gaps are inside the pieces"}


def summarize(name, w, res, K, peak_gbs):
    ms = res["total_ms"] / K
    alg = w.algorithmic_bytes()
    each = res["each_ms"]
    return {"workload": name, "us_per_step": ms * 1e3, "us_median": pct(each, 0.5) * 1e3,
            "us_p10": pct(each, 0.1) * 1e3, "us_p90": pct(each, 0.9) * 1e3,
            "algorithmic_bytes": alg, "tb_per_s": alg / (ms / 1e3) / 1e12,
            "frac": alg / (ms / 1e3) / 1e9 / peak_gbs, "steps": K, "l2": res["l2"],
            "n_seqs": w.n_seqs, "kv_heads_per_gpu": w.n_kv_heads, "max_seq_len": w.max_seq_len,
            "kv": f"K {w.k_mode} / V {w.v_mode}"}


def measure_append_loop(torch, ops, workloads, name, dev, K, W, barrier, peak_gbs, n_sub=64,
                        head_slice=None, fused=False):
    """Config 5 as stated: every step appends one new bf16 token per sequence to the cache
    (quantize-append, one launch for both planes) and then attends over the full cache, for
    ``n_sub`` consecutive steps with growing lengths.  The slots and lengths of all steps are
    precomputed on the device, the whole loop is one CUDA graph; a timed step is 1 / n_sub
    of a replay.  Replays rewrite the same slots with the same values."""
    w = workloads.config(name, dev, head_slice=head_slice, extra_blocks_per_seq=(n_sub + PAGE - 1) // PAGE + 1)
    kp, vp = w.planes()
    S, Hq, d = w.query.shape
    nblocks = w.key_cache.shape[0]
    L0 = torch.tensor(w.seq_lens_host, dtype=torch.int64)
    bt = w.block_table.cpu().to(torch.int64)
    lens, slots = [], []
    for i in range(n_sub):
        pos = L0 + i
        slots.append(bt[torch.arange(S), pos // PAGE] * PAGE + pos % PAGE)
        lens.append((pos + 1).to(torch.int32))
    lens_d = torch.stack(lens).to(dev)
    lens0_d = lens_d - 1
    slots_d = torch.stack(slots).to(dev)
    g = torch.Generator(device=dev).manual_seed(99)
    knew = torch.randn(n_sub, S, w.n_kv_heads, d, device=dev, generator=g).to(torch.bfloat16)
    vnew = torch.randn(n_sub, S, w.n_kv_heads, d, device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty((S, Hq, d), dtype=w.query.dtype, device=dev)
    max_len = w.max_seq_len + n_sub

    def loop():
        for i in range(n_sub):
            if fused:  # ONE launch appends the token and attends (lengths before the append)
                ops.decode_attention(w.query, kp, vp, nblocks, w.block_table, lens0_d[i],
                                     w.n_kv_heads, d, PAGE, max_seq_len=max_len, out=out,
                                     new_key=knew[i], new_value=vnew[i])
            else:
                ops.quant_append(knew[i], vnew[i], kp, vp, slots_d[i], PAGE)
                ops.decode_attention(w.query, kp, vp, nblocks, w.block_table, lens_d[i],
                                     w.n_kv_heads, d, PAGE, max_seq_len=max_len, out=out)

    replay, mode = capture(torch, loop, warm=1)
    for _ in range(max(1, W // 4)):
        replay()
    reps = max(2, K // 8)
    timed = Timed(torch, dev, need_flush=False)
    total_ms, each = timed.run(replay, reps, barrier)
    toks = sum(w.seq_lens_host)
    per_tok = w.kv_bytes_per_token_head() * w.n_kv_heads
    qo = w.query.numel() * w.query.element_size() * 2
    # per step i: the cache read at lengths L+i+1, the new token's bf16 K/V read and its codes written
    alg = sum((toks + S * (i + 1)) * per_tok + qo + S * w.n_kv_heads * (2 * d * 2) + S * per_tok
              for i in range(n_sub)) / n_sub
    ms = total_ms / reps / n_sub
    return {"workload": name + f" x {n_sub} append+attend steps, " +
                        ("append fused into the decode launch" if fused else "append launch + decode launch"),
            "us_per_step": ms * 1e3,
            "us_median": pct(each, 0.5) / n_sub * 1e3, "us_p10": pct(each, 0.1) / n_sub * 1e3,
            "us_p90": pct(each, 0.9) / n_sub * 1e3, "algorithmic_bytes": alg,
            "tb_per_s": alg / (ms / 1e3) / 1e12, "frac": alg / (ms / 1e3) / 1e9 / peak_gbs,
            "steps": reps * n_sub, "l2": "working set larger than L2", "mode": mode,
            "n_seqs": S, "kv_heads_per_gpu": w.n_kv_heads, "kv": f"K {w.k_mode} / V {w.v_mode}",
            "launches_per_step": 1 if fused else 2}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from knlp_b200 import ops, workloads
    from knlp_b200 import shard as shardlib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a short collective timeout: a rank that fell out of step ends the run in
        # minutes instead of holding the GPUs for NCCL's default ten
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    hq, total_kv_heads = shape_of(args.workload)[0:2]
    ctx_mode = args.shard == "context" and world > 1

    def head_slice_for(n_kv):
        if world == 1:
            return None
        if n_kv % world:
            raise SystemExit(f"--gpus must divide the {n_kv} kv heads")
        return shardlib.head_shard(n_kv, world, rank)

    # one spare page per sequence so the end-to-end leg can append a token
    w = workloads.config(args.workload, dev, scale=args.scale,
                         head_slice=None if ctx_mode else head_slice_for(total_kv_heads),
                         extra_blocks_per_seq=1, ctx_shard=(world, rank) if ctx_mode else None)
    S, Hq, d = w.query.shape
    K, W = args.steps, max(args.warmup, 3)
    peak_gbs, peak_kind = peaks()

    # warm the machine before the sampler starts, then time
    sampler = ClockSampler(local)
    if rank == 0 and not args.profile:
        sampler.start()
        time.sleep(0.25)
    res, replay = measure_decode(torch, ops, w, K, W, barrier, ctx_mode, shardlib)
    total_ms = res["total_ms"]
    # keep the load up for about a second more so the sampler sees the clocks.  The number
    # of extra steps is agreed between the ranks (a context shard has a collective per step).
    if not args.profile:
        extra = torch.tensor([min(20000, max(1, int(1000.0 / max(total_ms / K, 1e-3))))],
                             dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(extra, op=dist.ReduceOp.MAX)
        for _ in range(int(extra.item())):
            replay()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    head = summarize(args.workload, w, res, K, peak_gbs)
    if args.profile:
        # profiling run (under ncu): kernel timing only, no end-to-end, secondary or CPU legs
        if rank == 0:
            print(json.dumps({"profile_run": True, **head}), flush=True)
        teardown(torch, dist, world)
        return

    # ---------------- end to end through the operator API with host buffers
    # Per step the host supplies the query, the new token's K and V, its slots and the new
    # lengths in ONE pinned staging buffer (256-byte aligned regions): one h2d copy.  The
    # page table stays resident on the device, as a serving engine keeps it.
    kp, vp = w.planes()
    nblocks = w.key_cache.shape[0]
    L = w.seq_lens_host
    bt_h = w.block_table.cpu()
    q_h = w.query.cpu()
    knew_h = torch.randn(S, w.n_kv_heads, d, dtype=torch.float32).to(torch.bfloat16)
    vnew_h = torch.randn(S, w.n_kv_heads, d, dtype=torch.float32).to(torch.bfloat16)
    lens1_h = torch.tensor([x + 1 for x in L], dtype=torch.int32)
    slots_h = torch.tensor([int(bt_h[s, L[s] // PAGE]) * PAGE + L[s] % PAGE for s in range(S)],
                           dtype=torch.int64)
    host_inputs = (q_h, knew_h, vnew_h, lens1_h, slots_h)
    offs, total = [], 0
    for t in host_inputs:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    stage_h = torch.empty(total, dtype=torch.uint8).pin_memory()
    for t, o in zip(host_inputs, offs):
        nbytes = t.numel() * t.element_size()
        stage_h[o:o + nbytes].copy_(t.contiguous().view(-1).view(torch.uint8))
    out_h = torch.empty((S, Hq, d), dtype=w.query.dtype).pin_memory()
    stage_d = torch.empty(total, dtype=torch.uint8, device=dev)
    out_d = torch.empty((S, Hq, d), dtype=w.query.dtype, device=dev)
    packed_d = torch.empty((S, Hq, d + 2), dtype=torch.float32, device=dev) if ctx_mode else None
    h2d, d2h = total, out_h.numel() * out_h.element_size()

    def staged(i):
        t = host_inputs[i]
        nbytes = t.numel() * t.element_size()
        return stage_d[offs[i]:offs[i] + nbytes].view(t.dtype).view(t.shape)

    q_d, kn_d, vn_d, ln_d, sl_d = (staged(i) for i in range(5))
    # under a context shard only the rank that owns the end of a sequence appends to it
    append_here = (not ctx_mode) or rank == world - 1

    def e2e_step():
        stage_d.copy_(stage_h, non_blocking=True)
        if append_here:
            ops.quant_append(kn_d, vn_d, kp, vp, sl_d, PAGE)
        if ctx_mode:
            ops.decode_attention(q_d, kp, vp, nblocks, w.block_table,
                                 ln_d if append_here else w.seq_lens, w.n_kv_heads, d, PAGE,
                                 max_seq_len=w.max_seq_len + 1, emit_partial=True, out=packed_d)
            o = ops.combine_packed(shardlib.all_gather_packed(packed_d), out_dtype=w.query.dtype)
            out_h.copy_(o, non_blocking=True)
        else:
            ops.decode_attention(q_d, kp, vp, nblocks, w.block_table, ln_d, w.n_kv_heads, d, PAGE,
                                 max_seq_len=w.max_seq_len + 1, out=out_d)
            out_h.copy_(out_d, non_blocking=True)

    if args.e2e_eager:
        for _ in range(3):
            e2e_step()
        run_step, e2e_mode = e2e_step, "eager operator calls"
    else:
        run_step, e2e_mode = capture(torch, e2e_step)
        e2e_mode = "operator calls " + e2e_mode
    for _ in range(3):
        run_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    f0.record()
    for _ in range(K):
        run_step()
    f1.record()
    barrier()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(f0.elapsed_time(f1), e2e_wall_ms)  # host-side launch time counts too

    # ---------------- reduce over ranks
    alg_local = w.algorithmic_bytes()
    stats = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(alg_local), float(h2d), float(d2h)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms = stats.tolist()
    alg_total, h2d_total, d2h_total = tot.tolist()

    # ---------------- the other configurations, same method, same process
    secondary = []
    if not args.no_secondary and args.workload == "llama8b_b32_128k" and args.scale == 1.0:
        del w, kp, vp, replay, run_step
        torch.cuda.empty_cache()
        Ks, Ws = max(20, K), 5
        names = ["llama8b_b32_8k", "llama8b_b1_384k", "llama70b_ragged", "mixed_k8v4"]
        for name in names:
            n_kv = shape_of(name)[1]
            w2 = workloads.config(name, dev, head_slice=head_slice_for(n_kv))
            # the headline leaves the board at its power cap with the SM clock pulled down;
            # a short launch is not what holds it there, so let it settle and record the clock
            torch.cuda.synchronize()
            time.sleep(0.5)
            smp = ClockSampler(local)
            if rank == 0:
                smp.start()
            r2, rp2 = measure_decode(torch, ops, w2, Ks, Ws, barrier, False, shardlib)
            for _ in range(2000):
                rp2()
            torch.cuda.synchronize()
            row = summarize(name, w2, r2, Ks, peak_gbs)
            if rank == 0:
                c = smp.stop()
                row["sm_mhz"] = c.get("sm_mhz")
                row["clock_reasons"] = c.get("reasons")
            del rp2
            row["parallelism"] = "single GPU" if world == 1 else f"kv-head shard x{world}"
            secondary.append(row)
            del w2, r2, _
            torch.cuda.empty_cache()
        for fused in (False, True):
            row = measure_append_loop(torch, ops, workloads, "mixed_k8v4", dev, Ks, Ws, barrier,
                                      peak_gbs, head_slice=head_slice_for(8), fused=fused)
            row["parallelism"] = "single GPU" if world == 1 else f"kv-head shard x{world}"
            secondary.append(row)
            torch.cuda.empty_cache()
        if world > 1:
            # config 3 as stated: one long sequence split into contiguous context segments
            w3 = workloads.config("llama8b_b1_384k", dev, ctx_shard=(world, rank))
            r3, _ = measure_decode(torch, ops, w3, Ks, Ws, barrier, True, shardlib)
            row = summarize("llama8b_b1_384k", w3, r3, Ks, peak_gbs)
            row["parallelism"] = f"context shard x{world} (+1 NCCL all-gather of partials)"
            row["mode"] = r3["mode"]
            row["breakdown"] = ctx_breakdown(torch, ops, w3, shardlib, barrier)
            secondary.append(row)
            del w3, r3, _
            torch.cuda.empty_cache()
        side = []
        if world == 1:
            # the write path and the decode variants beside the headline (one GPU only)
            side += measure_write_path(torch, ops, workloads, dev, 10, 3)
            torch.cuda.empty_cache()
            side += measure_side_kernels(torch, ops, workloads, dev, Ks, peak_gbs)
            torch.cuda.empty_cache()
        # whole-job numbers: max time over ranks, bytes summed over ranks
        if world > 1:
            for row in secondary:
                t = torch.tensor([row["us_per_step"], row["us_median"]], dtype=torch.float64, device=dev)
                b = torch.tensor([float(row["algorithmic_bytes"])], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dist.all_reduce(b, op=dist.ReduceOp.SUM)
                row["us_per_step"], row["us_median"] = t.tolist()
                row["algorithmic_bytes"] = b.item()
                row["tb_per_s"] = b.item() / (row["us_per_step"] / 1e6) / 1e12
                row["frac_per_gpu"] = row["tb_per_s"] * 1e3 / world / peak_gbs
                row.pop("frac", None)
        secondary += side

    if rank == 0:
        ms_step = total_ms / K
        value = alg_total / (ms_step / 1e3) / 1e12
        # dominant kernel: the decode launch of ONE GPU (the step is that launch; with one
        # long sequence on the whole machine a ~3 us merge launch follows it inside the step)
        each = res["each_ms"]
        kern_ms = sum(each) / len(each)
        ach = alg_local / (kern_ms / 1e3) / 1e9
        cfg = job_config(args.workload, args.scale, world, args.shard)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
            "us_median": head["us_median"], "us_p10": head["us_p10"], "us_p90": head["us_p90"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u8 codes + f16 scales -> f16 mma, f32 accumulate", "data": "synthetic",
            "config": cfg,
            "run": {"kv_heads_per_gpu": head["kv_heads_per_gpu"], "l2": res["l2"],
                    "step": "decode_attention " + res["mode"],
                    "algorithmic_bytes_per_step": alg_total},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s",
                         "frac": ach / peak_gbs, "peak_kind": peak_kind,
                         "kernel": "decode_dq_kernel", "kernel_us": kern_ms * 1e3,
                         # DRAM bytes per launch on one GPU, scaled from the ncu capture of a
                         # smaller launch of the same kernel: reads = 1.0005 x the algorithmic
                         # bytes, writes = the partial slots (4 CTAs per SM + one per pair)
                         "traffic": int(1.0005 * alg_local + 4 * ops.decode_workspace_floats(
                             S, Hq, head["kv_heads_per_gpu"], d, PAGE, head["max_seq_len"])),
                         "traffic_source": "ncu dram__bytes of a smaller launch, scaled by tokens"},
            "e2e": {"value": alg_total / (e2e_ms / K / 1e3) / 1e12, "unit": UNIT,
                    "ms_per_step": e2e_ms / K, "mode": e2e_mode,
                    "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": int(d2h_total)},
            # kernels of this library in the timed region: one decode launch per step (plus
            # the all-gathered partials' merge under a context shard)
            "gpu_launches": (2 if ctx_mode else 1) * K,
            "secondary": secondary,
        }
        if world == 1 and not args.no_cpu:
            s = cpu_sample(args.workload, args.scale, 32768, repeats=40, warmup=3)
            line["cpu_baseline"] = {"value": s["value"], "unit": UNIT, "cores": s["cores"],
                                    "kind": "port", "sample": s["sample"],
                                    "ms_per_step_extrapolated": s["ms_per_step_extrapolated"],
                                    "cpu_extrapolated": s["cpu_extrapolated"]}
            # config 1 exactly as stated: GPT-2-small shape, the CPU path on the whole
            # workload (median of 50 after 5 warm-ups), beside this library on the same shape
            c1 = cpu_sample("gpt2_mha_1k", 1.0, 1024, repeats=50, warmup=5)
            w1 = workloads.config("gpt2_mha_1k", dev)
            r1, _ = measure_decode(torch, ops, w1, 50, 5, barrier, False, shardlib)
            line["config1_gpt2_mha_1k"] = {
                "cpu_us_median": c1["seconds_median"] * 1e6, "cpu_cores": c1["cores"],
                "cpu": "PyTorch eager fp32 dequantize -> SDPA, whole workload",
                "gpu_us_median": pct(r1["each_ms"], 0.5) * 1e3, "gpu": "decode_attention, " + r1["l2"]}
        print(json.dumps(line), flush=True)
    teardown(torch, dist, world)


def teardown(torch, dist, world):
    """Release every captured CUDA graph before the process group goes: a graph that holds
    a captured NCCL collective keeps the communicator busy and its destruction would wait
    for ever."""
    import gc
    torch.cuda.synchronize()
    for g in GRAPHS:
        g.reset()
    GRAPHS.clear()
    gc.collect()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def run_append_loop(args):
    """Side measurement: the append-then-attend loop of a workload (benchmark configuration
    5 is mixed_k8v4), with the append as its own launch and fused into the decode launch."""
    import torch
    from knlp_b200 import ops, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peak_gbs, _ = peaks()
    for fused in (False, True):
        row = measure_append_loop(torch, ops, workloads, args.workload, dev, max(args.steps, 20),
                                  args.warmup, torch.cuda.synchronize, peak_gbs, fused=fused)
        print(json.dumps(row), flush=True)
        torch.cuda.empty_cache()


def measure_write_path(torch, ops, workloads, dev, steps, warmup, scale=1.0):
    """The quantize-and-append kernel over a prefill-sized batch (tokens x 8 kv heads x 128,
    bf16, K and V, scattered slots): algorithmic read + write bytes per CUDA-event second,
    one row per quantizer."""
    n, h, d, P = int((1 << 20) * scale), 8, 128, 16
    g = torch.Generator(device=dev).manual_seed(1)
    k = torch.randn(n, h, d, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(n, h, d, device=dev, generator=g).to(torch.bfloat16)
    slots = torch.randperm(n, device=dev, generator=g).to(torch.int64)  # scattered pages
    nb = (n + P - 1) // P
    hbm_gbs, peak_kind = peaks()
    rows = []
    for mode, out_bytes in (("int4_asym", 160), ("int4_sym", 144), ("int8", 272)):
        kc, vc, ks, vs, kz, vz = workloads.alloc_cache(nb, h, d, mode, mode, dev)
        if mode == "int8":
            def step():
                ops.reshape_and_cache_k_int8(k, kc, ks, slots)
                ops.reshape_and_cache_v_int8(v, vc, vs, slots)
        else:
            asym = mode == "int4_asym"
            def step():
                ops.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz if asym else None,
                                           vz if asym else None, asymmetric=asym)
        for _ in range(max(warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        byts = n * h * (2 * d * 2 + out_bytes) + n * 8  # bf16 K and V in, codes/scales out, slots
        rows.append({"write_path": mode, "tokens": n, "kv_heads": h, "head_dim": d,
                     "src_dtype": "bf16", "ms_per_step": ms, "algorithmic_bytes": byts,
                     "value": byts / ms / 1e9, "unit": "TB/s",
                     "frac_of_hbm_peak": byts / ms / 1e6 / hbm_gbs, "peak": peak_kind,
                     "note": "inputs 4.3 GB > L2; K and V quantized per step"})
        del kc, vc, ks, vs, kz, vz
    return rows


def measure_side_kernels(torch, ops, workloads, dev, steps, peak_gbs):
    """Decode variants beside the headline, on the cache of llama8b_b32_8k (32 sequences x
    8192 tokens x 8 kv heads, shuffled 16-token pages), each one launch captured in a CUDA
    graph and replayed: an unquantized bf16 K plane with INT4 V, and routed decode (every kv
    head attends to its own top-64 blocks)."""
    from knlp_b200 import routing
    w = workloads.config("llama8b_b32_8k", dev)
    kp, vp = w.planes()
    S, Hq, d = w.query.shape
    Hkv, nb = w.n_kv_heads, w.key_cache.shape[0]
    rows = []

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        replay, _ = capture(torch, fn)
        for _ in range(3):
            replay()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(steps)]
        for a, b in ev:
            a.record()
            replay()
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in ev]

    # unquantized K: bf16 N(0,1) rows in the workload's own pages
    gen = torch.Generator(device=dev).manual_seed(3)
    kfp = torch.randn(nb, PAGE, Hkv, d, device=dev, generator=gen).to(torch.bfloat16)
    each = timed(lambda: ops.kfp16_vint4_decode(
        w.query, kfp, w.value_cache, w.v_scales, w.block_table, w.seq_lens, Hkv, d,
        v_zeros=w.v_zeros, asymmetric=True, max_seq_len=w.max_seq_len))
    tok = int(sum(w.seq_lens_host)) * Hkv
    byts = tok * (2 * d + d // 2 + (d // 32) * 4)
    us = pct(each, 0.5) * 1e3
    rows.append({"workload": "llama8b_b32_8k, K unquantized bf16 / V int4_asym (kfp16_vint4_decode)",
                 "us_median": us, "algorithmic_bytes": byts,
                 "tb_per_s": byts / us / 1e6, "frac": byts / us / 1e3 / peak_gbs, "steps": steps})
    del kfp
    # routed: 64 of each sequence's 512 blocks per kv head, drawn per head from the seed
    k_sel = 64
    prior = torch.rand(S, Hkv, w.block_table.shape[1], device=dev, generator=gen)
    idx = prior.topk(k_sel, dim=-1).indices
    tables = torch.gather(w.block_table[:, None, :].expand(-1, Hkv, -1).long(), 2, idx)
    tables = tables.to(torch.int32).contiguous()
    counts = torch.full((S, Hkv), k_sel, dtype=torch.int32, device=dev)
    each = timed(lambda: routing.fused_routed_decode(w.query, kp, vp, nb, PAGE, Hkv, tables, counts))
    byts = S * Hkv * k_sel * PAGE * w.kv_bytes_per_token_head()
    us = pct(each, 0.5) * 1e3
    rows.append({"workload": "llama8b_b32_8k, routed decode, 64 of 512 blocks per kv head",
                 "us_median": us, "algorithmic_bytes": byts,
                 "tb_per_s": byts / us / 1e6, "frac": byts / us / 1e3 / peak_gbs, "steps": steps})
    del w, kp, vp, tables, counts, prior, idx
    torch.cuda.empty_cache()
    # low-rank-V decode: 8 kv heads x 131072 tokens, bf16 K, rank-32 fp32 coefficients
    from knlp_b200 import lowrank
    hkv, nq, T, dh = 8, 4, 131072, 128
    Q = torch.randn(hkv, nq, dh, device=dev, generator=gen).to(torch.bfloat16)
    K = torch.randn(hkv, T, dh, device=dev, generator=gen).to(torch.bfloat16)
    proj = torch.randn(hkv, T, 32, device=dev, generator=gen)
    basis = torch.linalg.qr(torch.randn(hkv, dh, 32, device=dev, generator=gen)).Q.contiguous()
    each = timed(lambda: lowrank.lowrank_decode(Q, K, proj, basis))
    byts = hkv * T * (2 * dh + 4 * 32)
    us = pct(each, 0.5) * 1e3
    rows.append({"workload": "low-rank-V decode, 8 kv heads x 131072 tokens, bf16 K + rank-32 fp32",
                 "us_median": us, "algorithmic_bytes": byts,
                 "tb_per_s": byts / us / 1e6, "frac": byts / us / 1e3 / peak_gbs, "steps": steps})
    return rows


def run_side_kernels(args):
    """Side measurement: the decode variants beside the headline, one JSON line each."""
    import torch
    from knlp_b200 import ops, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peak_gbs, _ = peaks()
    for row in measure_side_kernels(torch, ops, workloads, dev, max(args.steps, 3), peak_gbs):
        print(json.dumps(row), flush=True)


def run_write_path(args):
    """Side measurement, not the headline: one JSON line per quantizer."""
    import torch
    from knlp_b200 import ops, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    for row in measure_write_path(torch, ops, workloads, dev, args.steps, args.warmup, args.scale):
        print(json.dumps(row))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b_b32_128k")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the other benchmark configurations measured after the headline")
    ap.add_argument("--shard", default="heads", choices=["heads", "context"],
                    help="how N > 1 GPUs split the work (default: kv heads, no exchange)")
    ap.add_argument("--profile", action="store_true",
                    help="short run for use under ncu: timed steps only, one JSON line of timings")
    ap.add_argument("--e2e-eager", action="store_true",
                    help="end-to-end leg as eager operator calls instead of one replayed CUDA graph")
    ap.add_argument("--append-loop", action="store_true",
                    help="time 64 append+attend steps of --workload, append separate and fused")
    ap.add_argument("--side-kernels", action="store_true",
                    help="time the decode variants beside the headline (unquantized K, routed, "
                         "low-rank V) and print one JSON line each")
    ap.add_argument("--write-path", action="store_true",
                    help="time the quantize-and-append kernel instead (side measurement)")
    args = ap.parse_args()
    shape_of(args.workload)  # unknown workloads are refused up front
    if args.side_kernels:
        run_side_kernels(args)
        return
    if args.write_path:
        run_write_path(args)
    elif args.append_loop:
        run_append_loop(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
