#!/usr/bin/env python
"""Benchmark of the packed-INT4-KV decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--scale F]

A step is one decode-attention pass (split-context kernel + combine) over one
batch.  Default workload: Llama-3-8B shape (32 q / 8 kv heads, d 128), batch 32,
every sequence at 131 072 tokens of asymmetric INT4 KV (group 32, fp16 scale and
zero), bf16 queries, paged cache with 16-token pages — 5.37 GB of packed KV per
step, far larger than L2, so no flush is needed between steps.

With N > 1 (launched under torchrun, one rank per GPU) the kv heads are sharded
across ranks: rank r owns heads [r*8/N, (r+1)*8/N) of the same seeded cache and
their q heads; attention needs no exchange under a head shard, each rank keeps
its output slice.  Total work is fixed (strong scaling).

Prints ONE JSON line on rank 0.  ``value`` is whole-job algorithmic HBM
throughput with inputs resident; ``e2e`` is the same through the public
operator API with host buffers (pinned h2d of the step's query, new K/V token,
slots, lengths and page table; quantize-append; decode; d2h of the output).
``--impl reference`` times the CPU restatement of the reference's
dequantize-then-attend path on a bounded sample of the same workload.
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


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


# ------------------------------------------------------------------ CPU oracle leg
def cpu_reference_sample(workload: str, scale: float, sample_tokens: int, repeats: int,
                         inner: int = 1):
    """Time the CPU restatement of the reference path (oracle/kv_oracle.py) on a
    bounded sample: one sequence, all kv heads, ``sample_tokens`` tokens of the
    workload's distribution, quantized on the CPU by the oracle's own quantizer.
    One worker thread per kv head; a timed run attends to the sample ``inner`` times
    (``inner`` sequences of a batch).  Returns (bytes one run reads, [seconds of each of
    the ``repeats`` runs], threads, description)."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import kv_oracle as O

    shapes = {"llama8b_b32_128k": (32, 8, 128, 131072), "llama8b_b32_8k": (32, 8, 128, 8192),
              "llama8b_b1_384k": (32, 8, 128, 393216)}
    hq, hkv, d, ctx = shapes.get(workload, (32, 8, 128, 131072))
    T = min(int(ctx * scale), sample_tokens)
    rng = np.random.default_rng(2000)
    chs = np.where(rng.random((hkv, d)) < 0.01, 10.0, 1.0).astype(np.float32)
    k = (rng.standard_normal((T, hkv, d), dtype=np.float32) * chs)
    v = (rng.standard_normal((T, hkv, d), dtype=np.float32) * chs)
    q = rng.standard_normal((1, hq, d), dtype=np.float32)
    nb = (T + PAGE - 1) // PAGE
    kc = np.zeros((nb, PAGE, hkv, d // 2), np.uint8); vc = np.zeros_like(kc)
    ks = np.zeros((nb, PAGE, hkv, d // 32), np.float16)
    vs, kz, vz = np.zeros_like(ks), np.zeros_like(ks), np.zeros_like(ks)
    O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, np.arange(T), kz, vz, asymmetric=True)
    del k, v
    bt = np.arange(nb, dtype=np.int32)[None]
    sl = np.array([T], np.int32)
    n_rep = hq // hkv
    threads = min(hkv * inner, os.cpu_count() or 1)  # every (sequence, kv head) is a work unit

    def one_head(h):
        sl_h = slice(h, h + 1)
        return O.fused_int4_decode(q[:, h * n_rep:(h + 1) * n_rep], kc[:, :, sl_h], vc[:, :, sl_h],
                                   ks[:, :, sl_h], vs[:, :, sl_h], bt, sl, 1, d,
                                   k_zeros=kz[:, :, sl_h], v_zeros=vz[:, :, sl_h], asymmetric=True)

    secs = []
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(ex.map(one_head, [h for _ in range(inner) for h in range(hkv)]))
            secs.append(time.perf_counter() - t0)
    nbytes = inner * (T * hkv * 160 + q.size * 4 * 2 + 4 * nb)
    desc = (f"{inner} x (1 sequence x {hkv} kv heads x {T} tokens of the workload's distribution) "
            f"= {inner * T / (32 * ctx * scale):.3g} of a step, numpy oracle, {threads} threads")
    return nbytes, secs, threads, desc


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # one step = as many sequences of the sample as keep every host core busy
    inner = max(1, (os.cpu_count() or 8) // 8)
    nbytes, secs, threads, desc = cpu_reference_sample(args.workload, args.scale, 16384,
                                                       args.warmup + args.steps, inner=inner)
    secs = secs[args.warmup:]
    ms = 1e3 * sum(secs) / len(secs)
    value = nbytes / (ms / 1e3) / 1e12  # bytes of the sample / mean step time
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u8 codes + f16 scales -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "scale": args.scale, "sample": desc,
                   "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from knlp_b200 import ops, workloads

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

    from knlp_b200 import shard as shardlib
    ctx_mode = args.shard == "context" and world > 1
    total_kv_heads = 8
    hs = None
    if world > 1 and not ctx_mode:
        if total_kv_heads % world:
            raise SystemExit("--gpus must divide the 8 kv heads")
        hs = shardlib.head_shard(total_kv_heads, world, rank)

    # one spare page per sequence so the end-to-end leg can append a token
    w = workloads.config(args.workload, dev, scale=args.scale, head_slice=hs,
                         extra_blocks_per_seq=1,
                         ctx_shard=(world, rank) if ctx_mode else None)
    S, Hq, d = w.query.shape
    n_splits = args.splits or ops.plan_splits(S, Hq, w.n_kv_heads, d, PAGE, w.max_seq_len)
    from knlp_b200.ops import _plane, _int4_mode, _lib
    asym = w.k_mode == "int4_asym"
    if w.k_mode == "int8":
        kp = _plane(w.key_cache, w.k_scales, None, _lib.KV_INT8_G32)
    else:
        kp = _plane(w.key_cache, w.k_scales, w.k_zeros if asym else None, _int4_mode(asym, w.k_zeros))
    vasym = w.v_mode == "int4_asym"
    if w.v_mode == "int8":
        vp = _plane(w.value_cache, w.v_scales, None, _lib.KV_INT8_G32)
    else:
        vp = _plane(w.value_cache, w.v_scales, w.v_zeros if vasym else None,
                    _int4_mode(vasym, w.v_zeros))
    nblocks = w.key_cache.shape[0]

    two_launches = (not args.single_launch) or ctx_mode

    def step(seq_lens, max_len, rec=None):
        if rec is not None:
            rec[0].record()
        if not two_launches:
            # one launch: split-context decode whose last CTA per row group merges the splits
            o = ops.decode_attention(w.query, kp, vp, nblocks, w.block_table, seq_lens,
                                     w.n_kv_heads, d, PAGE, max_seq_len=max_len,
                                     n_splits=n_splits)
            if rec is not None:
                rec[1].record()
            return o
        pm, pl, po = ops.decode_partials(w.query, kp, vp, nblocks, w.block_table, seq_lens,
                                         w.n_kv_heads, d, PAGE, max_seq_len=max_len,
                                         n_splits=n_splits)
        if rec is not None:
            rec[1].record()
        if ctx_mode:
            # context shard: one packed partial per rank, ONE NCCL all-gather, final merge
            return shardlib.context_sharded_decode((pm, pl, po), out_dtype=w.query.dtype)
        return ops.combine_partials(pm, pl, po, out_dtype=w.query.dtype)

    for _ in range(max(args.warmup, 3)):
        out = step(w.seq_lens, w.max_seq_len)
    barrier()

    K = args.steps
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0 and not args.profile:
        sampler.start()
        time.sleep(0.25)
    # L2 is 126 MB.  A working set of at least twice that is streamed without help;
    # a smaller one (a small shard of a small workload) gets L2 flushed by writing a
    # 256 MB buffer between the timed steps, and the steps are timed one by one.
    need_flush = w.algorithmic_bytes() < 2 * 126e6
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if need_flush else None
    sev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(K)]
    barrier()
    e0.record()
    for i in range(K):
        if need_flush:
            flush_buf.fill_(i & 0xFF)
        sev[i][0].record()
        out = step(w.seq_lens, w.max_seq_len, ev[i])
        sev[i][1].record()
    e1.record()
    barrier()
    total_ms = (sum(a.elapsed_time(b) for a, b in sev) if need_flush else e0.elapsed_time(e1))
    kern_ms = sum(a.elapsed_time(b) for a, b in ev) / K
    # keep the load up for about a second more so the sampler sees the clocks.  The
    # number of extra steps is agreed between the ranks (a context shard has a collective
    # in every step, so every rank must run the same count).
    if not args.profile:
        extra = torch.tensor([min(20000, max(1, int(1000.0 / max(total_ms / K, 1e-3))))],
                             dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(extra, op=dist.ReduceOp.MAX)
        for _ in range(int(extra.item())):
            step(w.seq_lens, w.max_seq_len)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if args.profile:
        # profiling run (under ncu): kernel timing only, no end-to-end or CPU legs
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload,
                              "ms_per_step": total_ms / K, "kernel_us": kern_ms * 1e3,
                              "n_splits": n_splits, "algorithmic_bytes": w.algorithmic_bytes()}),
                  flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- end to end through the operator API with host buffers
    L = w.seq_lens_host
    q_h = w.query.cpu().pin_memory()
    knew_h = torch.randn(S, w.n_kv_heads, d, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    vnew_h = torch.randn(S, w.n_kv_heads, d, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    bt_h = w.block_table.cpu().pin_memory()
    lens1_h = torch.tensor([x + 1 for x in L], dtype=torch.int32).pin_memory()
    slots_h = torch.tensor([int(bt_h[s, L[s] // PAGE]) * PAGE + L[s] % PAGE for s in range(S)],
                           dtype=torch.int64).pin_memory()
    out_h = torch.empty((S, Hq, d), dtype=w.query.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (q_h, knew_h, vnew_h, bt_h, lens1_h, slots_h))
    d2h = out_h.numel() * out_h.element_size()
    caches = (w.key_cache, w.value_cache, w.k_scales, w.v_scales, w.k_zeros, w.v_zeros)

    # The step's host inputs sit in ONE pinned staging buffer (256-byte aligned regions), as a
    # serving engine lays them out: one h2d copy per step instead of six.
    host_inputs = (q_h, knew_h, vnew_h, bt_h, lens1_h, slots_h)
    offs, total = [], 0
    for t in host_inputs:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    stage_h = torch.empty(total, dtype=torch.uint8).pin_memory()
    for t, o in zip(host_inputs, offs):
        nbytes = t.numel() * t.element_size()
        stage_h[o:o + nbytes].copy_(t.contiguous().view(-1).view(torch.uint8))
    h2d = total

    def staged(st, i):
        t = host_inputs[i]
        nbytes = t.numel() * t.element_size()
        return st[offs[i]:offs[i] + nbytes].view(t.dtype).view(t.shape)

    def e2e_step():
        st = stage_h.to(dev, non_blocking=True)
        q, kn, vn, bt, ln, sl = (staged(st, i) for i in range(6))
        workloads.append_tokens(caches, kn, vn, sl, w.k_mode, w.v_mode)
        if not two_launches:
            o = ops.decode_attention(q, kp, vp, nblocks, bt, ln, w.n_kv_heads, d, PAGE,
                                     max_seq_len=w.max_seq_len + 1, n_splits=n_splits)
        else:
            pm, pl, po = ops.decode_partials(q, kp, vp, nblocks, bt, ln, w.n_kv_heads, d, PAGE,
                                             max_seq_len=w.max_seq_len + 1, n_splits=n_splits)
            if ctx_mode:
                o = shardlib.context_sharded_decode((pm, pl, po), out_dtype=w.query.dtype)
            else:
                o = ops.combine_partials(pm, pl, po, out_dtype=w.query.dtype)
        out_h.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    run_step, e2e_mode = e2e_step, "eager operator calls"
    if not ctx_mode and not args.e2e_eager:
        # The library's calls neither allocate nor synchronise, so the whole step (pinned h2d
        # copies, quantize-append, decode, combine, d2h) is captured once in a CUDA graph and
        # replayed: one host call per step instead of a dozen.  The copies are graph nodes that
        # read the pinned host buffers at every replay.
        eager_out = out_h.clone()
        graph = torch.cuda.CUDAGraph()
        try:
            # thread-local: CUDA calls of other threads (a process group's watchdog) are theirs
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                e2e_step()
        except RuntimeError as exc:  # capture refused: the same calls run eagerly instead
            graph = None
            torch.cuda.synchronize()
            e2e_mode = f"eager operator calls (graph capture failed: {str(exc)[:80]})"
        if graph is not None:
            out_h.zero_()
            graph.replay()
            torch.cuda.synchronize()
            if not torch.equal(out_h, eager_out):
                raise RuntimeError("graph replay of the end-to-end step differs from the eager step")
            run_step, e2e_mode = graph.replay, "operator calls captured in one CUDA graph, replayed"
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
    stats = torch.tensor([total_ms, kern_ms, e2e_ms], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(alg_local), float(h2d), float(d2h)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    total_ms, kern_ms, e2e_ms = stats.tolist()
    alg_total, h2d_total, d2h_total = tot.tolist()

    if rank == 0:
        ms_step = total_ms / K
        peak_gbs, peak_kind = peaks()
        value = alg_total / (ms_step / 1e3) / 1e12
        # dominant kernel: the split-context decode kernel of ONE GPU
        ach = alg_local / (kern_ms / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u8 codes + f16 scales -> f16 mma, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "scale": args.scale, "n_seqs": S,
                       "q_heads_per_gpu": Hq, "kv_heads_per_gpu": w.n_kv_heads, "head_dim": d,
                       "context": w.max_seq_len, "kv": f"K {w.k_mode} / V {w.v_mode}, group 32",
                       "page": PAGE, "n_splits": n_splits,
                       "parallelism": (f"context shard x{world} (+1 NCCL all-gather of partials)"
                                       if ctx_mode else f"kv-head shard x{world}")
                       if world > 1 else "single GPU",
                       "l2": ("L2 flushed (256 MB write) between timed steps"
                              if need_flush else "inputs larger than L2 (no flush needed)"),
                       "algorithmic_bytes_per_step": alg_total},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s",
                         "frac": ach / peak_gbs, "peak_kind": peak_kind,
                         "kernel": "decode_mma_kernel", "kernel_us": kern_ms * 1e3,
                         # DRAM bytes per launch on one GPU, scaled from the ncu capture of
                         # the 8K-context case (profiles/decode_mma_kernel_*_ncu_full.md):
                         # reads = 0.9996 x algorithmic bytes, writes = the split partials
                         "traffic": int(0.9996 * alg_local + S * Hq * n_splits * (d + 2) * 4),
                         "traffic_source": "ncu dram__bytes of a smaller launch, scaled by tokens"},
            "e2e": {"value": alg_total / (e2e_ms / K / 1e3) / 1e12, "unit": UNIT,
                    "ms_per_step": e2e_ms / K, "mode": e2e_mode,
                    "h2d_bytes_per_step": int(h2d_total),
                    "d2h_bytes_per_step": int(d2h_total)},
            # kernels of this library in the timed region per step: decode + combine (a
            # context shard merges twice; --single-launch merges inside the decode kernel)
            "gpu_launches": (3 if ctx_mode else 2 if two_launches else 1) * K,
        }
        if world == 1 and not args.no_cpu:
            nbytes, secs, threads, desc = cpu_reference_sample(args.workload, args.scale, 65536, 4, inner=16)
            best = min(secs[1:])
            line["cpu_baseline"] = {"value": nbytes / best / 1e12, "unit": UNIT, "cores": threads,
                                    "kind": "port", "sample": desc + ", best of 3 after 1 warm-up",
                                    "seconds": best}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_write_path(args):
    """Side measurement, not the headline: the quantize-and-append kernel over a prefill-sized
    batch (tokens x 8 kv heads x 128, bf16, K and V), algorithmic read + write bytes per
    CUDA-event second.  One JSON line per quantizer."""
    import torch
    from knlp_b200 import ops, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    n, h, d, P = int((1 << 20) * args.scale), 8, 128, 16
    g = torch.Generator(device=dev).manual_seed(1)
    k = torch.randn(n, h, d, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(n, h, d, device=dev, generator=g).to(torch.bfloat16)
    slots = torch.randperm(n, device=dev, generator=g).to(torch.int64)  # scattered pages
    nb = (n + P - 1) // P
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
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        byts = n * h * (2 * d * 2 + out_bytes) + n * 8  # bf16 K and V in, codes/scales out, slots
        hbm_gbs, peak_kind = peaks()
        print(json.dumps({"write_path": mode, "tokens": n, "kv_heads": h, "head_dim": d,
                          "src_dtype": "bf16", "ms_per_step": ms, "algorithmic_bytes": byts,
                          "value": byts / ms / 1e9, "unit": "TB/s",
                          "frac_of_hbm_peak": byts / ms / 1e6 / hbm_gbs, "peak": peak_kind,
                          "note": "inputs 4.3 GB > L2; K and V quantized per step"}))
        del kc, vc, ks, vs, kz, vz


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b_b32_128k")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--single-launch", action="store_true",
                    help="merge the splits inside the decode kernel (its last CTA per row group) "
                         "instead of the separate combine kernel; measured slightly slower")
    ap.add_argument("--shard", default="heads", choices=["heads", "context"],
                    help="how N > 1 GPUs split the work (default: kv heads, no exchange)")
    ap.add_argument("--profile", action="store_true",
                    help="short run for use under ncu: timed steps only, one JSON line of timings")
    ap.add_argument("--e2e-eager", action="store_true",
                    help="end-to-end leg as eager operator calls instead of one replayed CUDA graph")
    ap.add_argument("--write-path", action="store_true",
                    help="time the quantize-and-append kernel instead (side measurement)")
    args = ap.parse_args()
    if args.write_path:
        run_write_path(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
