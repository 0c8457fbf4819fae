#!/usr/bin/env python
"""Benchmark of the paged KV decode path (append + GQA decode attention over pages).

Workload (N=1): batched decode at Qwen2.5-7B geometry — 28 layers, 28 q heads,
4 kv heads, head_dim 128, f16 K/V; 32 sequences per GPU with context lengths
uniform in [1024, 4096] from a seed; pages scattered over an arena of 8192 pages
(131072 tokens) by a seeded shuffle of the free-list.  One step = one token
appended per sequence + decode attention over every layer (28 fused launches).
With N GPUs every rank runs its own 32 sequences (sharded by sequence, no
collective in the path): weak scaling.

Prints ONE JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM;
`e2e` is the same step driven through the host-buffer entry point with the
host<->device copies inside the timed region; `roofline` is the decode kernel's
algorithmic bytes per launch over its CUDA-event duration against the measured
HBM copy bandwidth; `cpu_baseline` is the CPU oracle (a port of the reference
algorithm) timed on this box's host cores on a bounded sample.

`--impl reference` times that CPU port alone, with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, N_Q, N_KV, D, PAGE = 28, 28, 4, 128, 16
BATCH, CTX_LO, CTX_HI, ARENA_PAGES = 32, 1024, 4096, 8192
SEED = 0xC0B50002
SCALE = D ** -0.5
METRIC = "paged_decode_attention_tokens_per_s"
WINDOWS = None       # per-layer sliding windows (None = every layer global)
PREFIX = 0           # tokens of a prefix shared by page sharing (cfg5)
WORKLOAD = ("cfg2 qwen2.5-7b geometry batched decode: 28 layers, 28/4/128, batch 32 per GPU, "
            "ctx U[1024,4096], 8192-page arena, append + decode attention per layer")


def select_config(name: str) -> None:
    """cfg2 is the benchmark the headline metric is quoted on; cfg3 and cfg5 are run on request."""
    global LAYERS, N_Q, N_KV, D, BATCH, CTX_LO, CTX_HI, ARENA_PAGES, SEED, SCALE, WINDOWS, PREFIX, WORKLOAD
    if name == "cfg3":  # Gemma-3-4B-style: 5 local (w = 1024) : 1 global, batch 16 at 8192 tokens
        LAYERS, N_Q, N_KV, D, BATCH, CTX_LO, CTX_HI = 34, 8, 4, 256, 16, 8192, 8192
        ARENA_PAGES, SEED = 16 * 520, 0xC0B50003
        WINDOWS = [None if (i + 1) % 6 == 0 else 1024 for i in range(LAYERS)]
        WORKLOAD = ("cfg3 gemma-3-4b-style decode: 34 layers (5 local w=1024 : 1 global), 8/4/256, batch 16 per GPU, "
                    "ctx 8192, windows over paged KV")
    elif name == "cfg5":  # one GPU's shard of the churn workload: 64 sequences sharing a 1024-token prefix
        LAYERS, N_Q, N_KV, D, BATCH, CTX_LO, CTX_HI = 28, 28, 4, 128, 64, 128, 32768
        ARENA_PAGES, SEED, PREFIX = 40960, 0xC0B50005, 1024
        WORKLOAD = ("cfg5 qwen2.5-7b geometry serving shard: 64 sequences per GPU sharing a 1024-token prefix by page "
                    "sharing, suffix log-uniform [128,32768], decode step per sequence")
    SCALE = D ** -0.5


QUANT = False  # --quantize-kv: int8 KV pages (CacheConfig::quantize_kv)


def context_lengths(rank: int) -> np.ndarray:
    """Cached tokens per sequence before the first decode step (suffix lengths when a prefix is shared)."""
    rng = np.random.default_rng(SEED + 1000 * rank)
    if PREFIX:
        return np.round(np.exp(rng.uniform(np.log(CTX_LO), np.log(CTX_HI), BATCH))).astype(np.int64)
    return rng.integers(CTX_LO, CTX_HI + 1, BATCH)


def algorithmic_bytes_per_layer(lens_after: np.ndarray, window=None) -> float:
    """Per sequence: read K and V of the visible tokens, read Q / write O, read the new
    k,v and write them into the page, read the block-table ids."""
    L = lens_after.astype(np.float64)
    if window:
        L = np.minimum(L, float(window))
    if QUANT and not window:  # int8 pages: one byte per value plus one 2-byte scale per 32 values, K and V
        per = 2 * N_KV * (D + D // 16) * L + 4 * N_Q * D + 4 * N_KV * D + 2 * N_KV * (D + D // 16) + 4 * np.ceil(L / PAGE)
    else:
        per = 4 * N_KV * D * L + 4 * N_Q * D + 8 * N_KV * D + 4 * np.ceil(L / PAGE)
    return float(per.sum())


def algorithmic_bytes_per_step(lens_after: np.ndarray) -> float:
    wins = WINDOWS or [None] * LAYERS
    return sum(algorithmic_bytes_per_layer(lens_after, w) for w in wins)


# ------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons),
                "power_w_max": max(float(r[3]) for r in rows), "samples": len(rows)}


# ------------------------------------------------------------------ CPU port (oracle) timing
def time_cpu_port(n_seqs: int, n_layers: int, limit_s: float, lens: np.ndarray) -> dict:
    """The oracle's batch driver (a port of the reference algorithm: per-page scatter,
    materialised gather, repeat_kv, f32 upcast, scores, softmax, P.V) on host cores."""
    import oracle
    oracle.build()
    from oracle import OracleArena
    rng = np.random.default_rng(SEED)
    cores = oracle.set_threads(os.cpu_count() or 1)  # all host threads, whatever the launcher put in OMP_NUM_THREADS
    lens = lens[:n_seqs]
    pages = int(sum(-(-(int(n) + 64) // PAGE) for n in lens)) + 8
    arena = OracleArena(n_layers, N_KV, D, CTX_HI + 256, PAGE, pages, rolling=False, dtype="f16")
    seqs = [arena.new_seq() for _ in range(n_seqs)]
    arena.batch_begin(seqs, [int(n) for n in lens])
    for s, n in zip(seqs, lens):
        k = rng.standard_normal((N_KV, int(n), D)).astype(np.float16)
        v = rng.standard_normal((N_KV, int(n), D)).astype(np.float16)
        for layer in range(n_layers):
            s.append_only(layer, k, v, 0)
    ones = [1] * n_seqs
    q = rng.standard_normal(n_seqs * N_Q * D).astype(np.float16)
    k = rng.standard_normal(n_seqs * N_KV * D).astype(np.float16)
    v = rng.standard_normal(n_seqs * N_KV * D).astype(np.float16)
    steps, t0 = 0, time.perf_counter()
    while True:
        arena.batch_begin(seqs, ones)
        for layer in range(n_layers):
            arena.batch_layer(seqs, ones, layer, q, k, v, N_Q, SCALE)
        steps += 1
        el = time.perf_counter() - t0
        if el >= limit_s or steps >= 64:
            break
    # a token = one sequence advanced through all 28 layers
    value = n_seqs * steps * (n_layers / LAYERS) / el
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{n_seqs} sequences x {n_layers} of {LAYERS} layers x {steps} decode steps in {el:.1f} s, scaled by layers"}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    lens = context_lengths(0)
    # every "step" is a bounded sample: all 32 sequences, 2 of the 28 layers
    total_limit = 8.0 * max(1, args.steps + args.warmup)
    res = time_cpu_port(BATCH, 2, min(90.0, total_limit), lens)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": BATCH / res["value"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "cfg2 qwen2.5-7b geometry batched decode, batch 32, ctx U[1024,4096], 28 layers",
                   "note": "the reference (Rust on Burn/wgpu) cannot be built here; this is the CPU port of its algorithm"},
        "cpu_baseline": res,
        "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist
    from combsengine_b200 import KVArena, _lib, kv

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    lens = context_lengths(rank)
    total_steps = 3 * (args.steps + args.warmup) + 16
    arena = KVArena(LAYERS, N_Q, N_KV, D, PREFIX + CTX_HI + total_steps + 64, PAGE, ARENA_PAGES, windows=WINDOWS,
                    device=local_rank, sliding_popn_refuses=False, quantize_kv=QUANT)
    arena.set_free_list(np.random.default_rng(SEED + 7 + rank).permutation(ARENA_PAGES))
    if args.ctas_per_sm or args.stages or args.consumers or args.no_overlap or args.max_ctas:
        arena.set_decode_tuning(args.ctas_per_sm, args.stages, args.consumers, args.max_ctas, not args.no_overlap)
    if args.split:
        arena.set_decode_split(*[int(x) for x in args.split.split(",")])
    gen = torch.Generator(device=dev).manual_seed(SEED + rank)

    def fill(which, counts):
        """Cached context through the product path: one chunk step, append only."""
        ntok = int(sum(counts))
        kf = torch.randn(ntok * N_KV * D, device=dev, generator=gen).half()
        vf = torch.randn(ntok * N_KV * D, device=dev, generator=gen).half()
        arena.begin_step(which, [int(n) for n in counts])
        for layer in range(LAYERS):
            arena.append(layer, kf, vf)
        torch.cuda.synchronize()

    if PREFIX:  # every sequence forks the shared prefix (whole pages, refcounted), then gets its own suffix
        root = arena.new_seq()
        fill([root], [PREFIX])
        seqs = [root.fork_prefix(PREFIX) for _ in range(BATCH)]
    else:
        seqs = [arena.new_seq() for _ in range(BATCH)]
    fill(seqs, lens)
    lens = lens + PREFIX

    q = [torch.randn(BATCH * N_Q * D, device=dev, generator=gen).half() for _ in range(LAYERS)]
    k = [torch.randn(BATCH * N_KV * D, device=dev, generator=gen).half() for _ in range(LAYERS)]
    v = [torch.randn(BATCH * N_KV * D, device=dev, generator=gen).half() for _ in range(LAYERS)]
    out = [torch.empty_like(x) for x in q]
    qh = [x.cpu().pin_memory() for x in q]
    kh = [x.cpu().pin_memory() for x in k]
    vh = [x.cpu().pin_memory() for x in v]
    oh = [torch.empty_like(x).pin_memory() for x in qh]

    lib = _lib.load()
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    hs = (C.c_void_p * BATCH)(*[s._h for s in seqs])
    ones = (C.c_int64 * BATCH)(*([1] * BATCH))
    ah = C.c_void_p(arena._h)
    dargs = [(C.c_void_p(q[l].data_ptr()), C.c_void_p(k[l].data_ptr()), C.c_void_p(v[l].data_ptr()),
              C.c_void_p(out[l].data_ptr())) for l in range(LAYERS)]
    hargs = [(C.c_void_p(qh[l].data_ptr()), C.c_void_p(kh[l].data_ptr()), C.c_void_p(vh[l].data_ptr()),
              C.c_void_p(oh[l].data_ptr())) for l in range(LAYERS)]
    scale = C.c_double(SCALE)

    def step_device():
        _lib.check(lib.cbkv_begin_step(ah, hs, ones, None, BATCH, sp))
        for l in range(LAYERS):
            a = dargs[l]
            rc = lib.cbkv_attention(ah, l, a[0], a[1], a[2], a[3], scale, 0, sp)
            if rc:
                _lib.check(rc)

    def step_host():
        _lib.check(lib.cbkv_begin_step(ah, hs, ones, None, BATCH, sp))
        for l in range(LAYERS):
            a = hargs[l]
            rc = lib.cbkv_attention_host_async(ah, l, a[0], a[1], a[2], a[3], scale, 0, sp)
            if rc:
                _lib.check(rc)
        _lib.check(lib.cbkv_host_sync(ah))  # every layer's output is back in host memory

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, t0, t1

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = kv.launch_count()
    ms, t0, t1 = timed(step_device, args.steps, args.warmup)
    launches = kv.launch_count() - launches0
    launches_timed = launches * args.steps // (args.steps + args.warmup)
    clocks = sampler.summary(t0, t1) if rank == 0 else None
    assert arena.device_status() == 0, "kernel status word set"
    value = BATCH * world * args.steps / (ms * 1e-3)
    lens_mid = lens + 1 + args.warmup + args.steps // 2
    bytes_step = algorithmic_bytes_per_step(lens_mid)

    # roofline of the decode kernel: CUDA events around every launch, same steps again
    arena.profile_enable(True)
    for _ in range(args.steps):
        step_device()
    kms, kn = arena.profile_read()
    arena.profile_enable(False)
    lens_prof = lens + 1 + args.warmup + args.steps + args.steps // 2
    bytes_launch = algorithmic_bytes_per_step(lens_prof) / LAYERS  # mean over the layers of a step
    achieved = bytes_launch / (kms / kn * 1e-3) / 1e9

    # end to end: host buffers in, host buffers out, every layer
    ems, _, _ = timed(step_host, args.steps, args.warmup)
    e2e_value = BATCH * world * args.steps / (ems * 1e-3)
    h2d = LAYERS * (qh[0].numel() + kh[0].numel() + vh[0].numel()) * 2
    d2h = LAYERS * oh[0].numel() * 2
    assert arena.device_status() == 0
    if rank == 0:
        sampler.stop()

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"

    traffic = None
    tpath = os.path.join(ROOT, "profiles", f"decode_kernel_{args.config}_traffic.txt")
    if os.path.exists(tpath) and not args.layers and not QUANT:
        traffic = float(json.load(open(tpath))["traffic_bytes_per_launch"])  # from the committed ncu capture

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and args.config == "cfg2":
        cpu = time_cpu_port(8, 2, 12.0, context_lengths(0))

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD + (", int8 KV pages (quantize_kv): append quantises, decode reads records" if QUANT else ""),
                   "l2": f"inputs larger than L2 (about {bytes_step / 1e9:.1f} GB of KV read per step)",
                   "sharding": "by sequence, no collective"},
        "hbm_gbs": bytes_step * world / (ms / args.steps * 1e-3) / 1e9,
        "hbm_frac_of_8tbs": bytes_step / (ms / args.steps * 1e-3) / 8e12,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "kernel": f"decode_kernel<d={D},f16{',int8 pages' if QUANT else ''}>", "us_per_launch": kms / kn * 1e3,
                     "algorithmic_bytes_per_launch": bytes_launch, "peak_source": peak_src},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ems / args.steps},
        "gpu_launches": launches_timed,
        "clocks": clocks,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


def run_prefill(args, rank: int, world: int, local_rank: int) -> None:
    """cfg4: chunked prefill into the paged cache, Llama-3-8B geometry (32 layers, 32/8/128),
    8 prompts of 8192 tokens in 512-token chunks; per chunk and layer: append + causal attention
    over the paged prefix plus the chunk.  A step = one full pass over the 16 chunks."""
    import torch
    from combsengine_b200 import KVArena, _lib

    layers, n_q, n_kv, d, batch, prompt, chunk = 32, 32, 8, 128, 8, 8192, 512
    if args.layers:
        layers = args.layers
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    arena = KVArena(layers, n_q, n_kv, d, prompt + 64, 16, batch * (prompt // 16 + 4), device=local_rank,
                    quantize_kv=bool(args.quantize_kv))
    arena.set_free_list(np.random.default_rng(0xC0B50004).permutation(arena.num_pages))
    if args.chunk_kernel:
        arena.set_chunk_kernel(args.chunk_kernel)
    seqs = [arena.new_seq() for _ in range(batch)]
    gen = torch.Generator(device=dev).manual_seed(0xC0B50004)
    ntok = batch * chunk
    q = torch.randn(ntok * n_q * d, device=dev, generator=gen).half()
    k = torch.randn(ntok * n_kv * d, device=dev, generator=gen).half()
    v = torch.randn(ntok * n_kv * d, device=dev, generator=gen).half()
    out = torch.empty_like(q)
    scale = d ** -0.5
    stream = torch.cuda.current_stream()

    def one_pass():
        for c in range(prompt // chunk):
            arena.begin_step(seqs, [chunk] * batch)
            for layer in range(layers):
                arena.attention(layer, q, k, v, scale, out=out)
        for s in seqs:
            s.popn(prompt)

    for _ in range(max(1, args.warmup // 8)):
        one_pass()
    torch.cuda.synchronize()
    passes = max(1, args.steps // 16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(passes):
        one_pass()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / passes
    assert arena.device_status() == 0
    # Outside the timed region: the last chunk of one more pass, a few rows recomputed in float64.  Every
    # chunk appends the same k, v, so a prompt's cached K is its chunk of k repeated 16 times.
    for c in range(prompt // chunk):
        arena.begin_step(seqs, [chunk] * batch)
        for layer in range(layers):
            arena.attention(layer, q, k, v, scale, out=out)
    torch.cuda.synchronize()
    assert arena.device_status() == 0
    qh = q.cpu().numpy().reshape(batch, n_q, chunk, d).astype(np.float64)
    kh = np.tile(k.cpu().numpy().reshape(batch, n_kv, chunk, d).astype(np.float64), (1, 1, prompt // chunk, 1))
    vh = np.tile(v.cpu().numpy().reshape(batch, n_kv, chunk, d).astype(np.float64), (1, 1, prompt // chunk, 1))
    oh = out.cpu().numpy().reshape(batch, n_q, chunk, d).astype(np.float64)
    worst = 0.0
    for b, hq, r in ((0, 0, 0), (3, 17, 255), (7, 31, chunk - 1), (5, 9, 128)):
        p_abs = prompt - chunk + r
        sc = (kh[b, hq // (n_q // n_kv), :p_abs + 1] @ qh[b, hq, r]) * scale
        pr = np.exp(sc - sc.max())
        ref = (pr / pr.sum()) @ vh[b, hq // (n_q // n_kv), :p_abs + 1]
        err = np.abs(oh[b, hq, r] - ref)
        assert (err <= 2e-3 + 1e-2 * np.abs(ref)).all(), f"cfg4 spot check failed at prompt {b} head {hq} row {r}: {err.max()}"
        worst = max(worst, float(err.max()))
    for s in seqs:
        s.popn(prompt)
    pairs = prompt * (prompt + 1) // 2
    flops = 4.0 * n_q * d * pairs * layers * batch  # QK^T and PV over the causal pairs only
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks))["bf16_tflops"]) if os.path.exists(peaks) else 1590.0
    tfl = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "chunked_prefill_attention_tokens_per_s", "value": batch * prompt / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": passes, "warmup": max(1, args.warmup // 8), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"cfg4 llama-3-8b geometry chunked prefill: {layers} layers, 32/8/128, 8 prompts x 8192 in 512-token "
                               "chunks, append + causal attention over paged prefix + chunk"
                               + (", int8 KV pages (de-quantised per step into a float scratch layer)" if args.quantize_kv else ""),
                   "chunk_kernel": {0: "auto (tcgen05, two query tiles per CTA)", 1: "mma.sync", 2: "tcgen05, one query tile per CTA", 3: "tcgen05, two query tiles per CTA"}[args.chunk_kernel]},
        "roofline": {"bound": "tensor", "achieved": tfl, "peak": peak, "unit": "TFLOP/s", "frac": tfl / peak, "traffic": None,
                     "algorithmic_flops_per_pass": flops},
        "spot_check": {"rows": 4, "max_abs_err_vs_float64": worst, "tolerance": "2e-3 + 1e-2 |ref|"},
    }), flush=True)


def run_rope(args, rank: int, world: int, local_rank: int) -> None:
    """The step before the path, fused: per-head norm off, rotary embedding of q and k, k and v
    written into page slots, one launch per layer.  Workload: one 512-token chunk of each of the
    8 prompts of cfg4 (Llama-3-8B geometry 32/8/128, theta 500000), positions 4096..4607."""
    import time
    import torch
    from combsengine_b200 import KVArena
    from combsengine_b200 import rope as R

    layers, n_q, n_kv, d, batch, prefix, chunk = 32, 32, 8, 128, 8, 4096, 512
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    arena = KVArena(layers, n_q, n_kv, d, prefix + chunk, 16, batch * ((prefix + chunk) // 16), device=local_rank)
    arena.set_free_list(np.random.default_rng(0xC0B50004).permutation(arena.num_pages))
    seqs = [arena.new_seq() for _ in range(batch)]
    rope = R.RotaryEmbedding(arena, 500000.0, prefix + chunk)
    gen = torch.Generator(device=dev).manual_seed(0xC0B50004)
    ntok = batch * chunk
    nbuf = 4  # rotate over 4 input sets (4 x 50 MB) so that reads come from HBM, not L2
    q = [torch.randn(ntok * n_q * d, device=dev, generator=gen).half() for _ in range(nbuf)]
    k = [torch.randn(ntok * n_kv * d, device=dev, generator=gen).half() for _ in range(nbuf)]
    v = [torch.randn(ntok * n_kv * d, device=dev, generator=gen).half() for _ in range(nbuf)]
    qo = [torch.empty_like(q[0]) for _ in range(nbuf)]
    arena.begin_step(seqs, [prefix] * batch)       # the prefix's pages (contents irrelevant here)
    arena.begin_step(seqs, [chunk] * batch)
    stream = torch.cuda.current_stream()

    def one_pass():
        for layer in range(layers):
            i = layer % nbuf
            R.rope_append(arena, layer, rope, q[i], k[i], v[i], q_out=qo[i])

    for _ in range(max(3, args.warmup // 4)):
        one_pass()
    torch.cuda.synchronize()
    passes = max(2, args.steps // 4)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(passes):
        one_pass()
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (passes * layers)
    assert arena.device_status() == 0
    elems = ntok * d * 2
    alg = 2 * elems * n_q + 4 * elems * n_kv + ntok * (d // 2) * 4   # q r+w, k r+w, v r+w, one table row per token
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks))["hbm_gbs"]) if os.path.exists(peaks) else 6650.0
    gbs = alg / (us * 1e-6) / 1e9
    cpu = None
    if not args.no_cpu:
        import oracle
        oracle.build()
        cos, sin = oracle.rope_tables(d, 500000.0, prefix + chunk)
        xq = np.random.default_rng(1).standard_normal((n_q, chunk, d)).astype(np.float16)
        xk = xq[:n_kv].copy()
        t0 = time.perf_counter()
        oracle.rope_apply(xq, prefix, cos, sin); oracle.rope_apply(xk, prefix, cos, sin)
        dt = time.perf_counter() - t0
        cpu = {"value": chunk / dt, "unit": "tokens/s", "cores": 1, "kind": "port",
               "sample": f"rotation of q and k of one 512-token chunk of one prompt in {dt:.2f} s (scatter not included)"}
    print(json.dumps({
        "metric": "rope_append_tokens_per_s", "value": ntok / (us * 1e-6), "unit": "tokens/s", "n_gpus": 1,
        "steps": passes * layers, "warmup": max(3, args.warmup // 4) * layers, "ms_per_step": us * 1e-3,
        "higher_is_better": True, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "rotary embedding of q,k + append of k,v for a 512-token chunk of 8 prompts, 32/8/128, one launch per layer",
                   "l2": "four rotating input sets (200 MB) and 32 destination layers: larger than L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "kernel": "rope_append_kernel<f16>", "us_per_launch": us, "algorithmic_bytes_per_launch": alg},
        "gpu_launches": passes * layers, "cpu_baseline": cpu,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunk-kernel", type=int, default=0, help="cfg4 only: 1 = mma.sync, 2 = tcgen05 one tile per CTA, 3 = tcgen05 two tiles per CTA")
    ap.add_argument("--config", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5", "rope"],
                    help="cfg2 is the headline workload; cfg3 (windows, d=256) and cfg5 (shared prefix, long tails) on request")
    ap.add_argument("--ctas-per-sm", type=int, default=0, help="tuning: decode CTAs per SM (0 = default)")
    ap.add_argument("--stages", type=int, default=0, help="tuning: TMA ring stages (0 = default)")
    ap.add_argument("--consumers", type=int, default=0, help="tuning: consumer warps per decode CTA (4, 6, 8, 12)")
    ap.add_argument("--max-ctas", type=int, default=0, help="tuning: upper bound on the CTAs of a decode launch")
    ap.add_argument("--no-overlap", action="store_true", help="tuning: no programmatic dependent launch")
    ap.add_argument("--split", default="", help="tuning: tail_pct,min_item,max_levels of the decode work split (min_item 0 = static split)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quantize-kv", action="store_true", help="int8 KV pages (the reference's CacheConfig::quantize_kv)")
    ap.add_argument("--measure", action="store_true", help="load the measurement build (timers, CBKV_DEBUG switches)")
    ap.add_argument("--layers", type=int, default=0, help="profiling only: run fewer than the 28 layers (small ncu case)")
    args = ap.parse_args()
    if args.measure:
        from combsengine_b200 import _lib as _l
        _l.use_measure_build()
    if args.config == "cfg4":
        return run_prefill(args, int(os.environ.get("RANK", "0")), 1, int(os.environ.get("LOCAL_RANK", "0")))
    if args.config == "rope":
        return run_rope(args, int(os.environ.get("RANK", "0")), 1, int(os.environ.get("LOCAL_RANK", "0")))
    select_config(args.config)
    global QUANT
    QUANT = bool(args.quantize_kv)
    if args.layers:
        global LAYERS, WINDOWS
        LAYERS = args.layers
        if WINDOWS:
            WINDOWS = WINDOWS[:LAYERS]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
