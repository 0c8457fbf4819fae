#!/usr/bin/env python
"""Benchmark of the paged KV decode path (append + GQA decode attention over pages).

Headline workload (cfg2): batched decode at Qwen2.5-7B geometry — 28 layers, 28 q heads,
4 kv heads, head_dim 128, f16 K/V; 32 sequences per GPU with context lengths uniform in
[1024, 4096] from a seed; pages scattered over an arena of 8192 pages (131072 tokens) by a
seeded shuffle of the free-list.  One step = one token appended per sequence + decode
attention over every layer (28 fused launches).

With N GPUs ONE population of 32 * N sequences is drawn from one seed on every rank and
assigned to ranks by page count (longest processing time first); every rank builds only its
own sequences.  Nothing crosses GPUs inside the path (weak scaling); only the timing is
reduced (max over ranks).  A head-sharded leg (kv heads split across a group of ranks, one
NCCL all-gather of the outputs per layer) is measured next to it.

Prints ONE JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM; `e2e` is the
same step driven through the host-buffer entry point with the host<->device copies inside
the timed region; `roofline` is the decode kernel's algorithmic bytes per launch over its
CUDA-event duration against the measured HBM copy bandwidth, plus the step-level fraction;
`cpu_baseline` is the CPU oracle (a port of the reference algorithm) timed on this box's host
cores on a bounded sample; `also` holds short runs of the other configurations.

`--impl reference` times that CPU port alone, with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, replace
from typing import List, Optional

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PAGE = 16
METRIC = "paged_decode_attention_tokens_per_s"


@dataclass
class Workload:
    """One decode configuration: geometry, batch per GPU, context distribution, arena."""
    name: str
    layers: int
    n_q: int
    n_kv: int
    d: int
    batch: int
    ctx_lo: int
    ctx_hi: int
    arena_pages: int
    seed: int
    text: str
    windows: Optional[List[Optional[int]]] = None  # per-layer sliding windows (None = every layer global)
    prefix: int = 0                                # tokens of a prefix shared by page sharing (cfg5)
    quant: bool = False                            # int8 KV pages (CacheConfig::quantize_kv)

    @property
    def scale(self) -> float:
        return self.d ** -0.5

    def lengths(self, count: int) -> np.ndarray:
        """Cached tokens per sequence before the first decode step (suffix lengths when a prefix is shared);
        one seeded population, the same on every rank."""
        rng = np.random.default_rng(self.seed)
        if self.prefix:
            return np.round(np.exp(rng.uniform(np.log(self.ctx_lo), np.log(self.ctx_hi), count))).astype(np.int64)
        return rng.integers(self.ctx_lo, self.ctx_hi + 1, count)

    def bytes_per_layer(self, lens_after: np.ndarray, window=None, shared_prefix_once: bool = False) -> float:
        """Algorithmic bytes of one layer of one decode step.  Per sequence: read K and V of the visible tokens,
        read Q / write O, read the new k,v and write them into the page, read the block-table ids.
        shared_prefix_once: count the shared prefix's K/V once instead of once per sequence."""
        L = lens_after.astype(np.float64)
        if window:
            L = np.minimum(L, float(window))
        if self.quant and not window:  # int8 pages: one byte per value plus one 2-byte scale per 32 values, K and V
            kv_tok = 2 * self.n_kv * (self.d + self.d // 16)
            fixed = 4 * self.n_q * self.d + 4 * self.n_kv * self.d + kv_tok
        else:
            kv_tok = 4 * self.n_kv * self.d
            fixed = 4 * self.n_q * self.d + 8 * self.n_kv * self.d
        per = kv_tok * L + fixed + 4 * np.ceil(L / PAGE)
        total = float(per.sum())
        if shared_prefix_once and self.prefix and not window:
            total -= kv_tok * self.prefix * (len(L) - 1)
        return total

    def bytes_per_step(self, lens_after: np.ndarray, shared_prefix_once: bool = False) -> float:
        wins = self.windows or [None] * self.layers
        return sum(self.bytes_per_layer(lens_after, w, shared_prefix_once) for w in wins)


CFG2_TEXT = ("cfg2 qwen2.5-7b geometry batched decode: 28 layers, 28/4/128, batch 32 per GPU, "
             "ctx U[1024,4096], 8192-page arena, append + decode attention per layer")


def workload(name: str, layers: int = 0, quant: bool = False) -> Workload:
    if name == "cfg3":  # Gemma-3-4B-style: 5 local (w = 1024) : 1 global, batch 16 at 8192 tokens
        w = Workload("cfg3", 34, 8, 4, 256, 16, 8192, 8192, 16 * 640, 0xC0B50003,
                     "cfg3 gemma-3-4b-style decode: 34 layers (5 local w=1024 : 1 global), 8/4/256, batch 16 per GPU, "
                     "ctx 8192, windows over paged KV",
                     windows=[None if (i + 1) % 6 == 0 else 1024 for i in range(34)])
    elif name == "cfg1":  # the reference's own small case: one sequence, one layer; a step is bound by launch latency
        w = Workload("cfg1", 1, 9, 3, 64, 1, 512, 512, 64, 0xC0B50001,
                     "cfg1 smollm2-135m geometry: 1 layer, 9/3/64, one sequence, 512-token prefix, 64-page arena, append + "
                     "decode attention per step (0.4 MB per step: the time of a step is launch latency)")
    elif name == "cfg5":  # one GPU's shard of the churn workload: 64 sequences sharing a 1024-token prefix
        w = Workload("cfg5", 28, 28, 4, 128, 64, 128, 32768, 40960, 0xC0B50005,
                     "cfg5 qwen2.5-7b geometry serving shard: 64 sequences per GPU sharing a 1024-token prefix by page "
                     "sharing, suffix log-uniform [128,32768], decode step per sequence", prefix=1024)
    else:
        w = Workload("cfg2", 28, 28, 4, 128, 32, 1024, 4096, 8192, 0xC0B50002, CFG2_TEXT)
    if layers:
        w = replace(w, layers=layers, windows=w.windows[:layers] if w.windows else None)
    if quant:
        w = replace(w, quant=True, text=w.text + ", int8 KV pages (quantize_kv): append quantises, decode reads records")
    return w


def peak_sustained():
    """Dense bf16 TFLOP/s of a seconds-long cuBLAS loop under the power cap (MEASURED_PEAKS.json), or None."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        v = json.load(open(path)).get("bf16_tflops_sustained")
        return float(v) if v else None
    return 1400.0  # the fallback's sustained figure


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback"


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
CPU_SAMPLE_LAYERS = 2  # both CPU legs time all 32 sequences over this many of the 28 layers and scale by layers


def time_cpu_port(w: Workload, n_seqs: int, n_layers: int, limit_s: float, max_steps: int = 64) -> dict:
    """The oracle's batch driver (a port of the reference algorithm: per-page scatter,
    materialised gather, repeat_kv, f32 upcast, scores, softmax, P.V) on host cores."""
    import oracle
    oracle.build()
    from oracle import OracleArena
    rng = np.random.default_rng(w.seed)
    cores = oracle.set_threads(os.cpu_count() or 1)  # all host threads, whatever the launcher put in OMP_NUM_THREADS
    lens = w.lengths(w.batch)[:n_seqs]
    pages = int(sum(-(-(int(n) + max_steps + 16) // PAGE) for n in lens)) + 8
    arena = OracleArena(n_layers, w.n_kv, w.d, w.ctx_hi + 256, PAGE, pages, rolling=False, dtype="f16")
    seqs = [arena.new_seq() for _ in range(n_seqs)]
    arena.batch_begin(seqs, [int(n) for n in lens])
    for s, n in zip(seqs, lens):
        k = rng.standard_normal((w.n_kv, int(n), w.d)).astype(np.float16)
        v = rng.standard_normal((w.n_kv, int(n), w.d)).astype(np.float16)
        for layer in range(n_layers):
            s.append_only(layer, k, v, 0)
    ones = [1] * n_seqs
    q = rng.standard_normal(n_seqs * w.n_q * w.d).astype(np.float16)
    k = rng.standard_normal(n_seqs * w.n_kv * w.d).astype(np.float16)
    v = rng.standard_normal(n_seqs * w.n_kv * w.d).astype(np.float16)
    steps, t0 = 0, time.perf_counter()
    while True:
        arena.batch_begin(seqs, ones)
        for layer in range(n_layers):
            arena.batch_layer(seqs, ones, layer, q, k, v, w.n_q, w.scale)
        steps += 1
        el = time.perf_counter() - t0
        if el >= limit_s or steps >= max_steps:
            break
    # a token = one sequence advanced through all layers of the configuration
    value = n_seqs * steps * (n_layers / w.layers) / el
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{n_seqs} sequences x {n_layers} of {w.layers} layers x {steps} decode steps in {el:.1f} s, scaled by layers"}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    w = workload("cfg2")
    # every "step" is a bounded sample: all 32 sequences, 2 of the 28 layers
    total_limit = 8.0 * max(1, args.steps + args.warmup)
    res = time_cpu_port(w, w.batch, CPU_SAMPLE_LAYERS, min(90.0, total_limit))
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": w.batch / res["value"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": w.text,
                   "note": "the reference (Rust on Burn/wgpu) cannot be built here; this is the CPU port of its algorithm "
                           "on one host, whatever --gpus says"},
        "cpu_baseline": res,
        "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def _launch_count() -> int:
    from combsengine_b200 import kv
    return kv.launch_count()


def _partition(lens_total: np.ndarray, world: int) -> List[List[int]]:
    from combsengine_b200.sharding import partition_sequences
    return partition_sequences([int(x) for x in lens_total], world, PAGE)


class DecodeRun:
    """One workload built on this rank's GPU: arena, sequences, per-layer inputs, and the timed loops."""

    def __init__(self, w: Workload, lens: np.ndarray, local_rank: int, args, seed_salt: int = 0, host_buffers: bool = False,
                 n_q: Optional[int] = None, n_kv: Optional[int] = None):
        import torch
        from combsengine_b200 import KVArena, _lib
        self.torch, self.w, self.args = torch, w, args
        self.n_q, self.n_kv = n_q or w.n_q, n_kv or w.n_kv  # a head-sharded leg holds a slice of the heads
        self.dev = torch.device("cuda", local_rank)
        reserve = (args.steps + args.warmup) * 20 + 600
        self.arena = KVArena(w.layers, self.n_q, self.n_kv, w.d, w.prefix + w.ctx_hi + reserve, PAGE, w.arena_pages,
                             windows=w.windows, device=local_rank, sliding_popn_refuses=False, quantize_kv=w.quant)
        self.arena.set_free_list(np.random.default_rng(w.seed + 7 + seed_salt).permutation(w.arena_pages))
        if args.ctas_per_sm or args.stages or args.consumers or args.no_overlap or args.max_ctas:
            self.arena.set_decode_tuning(args.ctas_per_sm, args.stages, args.consumers, args.max_ctas, not args.no_overlap)
        if args.host_copies:
            self.arena.set_host_route(False)
        if args.split:
            self.arena.set_decode_split(*[int(x) for x in args.split.split(",")])
        self.gen = torch.Generator(device=self.dev).manual_seed(w.seed + seed_salt)
        if w.prefix:  # every sequence forks the shared prefix (whole pages, refcounted), then gets its own suffix
            self.root = self.arena.new_seq()
            self.fill([self.root], [w.prefix])
            self.seqs = [self.root.fork_prefix(w.prefix) for _ in range(len(lens))]
        else:
            self.root = None
            self.seqs = [self.arena.new_seq() for _ in range(len(lens))]
        self.fill(self.seqs, lens)
        self.lens = lens + w.prefix  # cached tokens per sequence before the first decode step
        self.lib = _lib.load()
        self._lib = _lib
        self.stream = torch.cuda.current_stream()
        self.sp = C.c_void_p(self.stream.cuda_stream)
        self.ah = C.c_void_p(self.arena._h)
        self.scale = C.c_double(w.scale)
        self.new_inputs()
        if host_buffers:
            self.qh = [x.cpu().pin_memory() for x in self.q]
            self.kh = [x.cpu().pin_memory() for x in self.k]
            self.vh = [x.cpu().pin_memory() for x in self.v]
            self.oh = [torch.empty_like(x).pin_memory() for x in self.qh]
            self.hargs = [(C.c_void_p(self.qh[l].data_ptr()), C.c_void_p(self.kh[l].data_ptr()), C.c_void_p(self.vh[l].data_ptr()),
                           C.c_void_p(self.oh[l].data_ptr())) for l in range(w.layers)]

    def new_inputs(self):
        """Per-layer q, k, v, out for the current sequences, and the ctypes arguments of a decode step."""
        torch, w, n = self.torch, self.w, len(self.seqs)
        mk = lambda heads: [torch.randn(n * heads * w.d, device=self.dev, generator=self.gen).half() for _ in range(w.layers)]
        self.q, self.k, self.v = mk(self.n_q), mk(self.n_kv), mk(self.n_kv)
        self.out = [torch.empty_like(x) for x in self.q]
        self.hs = (C.c_void_p * n)(*[s._h for s in self.seqs])
        self.ones = (C.c_int64 * n)(*([1] * n))
        self.dargs = [(C.c_void_p(self.q[l].data_ptr()), C.c_void_p(self.k[l].data_ptr()), C.c_void_p(self.v[l].data_ptr()),
                       C.c_void_p(self.out[l].data_ptr())) for l in range(w.layers)]

    def fill(self, which, counts):
        """Cached context through the product path: one chunk step, append only."""
        torch, w = self.torch, self.w
        ntok = int(sum(counts))
        kf = torch.randn(ntok * self.n_kv * w.d, device=self.dev, generator=self.gen).half()
        vf = torch.randn(ntok * self.n_kv * w.d, device=self.dev, generator=self.gen).half()
        self.arena.begin_step(which, [int(n) for n in counts])
        for layer in range(w.layers):
            self.arena.append(layer, kf, vf)
        torch.cuda.synchronize()

    def step_device(self):
        lib, n = self.lib, len(self.seqs)
        self._lib.check(lib.cbkv_begin_step(self.ah, self.hs, self.ones, None, n, self.sp))
        for l in range(self.w.layers):
            a = self.dargs[l]
            rc = lib.cbkv_attention(self.ah, l, a[0], a[1], a[2], a[3], self.scale, 0, self.sp)
            if rc:
                self._lib.check(rc)

    def step_host(self):
        lib, n = self.lib, len(self.seqs)
        self._lib.check(lib.cbkv_begin_step(self.ah, self.hs, self.ones, None, n, self.sp))
        for l in range(self.w.layers):
            a = self.hargs[l]
            rc = lib.cbkv_attention_host_async(self.ah, l, a[0], a[1], a[2], a[3], self.scale, 0, self.sp)
            if rc:
                self._lib.check(rc)
        self._lib.check(lib.cbkv_host_sync(self.ah))  # every layer's output is back in host memory

    def timed(self, fn, steps, warmup, barrier=None, world=1, repeats=1):
        """Device time of `steps` calls of fn after `warmup` untimed ones, bracketed by a barrier and a synchronise on
        both sides, maximum over ranks.  repeats > 1: the timed loop runs that many times; all times are returned."""
        torch = self.torch
        # a loop longer than the arena has room for drops its tokens part-way (popn is host bookkeeping: nothing is
        # enqueued, and the stream keeps later appends behind earlier reads of the freed pages)
        room = self.room()
        done = 0

        def run(n):
            nonlocal done
            for _ in range(n):
                if done >= room:
                    self.rollback(done, sync=False)
                    done = 0
                fn()
                done += 1

        run(warmup)
        self.rollback(done)
        done = 0
        out, t0 = [], None
        for _ in range(repeats):
            if barrier:
                barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = t0 or time.time()
            e0.record(self.stream)
            run(steps)
            e1.record(self.stream)
            if barrier:
                barrier()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                import torch.distributed as dist
                t = torch.tensor([ms], device=self.dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            out.append(ms)
            self.rollback(done)  # outside the timed region: every loop starts from the configured contexts
            done = 0
        return out, t0, time.time()

    def room(self):
        """Steps between two rollbacks inside a long timed loop: at most 64, so that the contexts stay within 64
        tokens of the configured ones whatever --steps is, and never more than the arena has pages for."""
        return min(64, max(16, (self.arena.num_free_pages() // max(1, len(self.seqs)) - 2) * 16))

    def rollback(self, n, sync=True):
        """Drop the n tokens the last n steps appended (popn, kv.rs:807-835), so that the contexts do not drift
        away from the configured ones over hundreds of steps."""
        if n <= 0:
            return
        if sync:
            self.torch.cuda.synchronize()
        for s in self.seqs:
            if s.popn(n) != n:
                raise RuntimeError("popn refused a rollback between timed loops")

    def kernel_level(self, steps):
        """CUDA events around every launch over `steps` more steps (this forbids the overlap of consecutive
        launches, so the mean is the launch's duration when it runs alone); microseconds per launch."""
        steps = min(steps, 64, self.room())
        self.arena.profile_enable(True)
        for _ in range(steps):
            self.step_device()
        kms, kn = self.arena.profile_read()
        self.arena.profile_enable(False)
        self.rollback(steps)
        return kms / kn * 1e3

    def close(self):
        self.torch.cuda.synchronize()
        self.arena.close()
        for name in ("q", "k", "v", "out", "qh", "kh", "vh", "oh", "dargs", "hargs"):
            if hasattr(self, name):
                delattr(self, name)
        self.torch.cuda.empty_cache()


def measure_decode(w: Workload, lens: np.ndarray, local_rank: int, args, steps: int, warmup: int, salt: int = 0) -> dict:
    """A short device-resident run of one configuration for the `also` object."""
    run = DecodeRun(w, lens, local_rank, args, seed_salt=salt)
    launches0 = _launch_count()
    (ms,), _, _ = run.timed(run.step_device, steps, warmup)
    launches = _launch_count() - launches0
    assert run.arena.device_status() == 0, f"kernel status word set ({w.name})"
    lens_mid = run.lens + 1 + min(steps, run.room()) // 2  # contexts at the middle of a timed loop (the loops are rolled back)
    bytes_step = w.bytes_per_step(lens_mid)
    ksteps = min(steps, 10)
    us = run.kernel_level(ksteps)
    bytes_launch = w.bytes_per_step(run.lens + 1 + min(ksteps, 64, run.room()) // 2) / w.layers
    peak, _, src = peaks()
    ms_step = ms / steps
    out = {
        "workload": w.text, "ms_per_step": ms_step, "tokens_per_s": len(lens) / (ms_step * 1e-3), "steps": steps, "warmup": warmup,
        "hbm_gbs": bytes_step / (ms_step * 1e-3) / 1e9, "hbm_frac_of_8tbs": bytes_step / (ms_step * 1e-3) / 8e12,
        "roofline": {"bound": "hbm", "achieved": bytes_launch / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bytes_launch / (us * 1e-6) / 1e9 / peak, "frac_step": bytes_step / (ms_step * 1e-3) / 1e9 / peak,
                     "us_per_launch_serialised": us, "algorithmic_bytes_per_launch": bytes_launch, "peak_source": src},
        "gpu_launches": launches * steps // (steps + warmup),
    }
    if w.prefix:  # the shared prefix is read by every sequence but comes from L2 after the first read: both counts
        once = w.bytes_per_step(lens_mid, shared_prefix_once=True)
        out["algorithmic_bytes_per_step"] = {"every_read_counted": bytes_step, "shared_prefix_counted_once": once}
        out["hbm_gbs_shared_prefix_counted_once"] = once / (ms_step * 1e-3) / 1e9
        out["roofline"]["frac_step_shared_prefix_counted_once"] = once / (ms_step * 1e-3) / 1e9 / peak
    run.close()
    return out


def measure_churn(w: Workload, lens_all: np.ndarray, parts: List[List[int]], rank: int, world: int, local_rank: int, args, barrier) -> dict:
    """cfg5 with its churn inside the timed loop: every 64 steps a seeded 10 % of the job's sequences are evicted
    (popn back to the shared prefix, pages returned to the LIFO free-list, sequence destroyed) and as many new ones
    are admitted, each to the rank with the most free pages, forking the prefix and appending a fresh suffix."""
    import torch
    from combsengine_b200.sharding import admit_to_rank
    run = DecodeRun(w, lens_all[parts[rank]], local_rank, args, seed_salt=rank)
    rng = np.random.default_rng(w.seed + 99)  # the same eviction and admission draws on every rank
    total = len(lens_all)
    owner = np.zeros(total, dtype=np.int64)
    for r, idxs in enumerate(parts):
        owner[idxs] = r
    live = {g: s for g, s in zip(parts[rank], run.seqs)}  # global sequence id -> this rank's sequence
    steps, every = 130, 64
    evicted_total = 0

    def churn():
        nonlocal evicted_total
        victims = rng.permutation(total)[: max(1, total // 10)]
        new_lens = np.round(np.exp(rng.uniform(np.log(w.ctx_lo), np.log(w.ctx_hi), len(victims)))).astype(np.int64)
        for g in victims:
            if owner[g] == rank:
                s = live.pop(int(g))
                n = s.seq_len() - w.prefix
                assert s.popn(n) == n and s.pages_used() == w.prefix // PAGE
                s.close()
        free = torch.tensor([run.arena.num_free_pages()], device=run.dev, dtype=torch.int64)
        if world > 1:
            import torch.distributed as dist
            allfree = [torch.zeros_like(free) for _ in range(world)]
            dist.all_gather(allfree, free)
            free_pages = [int(x.item()) for x in allfree]
        else:
            free_pages = [int(free.item())]
        admit, counts = [], []
        for g, n in zip(victims, new_lens):
            r = admit_to_rank(free_pages)
            free_pages[r] -= -(-int(n) // PAGE)
            owner[g] = r
            if r == rank:
                s = run.root.fork_prefix(w.prefix)
                live[int(g)] = s
                admit.append(s)
                counts.append(int(n))
        if admit:
            run.fill(admit, counts)
        evicted_total += len(victims)
        run.seqs = [live[g] for g in sorted(live)]
        run.new_inputs()

    for _ in range(5):
        run.step_device()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens = 0
    e0.record(run.stream)
    for i in range(steps):
        if i and i % every == 0:
            churn()
        run.step_device()
        tokens += len(run.seqs)
    e1.record(run.stream)
    barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist
        tm = torch.tensor([ms], device=run.dev, dtype=torch.float64)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        tt = torch.tensor([float(tokens)], device=run.dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        ms, tokens = float(tm.item()), float(tt.item())
    assert run.arena.device_status() == 0
    out = {"workload": w.text + f"; churn inside the timed loop: every {every} steps 10 % of the sequences evicted by popn to the "
                                "prefix and replaced (fork_prefix + suffix append), admission to the rank with most free pages",
           "steps": steps, "churn_events": (steps - 1) // every, "sequences_evicted": evicted_total,
           "ms_per_step": ms / steps, "tokens_per_s": tokens / (ms * 1e-3), "live_sequences_on_rank0_at_end": len(run.seqs)}
    run.close()
    return out


def measure_head_sharded(w: Workload, rank: int, world: int, local_rank: int, args, barrier) -> Optional[dict]:
    """KV heads split over groups of G ranks (G = the largest of 4, 2 that divides both the kv heads and the world
    size): every rank of a group holds n_kv / G kv heads (and the matching q heads) of the SAME 32 sequences, runs the
    decode kernel on its slice, and one NCCL all-gather per layer puts the outputs together on a side stream while
    the next layer's kernel runs.  The world / G groups are replicas with their own sequences."""
    import torch
    import torch.distributed as dist
    from combsengine_b200.sharding import kv_head_range
    G = next((g for g in (4, 2) if w.n_kv % g == 0 and world % g == 0), 0)
    if not G:
        return None
    groups = [dist.new_group(list(range(b, b + G))) for b in range(0, world, G)]  # every rank creates every group
    group, grank, replica = groups[rank // G], rank % G, rank // G
    heads = kv_head_range(w.n_kv, grank, G)
    rep = w.n_q // w.n_kv
    lens = replace(w, seed=w.seed + 31 * replica).lengths(w.batch)
    run = DecodeRun(w, lens, local_rank, args, seed_salt=500 + replica, n_q=len(heads) * rep, n_kv=len(heads))
    side = torch.cuda.Stream(device=run.dev)
    # shards arrive as [rank][tokens, n_q / G, d]: NCCL lands every shard in local memory, no peer memory is a kernel operand
    full = [torch.empty(G * run.out[0].numel(), device=run.dev, dtype=torch.float16) for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(w.layers)]
    gathered = [torch.cuda.Event() for _ in range(2)]

    def step(with_gather=True):
        n = len(run.seqs)
        run._lib.check(run.lib.cbkv_begin_step(run.ah, run.hs, run.ones, None, n, run.sp))
        for l in range(w.layers):
            a = run.dargs[l]
            rc = run.lib.cbkv_attention(run.ah, l, a[0], a[1], a[2], a[3], run.scale, 0, run.sp)
            if rc:
                run._lib.check(rc)
            if with_gather:
                done[l].record(run.stream)
                with torch.cuda.stream(side):
                    side.wait_event(done[l])
                    dist.all_gather_into_tensor(full[l & 1], run.out[l], group=group)
                    gathered[l & 1].record(side)
        if with_gather:  # the step ends when its last gathers have landed
            run.stream.wait_event(gathered[0])
            run.stream.wait_event(gathered[1])

    steps, warmup = args.steps, max(3, args.warmup)
    (ms,), _, _ = run.timed(step, steps, warmup, barrier, world)
    (ms_nog,), _, _ = run.timed(lambda: step(False), steps, 2, barrier, world)
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 200  # the all-gather alone, back to back, for its own cost per layer
    with torch.cuda.stream(side):
        for _ in range(20):
            dist.all_gather_into_tensor(full[0], run.out[0], group=group)
        e0.record(side)
        for _ in range(reps):
            dist.all_gather_into_tensor(full[0], run.out[0], group=group)
        e1.record(side)
    torch.cuda.synchronize()
    ag_us = e0.elapsed_time(e1) * 1e3 / reps
    assert run.arena.device_status() == 0
    shard_bytes = run.out[0].numel() * 2
    out = {"workload": f"cfg2 geometry with the {w.n_kv} kv heads split over groups of {G} ranks ({world // G} replica group(s) of "
                       f"{w.batch} sequences), one all-gather of [tokens, n_q/{G}, d] per layer on a side stream",
           "group_size": G, "replica_groups": world // G, "ms_per_step": ms / steps,
           "tokens_per_s": w.batch * (world // G) * steps / (ms * 1e-3),
           "ms_per_step_without_all_gather": ms_nog / steps,
           "collective": {"op": "ncclAllGather (torch.distributed.all_gather_into_tensor)", "us_per_layer_back_to_back": ag_us,
                          "bytes_gathered_per_layer": shard_bytes * G, "bytes_sent_per_rank_per_layer": shard_bytes * (G - 1),
                          "us_per_layer_added_to_the_step": (ms - ms_nog) / steps / w.layers * 1e3}}
    run.close()
    return out


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w = workload(args.config, args.layers, bool(args.quantize_kv))
    # one population for the whole job, assigned to ranks by page count (longest processing time first)
    lens_all = w.lengths(w.batch * world)
    parts = _partition(lens_all + w.prefix, world)
    run = DecodeRun(w, lens_all[parts[rank]], local_rank, args, seed_salt=rank, host_buffers=True)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = _launch_count()
    # a timed loop shorter than a quarter of a second is repeated and the median reported
    est = 1.1e-3 * args.steps * (w.layers / 28) * (3 if w.name == "cfg5" else 1)
    repeats = 1 if est >= 0.25 else min(15, max(3, int(0.25 / max(est, 1e-4)) | 1))
    times, t0, t1 = run.timed(run.step_device, args.steps, args.warmup, barrier, world, repeats)
    ms = statistics.median(times)
    launches = _launch_count() - launches0
    launches_timed = launches * args.steps // (args.steps * repeats + args.warmup)
    clocks = sampler.summary(t0, t1) if rank == 0 else None
    assert run.arena.device_status() == 0, "kernel status word set"
    n_total = w.batch * world
    value = n_total * args.steps / (ms * 1e-3)
    bytes_rank = w.bytes_per_step(run.lens + 1 + min(args.steps, run.room()) // 2)  # contexts at the middle of a timed loop (every loop is rolled back)
    if world > 1:  # every rank's own bytes: their sum for the job's GB/s, min and max to show the balance
        t = torch.tensor([bytes_rank], device=dev, dtype=torch.float64)
        allb = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allb, t)
        per_rank = [float(x.item()) for x in allb]
    else:
        per_rank = [bytes_rank]
    bytes_job = sum(per_rank)

    # roofline of the decode kernel: CUDA events around every launch, same steps again
    us = run.kernel_level(args.steps)
    bytes_launch = w.bytes_per_step(run.lens + 1 + min(args.steps, 64, run.room()) // 2) / w.layers  # mean over the layers of a step
    achieved = bytes_launch / (us * 1e-6) / 1e9

    # end to end: host buffers in, host buffers out, every layer
    etimes, _, _ = run.timed(run.step_host, args.steps, args.warmup, barrier, world, min(repeats, 5))
    ems = statistics.median(etimes)
    e2e_value = n_total * args.steps / (ems * 1e-3)
    h2d = w.layers * (run.qh[0].numel() + run.kh[0].numel() + run.vh[0].numel()) * 2
    d2h = w.layers * run.oh[0].numel() * 2
    assert run.arena.device_status() == 0
    if rank == 0:
        sampler.stop()
    run.close()

    peak, _, peak_src = peaks()
    traffic = None
    tpath = os.path.join(ROOT, "profiles", f"decode_kernel_{w.name}_traffic.txt")
    if os.path.exists(tpath) and not args.layers and not w.quant:
        traffic = float(json.load(open(tpath))["traffic_bytes_per_launch"])  # from the committed ncu capture

    # ---- the other configurations, briefly (device-resident, a fraction of a second of GPU time each)
    also = {}
    if args.config == "cfg2" and not args.layers and not args.quantize_kv and not args.no_also:
        if world > 1:
            also["head_sharded"] = measure_head_sharded(workload("cfg2"), rank, world, local_rank, args, barrier)
        w5 = workload("cfg5")
        lens5 = w5.lengths(w5.batch * world)
        also["cfg5_churn"] = measure_churn(w5, lens5, _partition(lens5 + w5.prefix, world), rank, world, local_rank, args, barrier)
        if world == 1:
            w3 = workload("cfg3")
            w1 = workload("cfg1")
            also["cfg1"] = measure_decode(w1, np.array([512]), local_rank, args, 60, 10)
            also["cfg1"]["us_per_step"] = also["cfg1"]["ms_per_step"] * 1e3
            also["cfg3"] = measure_decode(w3, w3.lengths(w3.batch), local_rank, args, 20, 5)
            also["cfg5_shard"] = measure_decode(w5, lens5, local_rank, args, 10, 4)
            wq = workload("cfg2", quant=True)
            also["int8"] = measure_decode(wq, wq.lengths(wq.batch), local_rank, args, 20, 5)
            also["cfg4_one_layer"] = prefill_record(args, local_rank, layers=1, passes=2, warm_passes=1)
            also["prefill_head_dim_256_one_layer"] = prefill_record(args, local_rank, layers=1, passes=2, warm_passes=1, geometry=(8, 4, 256),
                                                                    label="cfg3's gemma-3-4b-style geometry under the cfg4 schedule,")
            also["rope"] = rope_record(args, local_rank, cpu=False)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and args.config == "cfg2" and not args.layers:
        cpu = time_cpu_port(workload("cfg2"), w.batch, CPU_SAMPLE_LAYERS, 16.0)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    ms_step = ms / args.steps
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": w.text,
                   "l2": f"inputs larger than L2 (about {bytes_rank / 1e9:.1f} GB of KV read per step and GPU)",
                   "sharding": "one seeded population of 32 x N sequences, assigned to ranks by page count (LPT); no collective in the path",
                   "timing": (f"median of {repeats} timed loops of {args.steps} steps" if repeats > 1
                              else f"one timed loop of {args.steps} steps") +
                             "; the appended tokens are dropped again (popn: host bookkeeping, nothing enqueued) after the"
                             " warm-up, after every loop and every 64 steps of a longer loop, so the contexts stay within 64"
                             " tokens of the configured ones"},
        "repeats": repeats, "ms_per_step_all_repeats": [t / args.steps for t in times],
        "hbm_gbs": bytes_job / (ms_step * 1e-3) / 1e9,
        "hbm_frac_of_8tbs": bytes_job / world / (ms_step * 1e-3) / 8e12,
        "per_rank_bytes_per_step": {"min": min(per_rank), "max": max(per_rank), "spread": max(per_rank) / min(per_rank) - 1.0},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_step": bytes_rank / (ms_step * 1e-3) / 1e9 / peak,
                     "traffic": traffic, "kernel": f"decode_kernel<d={w.d},f16{',int8 pages' if w.quant else ''}>",
                     "us_per_launch_serialised": us, "algorithmic_bytes_per_launch": bytes_launch,
                     "peak_source": "copy bandwidth, " + peak_src,
                     "note": "frac: one launch alone between CUDA events (consecutive launches cannot overlap then); "
                             "frac_step: the step's algorithmic bytes over ms_per_step, launches overlapping as they do in use"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ems / args.steps},
        "gpu_launches": launches_timed,
        "clocks": clocks,
    }
    if also:
        line["also"] = also
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


def prefill_record(args, local_rank: int, layers: int = 32, passes: int = 1, warm_passes: int = 1, quant: bool = False,
                   chunk_kernel: int = 0, geometry=(32, 8, 128), label: str = "cfg4 llama-3-8b geometry") -> dict:
    """cfg4: chunked prefill into the paged cache, Llama-3-8B geometry (32 layers, 32/8/128),
    8 prompts of 8192 tokens in 512-token chunks; per chunk and layer: append + causal attention
    over the paged prefix plus the chunk.  A step = one full pass over the 16 chunks.  `geometry`
    runs the same schedule at other head counts / head_dim (cfg3's 8/4/256)."""
    import torch
    from combsengine_b200 import KVArena

    n_q, n_kv, d = geometry
    batch, prompt, chunk = 8, 8192, 512
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    arena = KVArena(layers, n_q, n_kv, d, prompt + 64, 16, batch * (prompt // 16 + 4), device=local_rank, quantize_kv=quant)
    arena.set_free_list(np.random.default_rng(0xC0B50004).permutation(arena.num_pages))
    if chunk_kernel:
        arena.set_chunk_kernel(chunk_kernel)
    if args.chunk_split:
        arena.set_chunk_split(args.chunk_split)
    seqs = [arena.new_seq() for _ in range(batch)]
    gen = torch.Generator(device=dev).manual_seed(0xC0B50004)
    ntok = batch * chunk
    q = torch.randn(ntok * n_q * d, device=dev, generator=gen).half()
    k = torch.randn(ntok * n_kv * d, device=dev, generator=gen).half()
    v = torch.randn(ntok * n_kv * d, device=dev, generator=gen).half()
    out = torch.empty_like(q)
    scale = d ** -0.5
    stream = torch.cuda.current_stream()

    def one_pass(pop=True):
        for c in range(prompt // chunk):
            arena.begin_step(seqs, [chunk] * batch)
            for layer in range(layers):
                arena.attention(layer, q, k, v, scale, out=out)
        if pop:
            for s in seqs:
                s.popn(prompt)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warm_passes):
        one_pass()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record(stream)
    for _ in range(passes):
        one_pass()
    e1.record(stream)
    torch.cuda.synchronize()
    t1 = time.time()
    clocks = sampler.summary(t0, t1)
    sampler.stop()
    ms = e0.elapsed_time(e1) / passes
    assert arena.device_status() == 0
    if args.measure:  # measurement build: per-role cycle counters of the last launch (CBKV_DEBUG=8), printed to stderr
        arena.profile_read()
    # Outside the timed region: the last chunk of one more pass, a few rows recomputed in float64.  Every
    # chunk appends the same k, v, so a prompt's cached K is its chunk of k repeated 16 times.
    one_pass(pop=False)
    torch.cuda.synchronize()
    assert arena.device_status() == 0
    qh = q.cpu().numpy().reshape(batch, n_q, chunk, d).astype(np.float64)
    kh = np.tile(k.cpu().numpy().reshape(batch, n_kv, chunk, d).astype(np.float64), (1, 1, prompt // chunk, 1))
    vh = np.tile(v.cpu().numpy().reshape(batch, n_kv, chunk, d).astype(np.float64), (1, 1, prompt // chunk, 1))
    oh = out.cpu().numpy().reshape(batch, n_q, chunk, d).astype(np.float64)
    worst = 0.0
    for b, hq, r in ((0, 0, 0), (3, 17 % n_q, 255), (7, n_q - 1, chunk - 1), (5, 9 % n_q, 128)):
        p_abs = prompt - chunk + r
        sc = (kh[b, hq // (n_q // n_kv), :p_abs + 1] @ qh[b, hq, r]) * scale
        pr = np.exp(sc - sc.max())
        ref = (pr / pr.sum()) @ vh[b, hq // (n_q // n_kv), :p_abs + 1]
        err = np.abs(oh[b, hq, r] - ref)
        tol = (5e-2 if quant else 2e-3) + 1e-2 * np.abs(ref)  # int8 pages: the reference's own bound, kv.rs:978
        assert (err <= tol).all(), f"cfg4 spot check failed at prompt {b} head {hq} row {r}: {err.max()}"
        worst = max(worst, float(err.max()))
    arena.close()
    del q, k, v, out
    torch.cuda.empty_cache()
    pairs = prompt * (prompt + 1) // 2
    flops = 4.0 * n_q * d * pairs * layers * batch  # QK^T and PV over the causal pairs only
    _, peak, src = peaks()
    sustained = peak_sustained()
    tfl = flops / (ms * 1e-3) / 1e12
    # The denominator: the burst figure for a short run, the sustained one (a seconds-long cuBLAS loop under the
    # power cap) when this run is itself long or was seen to hit the power cap.
    long_run = ms * passes >= 500.0 or "sw_power_cap" in (clocks.get("reasons") or [])
    use = sustained if (long_run and sustained) else peak
    return {
        "metric": "chunked_prefill_attention_tokens_per_s", "value": batch * prompt / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": passes, "warmup": warm_passes, "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"{label} chunked prefill: {layers} layers, {n_q}/{n_kv}/{d}, 8 prompts x 8192 in 512-token "
                               "chunks, append + causal attention over paged prefix + chunk"
                               + (", int8 KV pages" if quant else ""),
                   "chunk_kernel": {0: "auto", 1: "mma.sync", 2: "tcgen05, one query tile per CTA",
                                    3: "tcgen05, two query tiles per CTA",
                                    4: "tcgen05, two query tiles per CTA, int8 records converted in the kernel"}[chunk_kernel]},
        "roofline": {"bound": "tensor", "achieved": tfl, "peak": use, "unit": "TFLOP/s", "frac": tfl / use, "traffic": None,
                     "algorithmic_flops_per_pass": flops,
                     "peak_source": ("cuBLAS bf16 sustained under the power cap, " if use is not peak else "cuBLAS bf16 burst, ") + src,
                     "frac_of_burst_peak": tfl / peak, "frac_of_sustained_peak": (tfl / sustained) if sustained else None},
        "clocks": clocks,
        "spot_check": {"rows": 4, "max_abs_err_vs_float64": worst, "tolerance": ("5e-2" if quant else "2e-3") + " + 1e-2 |ref|"},
    }


def rope_record(args, local_rank: int, cpu: bool = True) -> dict:
    """The step before the path, fused: per-head norm off, rotary embedding of q and k, k and v
    written into page slots, one launch per layer.  Workload: one 512-token chunk of each of the
    8 prompts of cfg4 (Llama-3-8B geometry 32/8/128, theta 500000), positions 4096..4607."""
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

    warm = max(3, args.warmup // 4)
    for _ in range(warm):
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
    peak, _, src = peaks()
    gbs = alg / (us * 1e-6) / 1e9
    base = None
    if cpu:
        import oracle
        oracle.build()
        cos, sin = oracle.rope_tables(d, 500000.0, prefix + chunk)
        xq = np.random.default_rng(1).standard_normal((n_q, chunk, d)).astype(np.float16)
        xk = xq[:n_kv].copy()
        t0 = time.perf_counter()
        oracle.rope_apply(xq, prefix, cos, sin); oracle.rope_apply(xk, prefix, cos, sin)
        dt = time.perf_counter() - t0
        base = {"value": chunk / dt, "unit": "tokens/s", "cores": 1, "kind": "port",
                "sample": f"rotation of q and k of one 512-token chunk of one prompt in {dt:.2f} s (scatter not included)"}
    arena.close()
    del q, k, v, qo
    torch.cuda.empty_cache()
    return {
        "metric": "rope_append_tokens_per_s", "value": ntok / (us * 1e-6), "unit": "tokens/s", "n_gpus": 1,
        "steps": passes * layers, "warmup": warm * layers, "ms_per_step": us * 1e-3,
        "higher_is_better": True, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "rotary embedding of q,k + append of k,v for a 512-token chunk of 8 prompts, 32/8/128, one launch per layer",
                   "l2": "four rotating input sets (200 MB) and 32 destination layers: larger than L2"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "kernel": "rope_append_kernel<f16>", "us_per_launch_serialised": us, "algorithmic_bytes_per_launch": alg,
                     "peak_source": "copy bandwidth, " + src},
        "gpu_launches": passes * layers, "cpu_baseline": base,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chunk-kernel", type=int, default=0, help="cfg4 only: 1 = mma.sync, 2 = tcgen05 one tile per CTA, 3 = tcgen05 two tiles per CTA, 4 = as 3 with int8 records converted in the kernel")
    ap.add_argument("--config", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5", "rope"],
                    help="cfg2 is the headline workload; the others on request (short runs of them ride in the default line's `also`)")
    ap.add_argument("--ctas-per-sm", type=int, default=0, help="tuning: decode CTAs per SM (0 = default)")
    ap.add_argument("--stages", type=int, default=0, help="tuning: TMA ring stages (0 = default)")
    ap.add_argument("--consumers", type=int, default=0, help="tuning: consumer warps per decode CTA (4, 6, 8, 12)")
    ap.add_argument("--max-ctas", type=int, default=0, help="tuning: upper bound on the CTAs of a decode launch")
    ap.add_argument("--chunk-split", type=int, default=0, help="cfg4 only: most K/V slices per item of a launch's last wave (1 = never cut; default: the library's 4)")
    ap.add_argument("--no-overlap", action="store_true", help="tuning: no programmatic dependent launch")
    ap.add_argument("--host-copies", action="store_true", help="e2e leg: the compute stream waits for the input copies before every kernel instead of the kernels reading a flag")
    ap.add_argument("--split", default="", help="tuning: tail_pct,min_item,max_levels of the decode work split (min_item 0 = static split)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-also", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--quantize-kv", action="store_true", help="int8 KV pages (the reference's CacheConfig::quantize_kv)")
    ap.add_argument("--head-dim-256", action="store_true", help="cfg4 only: run the schedule at cfg3's geometry (8/4/256)")
    ap.add_argument("--measure", action="store_true", help="load the measurement build (timers, CBKV_DEBUG switches)")
    ap.add_argument("--layers", type=int, default=0, help="profiling only: run fewer layers than the configuration has (small ncu case)")
    args = ap.parse_args()
    if args.measure:
        from combsengine_b200 import _lib as _l
        _l.use_measure_build()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.config == "cfg4":
        if rank == 0:
            geo = dict(geometry=(8, 4, 256), label="cfg3's gemma-3-4b-style geometry under the cfg4 schedule,") if args.head_dim_256 else {}
            print(json.dumps(prefill_record(args, local_rank, layers=args.layers or 32, passes=max(1, args.steps // 16),
                                            warm_passes=max(1, args.warmup // 8), quant=bool(args.quantize_kv),
                                            chunk_kernel=args.chunk_kernel, **geo)), flush=True)
        return
    if args.config == "rope":
        if rank == 0:
            print(json.dumps(rope_record(args, local_rank, cpu=not args.no_cpu)), flush=True)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
