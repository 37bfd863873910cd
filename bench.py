#!/usr/bin/env python
"""Benchmark of the attention hot path: decode attention over the q8_0 KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the decode-attention context sweep -- batch 1, 32 query heads / 8 KV heads,
head_dim 128, contexts 8K..256K, a full-causal layer and a sliding-window layer (window 4096) per
context; fp16 Q, fp32 accumulation, fp16 output.  One *step* = one decode-attention call on every
(context, layer) of the sweep, i.e. one pass of the hot path over the whole batch of caches.
The metric is the KV stream rate: algorithmic KV bytes (visible keys x 2176 B) / time.

    value      device-timed, inputs resident in HBM
    e2e        the same sweep through the C ABI with HOST buffers: per step the query rows, the new
               K/V rows and the positions of all calls are copied from one pinned host buffer, every
               row is appended to its cache, attention runs, and the output rows are copied back
    roofline   the flash-decode kernel at the longest context, timed live with CUDA event pairs
               around each of its launches inside the timed region
    cpu_baseline  the CPU oracle (a scalar restatement of the reference arithmetic) on a bounded
               sample of the same sweep, on this machine's host cores

With N > 1 (torchrun, one rank per GPU) every rank serves its own sequence (slots are sharded over
GPUs, no collective on the data path): weak scaling, value = bytes of all ranks / max time.

`--impl reference` times the reference arithmetic on the host cores (the reference engine is CUDA
only and has no CPU implementation of this path; its attention math is restated in oracle/).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CTXS = [8192, 16384, 32768, 65536, 131072, 262144]
CPU_SAMPLE_CTXS = [8192, 16384, 32768, 65536]
WINDOW = 4096
POS_BYTES = 2176                      # K+V bytes per cached position per layer
METRIC = "decode-attn HBM TB/s (ctx sweep 8K-256K, full + window-4096 layer per ctx)"
# DRAM bytes (read + write) of one flash-decode launch at 256K, from an ncu capture of the library revision named
# beside it (dram__bytes_read.sum + dram__bytes_write.sum).  Reported as roofline.traffic only while the loaded
# library still is that revision (battn_version()); a changed kernel needs a new capture.
NCU_TRAFFIC_256K = {"lib_version": 4, "bytes": 570502144 + 4255488}
MIN_TIMED_S = 0.5                     # the K-step block is repeated until the timed region is at least this long


def visible(ctx: int, is_swa: bool) -> int:
    return min(ctx, WINDOW) if is_swa else ctx


def step_bytes(ctxs) -> int:
    return sum((visible(c, False) + visible(c, True)) * POS_BYTES for c in ctxs)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons through NVML (read-only) every few
    milliseconds while the timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, torch, local: int):
        self.samples, self.stop_flag, self.t, self.h = [], False, None, None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                pr = torch.cuda.get_device_properties(local)
                bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
                self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(local)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.h = None

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((mhz, bits))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.h is None:
            return
        self.samples, self.stop_flag = [], False
        self.t = threading.Thread(target=self._poll, daemon=True)
        self.t.start()

    def stop(self):
        if self.h is None or self.t is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.stop_flag = True
        self.t.join(timeout=2)
        sm = [m for m, _ in self.samples]
        reasons = set()
        for _, bits in self.samples:
            for bit, name in self.REASONS.items():
                if bits & bit:
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm (oracle): used for cpu_baseline and for --impl reference
# ------------------------------------------------------------------------------------------------
def cpu_workload(ctxs):
    """Host-side caches for the sample contexts: valid q8_0 records with random payload."""
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    items = []
    for ctx in ctxs:
        g = O.Geom(n_head=32, n_kv=8, head_dim=128, window=WINDOW, slot_ctx=ctx, n_slots=1)
        q = rng.standard_normal((1, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
        for is_swa in (False, True):
            caches = []
            for _ in range(2):
                c = O.new_cache(g, is_swa)
                view = O.np_cache_view(g, c, is_swa)
                view[...] = rng.integers(0, 256, size=view.shape, dtype=np.uint8)
                view[..., :8] = np.full(4, 0.0236, np.float16).view(np.uint8)     # ~ amax 3 / 127
                caches.append(c)
            items.append((g, q, caches[0], caches[1], ctx - 1, is_swa))
    return items


def cpu_threads():
    """(pool workers, OpenMP threads per oracle call, host threads used).  One oracle call runs its 8 KV heads on
    up to 8 OpenMP threads; calls on different (context, layer) items run side by side from a thread pool, so that
    all host cores are used whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)."""
    cores = os.cpu_count() or 1
    per_call = min(8, cores)
    workers = max(1, cores // per_call)
    return workers, per_call, workers * per_call


def cpu_step(items):
    from concurrent.futures import ThreadPoolExecutor

    from oracle import oracle as O
    workers, per_call, _ = cpu_threads()

    def one(it):
        g, q, kvk, kvv, pos, is_swa = it
        O.attend(g, q, kvk, kvv, [pos], rows=1, is_swa=is_swa, nthreads=per_call)

    if workers == 1:
        for it in items:
            one(it)
    else:
        with ThreadPoolExecutor(max_workers=workers) as ex:
            list(ex.map(one, sorted(items, key=lambda it: -it[4])))      # longest contexts first


def cpu_baseline(budget_s: float = 10.0):
    from oracle import oracle as O
    items = cpu_workload(CPU_SAMPLE_CTXS)
    cpu_step(items)                                    # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        cpu_step(items)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or n >= 200:
            break
    tbs = n * step_bytes(CPU_SAMPLE_CTXS) / dt / 1e12
    return {"value": tbs, "unit": "TB/s", "cores": cpu_threads()[2], "kind": "port",
            "sample": f"decode sweep restricted to ctx {CPU_SAMPLE_CTXS} (full + window layer), {n} passes in {dt:.1f} s, "
                      "double-accumulating scalar C oracle, OpenMP over KV heads x a thread pool over (context, layer)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as O
    items = cpu_workload(CPU_SAMPLE_CTXS)
    for _ in range(max(1, args.warmup)):
        cpu_step(items)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(items)
    dt = time.perf_counter() - t0
    val = args.steps * step_bytes(CPU_SAMPLE_CTXS) / dt / 1e12
    sample = (f"each step = decode sweep restricted to ctx {CPU_SAMPLE_CTXS} (full + window layer); the reference "
              "engine is CUDA-only, so its attention arithmetic runs here as the scalar C restatement in oracle/")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (int8 KV, fp16 scales)",
        "data": "synthetic",
        "config": {"workload": "decode-attention context sweep (BASELINE config 1), CPU sample", "ctxs": CPU_SAMPLE_CTXS,
                   "n_head": 32, "n_kv": 8, "head_dim": 128, "window": WINDOW, "batch": 1},
        "cpu_baseline": {"value": val, "unit": "TB/s", "cores": cpu_threads()[2], "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class Layer:
    """One (context, layer kind) of the sweep: its own engine, cache, query, output and scratch."""

    def __init__(self, ctx, is_swa, gen, torch, AttnEngine, G_B, device):
        self.ctx, self.is_swa = ctx, is_swa
        g = G_B.with_(slot_ctx=ctx, window=WINDOW)
        self.g = g
        self.eng = AttnEngine(g, device)
        dev = self.eng.device
        self.kvk, self.kvv = self.eng.alloc_kv_layer(is_swa)
        start = max(0, ctx - 2 * WINDOW) if is_swa else 0
        pos = torch.zeros(1, dtype=torch.int32, device=dev)
        for a in range(start, ctx, 512):
            n = min(512, ctx - a)
            k = torch.randn((1, n, g.n_kv, g.head_dim), generator=gen, device=dev, dtype=torch.float32)
            v = torch.randn((1, n, g.n_kv, g.head_dim), generator=gen, device=dev, dtype=torch.float32)
            pos.fill_(a)
            self.eng.qkv_prep_store(k, v, self.kvk, self.kvv, pos, rows=n, is_swa=is_swa)
        self.pos = torch.full((1,), ctx - 1, dtype=torch.int32, device=dev)
        self.q = torch.randn((1, 1, g.n_head, g.head_dim), generator=gen, device=dev, dtype=torch.float32).half()
        self.out = torch.zeros((1, 1, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
        self.part = self.eng.alloc_part(1, 1)
        self.bytes = visible(ctx, is_swa) * POS_BYTES
        # positions reach the device by a copy at the start of a step and the kernel before an attention call is the
        # append of that call's row (or the previous call's merge): the order early KV streaming asks for
        self.eng.set_early_kv_stream(True)

    # ---- end-to-end path: this layer's inputs and output are views into one staging buffer per step ----
    E2E_Q, E2E_K, E2E_V, E2E_POS = 0, 8192, 8192 + 4096, 8192 + 2 * 4096       # byte offsets inside a slot
    E2E_IN_BYTES, E2E_OUT_BYTES = 8192 + 2 * 4096 + 256, 8192

    def bind_staging(self, torch, d_in, d_out, idx):
        g = self.g
        a = idx * self.E2E_IN_BYTES
        self.s_q = d_in[a + self.E2E_Q:a + self.E2E_Q + 8192].view(torch.float16).view(1, 1, g.n_head, g.head_dim)
        self.s_k = d_in[a + self.E2E_K:a + self.E2E_K + 4096].view(torch.float32).view(1, 1, g.n_kv, g.head_dim)
        self.s_v = d_in[a + self.E2E_V:a + self.E2E_V + 4096].view(torch.float32).view(1, 1, g.n_kv, g.head_dim)
        self.s_pos = d_in[a + self.E2E_POS:a + self.E2E_POS + 4].view(torch.int32)
        b = idx * self.E2E_OUT_BYTES
        self.s_out = d_out[b:b + 8192].view(torch.float16).view(1, 1, g.n_head, g.head_dim)

    def fill_host(self, torch, h_in, idx):
        a = idx * self.E2E_IN_BYTES
        h_in[a + self.E2E_Q:a + self.E2E_Q + 8192].view(torch.float16).copy_(self.q.cpu().reshape(-1))
        h_in[a + self.E2E_K:a + self.E2E_K + 4096].view(torch.float32).copy_(torch.randn(self.g.n_kv * self.g.head_dim))
        h_in[a + self.E2E_V:a + self.E2E_V + 4096].view(torch.float32).copy_(torch.randn(self.g.n_kv * self.g.head_dim))
        h_in[a + self.E2E_POS:a + self.E2E_POS + 4].view(torch.int32).fill_(self.ctx - 1)

    def decode(self):
        self.eng.launch_attn_m(self.out, self.q, self.kvk, self.kvv, self.pos, self.part, 1, self.is_swa)

    def decode_e2e(self, two_calls: bool = False):
        """Append the step's new K/V row and attend, on the staged inputs (no copies here): one call whose decode
        kernel appends the row itself, or (two_calls) battn_kv_append followed by battn_decode."""
        if two_calls:
            self.eng.qkv_prep_store(self.s_k, self.s_v, self.kvk, self.kvv, self.s_pos, rows=1, is_swa=self.is_swa)
            self.eng.launch_attn_m(self.s_out, self.s_q, self.kvk, self.kvv, self.s_pos, self.part, 1, self.is_swa)
        else:
            self.eng.decode_append(self.s_out, self.s_q, self.s_k, self.s_v, self.kvk, self.kvv, self.s_pos,
                                   self.part, is_swa=self.is_swa)


PREFILL_PROMPT, PREFILL_CHUNK = 16384, 512


def prefill_pairs(n_prompt: int, window: int | None) -> int:
    """Unmasked (query, key) pairs of a causal (optionally windowed) prompt."""
    if window is None or window >= n_prompt:
        return n_prompt * (n_prompt + 1) // 2
    return window * (window + 1) // 2 + (n_prompt - window) * window


def bench_prefill(torch, AttnEngine, G_B, device, reps: int, window: int = WINDOW):
    """BASELINE config 2: a 16,384-token prompt in 512-row chunks against a growing q8_0 cache, one
    full-causal layer and one sliding-window layer (window 4096 on the bench geometry); each chunk =
    append 512 K/V rows, then attend."""
    WINDOW = window
    g = G_B.with_(slot_ctx=PREFILL_PROMPT, window=WINDOW)
    eng = AttnEngine(g, device)
    eng.set_early_kv_stream(True)      # append -> attention on one position buffer: the order the option asks for
    dev = eng.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    n_chunks = PREFILL_PROMPT // PREFILL_CHUNK
    q = torch.randn((n_chunks, PREFILL_CHUNK, g.n_head, g.head_dim), generator=gen, device=dev).half()
    k = torch.randn((n_chunks, PREFILL_CHUNK, g.n_kv, g.head_dim), generator=gen, device=dev)
    v = torch.randn((n_chunks, PREFILL_CHUNK, g.n_kv, g.head_dim), generator=gen, device=dev)
    out = torch.zeros((1, PREFILL_CHUNK, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
    part = eng.alloc_part(1, PREFILL_CHUNK)
    pos = [torch.full((1,), c * PREFILL_CHUNK, dtype=torch.int32, device=dev) for c in range(n_chunks)]
    flop_per_pair = 4 * g.head_dim * g.n_head
    res = {}
    for is_swa in (False, True):
        kvk, kvv = eng.alloc_kv_layer(is_swa)

        def prompt():
            for c in range(n_chunks):
                eng.qkv_prep_store(k[c:c + 1], v[c:c + 1], kvk, kvv, pos[c], rows=PREFILL_CHUNK, is_swa=is_swa)
                eng.launch_attn_m(out, q[c:c + 1], kvk, kvv, pos[c], part, PREFILL_CHUNK, is_swa)

        prompt()                                   # warm-up (also fills the cache)
        torch.cuda.synchronize()
        # per-kernel times: an eager pass with an event pair around every attention launch
        eng.profile_start(n_chunks * reps)
        for _ in range(reps):
            prompt()
        torch.cuda.synchronize()
        kms = eng.profile_stop()
        # prompt time: the 32 x (append + attend) launches captured once into a CUDA graph (positions are
        # device-resident, one tensor per chunk) and replayed, as the reference replays its captured chunk steps;
        # launched call by call from Python the host's launch rate, not the GPU, would bound the early chunks
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            prompt()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        del graph
        pairs = prefill_pairs(PREFILL_PROMPT, WINDOW if is_swa else None)
        flops = pairs * flop_per_pair
        last = [kms[r * n_chunks + n_chunks - 1] for r in range(reps)]
        c_last = n_chunks - 1
        if is_swa:
            pairs_last = PREFILL_CHUNK * WINDOW
        else:
            pairs_last = PREFILL_CHUNK * c_last * PREFILL_CHUNK + PREFILL_CHUNK * (PREFILL_CHUNK + 1) // 2
        t_last = statistics.mean(last) * 1e-3
        res["swa" if is_swa else "full"] = {
            "prompt_ms": ms, "tflop": flops / 1e12, "TFLOPS": flops / (ms * 1e-3) / 1e12,
            "prefill_tok_per_s": PREFILL_PROMPT / (ms * 1e-3),
            "last_chunk_kernel_us": t_last * 1e6, "last_chunk_TFLOPS": pairs_last * flop_per_pair / t_last / 1e12}
        del kvk, kvv
    assert eng.device_status() == 0
    return res


def bench_prefill_short_chunks(torch, AttnEngine, G_B, device, reps: int):
    """Short prompt chunks (64, 128, 256 rows) against 16,384 cached keys, full-causal layer: microseconds per
    attention call (eager, CUDA events around `reps` back-to-back calls) and TFLOPS.  These shapes leave most SMs
    without an M tile, which is what the key splits of the prompt kernel are for."""
    depth = 16384
    res = {}
    g = G_B.with_(slot_ctx=depth + 256, window=WINDOW)
    eng = AttnEngine(g, device)
    dev = eng.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(13)
    kvk, kvv = eng.alloc_kv_layer(False)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    for a in range(0, depth, 512):
        k = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        v = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        pos.fill_(a)
        eng.qkv_prep_store(k, v, kvk, kvv, pos, rows=512)
    pos.fill_(depth)
    for rows in (64, 128, 256):
        k = torch.randn((1, rows, g.n_kv, g.head_dim), generator=gen, device=dev)
        eng.qkv_prep_store(k, k, kvk, kvv, pos, rows=rows)
        q = torch.randn((1, rows, g.n_head, g.head_dim), generator=gen, device=dev).half()
        out = torch.zeros_like(q)
        part = eng.alloc_part(1, rows)
        for _ in range(3):
            eng.launch_attn_m(out, q, kvk, kvv, pos, part, rows, False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            eng.launch_attn_m(out, q, kvk, kvv, pos, part, rows, False)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        flops = 4.0 * g.head_dim * g.n_head * (rows * depth + rows * (rows + 1) // 2)
        res[f"rows_{rows}"] = {"us_per_call": us, "TFLOPS": flops / us / 1e6}
    assert eng.device_status() == 0
    return res


def bench_qkv_prep(torch, AttnEngine, G_B, device, reps: int):
    """The fused QKV prologue + append (L2 scale, RoPE, sqk, q8_0 store, fp16 q for the attention kernels) on a
    512-row prompt chunk and on a 64-slot decode batch: microseconds per call and algorithmic HBM bytes per second
    (q in and out, k, v, the row's tables, the records written)."""
    res = {}
    for name, n_seq, rows in (("prompt_chunk_512_rows", 1, 512), ("decode_64_slots", 64, 1)):
        g = G_B.with_(slot_ctx=4096, window=WINDOW, n_slots=n_seq)
        eng = AttnEngine(g, device)
        dev = eng.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(11)
        m = n_seq * rows
        q = torch.randn((m, g.n_head, g.head_dim), generator=gen, device=dev)
        k = torch.randn((m, g.n_kv, g.head_dim), generator=gen, device=dev)
        v = torch.randn((m, g.n_kv, g.head_dim), generator=gen, device=dev)
        sqk = torch.ones((g.n_head, g.head_dim), device=dev)
        q16 = torch.empty((m, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
        cs = torch.zeros((m, g.head_dim), device=dev)
        sn = torch.zeros((m, g.head_dim), device=dev)
        pos = torch.full((n_seq,), 1000, dtype=torch.int32, device=dev)
        kslot = torch.arange(n_seq, dtype=torch.int32, device=dev) if n_seq > 1 else None
        kvk, kvv = eng.alloc_kv_layer(False)
        eng.rope_tables(cs, sn, pos, rows=rows)

        def call():
            eng.qkv_prep(q16, q, k, v, sqk, cs, sn, kvk, kvv, pos, kslot=kslot, rows=rows)

        for _ in range(5):
            call()
        torch.cuda.synchronize()
        # 20 calls per graph, so that the figure is device time and not the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(20):
                call()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * 20)
        del graph
        per_row = g.n_head * g.head_dim * (4 + 2) + 2 * g.n_kv * g.head_dim * 4 + 2 * (g.head_dim // 2) * 4 + \
            2 * g.n_kv * (g.head_dim + g.head_dim // 16)
        res[name] = {"us_per_call": us, "bytes": m * per_row, "GBps": m * per_row / (us * 1e-6) / 1e9,
                     "rows_per_s": m / (us * 1e-6)}
        assert eng.device_status() == 0
    return res


def bench_verify(torch, AttnEngine, G_B, device, reps: int):
    """BASELINE config 3: 8 query rows (1 accepted + 7 drafts, causal among themselves) against a 64K q8_0
    context, batch 1 and batch 8 (independent slots); the KV is streamed once per sequence."""
    ctx, rows = 65536, 8
    res = {}
    for batch in (1, 8):
        g = G_B.with_(slot_ctx=ctx + 64, window=WINDOW, n_slots=batch)
        eng = AttnEngine(g, device)
        dev = eng.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(batch)
        kvk, kvv = eng.alloc_kv_layer(False)
        kb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        vb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        pos1 = torch.zeros(1, dtype=torch.int32, device=dev)
        ks1 = torch.zeros(1, dtype=torch.int32, device=dev)
        for b in range(batch):
            ks1.fill_(b)
            for a in range(0, ctx + rows, 512):
                pos1.fill_(a)
                eng.qkv_prep_store(kb, vb, kvk, kvv, pos1, kslot=ks1, rows=min(512, ctx + rows - a))
        q = torch.randn((batch, rows, g.n_head, g.head_dim), generator=gen, device=dev).half()
        out = torch.zeros_like(q)
        pos = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
        kslot = torch.arange(batch, dtype=torch.int32, device=dev)
        part = eng.alloc_part(batch, rows)
        step = lambda: eng.launch_attn_ms(out, q, kvk, kvv, pos, kslot, None, part, batch, False, rows_per_seq=rows)  # noqa: E731
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        eng.profile_start(reps)
        for _ in range(reps):
            step()
        kms = eng.profile_stop()
        t = statistics.mean(kms) * 1e-3
        nbytes = batch * (ctx + rows) * POS_BYTES
        res[f"batch{batch}"] = {"kernel_us": t * 1e6, "bytes": nbytes, "TBps": nbytes / t / 1e12,
                                "verified_rows_per_s": batch * rows / t}
        assert eng.device_status() == 0
        del kvk, kvv
    return res


def bench_paged(torch, AttnEngine, G_B, device, reps: int, ctx: int = 262144, page_len: int = 256):
    """Decode at context `ctx` over a paged cache (pages of `page_len` positions, table = a random permutation of the
    pool) next to the same call on a contiguous partition holding the same records; the outputs must be equal."""
    g = G_B.with_(slot_ctx=ctx + page_len, window=WINDOW, n_slots=1)
    eng = AttnEngine(g, device)
    dev = eng.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    n_pages = (ctx + page_len) // page_len
    table = torch.randperm(n_pages, generator=gen, device=dev).to(torch.int32).reshape(1, n_pages).contiguous()
    pages, pool_k, pool_v = eng.alloc_pages(n_pages, page_len, table)
    kvk, kvv = eng.alloc_kv_layer(False)
    kb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
    vb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
    pos1 = torch.zeros(1, dtype=torch.int32, device=dev)
    for a in range(0, ctx + 1, 512):
        pos1.fill_(a)
        n = min(512, ctx + 1 - a)
        eng.qkv_prep_store(kb, vb, kvk, kvv, pos1, rows=n)
        eng.kv_append_paged(pages, kb, vb, pos1, rows=n)
    q = torch.randn((1, 1, g.n_head, g.head_dim), generator=gen, device=dev).half()
    out_c, out_p = torch.zeros_like(q), torch.zeros_like(q)
    pos = torch.full((1,), ctx, dtype=torch.int32, device=dev)
    part = eng.alloc_part(1, 1)
    res = {"ctx": ctx, "page_len": page_len, "n_pages": n_pages}
    for name, step in (("contiguous", lambda: eng.launch_attn_m(out_c, q, kvk, kvv, pos, part, 1)),
                       ("paged", lambda: eng.attn_paged(out_p, q, pages, pos, part, rows=1))):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        eng.profile_start(reps)
        for _ in range(reps):
            step()
        t = statistics.mean(eng.profile_stop()) * 1e-3
        res[name] = {"kernel_us": t * 1e6, "TBps": (ctx + 1) * POS_BYTES / t / 1e12}
    res["outputs_equal"] = bool(torch.equal(out_c, out_p))
    assert eng.device_status() == 0
    return res


def fill_positions(torch, eng, kvk, kvv, seed: int, start: int, end: int, kslot=None, local_start: int = 0):
    """Appends deterministic N(0,1) K/V rows for global positions [start, end) of one sequence: the rows of every
    512-position block come from a generator seeded by (seed, block index), so the data at a position does not
    depend on how the sequence is sharded over ranks.  `local_start`: global position held at local position 0."""
    g, dev = eng.geom, eng.device
    gen = torch.Generator(device=dev)
    pos1 = torch.zeros(1, dtype=torch.int32, device=dev)
    for blk in range(start // 512, (end + 511) // 512):
        gen.manual_seed(seed * 1000003 + blk)
        kb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        vb = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device=dev)
        a, b = max(start, blk * 512), min(end, blk * 512 + 512)
        pos1.fill_(a - local_start)
        eng.qkv_prep_store(kb[:, a - blk * 512:b - blk * 512].contiguous(), vb[:, a - blk * 512:b - blk * 512].contiguous(),
                           kvk, kvv, pos1, kslot=kslot, rows=b - a)


def seeded_q(torch, dev, seed: int, shape):
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    return torch.randn(shape, generator=gen, device=dev).half()


def time_steps(torch, dist, world, step, reps: int):
    """Device time per step (ms), max over ranks: warm-up, barrier, CUDA events around `reps` steps."""
    for _ in range(3):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), ms


MIX_SLOTS, MIX_CAP = 64, 131072


def mix_contexts():
    return np.random.default_rng(0).integers(1024, 131073, size=MIX_SLOTS)


def run_mix(torch, AttnEngine, G_B, local, ctx, mine):
    """The slots `mine` of the 64-slot mix on this GPU: caches (slot s from seed 1000 + s), queries (seed 5000 + s),
    the decode step, and the output rows."""
    n = len(mine)
    g = G_B.with_(slot_ctx=MIX_CAP, window=WINDOW, n_slots=max(1, n))
    eng = AttnEngine(g, local)
    dev = eng.device
    kvk, kvv = eng.alloc_kv_layer(False)
    ks1 = torch.zeros(1, dtype=torch.int32, device=dev)
    for j, s in enumerate(mine):
        ks1.fill_(j)
        fill_positions(torch, eng, kvk, kvv, 1000 + int(s), 0, int(ctx[s]), kslot=ks1)
    pos = torch.tensor([int(ctx[s]) - 1 for s in mine], dtype=torch.int32, device=dev)
    kslot = torch.arange(n, dtype=torch.int32, device=dev)
    q = torch.cat([seeded_q(torch, dev, 5000 + int(s), (1, 1, g.n_head, g.head_dim)) for s in mine]) if n else \
        torch.zeros((0, 1, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
    out = torch.zeros_like(q)
    part = eng.alloc_part(max(1, n), 1)

    def step():
        if n:
            eng.launch_attn_ms(out, q, kvk, kvv, pos, kslot, None, part, n, False)

    return eng, step, out, (q, kvk, kvv, pos, kslot)


def bench_serving_mix(torch, dist, AttnEngine, G_B, bd, local, rank, world, reps: int):
    """BASELINE config 4a: 64 decode slots with context lengths uniform in [1K, 128K] (seed 0), slots dealt
    to the ranks by length (no collective); one multi-slot decode call per rank per step.  Slot s holds the same
    data whichever rank serves it, so at N > 1 rank 0 also runs all 64 slots alone: that gives the 1-GPU time the
    scaling is measured against and the outputs the sharded run must reproduce bit for bit; three slots are
    compared with the exact fp32 device path as well."""
    ctx = mix_contexts()
    mine = bd.balance_slots(ctx, world)[rank]
    eng, step, out, extra = run_mix(torch, AttnEngine, G_B, local, ctx, mine)
    ms_max, ms = time_steps(torch, dist, world, step, reps)
    total_bytes = int(ctx.sum()) * POS_BYTES
    assert eng.device_status() == 0
    res = {"slots": MIX_SLOTS, "ctx_sum": int(ctx.sum()), "bytes": total_bytes, "ms_per_step": ms_max,
           "TBps": total_bytes / (ms_max * 1e-3) / 1e12, "tok_per_s": MIX_SLOTS / (ms_max * 1e-3),
           "rank0_ms": ms, "rank0_slots": len(mine), "rank0_bytes": int(sum(int(ctx[s]) for s in mine)) * POS_BYTES,
           "scaling": "strong (64 slots dealt over the ranks by context length)"}
    # ---- parity: every rank's rows against the all-slots run on rank 0, and against the exact path --------------
    g = eng.geom

    def exact_check(e, o, q_, kvk_, kvv_, pos_, kslot_):
        worst = 0.0
        for s in (0, 31, 63):
            ref = torch.empty_like(o[s:s + 1])
            ws = torch.empty(e.exact_workspace_bytes(1, 1, 64), dtype=torch.uint8, device="cuda")
            e.attn_exact(ref, q_[s:s + 1], kvk_, kvv_, pos_[s:s + 1], ws, 1, 1, 64, False, kslot=kslot_[s:s + 1])
            worst = max(worst, float((ref.float() - o[s:s + 1].float()).abs().max()))
        assert e.device_status() == 0
        return worst

    if world == 1:
        res["parity_vs_exact_path_max_abs"] = exact_check(eng, out, *extra)
        return res
    mine_out = out.clone()
    del eng, step, out, extra
    torch.cuda.empty_cache()
    full = torch.zeros((MIX_SLOTS, 1, g.n_head, g.head_dim), dtype=torch.float16, device="cuda")
    if rank == 0:
        eng1, step1, out1, extra1 = run_mix(torch, AttnEngine, G_B, local, ctx, list(range(MIX_SLOTS)))
        res["ms_per_step_1gpu"] = time_steps(torch, None, 1, step1, reps)[1]
        full.copy_(out1)
        res["parity_vs_exact_path_max_abs"] = exact_check(eng1, out1, *extra1)
        del eng1, step1, out1, extra1
        torch.cuda.empty_cache()
    dist.broadcast(full, 0)
    err = float((full[torch.tensor(mine, dtype=torch.long, device="cuda")].float() - mine_out.float()).abs().max()) if len(mine) else 0.0
    t = torch.tensor([err], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["parity_sharded_vs_1gpu_max_abs"] = float(t.item())
    return res


SPLIT_TOKENS = 1 << 20


def bench_seq_split(torch, dist, AttnEngine, G_B, bd, local, rank, world, reps: int):
    """BASELINE config 4b: one 1,048,576-token sequence, KV split evenly by position range over the ranks; a decode
    step = local split-K decode whose merge epilogue pushes the shard's (o, m, l) records into every peer's receive
    area over NVLink and merges what the peers pushed (battn_partials_push, one CUDA graph per step).  The NCCL
    all-gather form of the same step is timed beside it.  Position p holds the same data however the sequence is
    sharded, so at N > 1 rank 0 also decodes the whole sequence alone: the 1-GPU time, and the reference output
    (flash kernel and exact fp32 path) the split result is compared with."""
    n_total = SPLIT_TOKENS
    sh = bd.shard_of(n_total, rank, world)
    g = G_B.with_(slot_ctx=sh.capacity, window=WINDOW)
    eng = AttnEngine(g, local)
    dev = eng.device
    kvk, kvv = eng.alloc_kv_layer(False)
    fill_positions(torch, eng, kvk, kvv, 2000, sh.start, sh.end, local_start=sh.start)
    q = seeded_q(torch, dev, 2999, (1, g.n_head, g.head_dim))
    out = torch.zeros_like(q)
    res = {"tokens": n_total, "bytes": n_total * POS_BYTES, "exchange_bytes_per_rank": g.n_head * (g.head_dim + 2) * 8}
    if world > 1:
        dec = bd.SeqSplitDecoder(eng, n_total, exchange="push")
        ms, _ = time_steps(torch, dist, world, lambda: dec.decode(out, q, kvk, kvv, n_total - 1, 1), reps)
        # phases of one step on this rank: the local decode alone (no exchange), then exchange + merge as the rest
        part = eng.alloc_part(1, 1)
        pos = torch.tensor([sh.capacity - 1], dtype=torch.int32, device=dev)
        o2 = torch.zeros((1, 1, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
        ms_local, _ = time_steps(torch, dist, world, lambda: eng.launch_attn_m(o2, q[None], kvk, kvv, pos, part, 1, False), reps)
        dec_n = bd.SeqSplitDecoder(eng, n_total, exchange="nccl")
        out_n = torch.zeros_like(q)
        ms_nccl, _ = time_steps(torch, dist, world, lambda: dec_n.decode(out_n, q, kvk, kvv, n_total - 1, 1), reps)
        res.update({"ms_per_step": ms, "ms_local_decode_only": ms_local, "ms_exchange_and_merge": max(0.0, ms - ms_local),
                    "ms_per_step_nccl_allgather": ms_nccl,
                    "exchange": "push: peer stores from the merge epilogue, every word paired with the step number (no fence, no "
                                "flag), bounded spin on the words, CUDA graph"})
        nccl_vs_push = float((out_n.float() - out.float()).abs().max())
        dec.close()
    else:
        part = eng.alloc_part(1, 1)
        pos = torch.tensor([n_total - 1], dtype=torch.int32, device=dev)
        ms, _ = time_steps(torch, dist, world, lambda: eng.launch_attn_m(out[None], q[None], kvk, kvv, pos, part, 1, False), reps)
        res.update({"ms_per_step": ms})
    assert eng.device_status() == 0
    res["TBps"] = n_total * POS_BYTES / (res["ms_per_step"] * 1e-3) / 1e12
    res["scaling"] = "strong (position range split evenly over the ranks)"
    # ---- parity: the split result against the whole sequence on one GPU (flash kernel and exact fp32 path) ---------
    if world == 1:
        ws = torch.empty(eng.exact_workspace_bytes(1, 1, 128), dtype=torch.uint8, device=dev)
        oe = torch.zeros_like(out)
        eng.attn_exact(oe[None], q[None], kvk, kvv, pos, ws, 1, 1, 128, False)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        res["parity_vs_exact_path_max_abs"] = float((out.float() - oe.float()).abs().max())
        return res
    mine_out = out.clone()
    del kvk, kvv
    torch.cuda.empty_cache()
    ref2 = torch.zeros((2,) + tuple(q.shape), dtype=torch.float16, device=dev)
    if rank == 0:
        g1 = G_B.with_(slot_ctx=n_total, window=WINDOW)
        eng1 = AttnEngine(g1, local)
        kvk1, kvv1 = eng1.alloc_kv_layer(False)
        fill_positions(torch, eng1, kvk1, kvv1, 2000, 0, n_total)
        part1 = eng1.alloc_part(1, 1)
        pos1 = torch.tensor([n_total - 1], dtype=torch.int32, device=dev)
        o1 = torch.zeros((1, 1, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
        res["ms_per_step_1gpu"] = time_steps(torch, None, 1, lambda: eng1.launch_attn_m(o1, q[None], kvk1, kvv1, pos1, part1, 1, False), reps)[1]
        ws = torch.empty(eng1.exact_workspace_bytes(1, 1, 128), dtype=torch.uint8, device=dev)
        oe = torch.zeros_like(o1)
        eng1.attn_exact(oe, q[None], kvk1, kvv1, pos1, ws, 1, 1, 128, False)
        torch.cuda.synchronize()
        assert eng1.device_status() == 0
        ref2[0].copy_(o1[0]); ref2[1].copy_(oe[0])
        del eng1, kvk1, kvv1
        torch.cuda.empty_cache()
    dist.broadcast(ref2, 0)
    errs = torch.tensor([float((mine_out.float() - ref2[0].float()).abs().max()),
                         float((mine_out.float() - ref2[1].float()).abs().max())], dtype=torch.float64, device=dev)
    dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    res["parity_nccl_vs_push_max_abs"] = nccl_vs_push
    res["parity_split_vs_1gpu_max_abs"] = float(errs[0].item())
    res["parity_split_vs_exact_path_max_abs"] = float(errs[1].item())
    return res


def bench_legacy_reference_kernels(torch, AttnEngine, reps: int = 20):
    """The reference's OWN shipping kernels (engine/src/bruce.cu built unmodified for sm_100a into oracle/_ref by
    oracle/ref_build.py) timed on this GPU beside this library on the same cache and queries, in the reference's
    geometry (16/4/256, window 1024): decode at 64K (launch_attn_m rows = 1 + k_attn_combine_rows) and a 512-row
    prompt chunk at depth 16K (launch_attn_m rows = 512).  The checker's leg of the benchmark: nothing here is part
    of a product timed region."""
    import ctypes as C

    from bruce_engine_b200.layout import G_R
    path = os.path.join(ROOT, "oracle", "_ref", "libbruce_ref.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libbruce_ref.so not built (the reference tree was not present at build time)"}
    lib = C.CDLL(path)
    P = lambda t: C.c_void_p(t.data_ptr())   # noqa: E731
    res = {"geometry": "n_head 16, n_kv 4, head_dim 256, window 1024 (the only one the reference's kernels exist in)"}
    for name, n, rows, splits in (("decode_64k", 65536, 1, (56, 128)), ("prompt_chunk_512_rows_at_16k", 16384, 512, (1, 3, 8))):
        g = G_R.with_(slot_ctx=n)
        eng = AttnEngine(g, 0)
        dev = eng.device
        kvk, kvv = eng.alloc_kv_layer(False)
        fill_positions(torch, eng, kvk, kvv, 3000, 0, n)
        gen = torch.Generator(device=dev)
        gen.manual_seed(77)
        q = torch.randn((rows, g.n_head, g.head_dim), generator=gen, device=dev)
        pos = torch.tensor([n - rows], dtype=torch.int32, device=dev)
        best = None
        for ns in splits:
            out_r = torch.zeros((rows, g.n_head, g.head_dim), device=dev)
            part_r = torch.zeros(rows * ns * g.n_kv * 4 * (g.head_dim + 2), device=dev)
            ms = C.c_float()
            rc = lib.ref_attn_shipping(P(out_r), P(q), P(kvk), P(kvv), P(pos), P(part_r), rows, ns, 0, g.slot_ctx, reps, C.byref(ms))
            if rc == 0 and (best is None or ms.value / reps < best[0]):
                best = (ms.value / reps, ns)
        out = torch.zeros((1, rows, g.n_head, g.head_dim), device=dev)
        part = eng.alloc_part(1, rows)
        step = lambda: eng.launch_attn_m(out, q[None], kvk, kvv, pos, part, rows, False)       # noqa: E731
        _, ms_here = time_steps(torch, None, 1, step, reps)
        assert eng.device_status() == 0
        if rows == 1:
            work, unit = n * g.pos_bytes / 1e12, "TB/s"
        else:
            work, unit = 4.0 * g.head_dim * g.n_head * (rows * (n - rows) + rows * (rows + 1) // 2) / 1e12, "TFLOP/s"
        res[name] = {"reference_us": None if best is None else best[0] * 1e3, "reference_splits": None if best is None else best[1],
                     "here_us": ms_here * 1e3, "unit": unit,
                     "reference_rate": None if best is None else work / (best[0] * 1e-3), "here_rate": work / (ms_here * 1e-3),
                     "speedup": None if best is None else best[0] / ms_here}
        del eng, kvk, kvv
        torch.cuda.empty_cache()
    return res


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from bruce_engine_b200 import dist as bd
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL may print a version banner on stdout when its communicator comes up; stdout carries the one
        # JSON line, so it points at stderr while the process group and the first collective are set up
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    gen = torch.Generator(device=f"cuda:{local}")
    gen.manual_seed(1000 + rank)                   # every rank serves its own sequence
    ctxs = [args.only_ctx] if args.only_ctx else CTXS
    if args.case == "verify":
        print(json.dumps({"verify": bench_verify(torch, AttnEngine, G_B, local, max(1, args.steps)),
                          "qkv_prep": bench_qkv_prep(torch, AttnEngine, G_B, local, 50),
                          "paged_decode_256k": bench_paged(torch, AttnEngine, G_B, local, max(1, args.steps))}))
        return 0
    if args.case == "prefill":                      # light run for profiling the prompt-chunk kernel
        from bruce_engine_b200.layout import G_R
        print(json.dumps({"prefill": bench_prefill(torch, AttnEngine, G_B, local, max(1, args.steps)),
                          "prefill_hd256_w1024": bench_prefill(torch, AttnEngine, G_R, local, max(1, args.steps), window=1024),
                          "short_chunks_at_16k": bench_prefill_short_chunks(torch, AttnEngine, G_B, local, 10)}))
        return 0
    layers = [Layer(c, s, gen, torch, AttnEngine, G_B, local) for c in ctxs for s in (False, True)]
    torch.cuda.synchronize()

    def step():
        for L in layers:
            L.decode()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    K, W = args.steps, max(3, args.warmup)
    sampler = ClockSampler(torch, local)

    # One step is captured into a CUDA graph after an eager warm-up, as the reference engine does with
    # every step it runs (bruce.cu:8046-8055): replaying it removes the per-launch host cost.
    def capture(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph

    l0 = sum(L.eng.launch_count() for L in layers)
    step()
    launches_per_step = sum(L.eng.launch_count() for L in layers) - l0

    class _Eager:                                   # --light: no graph, the step is launched eagerly
        @staticmethod
        def replay():
            step()

    graph = _Eager if args.light else capture(step)

    # ---- device-resident timed region: K graph replays of the step ------------------------------------
    for _ in range(W):
        graph.replay()
    barrier()
    # The block of K steps is repeated until the timed region is at least MIN_TIMED_S long (the clock sampler needs
    # more than a handful of samples): the repeat count comes from a probe of one block and is the same on all ranks.
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        graph.replay()
    ev1.record()
    barrier()
    probe_ms = max_over_ranks(ev0.elapsed_time(ev1))
    repeats = 1 if args.light else max(1, int(np.ceil(MIN_TIMED_S * 1e3 / max(probe_ms, 1e-3))))
    barrier()
    if rank == 0:
        sampler.start()
    ev0.record()
    for _ in range(K * repeats):
        graph.replay()
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(ev0.elapsed_time(ev1)) / repeats          # time of ONE block of K steps
    launches = launches_per_step * K * repeats

    # ---- the same K steps launched eagerly with an event pair around every flash-decode launch ----------
    for L in layers:
        L.eng.profile_start(K)
    barrier()
    for _ in range(K):
        step()
    barrier()
    kernel_ms = {(L.ctx, L.is_swa): L.eng.profile_stop() for L in layers}

    if args.light:                                  # profiling run: kernel timings only
        if rank == 0:
            print(json.dumps({"light": True, "ms_per_step": ms / K, "kernel_us": {
                f"{c}{'_swa' if w else ''}": statistics.mean(v) * 1e3 for (c, w), v in kernel_ms.items()}}))
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end-to-end timed region: host buffers, copies inside, one graph replay + host sync per step ------
    # The host stages a step's inputs (q, new k/v row, position of every call) in ONE pinned buffer; the
    # step is: the H2D copy (in two parts), 12 x (append + attention) on views of the staged data, the D2H copy of the
    # 12 output rows, host sync.
    n_l = len(layers)
    h_in = torch.empty(n_l * Layer.E2E_IN_BYTES, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n_l * Layer.E2E_OUT_BYTES, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(n_l * Layer.E2E_IN_BYTES, dtype=torch.uint8, device=f"cuda:{local}")
    d_out = torch.empty(n_l * Layer.E2E_OUT_BYTES, dtype=torch.uint8, device=f"cuda:{local}")
    for i, L in enumerate(layers):
        L.bind_staging(torch, d_in, d_out, i)
        L.fill_host(torch, h_in, i)

    copy_stream = torch.cuda.Stream()
    IN1, OUT1 = Layer.E2E_IN_BYTES, (n_l - 1) * Layer.E2E_OUT_BYTES

    def e2e_enqueue():
        # The copies overlap the first and the last call: the first call's inputs go ahead on the step's stream,
        # the other eleven calls' inputs follow on a second stream while the first call runs; the outputs of the
        # first eleven calls leave while the twelfth runs.  Same bytes, all inside the step.
        main = torch.cuda.current_stream()
        copy_stream.wait_stream(main)
        d_in[:IN1].copy_(h_in[:IN1], non_blocking=True)
        with torch.cuda.stream(copy_stream):
            d_in[IN1:].copy_(h_in[IN1:], non_blocking=True)
        layers[0].decode_e2e(args.e2e_two_calls)
        main.wait_stream(copy_stream)
        for L in layers[1:-1]:
            L.decode_e2e(args.e2e_two_calls)
        copy_stream.wait_stream(main)
        with torch.cuda.stream(copy_stream):
            h_out[:OUT1].copy_(d_out[:OUT1], non_blocking=True)
        layers[-1].decode_e2e(args.e2e_two_calls)
        h_out[OUT1:].copy_(d_out[OUT1:], non_blocking=True)
        main.wait_stream(copy_stream)

    graph_e2e = capture(e2e_enqueue)
    stream = torch.cuda.current_stream()
    h_q0 = h_in[Layer.E2E_Q:Layer.E2E_Q + 8192].view(torch.float16)
    h_o_last = h_out[(n_l - 1) * Layer.E2E_OUT_BYTES:(n_l - 1) * Layer.E2E_OUT_BYTES + 8192].view(torch.float16)

    def step_e2e(i):
        h_q0[0] = 0.001 * (i & 7)                     # the host produces this step's inputs in pinned memory
        graph_e2e.replay()
        stream.synchronize()                          # ... and reads this step's outputs
        return float(h_o_last[0])

    for i in range(W):
        step_e2e(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K * repeats):
        step_e2e(i)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / repeats

    status = sum(L.eng.device_status() for L in layers)
    sb = step_bytes(ctxs)
    value = world * K * sb / (ms * 1e-3) / 1e12
    e2e_value = world * K * sb / (ms_e2e * 1e-3) / 1e12
    h2d = h_in.numel()
    d2h = h_out.numel()

    peak, peak_kind = measured_peak()
    # whole call (decode kernel + merge) of every layer, back to back: a graph of 20 calls of that layer alone
    call_us = {}
    for L in layers:
        for _ in range(2):
            L.decode()
        g20 = capture(lambda L=L: [L.decode() for _ in range(20)])
        g20.replay()
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(10):
            g20.replay()
        c1.record()
        torch.cuda.synchronize()
        call_us[(L.ctx, L.is_swa)] = c0.elapsed_time(c1) * 1e3 / 200
        del g20
    sweep = []
    for c in ctxs:
        tf = statistics.mean(kernel_ms[(c, False)]) * 1e-3
        ts = statistics.mean(kernel_ms[(c, True)]) * 1e-3
        sweep.append({"ctx": c, "full_us": tf * 1e6, "full_TBps": c * POS_BYTES / tf / 1e12,
                      "full_frac_of_peak": c * POS_BYTES / tf / 1e9 / peak,
                      "swa_us": ts * 1e6, "swa_TBps": visible(c, True) * POS_BYTES / ts / 1e12,
                      "full_call_us_in_graph": call_us[(c, False)], "swa_call_us_in_graph": call_us[(c, True)],
                      "full_call_frac_of_peak": c * POS_BYTES / (call_us[(c, False)] * 1e-6) / 1e9 / peak,
                      "attn_tok_per_s_layer_pair": 1.0 / (tf + ts)})
    top = ctxs[-1]
    t_top = statistics.mean(kernel_ms[(top, False)]) * 1e-3
    alg_bytes = top * POS_BYTES + 2 * 32 * 128 * 2
    achieved = alg_bytes / t_top / 1e9
    lib_version = int(layers[0].eng.lib.battn_version())
    traffic = NCU_TRAFFIC_256K["bytes"] if NCU_TRAFFIC_256K["lib_version"] == lib_version else None
    roofline = {"bound": "hbm", "kernel": "k_flash_decode<128,1> @ ctx 262144, full layer", "achieved": achieved,
                "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                "timed": "CUDA event pair around each launch, eager pass of the same K steps (sweep[].full_us / swa_us "
                         "are these kernel-alone times, event overhead included; *_call_us_in_graph is the whole call, "
                         "decode kernel + merge, from a graph of 20 calls of that layer)",
                "frac_of_nominal_8TBps": achieved / 8000.0, "launch_us": t_top * 1e6,
                "algorithmic_bytes_per_launch": alg_bytes, "traffic": traffic,
                "traffic_from": f"ncu capture of library revision {NCU_TRAFFIC_256K['lib_version']}; loaded revision {lib_version}"}

    del layers, graph, graph_e2e
    torch.cuda.empty_cache()
    serving = bench_serving_mix(torch, dist, AttnEngine, G_B, bd, local, rank, world, 20)
    torch.cuda.empty_cache()
    seqsplit = bench_seq_split(torch, dist, AttnEngine, G_B, bd, local, rank, world, 20)
    torch.cuda.empty_cache()
    prefill = bench_prefill(torch, AttnEngine, G_B, local, 2) if rank == 0 else None
    verify = bench_verify(torch, AttnEngine, G_B, local, 20) if rank == 0 else None
    qkv_prep = bench_qkv_prep(torch, AttnEngine, G_B, local, 50) if rank == 0 else None
    paged = bench_paged(torch, AttnEngine, G_B, local, 20) if rank == 0 else None
    legacy = bench_legacy_reference_kernels(torch, AttnEngine) if rank == 0 and world == 1 else None
    if prefill is not None:
        bf16_peak = None
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                bf16_peak = float(json.load(f)["bf16_tflops_sustained"])
        except Exception:
            bf16_peak = 1400.0
        for kind in prefill.values():
            kind["frac_of_measured_dense_bf16_sustained"] = kind["TFLOPS"] / bf16_peak
            kind["frac_of_nominal_dense_fp16_2250"] = kind["TFLOPS"] / 2250.0
    if rank == 0:
        cpu = cpu_baseline() if world == 1 else None
        scaling_detail = None
        if world > 1:
            scaling_detail = {
                "note": "headline `value` at N > 1 is N replicas of the N = 1 sweep (one sequence set per GPU, no "
                        "collective): weak scaling of independent sequences.  The SHARDED workloads are these two; "
                        "efficiency = 1-GPU time / (N x N-GPU time), the 1-GPU time measured by rank 0 in this same run.",
                "serving_mix": {"ms": serving["ms_per_step"], "ms_1gpu": serving.get("ms_per_step_1gpu"),
                                "speedup": serving.get("ms_per_step_1gpu", 0) / serving["ms_per_step"],
                                "efficiency": serving.get("ms_per_step_1gpu", 0) / serving["ms_per_step"] / world},
                "seq_split": {"ms": seqsplit["ms_per_step"], "ms_1gpu": seqsplit.get("ms_per_step_1gpu"),
                              "ms_nccl_allgather": seqsplit.get("ms_per_step_nccl_allgather"),
                              "speedup": seqsplit.get("ms_per_step_1gpu", 0) / seqsplit["ms_per_step"],
                              "efficiency": seqsplit.get("ms_per_step_1gpu", 0) / seqsplit["ms_per_step"] / world}}
        parity = {"mix_max_abs": serving.get("parity_sharded_vs_1gpu_max_abs"),
                  "mix_vs_exact_path_max_abs": serving.get("parity_vs_exact_path_max_abs"),
                  "seq_split_max_abs": seqsplit.get("parity_split_vs_1gpu_max_abs"),
                  "seq_split_vs_exact_path_max_abs": seqsplit.get("parity_split_vs_exact_path_max_abs",
                                                                  seqsplit.get("parity_vs_exact_path_max_abs")),
                  "tolerance_max_abs": 2e-3,
                  "what": "sharded result vs the same data on one GPU (rank 0, same run) and vs the exact fp32 device path"}
        line = {
            "metric": METRIC, "value": value, "unit": "TB/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (int8 KV, fp16 scales, fp16 MMA operands, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "decode-attention context sweep (BASELINE config 1)", "ctxs": CTXS, "n_head": 32,
                       "n_kv": 8, "head_dim": 128, "window": WINDOW, "batch": 1, "q_dtype": "f16", "out_dtype": "f16",
                       "parallelism": f"one sequence per GPU x{world}" if world > 1 else "1 GPU",
                       "l2": "each (context, layer) has its own cache; 1.18 GB are streamed between two reads of "
                             "the same buffer (inputs larger than L2)",
                       "launch": "one CUDA graph per step (12 decode calls through the C ABI), replayed K times",
                       "timed_region": f"{repeats} x the block of K = {K} steps (repeated until >= {MIN_TIMED_S} s); "
                                       "ms_per_step and value are per step of one block",
                       "block_repeats": repeats,
                       "early_kv_stream": True,
                       "e2e_call": "battn_kv_append + battn_decode" if args.e2e_two_calls else
                                   "battn_decode_append (the decode kernel quantises and stores the step's row)",
                       "n_gt_1": "value at N > 1 = N replicas of this sweep (one sequence set per GPU); the sharded "
                                 "workloads and their efficiency are in scaling_detail"},
            "e2e": {"value": e2e_value, "unit": "TB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / K},
            "gpu_launches": launches, "roofline": roofline, "sweep": sweep, "prefill": prefill, "verify_8rows_64k": verify, "qkv_prep": qkv_prep, "paged_decode_256k": paged, "serving_mix_64_slots": serving, "seq_split_1m": seqsplit,
            "clocks": clocks,
            "device_status": status,
            "parity": parity,
        }
        if scaling_detail is not None:
            line["scaling_detail"] = scaling_detail
        if legacy is not None:
            line["legacy_reference_kernels"] = legacy
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-two-calls", action="store_true",
                    help="end-to-end region with battn_kv_append + battn_decode instead of battn_decode_append")
    ap.add_argument("--light", action="store_true", help="profiling run: eager launches, kernel timings only")
    ap.add_argument("--only-ctx", type=int, default=0, help="restrict the decode sweep to one context")
    ap.add_argument("--case", default="decode", choices=["decode", "prefill", "verify"], help="light run of one kernel family")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
