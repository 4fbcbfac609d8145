"""Benchmark of the paged-KV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--blocks R] [--batch B] [--profile]

With no --workload the line is the headline workload `decode_c2` -- large-batch paged
decode with float16 KV: 256 sequences, context lengths uniform in [512, 8192], block size
16, head_dim 128, 32 query / 8 KV heads, non-contiguous block tables, seeded synthetic
N(0,1) data -- and its `also` object carries one entry per other workload of the metric
(`prefill_c3`, `decode_c4`, `step_c4`, `append_c1`), each with its own time, roofline,
clocks, end-to-end figure and bounded CPU baseline.  With --workload NAME the line is that
workload alone.

With N GPUs (one process per GPU, torch.distributed.run) the KV heads are split into N
groups, one per GPU; every GPU holds its heads' pages and an identical copy of the block
tables, and no collective runs on the attention path, so the total work is fixed (strong
scaling).  `value` is the whole job: the units of one step divided by the step time of the
slowest rank.

Timing: W warm-up steps, a half-second settling loop (so that the clock sampler sees the
clocks of the timed region), then R blocks (default 10) of exactly K steps, each block
bracketed by a barrier and a device synchronisation and timed with CUDA events on the
launching stream, maximum over ranks per block; `ms_per_step` is the median block,
`ms_per_step_min` / `_max` the fastest and slowest.

`e2e` is the same step through the reference-shaped C-ABI calls with queries, new K/V rows
and outputs in page-locked host memory, copies inside the timed region.  `roofline` relates
the dominant kernel's algorithmic bytes (or flops) to the measured peaks.  `cpu_baseline`
is the C oracle (a restatement of the reference's CPU path) on this host's cores on a
bounded sample (rank 0, N = 1 only).

`--impl reference` times that CPU path alone (rank 0 only), for the same workloads.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEAD_DIM, BLOCK, KV_HEADS = 128, 16, 8
# decode_c2
SEED, BATCH, LEN_LO, LEN_HI, HEADS, SPARE_BLOCKS, CPU_SAMPLE_SEQS = 1002, 256, 512, 8192, 32, 1024, 32
# prefill_c3
PF_SEQS, PF_LEN, PF_CHUNK, PF_PREFIX = 16, 2048, 512, 1024
# append_c1
C1_TOKENS, C1_BLOCKS, C1_COPIES = 4096, 4096, 512
# decode_c4 / step_c4
C4_SEQS, C4_LO, C4_HI, C4_WINDOW, C4_HEADS, C4_CHUNK = 64, 32768, 131072, 4096, 64, 2048

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM traffic of one decode launch from its algorithmic bytes, after ncu captures
# (dram__bytes_read.sum, dram__bytes_write.sum) of decodeStreamKernel on cuts of the two
# workloads (64 sequences of decode_c2, 16 of decode_c4): the bytes read grow in proportion to
# the context tokens (factor), the bytes written are the outputs plus the records of the
# pieces, whose number is that of the grid's warps whatever the batch (constant).
DECODE_TRAFFIC = {"f16": (1.0032, 5.8e6), "fp8": (1.0042, 4.6e6)}


def decode_traffic(kind, algorithmic_bytes):
    factor, written = DECODE_TRAFFIC[kind]
    return algorithmic_bytes * factor + written


WORKLOADS = ("decode_c2", "prefill_c3", "decode_c4", "step_c4", "append_c1")


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
        return {k: float(mp[k]) for k in FALLBACK}, "measured"
    except Exception:
        return dict(FALLBACK), "fallback"


def host_cores() -> int:
    # all host cores this process may run on (a launcher may have set OMP_NUM_THREADS=1)
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs: NVML read every
    20 ms by a thread of this process (the figures `nvidia-smi --query-gpu=clocks.sm,
    clocks.max.sm,clocks_event_reasons.*` prints), with `nvidia-smi -lms 100` as the fallback
    when the NVML binding is missing.  Nothing is set, only read."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None
        self.sm, self.mx, self.reasons = [], [], set()
        self.stopping, self.thread = threading.Event(), None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            pr = torch.cuda.get_device_properties(self.index)
            bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll(self, nv, h):
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        while True:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.mx.append(float(mx))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            if self.stopping.wait(0.02):
                return

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll, args=(nv, h), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.thread:
            self.stopping.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# ===================================================================== CPU arm

def c2_lengths(batch=None):
    rng = np.random.default_rng(SEED)
    return rng.integers(LEN_LO, LEN_HI + 1, size=batch or BATCH).astype(np.int64)


def cpu_decode_c2(steps, warmup, n_seqs=CPU_SAMPLE_SEQS):
    """The reference's decode loop (restated in C, OpenMP over (sequence, kv head)) on all
    host cores, on the first sequences of the workload; tokens/s over the sample."""
    from oracle import c_oracle as co

    lens = c2_lengths()
    n_seqs = min(n_seqs, len(lens))
    sub = lens[:n_seqs]
    nblk = (sub + BLOCK - 1) // BLOCK
    n_pool = int(nblk.sum()) + 16
    rng = np.random.default_rng(SEED + 1)
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.zeros((n_seqs, int(nblk.max())), dtype=np.int32)
    o = 0
    for i in range(n_seqs):
        tables[i, : nblk[i]] = perm[o: o + nblk[i]]
        o += int(nblk[i])
    shape = (n_pool, KV_HEADS, BLOCK, HEAD_DIM)
    k_pool = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    v_pool = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((n_seqs, HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    l = sub.astype(np.uint32)
    cores = host_cores()
    for _ in range(max(warmup, 1)):
        co.decode(q, k_pool, v_pool, tables, l, KV_HEADS, BLOCK, 1, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        co.decode(q, k_pool, v_pool, tables, l, KV_HEADS, BLOCK, 1, nthreads=cores)
    dt = (time.perf_counter() - t0) / steps
    return {"value": n_seqs / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {n_seqs} of {len(lens)} sequences of the workload ({int(l.sum())} context tokens), "
                      f"{steps} timed passes of {dt * 1e3:.1f} ms (oracle/paged_oracle.c orc_decode)",
            "ms_per_step_sample": dt * 1e3, "sample_fraction": n_seqs / len(lens)}


def cpu_prefill_c3(budget_s=8.0):
    """orc_prefill on every 8th row of one 2048-token sequence (256 rows x 32 heads, causal,
    bf16), repeated for about budget_s seconds; TFLOP/s over the rows computed."""
    from oracle import c_oracle as co
    from oracle import paged_oracle as po

    rng = np.random.default_rng(1003)
    nb = PF_LEN // BLOCK
    k_pool = po.to_bf16_bits(rng.standard_normal((nb, KV_HEADS, BLOCK, HEAD_DIM), dtype=np.float32))
    v_pool = po.to_bf16_bits(rng.standard_normal((nb, KV_HEADS, BLOCK, HEAD_DIM), dtype=np.float32))
    table = rng.permutation(nb).astype(np.int32)
    rows = np.arange(0, PF_LEN, 8)
    q = po.to_bf16_bits(rng.standard_normal((len(rows), HEADS, HEAD_DIM), dtype=np.float32))
    cores = host_cores()

    def one_pass():
        # rows are not contiguous: one call per row (q_start selects the sequence position)
        for i, r in enumerate(rows):
            co.prefill(q[i:i + 1], k_pool, v_pool, table, PF_LEN, KV_HEADS, BLOCK, 3, q_start=int(r), nthreads=cores)

    one_pass()
    passes, t0 = 0, time.perf_counter()
    while passes < 1 or time.perf_counter() - t0 < budget_s:
        one_pass()
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    flops = int((rows + 1).sum()) * HEADS * 4 * HEAD_DIM
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"every 8th row of one 2048-token sequence (256 rows x 32 heads, causal, {flops / 1e9:.2f} GFLOP), "
                      f"{passes} timed passes of {dt * 1e3:.0f} ms (oracle/paged_oracle.c orc_prefill)",
            "ms_per_step_sample": dt * 1e3, "sample_fraction": flops / c3_flops()}


def cpu_decode_c4(budget_s=6.0, n_seqs=4):
    """orc_decode with FP8 KV and the 4096-token window on the first sequences of the
    workload (only the visible pages are materialised)."""
    from oracle import c_oracle as co
    from oracle import paged_oracle as po

    lens = np.random.default_rng(1004).integers(C4_LO, C4_HI + 1, size=C4_SEQS).astype(np.int64)[:n_seqs]
    rng = np.random.default_rng(1004 + 1)
    vis_blocks = C4_WINDOW // BLOCK + 1
    n_pool = n_seqs * vis_blocks
    nblk = (lens + BLOCK - 1) // BLOCK
    tables = np.zeros((n_seqs, int(nblk.max())), np.int32)
    for i in range(n_seqs):
        first = (int(lens[i]) - C4_WINDOW) // BLOCK
        tables[i, first: nblk[i]] = i * vis_blocks + np.arange(int(nblk[i]) - first)
    kc = rng.integers(0, 256, size=(n_pool, KV_HEADS, BLOCK, HEAD_DIM), dtype=np.uint8)
    vc = rng.integers(0, 256, size=(n_pool, KV_HEADS, BLOCK, HEAD_DIM), dtype=np.uint8)
    kc[(kc & 0x7F) == 0x7F] = 0x3C                      # no NaN codes
    vc[(vc & 0x7F) == 0x7F] = 0x3C
    scale = np.full((n_pool, KV_HEADS), 1.0 / 128, np.float16).view(np.uint16)
    q = rng.standard_normal((n_seqs, C4_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    l = lens.astype(np.uint32)
    cores = host_cores()
    run = lambda: co.decode(q, kc, vc, tables, l, KV_HEADS, BLOCK, 2, window=C4_WINDOW, k_scale=scale, v_scale=scale,
                            nthreads=cores)
    run()
    passes, t0 = 0, time.perf_counter()
    while passes < 1 or time.perf_counter() - t0 < budget_s:
        run()
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    _ = po
    return {"value": n_seqs / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {n_seqs} of {C4_SEQS} sequences, FP8 KV, window {C4_WINDOW}, 64 q / 8 kv heads, "
                      f"{passes} timed passes of {dt * 1e3:.1f} ms (oracle/paged_oracle.c orc_decode)",
            "ms_per_step_sample": dt * 1e3, "sample_fraction": n_seqs / C4_SEQS}


def c1_inputs():
    rng = np.random.default_rng(1001)
    k = rng.standard_normal((C1_TOKENS, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((C1_TOKENS, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    slots = rng.choice(C1_BLOCKS * BLOCK, C1_TOKENS, replace=False).astype(np.int64)
    perm = rng.permutation(C1_BLOCKS)
    return rng, k, v, slots, perm[:C1_COPIES].astype(np.int32), perm[C1_COPIES:2 * C1_COPIES].astype(np.int32)


def c1_bytes(kv_heads, tokens=C1_TOKENS, copies=C1_COPIES):
    row = kv_heads * HEAD_DIM
    f16 = 2 * (tokens * row * 2) * 2                       # K and V: read + write
    fp8 = 2 * (tokens * row * 2) + 2 * (tokens * row) + 2 * 2 * tokens * kv_heads * 2   # read once, codes, scales (upper bound)
    cow = 2 * copies * kv_heads * BLOCK * HEAD_DIM * 2 * 2 # K and V blocks: read + write
    return f16 + fp8 + cow + tokens * 8 * 2


def cpu_append_c1(budget_s=5.0):
    """The three parts of the step with the C oracle (scatter, FP8 scale + quantise with the
    reference's software codec, block copies), one thread (the oracle's loops are scalar)."""
    from oracle import c_oracle as co

    _, k, v, slots, src, dst = c1_inputs()
    kp = np.zeros((C1_BLOCKS, KV_HEADS, BLOCK, HEAD_DIM), np.float16)
    vp = np.zeros_like(kp)
    kc = np.zeros((C1_BLOCKS, KV_HEADS, BLOCK, HEAD_DIM), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((C1_BLOCKS, KV_HEADS), np.uint16)
    vs = np.zeros_like(ks)

    def run():
        co.reshape_and_cache(k, v, kp, vp, slots, BLOCK)
        co.reshape_and_cache_fp8(k, v, kc, vc, ks, vs, slots, BLOCK)
        co.copy_blocks(kp, vp, src, dst)

    run()
    passes, t0 = 0, time.perf_counter()
    while passes < 1 or time.perf_counter() - t0 < budget_s:
        run()
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    return {"value": c1_bytes(KV_HEADS) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"the whole step, {passes} timed passes of {dt * 1e3:.1f} ms (oracle/paged_oracle.c orc_reshape_and_cache, "
                      "orc_reshape_and_cache_fp8, orc_copy_blocks)",
            "ms_per_step_sample": dt * 1e3, "sample_fraction": 1.0}


def cpu_backward(budget_s=5.0, rows=512):
    """The backward restatement (numpy, float64 matrix products on the host's BLAS threads) on the
    first `rows` tokens of a sequence of the workload's shape."""
    from oracle import paged_oracle as po

    rng = np.random.default_rng(1005)
    nb = rows // BLOCK
    table = rng.permutation(nb + 8)[:nb].astype(np.int32)
    kp = rng.standard_normal((nb + 8, KV_HEADS, BLOCK, HEAD_DIM)).astype(np.float16)
    vp = rng.standard_normal((nb + 8, KV_HEADS, BLOCK, HEAD_DIM)).astype(np.float16)
    q = rng.standard_normal((rows, HEADS, HEAD_DIM)).astype(np.float16)
    d_out = (0.1 * rng.standard_normal((rows, HEADS, HEAD_DIM))).astype(np.float16)
    m, l = po.attention_stats(q, kp, table, rows, KV_HEADS, BLOCK)
    run = lambda: po.paged_backward(q, kp, vp, table, d_out, m, l, rows, KV_HEADS, BLOCK)
    run()
    passes, t0 = 0, time.perf_counter()
    while passes < 1 or time.perf_counter() - t0 < budget_s:
        run()
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    flops = 5 * 2 * rows * rows * HEAD_DIM * HEADS
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"the first {rows} tokens of a sequence ({rows} x {rows} pairs per head, 32 q / 8 kv heads), {passes} timed "
                      f"passes of {dt * 1e3:.1f} ms (oracle/paged_oracle.py paged_backward, numpy)",
            "ms_per_step_sample": dt * 1e3, "sample_fraction": (rows / 2048.0) ** 2}


def c3_flops(heads=HEADS, seqs=None):
    return (seqs or PF_SEQS) * heads * (PF_LEN * (PF_LEN + 1) // 2) * 4 * HEAD_DIM


CPU_ARMS = {"decode_c2": lambda a: cpu_decode_c2(max(a.steps, 1), a.warmup), "prefill_c3": lambda a: cpu_prefill_c3(),
            "decode_c4": lambda a: cpu_decode_c4(), "append_c1": lambda a: cpu_append_c1(), "backward": lambda a: cpu_backward()}
CPU_META = {
    "decode_c2": ("paged decode tokens/s", "f16", lambda cb: BATCH),
    "prefill_c3": ("prefill TFLOP/s", "bf16", None),
    "decode_c4": ("paged decode tokens/s", "fp8-e4m3 KV, f16 q/out", lambda cb: C4_SEQS),
    "append_c1": ("KV append GB/s", "f16 -> f16 / fp8-e4m3", None),
    "backward": ("backward TFLOP/s", "f16", None),
}


def reference_line(name, args):
    """One JSON object of the CPU arm for workload `name` (step_c4 has no CPU restatement of
    its own: its decode half is decode_c4)."""
    key = "decode_c4" if name == "step_c4" else name
    cb = CPU_ARMS[key](args)
    metric, dtype, _ = CPU_META[key]
    ms_full = cb["ms_per_step_sample"] / max(cb["sample_fraction"], 1e-12)
    return {"impl": "reference", "metric": metric, "value": cb["value"], "unit": cb["unit"], "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_full,
            "ms_per_step_note": "time of the sample divided by the fraction of the workload it covers (subsampled)",
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": CONFIG_TEXT[key], "sample": cb["sample"]}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": cb["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    primary = args.workload or "decode_c2"
    line = reference_line(primary, args)
    if not args.workload:
        line["also"] = {n: reference_line(n, args) for n in ("prefill_c3", "decode_c4", "append_c1")}
    print(json.dumps(line))


CONFIG_TEXT = {
    "decode_c2": "decode_c2: batch 256, context U[512,8192], block 16, head_dim 128, 32 q / 8 kv heads, float16 KV, "
                 "random non-contiguous block tables",
    "prefill_c3": "prefill_c3: 16 seqs x 2048 tokens, chunks of 512, shared 1024-token prefix, bf16, 32 q / 8 kv heads, "
                  "head_dim 128, block 16",
    "decode_c4": "decode_c4: 64 seqs, context U[32768,131072], window 4096, FP8 e4m3 KV with (block, kv_head) scales, "
                 "64 q / 8 kv heads, head_dim 128, block 16",
    "step_c4": "step_c4: one scheduler step = append + prefill of a 2048-token chunk of a new sequence, and the 64 "
               "windowed FP8 decodes of decode_c4",
    "append_c1": "append_c1: 4096 tokens x 8 kv heads x 128 scattered to random distinct slots of a 4096-block pool as "
                 "float16 and as FP8 e4m3 with (block, kv_head) scales, plus a copy of 512 random blocks",
    "backward": "backward: gradients of one 2048-token sequence (no causal mask), 32 q / 8 kv heads, head_dim 128, float16, "
                "block 16 (not a term of the headline metric; only with --workload backward)",
}


# ===================================================================== GPU arm

class Runtime:
    """Process group, device, the stream shared with the library, and the timing rules."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import pagedattentionmetal_b200 as pam

        self.torch, self.dist, self.pam, self.args = torch, dist, pam, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
        assert KV_HEADS % self.world == 0, "the KV heads must divide over the GPUs"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.engine = pam.PagedAttentionEngine(self.local)
        # a stream of torch's that is not the legacy default stream, shared with the library so
        # that torch's events time the library's kernels
        self.stream = torch.cuda.Stream(self.dev)
        torch.cuda.set_stream(self.stream)
        self.engine.setStream(self.stream.cuda_stream)
        # --shards M (single process only): this GPU takes KV-head group 0 of M, the share it
        # would have in an M-GPU job, for profiling the small per-GPU steps of large N alone
        self.shards = args.shards if (args.shards and self.world == 1) else self.world
        assert KV_HEADS % self.shards == 0
        self.kvh = KV_HEADS // self.shards
        self.peaks, self.peak_kind = peaks()
        self.comm = None

    def heads(self, total):
        return total // self.shards

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def settle(self, step, burst=10):
        """Keep the GPU busy for about half a second, so that the clock sampler sees the
        clocks the timed region runs at; returns the number of steps run."""
        n, t0 = 0, time.perf_counter()
        while not self.args.profile and time.perf_counter() - t0 < 0.5:
            for _ in range(burst):
                step()
            self.torch.cuda.synchronize(self.dev)
            n += burst
        return n

    def timed(self, step, flush=None):
        """args.blocks blocks of exactly args.steps steps; per block the device time between
        two events on the launching stream, maximum over ranks.  With `flush` every step is
        timed with its own event pair and `flush()` runs before each (inputs smaller than
        L2).  Returns per-step milliseconds: (median, min, max, all blocks)."""
        torch, K = self.torch, self.args.steps
        blocks = []
        for _ in range(1 if self.args.profile else self.args.blocks):
            self.barrier()
            if flush is None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                for _ in range(K):
                    step()
                e1.record(self.stream)
                self.barrier()
                ms = e0.elapsed_time(e1)
            else:
                ms = 0.0
                for _ in range(K):
                    flush()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(self.stream)
                    step()
                    e1.record(self.stream)
                    torch.cuda.synchronize(self.dev)
                    ms += e0.elapsed_time(e1)
                self.barrier()
            blocks.append(self.max_over_ranks(ms) / K)
        self.engine.synchronize()          # raises if a kernel of the timed region reported an error
        return statistics.median(blocks), min(blocks), max(blocks), blocks

    def timed_host(self, step):
        """The same blocks for the end-to-end legs: synchronous calls with host buffers, wall
        clock between barriers, maximum over ranks."""
        K, blocks = self.args.steps, []
        if self.args.profile:
            return None, None, None
        for _ in range(max(self.args.warmup, 3)):
            step()
        for _ in range(self.args.blocks):
            self.barrier()
            t0 = time.perf_counter()
            for _ in range(K):
                step()
            self.barrier()
            blocks.append(self.max_over_ranks((time.perf_counter() - t0) * 1e3) / K)
        return statistics.median(blocks), min(blocks), max(blocks)

    def base_line(self, name, metric, value, unit, ms, dtype, warm_steps, launches, clocks, extra_config=None):
        med, lo, hi, blocks = ms
        cfg = {"workload": CONFIG_TEXT[name], "sharding": f"kv-head groups over {self.world} GPU(s), no collective on the attention path",
               "timed_blocks": len(blocks), "settle_steps": warm_steps}
        cfg.update(extra_config or {})
        if self.shards != self.world:
            cfg["sharding"] = f"KV-head group 0 of {self.shards} on one GPU (the per-GPU share of a {self.shards}-GPU job, run alone)"
        return {"metric": metric, "value": value, "unit": unit, "n_gpus": self.world, "steps": self.args.steps,
                "warmup": self.args.warmup, "ms_per_step": med, "ms_per_step_min": lo, "ms_per_step_max": hi,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
                "config": cfg, "gpu_launches": int(launches), "clocks": clocks}

    def close(self):
        if self.comm is not None:
            self.pam.PagedAttentionEngine.leaveComm(self.comm)
        self.engine.close()
        if self.world > 1:
            self.dist.destroy_process_group()


def scramble_free_list(cache, n_blocks, rng):
    """Make the allocator hand out blocks in a random order, as after a long run of a server:
    take every block with one-block sequences, free them in a random order (the fifo policy
    re-uses blocks in the order they were freed)."""
    base = 1 << 40
    for i in range(n_blocks):
        cache.allocateSequence(base + i)
        cache.appendTokens(base + i, 1)
    for i in rng.permutation(n_blocks):
        cache.freeSequence(base + int(i))


def fetch_pages(rt, cache, blocks, elem_bytes, with_scales):
    """Pages `blocks` of this rank's device pools as a compact host pool (guards only)."""
    from pagedattentionmetal_b200._cabi import lib

    kvh = rt.kvh
    page = kvh * BLOCK * HEAD_DIM * elem_bytes
    dt = np.uint8 if elem_bytes == 1 else np.float16
    k = np.empty((len(blocks), kvh, BLOCK, HEAD_DIM), dt)
    v = np.empty_like(k)
    ks = np.empty((len(blocks), kvh), np.float16) if with_scales else None
    vs = np.empty_like(ks) if with_scales else None
    ctx = rt.engine._ctx
    for i, b in enumerate(blocks):
        lib.pamc_memcpy(ctx, k[i].ctypes.data, cache.kPoolBuffer.ptr + int(b) * page, page, 1)
        lib.pamc_memcpy(ctx, v[i].ctypes.data, cache.vPoolBuffer.ptr + int(b) * page, page, 1)
        if with_scales:
            lib.pamc_memcpy(ctx, ks[i].ctypes.data, cache.kScaleBuffer.ptr + int(b) * kvh * 2, kvh * 2, 1)
            lib.pamc_memcpy(ctx, vs[i].ctypes.data, cache.vScaleBuffer.ptr + int(b) * kvh * 2, kvh * 2, 1)
    return k, v, ks, vs


def guard_decode(rt, cache, sample, tables, lens, q_host, out_host, dtype, tol, window=0):
    """Correctness guard: the sequences `sample` against the oracle on this rank's heads."""
    from oracle import c_oracle as co

    first = [((int(lens[i]) - window) // BLOCK if window and lens[i] > window else 0) for i in sample]
    last = [(int(lens[i]) + BLOCK - 1) // BLOCK for i in sample]
    used = np.unique(np.concatenate([tables[i, f:l] for i, f, l in zip(sample, first, last)]))
    remap = np.zeros(int(tables.max()) + 1, np.int32)
    remap[used] = np.arange(len(used), dtype=np.int32)
    fp8 = dtype == 2
    k, v, ks, vs = fetch_pages(rt, cache, used, 1 if fp8 else 2, fp8)
    ref = co.decode(np.ascontiguousarray(q_host[sample]), k, v, remap[tables[sample]], lens[sample].astype(np.uint32), rt.kvh,
                    BLOCK, dtype, window=window, k_scale=None if ks is None else ks.view(np.uint16),
                    v_scale=None if vs is None else vs.view(np.uint16))
    err = float(np.abs(out_host[sample].astype(np.float32) - ref).max())
    assert err <= tol, f"decode differs from the oracle by {err}"


# ------------------------------------------------------------------ decode_c2

def algorithmic_bytes_c2(lens, heads, kv_heads):
    """Bytes one decode step must move for `kv_heads` KV heads and `heads` query heads: K and V
    of every context token once, queries, outputs, the touched block-table entries and the
    lengths."""
    kv = int(lens.sum()) * 2 * kv_heads * HEAD_DIM * 2
    qo = 2 * len(lens) * heads * HEAD_DIM * 2
    tables = int(((lens + BLOCK - 1) // BLOCK).sum()) * 4
    return kv + qo + tables + len(lens) * 4


def run_decode_c2(rt, with_cpu):
    torch, pam, engine, dev, args = rt.torch, rt.pam, rt.engine, rt.dev, rt.args
    DT = pam.PagedAttentionDataType
    kvh, heads, rank = rt.kvh, rt.heads(HEADS), rt.rank
    lens = c2_lengths(args.batch)
    B = len(lens)
    nblk = (lens + BLOCK - 1) // BLOCK
    n_pool = int(nblk.sum()) + SPARE_BLOCKS
    cache = pam.KVCacheManager(engine, n_pool, BLOCK, HEAD_DIM, kvh, DT.float16)
    scramble_free_list(cache, n_pool, np.random.default_rng(SEED + 2))
    ids = list(range(B))
    gen = torch.Generator(device=dev)
    for sid in ids:
        L = int(lens[sid])
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        gen.manual_seed(SEED * 1000 + sid)
        # the full [L][KV_HEADS][D] tensor of the sequence, of which this GPU keeps its heads
        kv = torch.randn((2, L, KV_HEADS, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32)
        kv = kv[:, :, rank * kvh:(rank + 1) * kvh, :].to(torch.float16).contiguous()
        engine.appendKV(cache, sid, kv[0], kv[1], 0, L, heads)
    gen.manual_seed(SEED * 1000 + 999983)
    q_full = torch.randn((B, HEADS, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    q_dev = q_full[:, rank * heads:(rank + 1) * heads, :].contiguous()
    out_dev = torch.empty_like(q_dev)
    max_nb = int(nblk.max())
    tables_h, lens_h = cache.batchTables(ids, max_nb)
    assert np.array_equal(lens_h.astype(np.int64), lens)
    tables_dev = torch.from_numpy(tables_h).to(dev)
    layer = pam.PagedLayerSpec(HEAD_DIM, heads, kvh, BLOCK, DT.float16)
    # K/V pools, queries, outputs, block tables and lengths resident in HBM
    lens_dev = torch.from_numpy(lens_h.view(np.int32)).to(dev)
    req = pam.PagedAttentionDecodeRequest(q_dev, cache.kPoolBuffer, cache.vPoolBuffer, tables_dev, lens_dev, out_dev,
                                          B, max_nb, layer)
    q_pin = torch.empty((B, heads, HEAD_DIM), dtype=torch.float16, pin_memory=True)
    q_pin.copy_(q_dev)
    out_pin = torch.empty_like(q_pin, pin_memory=True)

    engine.decode(req)
    sample = [int(np.argmin(lens)), int(np.argmax(lens)), 3 % B]
    guard_decode(rt, cache, sample, tables_h, lens_h, q_dev.cpu().numpy(), out_dev.cpu().numpy(), 1, 2e-3)

    # ---- value: inputs resident in HBM ----
    engine.setAsync(True)
    sampler = ClockSampler(rt.local).start()
    step = lambda: engine.decode(req)
    for _ in range(max(args.warmup, 3)):
        step()
    settled = rt.settle(step)
    launches0 = engine.kernelLaunches
    ms = rt.timed(step)
    launches = engine.kernelLaunches - launches0
    engine.setAsync(False)
    clocks = sampler.stop()

    # ---- e2e: the reference-shaped call with host buffers ----
    e2e_step = lambda: engine.decodeBatch(cache, ids, q_pin.data_ptr(), out_pin.data_ptr(), heads)
    e2e = rt.timed_host(e2e_step)
    if not args.profile:
        assert torch.equal(out_pin.to(dev), out_dev), "host-buffer path and device path disagree"

    # ---- all-gather of the head slices, for a caller that wants the whole output on every GPU ----
    gather = None
    if rt.world > 1 and not args.profile:
        gather = gather_leg(rt, out_dev, B, heads)

    line = None
    if rank == 0:
        bytes_gpu = algorithmic_bytes_c2(lens, heads, kvh)
        achieved = bytes_gpu / (ms[0] * 1e-3) / 1e9
        peak = rt.peaks["hbm_gbs"]
        io_bytes = B * heads * HEAD_DIM * 2
        line = rt.base_line("decode_c2", "paged decode tokens/s", B / (ms[0] * 1e-3), "tokens/s", ms, "f16", settled,
                            launches, clocks,
                            {"seed": SEED, "l2": "inputs larger than L2 (KV read per step per GPU exceeds 126 MB); no flush needed",
                             })
        line["kv_read_gbs_total"] = achieved * rt.world
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                            "peak_source": f"{rt.peak_kind} copy bandwidth", "per": "GPU",
                            "kernel": "decodeStreamKernel (float16 tiles)",
                            "algorithmic_bytes_per_launch": bytes_gpu,
                            "traffic": decode_traffic("f16", bytes_gpu),
                            "traffic_source": "ncu on a 64-sequence cut: bytes read scaled by context tokens, bytes written constant"}
        line["e2e"] = {"value": B / (e2e[0] * 1e-3) if e2e[0] else None, "unit": "tokens/s", "ms_per_step": e2e[0],
                       "ms_per_step_min": e2e[1], "ms_per_step_max": e2e[2],
                       "h2d_bytes_per_step": io_bytes + lens_h.nbytes, "d2h_bytes_per_step": io_bytes,
                       "call": "pam_decode with page-locked host q/out: block tables resident on the device (only changed "
                               "entries are sent), lengths sent per call, output written by the kernels into the host buffer"}
        if gather:
            line["gather"] = gather
        if with_cpu:
            line["cpu_baseline"] = cpu_decode_c2(90, 2)        # about 10 s of CPU work
    cache.close()
    return line


def gather_leg(rt, out_dev, rows, heads):
    """pamc_allgather_heads on the decode output: checked against the ranks' outputs put side
    by side (torch.distributed as the checker), then timed."""
    torch, dist, engine, pam = rt.torch, rt.dist, rt.engine, rt.pam
    if rt.comm is None:
        raw = torch.zeros(128, dtype=torch.uint8, device=rt.dev)
        if rt.rank == 0:
            raw.copy_(torch.frombuffer(bytearray(pam.PagedAttentionEngine.makeCommId()), dtype=torch.uint8))
        dist.broadcast(raw, 0)
        rt.comm = engine.joinComm(bytes(raw.cpu().numpy().tobytes()), rt.rank, rt.world)
    full = torch.empty((rows, heads * rt.world, HEAD_DIM), dtype=out_dev.dtype, device=rt.dev)
    DT = pam.PagedAttentionDataType
    call = lambda: engine.allGatherHeads(rt.comm, out_dev, full, rows, heads, HEAD_DIM, DT.float16)
    call()
    parts = [torch.empty_like(out_dev) for _ in range(rt.world)]
    dist.all_gather(parts, out_dev)
    assert torch.equal(full, torch.cat(parts, dim=1)), "gathered tensor differs from the ranks' outputs side by side"
    engine.setAsync(True)
    for _ in range(3):
        call()
    ms = rt.timed(call)
    engine.setAsync(False)
    bytes_moved = full.numel() * full.element_size()
    return {"ms": ms[0], "ms_min": ms[1], "ms_max": ms[2], "bytes_gathered_per_gpu": bytes_moved,
            "gbs_per_gpu": bytes_moved / (ms[0] * 1e-3) / 1e9,
            "call": "pamc_allgather_heads: ncclAllGather over NVLink + one interleave kernel; verified against the ranks' slices"}


# ------------------------------------------------------------------ prefill_c3

def run_prefill_c3(rt, with_cpu):
    """Chunked causal prefill with prefix caching (`configs[3]`): 16 sequences x 2048 prompt
    tokens in 512-token chunks, all sharing an identical 1024-token prefix (its pages are
    shared through the manager's prefix cache and written once), bf16.  A step is the four
    chunk launches (one launch per chunk for all 16 sequences); the metric is algorithmic
    TFLOP/s: 16 x 32 x (2048 x 2049 / 2) x 4 x 128 = 550.0 GFLOP per step, masked pairs and
    softmax not counted.  Tensor-bound."""
    torch, pam, engine, dev, args = rt.torch, rt.pam, rt.engine, rt.dev, rt.args
    DT = pam.PagedAttentionDataType
    kvh, heads, rank = rt.kvh, rt.heads(HEADS), rt.rank
    seqs = PF_SEQS if args.batch is None or args.workload != "prefill_c3" else args.batch
    nblk_seq = PF_LEN // BLOCK
    cache = pam.KVCacheManager(engine, seqs * nblk_seq + 64, BLOCK, HEAD_DIM, kvh, DT.bfloat16)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1003)
    ksl, qsl = slice(rank * kvh, (rank + 1) * kvh), slice(rank * heads, (rank + 1) * heads)
    prefix_kv = torch.randn((2, PF_PREFIX, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
    prefix_q = torch.randn((PF_PREFIX, HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)[:, qsl]
    qs = []
    hashes = list(range(PF_PREFIX // BLOCK))
    for sid in range(seqs):
        cache.allocateSequence(sid)
        cache.appendTokens(sid, PF_PREFIX, hashes)              # followers hit the leader's pages
        if sid == 0:
            engine.appendKV(cache, 0, prefix_kv[0][:, ksl].contiguous(), prefix_kv[1][:, ksl].contiguous(), 0, PF_PREFIX, heads)
        cache.appendTokens(sid, PF_LEN - PF_PREFIX)
        kv = torch.randn((2, PF_LEN - PF_PREFIX, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
        engine.appendKV(cache, sid, kv[0][:, ksl].contiguous(), kv[1][:, ksl].contiguous(), PF_PREFIX, PF_LEN - PF_PREFIX, heads)
        q_own = torch.randn((PF_LEN - PF_PREFIX, HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)[:, qsl]
        qs.append(torch.cat([prefix_q, q_own]).contiguous())
    stats = cache.memoryStats()
    assert stats.sharedBlocks == (PF_PREFIX // BLOCK if seqs > 1 else 0)
    assert stats.prefixCacheHits == (seqs - 1) * (PF_PREFIX // BLOCK)
    tables_h, _ = cache.batchTables(list(range(seqs)), nblk_seq)
    tables = torch.from_numpy(tables_h).to(dev)
    layer = pam.PagedLayerSpec(HEAD_DIM, heads, kvh, BLOCK, DT.bfloat16)
    n_chunks = PF_LEN // PF_CHUNK
    q_chunks = [torch.cat([qs[s][c * PF_CHUNK:(c + 1) * PF_CHUNK] for s in range(seqs)]).contiguous() for c in range(n_chunks)]
    outs = [torch.empty_like(q_chunks[c]) for c in range(n_chunks)]

    def make_step(q_list, out_list):
        def step():
            for c in range(n_chunks):
                engine.prefillBatch(q_list[c], cache.kPoolBuffer, cache.vPoolBuffer, tables, out_list[c],
                                    [(c + 1) * PF_CHUNK] * seqs, [c * PF_CHUNK] * seqs, [PF_CHUNK] * seqs,
                                    nblk_seq, layer, True)
        return step

    step = make_step(q_chunks, outs)
    # correctness guard: a few rows of one follower sequence against the oracle
    step()
    engine.synchronize()
    from oracle import c_oracle as co
    from oracle import paged_oracle as po
    tensor_path = engine.lastStats.operation == pam.Operation.prefillMMA
    sid, c, r0, n = min(5, seqs - 1), 2, 100, 8
    used = tables_h[sid]
    k, v, _, _ = fetch_pages(rt, cache, used, 2, False)
    ref = co.prefill(qs[sid][c * PF_CHUNK + r0: c * PF_CHUNK + r0 + n].view(torch.uint16).cpu().numpy(), k.view(np.uint16),
                     v.view(np.uint16), np.arange(len(used), dtype=np.int32), (c + 1) * PF_CHUNK, kvh, BLOCK, 3,
                     q_start=c * PF_CHUNK + r0)
    got = po.from_bf16_bits(outs[c][sid * PF_CHUNK + r0: sid * PF_CHUNK + r0 + n].view(torch.uint16).cpu().numpy())
    err = float(np.abs(got - ref).max())
    assert err <= 2e-3 + 2.0 ** -8, f"prefill differs from the oracle by {err}"

    engine.setAsync(True)
    sampler = ClockSampler(rt.local).start()
    for _ in range(max(args.warmup, 3)):
        step()
    settled = rt.settle(step, burst=2)
    launches0 = engine.kernelLaunches
    ms = rt.timed(step)
    launches = engine.kernelLaunches - launches0
    engine.setAsync(False)
    clocks = sampler.stop()

    # ---- e2e: the same four chunk calls with q and the output in page-locked host memory ----
    e2e = (None, None, None)
    io_bytes = sum(q.numel() * 2 for q in q_chunks)
    if not args.profile:
        q_pin = [q.cpu().pin_memory() for q in q_chunks]
        out_pin = [torch.empty_like(q).pin_memory() for q in q_pin]
        e2e = rt.timed_host(make_step(q_pin, out_pin))
        assert torch.equal(out_pin[n_chunks - 1].to(dev), outs[n_chunks - 1]), "host-buffer path and device path disagree"

    line = None
    if rank == 0:
        flops = c3_flops(HEADS, seqs)                      # whole job, all GPUs
        tflops = flops / (ms[0] * 1e-3) / 1e12
        flops = flops * rt.world // rt.shards              # (with --shards: the share that ran)
        tflops = flops / (ms[0] * 1e-3) / 1e12
        per_gpu = tflops / rt.world
        peak, sustained = rt.peaks["bf16_tflops"], rt.peaks["bf16_tflops_sustained"]
        line = rt.base_line("prefill_c3", "prefill TFLOP/s", tflops, "TFLOP/s", ms, "bf16", settled, launches, clocks,
                            {"seed": 1003, "l2": "K/V of a step (16 x 2048 tokens x 8 kv heads) is re-read from L2 by design; "
                                                 "q and out stream through HBM"})
        line["tokens_per_s"] = seqs * PF_LEN / (ms[0] * 1e-3)
        line["roofline"] = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                            "peak_source": f"{rt.peak_kind} cuBLAS bf16 burst", "per": "GPU",
                            "kernel": "prefillTcKernel" if tensor_path else "prefillGeneralKernel",
                            "algorithmic_flops_per_step": flops // rt.world, "traffic": None,
                            # the step is timed inside a loop of back-to-back steps: the fraction of the sustained
                            # cuBLAS figure is given beside the fraction of its burst figure
                            "frac_of_sustained": per_gpu / sustained if sustained else None, "peak_sustained": sustained}
        line["e2e"] = {"value": flops / (e2e[0] * 1e-3) / 1e12 if e2e[0] else None, "unit": "TFLOP/s", "ms_per_step": e2e[0],
                       "ms_per_step_min": e2e[1], "ms_per_step_max": e2e[2],
                       "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                       "call": "pamc_prefill_batch per chunk with page-locked host q/out (copied to and from the device inside the call; "
                               "block tables resident): 268 MB each way per step, bound by the host link"}
        if with_cpu:
            line["cpu_baseline"] = cpu_prefill_c3()
    cache.close()
    return line


# ------------------------------------------------------------------ append_c1

def run_append_c1(rt, with_cpu):
    """`configs[1]`: 4096 new tokens (float16 K/V) scattered by a slot mapping of random
    distinct slots into a pool of 4096 blocks x 16, once as float16 and once quantised to FP8
    e4m3 with per-(block, kv_head) scales, plus the copy of 512 random blocks (copy-on-write).
    A step is the three calls; the working set is smaller than L2, so L2 is flushed (a 512 MB
    buffer is written) before every timed step and every step is timed with its own pair of
    CUDA events.  Metric: algorithmic GB/s (this GPU's KV heads)."""
    torch, pam, engine, dev, args = rt.torch, rt.pam, rt.engine, rt.dev, rt.args
    DT = pam.PagedAttentionDataType
    kvh, rank = rt.kvh, rt.rank
    T, nblk = C1_TOKENS, C1_BLOCKS
    rng, k_full, v_full, slots_h, src, dst = c1_inputs()
    k_h = np.ascontiguousarray(k_full[:, rank * kvh:(rank + 1) * kvh])
    v_h = np.ascontiguousarray(v_full[:, rank * kvh:(rank + 1) * kvh])
    k, v, slots = torch.from_numpy(k_h).to(dev), torch.from_numpy(v_h).to(dev), torch.from_numpy(slots_h).to(dev)
    c16 = pam.KVCacheManager(engine, nblk, BLOCK, HEAD_DIM, kvh, DT.float16)
    c8 = pam.KVCacheManager(engine, nblk, BLOCK, HEAD_DIM, kvh, DT.float8)

    def step():
        engine.reshapeAndCache(c16, k, v, slots, T)
        engine.reshapeAndCache(c8, k, v, slots, T)
        engine.copyBlocks(c16, src, dst)

    # correctness guard: pools, codes and scales bit for bit against the oracle
    step()
    engine.synchronize()
    from oracle import c_oracle as co
    kp = np.zeros((nblk, kvh, BLOCK, HEAD_DIM), np.float16)
    vp = np.zeros_like(kp)
    co.reshape_and_cache(k_h, v_h, kp, vp, slots_h, BLOCK)
    co.copy_blocks(kp, vp, src, dst)
    gk, gv, _, _ = c16.readPools()
    assert np.array_equal(gk, kp) and np.array_equal(gv, vp), "float16 append or block copy differs from the oracle"
    kc = np.zeros((nblk, kvh, BLOCK, HEAD_DIM), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((nblk, kvh), np.float16)
    vs = np.zeros_like(ks)
    co.reshape_and_cache_fp8(k_h, v_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots_h, BLOCK)
    gk8, gv8, gks, gvs = c8.readPools()
    assert np.array_equal(gk8, kc) and np.array_equal(gv8, vc), "FP8 codes differ from the oracle"
    assert np.array_equal(gks, ks) and np.array_equal(gvs, vs), "FP8 scales differ from the oracle"

    engine.setAsync(True)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: flush_buf.fill_(1)
    sampler = ClockSampler(rt.local).start()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(dev)
    launches0 = engine.kernelLaunches
    ms = rt.timed(step, flush=flush)
    launches = engine.kernelLaunches - launches0
    clocks = sampler.stop()

    # ---- the same scatters with 16 times the tokens: 65 536 tokens that fill every slot of the
    # pool (a permutation of all slots), where the kernels run long enough for HBM to bound them
    x16 = None
    if not args.profile:
        T16 = nblk * BLOCK
        k16_h = rng.standard_normal((T16, kvh, HEAD_DIM), dtype=np.float32).astype(np.float16)
        v16_h = rng.standard_normal((T16, kvh, HEAD_DIM), dtype=np.float32).astype(np.float16)
        slots16_h = rng.permutation(T16).astype(np.int64)
        k16, v16 = torch.from_numpy(k16_h).to(dev), torch.from_numpy(v16_h).to(dev)
        slots16 = torch.from_numpy(slots16_h).to(dev)

        def step16():
            engine.reshapeAndCache(c16, k16, v16, slots16, T16)
            engine.reshapeAndCache(c8, k16, v16, slots16, T16)

        step16()
        engine.synchronize()
        kp16 = np.zeros((nblk, kvh, BLOCK, HEAD_DIM), np.float16)
        vp16 = np.zeros_like(kp16)
        co.reshape_and_cache(k16_h, v16_h, kp16, vp16, slots16_h, BLOCK)
        gk, gv, _, _ = c16.readPools()
        assert np.array_equal(gk, kp16) and np.array_equal(gv, vp16), "x16 float16 append differs from the oracle"
        # the FP8 pool already holds codes and scales of the steps before (same tokens to the same
        # slots: a second pass of the oracle leaves what every later pass leaves)
        co.reshape_and_cache_fp8(k_h, v_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots_h, BLOCK)
        co.reshape_and_cache_fp8(k16_h, v16_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots16_h, BLOCK)
        gk8, gv8, gks, gvs = c8.readPools()
        assert np.array_equal(gk8, kc) and np.array_equal(gv8, vc), "x16 FP8 codes differ from the oracle"
        assert np.array_equal(gks, ks) and np.array_equal(gvs, vs), "x16 FP8 scales differ from the oracle"
        for _ in range(3):
            step16()
        ms16 = rt.timed(step16, flush=flush)
        row = kvh * HEAD_DIM
        bytes16 = 2 * (T16 * row * 2) * 2 + 2 * (T16 * row * 2) + 2 * (T16 * row) + 2 * 2 * nblk * kvh * 2 + T16 * 8 * 2
        x16 = {"tokens": T16, "ms_per_step": ms16[0], "ms_per_step_min": ms16[1], "ms_per_step_max": ms16[2],
               "algorithmic_bytes": bytes16, "gbs": bytes16 / (ms16[0] * 1e-3) / 1e9,
               "frac": bytes16 / (ms16[0] * 1e-3) / 1e9 / rt.peaks["hbm_gbs"],
               "what": "float16 scatter + FP8 scatter of 65 536 tokens over all slots of the pool, no block copies"}
    engine.setAsync(False)

    # ---- e2e: new K/V rows in page-locked host memory through pamc_reshape_and_cache ----
    e2e = (None, None, None)
    if not args.profile:
        k_pin, v_pin = torch.from_numpy(k_h).pin_memory(), torch.from_numpy(v_h).pin_memory()

        def step_host():
            engine.reshapeAndCache(c16, k_pin, v_pin, slots_h, T)
            engine.reshapeAndCache(c8, k_pin, v_pin, slots_h, T)
            engine.copyBlocks(c16, src, dst)

        e2e = rt.timed_host(step_host)

    line = None
    if rank == 0:
        total = c1_bytes(kvh)
        peak = rt.peaks["hbm_gbs"]
        achieved = total / (ms[0] * 1e-3) / 1e9
        line = rt.base_line("append_c1", "KV append GB/s", achieved * rt.world, "GB/s", ms, "f16 -> f16 / fp8-e4m3", 0, launches,
                            clocks, {"seed": 1001, "l2": "flushed before every timed step (512 MB written)"})
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                            "peak_source": f"{rt.peak_kind} copy bandwidth", "per": "GPU",
                            "kernel": "reshapeAndCacheKernel, fp8AbsmaxPiecesKernel + fp8QuantizePiecesKernel, copyBlocksKernel",
                            "algorithmic_bytes_per_launch": total, "traffic": None,
                            "note": "four short kernels per step: launch latency, not HBM, bounds this size; see x16"}
        line["tokens_per_s"] = T / (ms[0] * 1e-3)
        io = 2 * 2 * T * kvh * HEAD_DIM * 2 + 2 * T * 8 + 2 * C1_COPIES * 4
        line["e2e"] = {"value": total * rt.world / (e2e[0] * 1e-3) / 1e9 if e2e[0] else None, "unit": "GB/s", "ms_per_step": e2e[0],
                       "ms_per_step_min": e2e[1], "ms_per_step_max": e2e[2], "h2d_bytes_per_step": io, "d2h_bytes_per_step": 0,
                       "call": "pamc_reshape_and_cache (float16 and FP8 cache) with page-locked host K/V rows and a host slot "
                               "list, pamc_copy_blocks with host block lists"}
        if x16 is not None:
            line["x16"] = x16
        if with_cpu:
            line["cpu_baseline"] = cpu_append_c1()
    c16.close()
    c8.close()
    return line


# ------------------------------------------------------------------ backward

BW_LEN = 2048


def run_backward(rt, with_cpu):
    """PagedAttentionEngine.backward on one 2048-token float16 sequence: a step is one call
    (row sums, the key-tile kernel, the store of dQ).  Algorithmic flops = five L x L x d
    products per head (S, dP, dV, dK, dQ).  The guard compares dQ and the pool gradients with
    automatic differentiation of the same attention in float32 torch."""
    torch, pam, engine, dev, args = rt.torch, rt.pam, rt.engine, rt.dev, rt.args
    DT = pam.PagedAttentionDataType
    kvh, heads, rank = rt.kvh, rt.heads(HEADS), rt.rank
    L, nb = BW_LEN, BW_LEN // BLOCK
    gen = torch.Generator(device=dev)
    gen.manual_seed(1005 * 1000 + rank)
    table_h = np.random.default_rng(1005).permutation(nb + 8)[:nb].astype(np.int32)
    table = torch.from_numpy(table_h).to(dev)
    rnd = lambda *shape: torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)
    k_pool = rnd(nb + 8, kvh, BLOCK, HEAD_DIM).to(torch.float16)
    v_pool = rnd(nb + 8, kvh, BLOCK, HEAD_DIM).to(torch.float16)
    q = rnd(L, heads, HEAD_DIM).to(torch.float16)
    d_out = (0.1 * rnd(L, heads, HEAD_DIM)).to(torch.float16)
    dq = torch.empty_like(q)
    dk_pool, dv_pool = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    # the forward pass's row statistics and the float32 reference gradients
    G = heads // kvh
    idx = torch.from_numpy(table_h.astype(np.int64)).to(dev)
    kd = k_pool[idx].permute(1, 0, 2, 3).reshape(kvh, L, HEAD_DIM).float().requires_grad_(True)
    vd = v_pool[idx].permute(1, 0, 2, 3).reshape(kvh, L, HEAD_DIM).float().requires_grad_(True)
    qf = q.float().permute(1, 0, 2).reshape(kvh, G, L, HEAD_DIM).requires_grad_(True)
    sc = torch.einsum("kgid,kjd->kgij", qf, kd) / float(np.sqrt(np.float32(HEAD_DIM)))
    m = sc.max(dim=-1).values
    l = torch.exp(sc - m[..., None]).sum(dim=-1)
    out = torch.einsum("kgij,kjd->kgid", torch.softmax(sc, dim=-1), vd)
    (out * d_out.float().permute(1, 0, 2).reshape(kvh, G, L, HEAD_DIM)).sum().backward()
    m_dev = m.detach().reshape(heads, L).t().contiguous()
    l_dev = l.detach().reshape(heads, L).t().contiguous()
    step = lambda: engine.backward(q, k_pool, v_pool, table, d_out, m_dev, l_dev, dq, dk_pool, dv_pool, L, HEAD_DIM, heads, kvh,
                                   BLOCK, DT.float16, 0)
    step()
    engine.synchronize()
    ref_dq = qf.grad.reshape(heads, L, HEAD_DIM).permute(1, 0, 2)
    err_q = float((dq.float() - ref_dq).abs().max())
    got_dk = dk_pool[idx].permute(1, 0, 2, 3).reshape(kvh, L, HEAD_DIM).float()
    got_dv = dv_pool[idx].permute(1, 0, 2, 3).reshape(kvh, L, HEAD_DIM).float()
    err_k, err_v = float((got_dk - kd.grad).abs().max()), float((got_dv - vd.grad).abs().max())
    scale_k, scale_v = float(kd.grad.abs().max()), float(vd.grad.abs().max())
    assert err_q <= 2e-3 and err_k <= 2e-3 + scale_k * 2 ** -10 and err_v <= 2e-3 + scale_v * 2 ** -10, \
        f"backward differs from float32 autograd: dQ {err_q}, dK {err_k}, dV {err_v}"
    del sc, out, qf, kd, vd

    engine.setAsync(True)
    sampler = ClockSampler(rt.local).start()
    for _ in range(max(args.warmup, 3)):
        step()
    settled = rt.settle(step, burst=2)
    launches0 = engine.kernelLaunches
    ms = rt.timed(step)
    launches = engine.kernelLaunches - launches0
    engine.setAsync(False)
    clocks = sampler.stop()
    line = None
    if rank == 0:
        flops = 5 * 2 * L * L * HEAD_DIM * heads * rt.world           # whole job
        tflops = flops / (ms[0] * 1e-3) / 1e12
        line = rt.base_line("backward", "backward TFLOP/s", tflops, "TFLOP/s", ms, "f16", settled, launches, clocks,
                            {"seed": 1005, "l2": "the sequence's K/V and gradients (a few MB per KV head) stay in L2 by design"})
        peak = rt.peaks["bf16_tflops"]
        line["roofline"] = {"bound": "tensor", "achieved": tflops / rt.world, "peak": peak, "unit": "TFLOP/s",
                            "frac": tflops / rt.world / peak, "peak_source": f"{rt.peak_kind} cuBLAS bf16 burst", "per": "GPU",
                            "kernel": "backwardMmaKeyTileKernel (+ backwardMmaRowSumKernel, backwardMmaStoreKernel)",
                            "algorithmic_flops_per_step": flops // rt.world, "traffic": None,
                            "note": "mma.sync.m16n8k16 products (legacy tensor path) with float32 accumulation, seven products "
                                    "of which five are counted (S and dP are computed twice)"}
        line["e2e"] = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                       "note": "not measured for this workload"}
        if with_cpu:
            line["cpu_baseline"] = cpu_backward()
    return line


# ------------------------------------------- long-context FP8 decode and step (c4)

def run_c4(rt, with_cpu, want=("decode_c4", "step_c4")):
    """`configs[4]`: 64 sequences with contexts uniform in [32768, 131072], sliding window
    4096, FP8 e4m3 KV with per-(block, kv_head) scales, 64 query / 8 KV heads.  Every block of
    every context is allocated through the manager (the pool holds all tokens, about 10.7 GB
    over all GPUs, as the reference never frees out-of-window blocks); K/V is written
    (quantised by the append kernel) only for the tokens a decode can see, the rest of the
    pool is never read.  `decode_c4` is the 64 decodes; `step_c4` adds the waiting sequence of
    the scheduler's batch: its first 2048-token chunk is appended (quantised) and prefilled
    in the same step.  Returns {name: line}."""
    torch, pam, engine, dev, args = rt.torch, rt.pam, rt.engine, rt.dev, rt.args
    DT = pam.PagedAttentionDataType
    kvh, heads, rank = rt.kvh, rt.heads(C4_HEADS), rt.rank
    ksl, qsl = slice(rank * kvh, (rank + 1) * kvh), slice(rank * heads, (rank + 1) * heads)
    rng = np.random.default_rng(1004)
    n_seq = C4_SEQS if args.batch is None or args.workload not in ("decode_c4", "step_c4") else min(C4_SEQS, args.batch)
    lens = rng.integers(C4_LO, C4_HI + 1, size=C4_SEQS).astype(np.int64)[:n_seq]
    nblk = (lens + BLOCK - 1) // BLOCK
    cache = pam.KVCacheManager(engine, int(nblk.sum()) + 256 + C4_CHUNK // BLOCK, BLOCK, HEAD_DIM, kvh, DT.float8)
    gen = torch.Generator(device=dev)
    for sid in range(n_seq):
        L = int(lens[sid])
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        first = ((L - C4_WINDOW) // BLOCK) * BLOCK                      # first token of the first visible block
        gen.manual_seed(1004 * 1000 + sid)
        kv = torch.randn((2, L - first, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        engine.appendKV(cache, sid, kv[0][:, ksl].contiguous(), kv[1][:, ksl].contiguous(), first, L - first, heads)
    ids = list(range(n_seq))
    max_nb = int(nblk.max())
    tables_h, lens_h = cache.batchTables(ids, max_nb)
    tables = torch.from_numpy(tables_h).to(dev)
    gen.manual_seed(1004 * 1000 + 999983)
    q = torch.randn((n_seq, C4_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)[:, qsl].contiguous()
    out = torch.empty_like(q)
    layer = pam.PagedLayerSpec(HEAD_DIM, heads, kvh, BLOCK, DT.float8, C4_WINDOW)
    lens_dev = torch.from_numpy(lens_h.view(np.int32)).to(dev)
    req = pam.PagedAttentionDecodeRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, tables, lens_dev, out, n_seq, max_nb,
                                          layer, cache.kScaleBuffer, cache.vScaleBuffer)
    decode = lambda: engine.decode(req)
    decode()
    guard_decode(rt, cache, [int(np.argmin(lens)), int(np.argmax(lens))], tables_h, lens_h, q.cpu().numpy(), out.cpu().numpy(),
                 2, 1e-2, window=C4_WINDOW)
    q_pin = q.cpu().pin_memory()
    out_pin = torch.empty_like(q_pin).pin_memory()
    engine.defaultWindowSize = C4_WINDOW                       # pam_decode takes the engine's default window
    decode_host = lambda: engine.decodeBatch(cache, ids, q_pin.data_ptr(), out_pin.data_ptr(), heads)
    # visible tokens per sequence: tokens in blocks >= floor((L - W) / 16); K and V codes, scales, q, out, tables
    nvis = np.array([int(l) - ((int(l) - C4_WINDOW) // BLOCK) * BLOCK for l in lens])
    bytes_decode = int(nvis.sum()) * 2 * kvh * HEAD_DIM + int(((nvis + BLOCK - 1) // BLOCK).sum()) * (kvh * 4 + 4) \
        + 2 * n_seq * heads * HEAD_DIM * 2 + n_seq * 4
    peak = rt.peaks["hbm_gbs"]
    io_decode = n_seq * heads * HEAD_DIM * 2
    lines = {}

    def decode_roofline(ms_decode):
        achieved = bytes_decode / (ms_decode * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"{rt.peak_kind} copy bandwidth", "per": "GPU",
                "kernel": "decodeStreamKernel (FP8 tiles)",
                "algorithmic_bytes_per_launch": bytes_decode, "traffic": decode_traffic("fp8", bytes_decode),
                "traffic_source": "ncu on a 16-sequence cut: bytes read scaled by visible tokens, bytes written constant"}

    l2_note = {"seed": 1004, "l2": "window bytes per step (0.54 GB over all GPUs) exceed L2 up to 4 GPUs; at 8 GPUs a GPU's 67 MB "
                                   "share fits L2 and L2 is flushed between timed steps"}
    small = bytes_decode < 126e6
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None
    flush = (lambda: flush_buf.fill_(1)) if small else None

    if "decode_c4" in want:
        engine.setAsync(True)
        sampler = ClockSampler(rt.local).start()
        for _ in range(max(args.warmup, 3)):
            decode()
        settled = rt.settle(decode)
        launches0 = engine.kernelLaunches
        ms = rt.timed(decode, flush=flush)
        launches = engine.kernelLaunches - launches0
        engine.setAsync(False)
        clocks = sampler.stop()
        e2e = rt.timed_host(decode_host)
        if not args.profile:
            assert torch.equal(out_pin.to(dev), out), "host-buffer path and device path disagree"
        if rank == 0:
            line = rt.base_line("decode_c4", "paged decode tokens/s", n_seq / (ms[0] * 1e-3), "tokens/s", ms,
                                "fp8-e4m3 KV, f16 q/out", settled, launches, clocks, l2_note)
            line["roofline"] = decode_roofline(ms[0])
            line["kv_read_gbs_total"] = line["roofline"]["achieved"] * rt.world
            line["e2e"] = {"value": n_seq / (e2e[0] * 1e-3) if e2e[0] else None, "unit": "tokens/s", "ms_per_step": e2e[0],
                           "ms_per_step_min": e2e[1], "ms_per_step_max": e2e[2],
                           "h2d_bytes_per_step": io_decode + lens_h.nbytes, "d2h_bytes_per_step": io_decode,
                           "call": "pam_decode (engine default window 4096) with page-locked host q/out"}
            if with_cpu:
                line["cpu_baseline"] = cpu_decode_c4()
            lines["decode_c4"] = line

    if "step_c4" in want:
        new_id = n_seq
        sched = pam.ContinuousBatchingScheduler(n_seq + 1, n_seq + 1)
        sids = [sched.addRequest(int(l), 1) for l in lens]
        for q_s in sched.step():
            sched.markPrefilled(q_s.id)
        wid = sched.addRequest(8192, 1)
        batch = [q_s.id for q_s in sched.step()]              # Scheduler.swift:78-114: waiting first, then running
        assert batch == [wid] + sids and sched.waitingCount == 0, "scheduler batch order"
        cache.allocateSequence(new_id)
        cache.appendTokens(new_id, C4_CHUNK)
        gen.manual_seed(1004 * 1000 + new_id)
        kv_new = torch.randn((2, C4_CHUNK, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        k_new, v_new = kv_new[0][:, ksl].contiguous(), kv_new[1][:, ksl].contiguous()
        q_new = torch.randn((C4_CHUNK, C4_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)[:, qsl].contiguous()
        o_new = torch.empty_like(q_new)
        t_new_h, _ = cache.batchTables([new_id], C4_CHUNK // BLOCK)
        t_new = torch.from_numpy(t_new_h).to(dev)

        def make_step(kk, vv, qq, oo, dec):
            def step():
                engine.appendKV(cache, new_id, kk, vv, 0, C4_CHUNK, heads)
                engine.prefillBatch(qq, cache.kPoolBuffer, cache.vPoolBuffer, t_new, oo, [C4_CHUNK], [0], [C4_CHUNK],
                                    C4_CHUNK // BLOCK, layer, True, cache.kScaleBuffer, cache.vScaleBuffer)
                dec()
            return step

        step = make_step(k_new, v_new, q_new, o_new, decode)
        step()
        engine.synchronize()
        # correctness guard for the chunk: a few rows against the oracle on the quantised pages
        from oracle import c_oracle as co
        kc2, vc2, ks2, vs2 = fetch_pages(rt, cache, t_new_h[0], 1, True)
        r0, nr = C4_CHUNK - 8, 8
        refp = co.prefill(q_new[r0:r0 + nr].cpu().numpy(), kc2, vc2, np.arange(len(t_new_h[0]), dtype=np.int32), C4_CHUNK,
                          kvh, BLOCK, 2, q_start=r0, k_scale=ks2.view(np.uint16), v_scale=vs2.view(np.uint16))
        errp = float(np.abs(o_new[r0:r0 + nr].float().cpu().numpy() - refp).max())
        assert errp <= 1e-2, f"FP8 prefill chunk differs from the oracle by {errp}"

        engine.setAsync(True)
        sampler = ClockSampler(rt.local).start()
        for _ in range(max(args.warmup, 3)):
            step()
        settled = rt.settle(step)
        launches0 = engine.kernelLaunches
        ms = rt.timed(step, flush=flush)
        launches = engine.kernelLaunches - launches0
        ms_dec = rt.timed(decode, flush=flush)              # the decode launches alone, for the roofline of the HBM-bound part
        engine.setAsync(False)
        clocks = sampler.stop()
        e2e = (None, None, None)
        io_new = C4_CHUNK * heads * HEAD_DIM * 2
        kv_new_bytes = 2 * C4_CHUNK * kvh * HEAD_DIM * 2
        if not args.profile:
            pins = [t.cpu().pin_memory() for t in (k_new, v_new, q_new)]
            o_pin = torch.empty_like(pins[2]).pin_memory()
            e2e = rt.timed_host(make_step(pins[0], pins[1], pins[2], o_pin, decode_host))
            assert torch.equal(o_pin.to(dev), o_new), "host-buffer path and device path disagree"
        if rank == 0:
            tokens = n_seq + C4_CHUNK
            line = rt.base_line("step_c4", "step tokens/s", tokens / (ms[0] * 1e-3), "tokens/s", ms, "fp8-e4m3 KV, f16 q/out",
                                settled, launches, clocks, l2_note)
            line["roofline"] = decode_roofline(ms_dec[0])
            pf_flops = C4_HEADS * (C4_CHUNK * (C4_CHUNK + 1) // 2) * 4 * HEAD_DIM
            rest = ms[0] - ms_dec[0]
            line["step_parts"] = {"decode_ms": ms_dec[0], "append_and_prefill_ms": rest,
                                  "prefill_chunk_gflop": pf_flops / 1e9,
                                  "prefill_chunk_tflops_lower_bound": pf_flops / (rest * 1e-3) / 1e12 if rest > 0 else None,
                                  "prefill_path": "FP8 pages dequantised to float16 scratch, then prefillTcKernel"}
            line["e2e"] = {"value": tokens / (e2e[0] * 1e-3) if e2e[0] else None, "unit": "tokens/s", "ms_per_step": e2e[0],
                           "ms_per_step_min": e2e[1], "ms_per_step_max": e2e[2],
                           "h2d_bytes_per_step": io_decode + lens_h.nbytes + io_new + kv_new_bytes,
                           "d2h_bytes_per_step": io_decode + io_new,
                           "call": "pam_append_kv + pamc_prefill_batch + pam_decode with page-locked host K/V rows, q and out"}
            lines["step_c4"] = line
    engine.defaultWindowSize = 0
    cache.close()
    return lines


def run_ours(args):
    rt = Runtime(args)
    with_cpu = rt.world == 1 and not args.profile
    names = [args.workload] if args.workload else list(WORKLOADS)
    results = {}
    for name in names:
        if name in results:
            continue
        if name == "decode_c2":
            results[name] = run_decode_c2(rt, with_cpu)
        elif name == "prefill_c3":
            results[name] = run_prefill_c3(rt, with_cpu)
        elif name == "append_c1":
            results[name] = run_append_c1(rt, with_cpu)
        elif name == "backward":
            results[name] = run_backward(rt, with_cpu)
        else:
            want = [n for n in names if n in ("decode_c4", "step_c4")]
            out = run_c4(rt, with_cpu, want)
            for n in want:
                results[n] = out.get(n)
        rt.torch.cuda.empty_cache()
    if rt.rank == 0:
        line = results[names[0]]
        if len(names) > 1:
            line["also"] = {n: results[n] for n in names[1:]}
        print(json.dumps(line))
    rt.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--blocks", type=int, default=10, help="timed blocks of --steps steps each; the median block is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None,
                    help="number of sequences of the chosen workload (smaller values are for profiler captures)")
    ap.add_argument("--workload", default=None, choices=list(WORKLOADS) + ["backward"],
                    help="one workload alone; default: decode_c2 with the others under `also`")
    ap.add_argument("--shards", type=int, default=None,
                    help="single process only: run KV-head group 0 of this many (the per-GPU share of a larger job)")
    ap.add_argument("--profile", action="store_true",
                    help="profiler run: one timed block, no clock-settling loop, no end-to-end leg, no CPU baseline")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
