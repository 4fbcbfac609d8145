"""Benchmark of the paged-KV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B] [--profile]

Default workload `decode_c2`: large-batch paged decode with float16 KV -- 256
sequences, context lengths uniform in [512, 8192], block size 16, head_dim 128,
32 query / 8 KV heads, non-contiguous block tables, seeded synthetic N(0,1)
data.  With N GPUs the KV heads are split into N groups, one per GPU; no
collective runs on the attention path, so the total work is fixed (strong
scaling).  A step is one decode of the whole batch (one new token per
sequence); the metric is decode tokens per second of the whole job.

Prints ONE JSON line: `value` is measured with every input resident in HBM
(CUDA events around exactly K steps on the launching stream, max over ranks);
`e2e` is the same step through the reference-shaped C-ABI call `pam_decode`
with queries and outputs in pinned host memory, copies inside the timed
region; `roofline` relates the decode kernel's algorithmic bytes to the
measured HBM copy bandwidth; `cpu_baseline` is the C oracle (a restatement of
the reference's CPU path) timed on this host's cores on a bounded sample.

`--impl reference` times that CPU path alone (rank 0 only).
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

SEED = 1002
BATCH, LEN_LO, LEN_HI = 256, 512, 8192
HEADS, KV_HEADS, HEAD_DIM, BLOCK = 32, 8, 128, 16
SPARE_BLOCKS = 1024
CPU_SAMPLE_SEQS = 32
FALLBACK_HBM_GBS = 6650.0


def workload_lengths():
    rng = np.random.default_rng(SEED)
    return rng.integers(LEN_LO, LEN_HI + 1, size=BATCH).astype(np.int64)


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(lens, heads, kv_heads):
    """Bytes one decode step must move for `kv_heads` KV heads and `heads` query
    heads: K and V of every context token once, queries, outputs, the touched
    block-table entries and the lengths."""
    kv = int(lens.sum()) * 2 * kv_heads * HEAD_DIM * 2
    qo = 2 * len(lens) * heads * HEAD_DIM * 2
    tables = int(((lens + BLOCK - 1) // BLOCK).sum()) * 4
    return kv + qo + tables + len(lens) * 4


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
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
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------- CPU arm

def cpu_sample_inputs(lens, n_seqs):
    """K/V pools, tables, lengths and queries for the first n_seqs sequences of
    the workload (same lengths, same shapes, N(0,1) float16)."""
    from oracle import paged_oracle as po

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
    return q, k_pool, v_pool, tables, sub.astype(np.uint32)


def time_cpu_path(lens, steps, warmup, n_seqs=CPU_SAMPLE_SEQS):
    n_seqs = min(n_seqs, len(lens))
    """The reference's CPU path (its decode loop restated in C, OpenMP over
    (sequence, kv head)) on all host cores; tokens/s over the sample."""
    from oracle import c_oracle as co

    q, k_pool, v_pool, tables, l = cpu_sample_inputs(lens, n_seqs)
    # all host cores this process may run on (a launcher may have set OMP_NUM_THREADS=1)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    for _ in range(max(warmup, 1)):
        co.decode(q, k_pool, v_pool, tables, l, KV_HEADS, BLOCK, 1, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        co.decode(q, k_pool, v_pool, tables, l, KV_HEADS, BLOCK, 1, nthreads=cores)
    dt = (time.perf_counter() - t0) / steps
    return {"value": n_seqs / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {n_seqs} of {BATCH} sequences of the workload ({int(l.sum())} context tokens), "
                      f"{steps} timed passes of {dt * 1e3:.1f} ms",
            "ms_per_step_sample": dt * 1e3}


def config_dict(n_gpus):
    return {"workload": f"decode_c2: batch {BATCH}, context U[512,8192], block 16, head_dim 128, 32 q / 8 kv heads, "
                        "float16 KV, random non-contiguous block tables",
            "seed": SEED, "sharding": f"kv-head groups over {n_gpus} GPU(s), no collective on the attention path",
            "l2": "inputs larger than L2 (KV read per step per GPU exceeds 126 MB); no flush needed"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lens = workload_lengths()
    cb = time_cpu_path(lens, max(args.steps, 1), args.warmup)
    line = {"impl": "reference", "metric": "paged decode tokens/s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": cb["ms_per_step_sample"] * BATCH / min(CPU_SAMPLE_SEQS, BATCH),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config_dict(args.gpus), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# --------------------------------------------------------------------- GPU arm

def scramble_free_list(cache, n_blocks, rng):
    """Make the allocator hand out blocks in a random order, as after a long
    run of a server: take every block with one-block sequences, free them in a
    random order (the fifo policy re-uses blocks in the order they were freed)."""
    base = 1 << 40
    for i in range(n_blocks):
        cache.allocateSequence(base + i)
        cache.appendTokens(base + i, 1)
    for i in rng.permutation(n_blocks):
        cache.freeSequence(base + int(i))


def run_ours(args):
    import torch
    import torch.distributed as dist

    import pagedattentionmetal_b200 as pam

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    assert KV_HEADS % world == 0, "the KV heads must divide over the GPUs"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    kvh = KV_HEADS // world
    heads = HEADS // world
    DT = pam.PagedAttentionDataType

    lens = workload_lengths()
    nblk = (lens + BLOCK - 1) // BLOCK
    n_pool = int(nblk.sum()) + SPARE_BLOCKS
    engine = pam.PagedAttentionEngine(local)
    # a stream of torch's that is not the legacy default stream, shared with the
    # library so that torch's events time the library's kernels
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    engine.setStream(stream.cuda_stream)
    cache = pam.KVCacheManager(engine, n_pool, BLOCK, HEAD_DIM, kvh, DT.float16)
    scramble_free_list(cache, n_pool, np.random.default_rng(SEED + 2))
    ids = list(range(BATCH))
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
    q_full = torch.randn((BATCH, HEADS, HEAD_DIM), generator=gen, device=dev, dtype=torch.float32).to(torch.float16)
    q_dev = q_full[:, rank * heads:(rank + 1) * heads, :].contiguous()
    out_dev = torch.empty_like(q_dev)
    max_nb = int(nblk.max())
    tables_h, lens_h = cache.batchTables(ids, max_nb)
    assert np.array_equal(lens_h.astype(np.int64), lens)
    tables_dev = torch.from_numpy(tables_h).to(dev)
    lens_dev = torch.from_numpy(lens_h.view(np.int32)).to(dev)
    layer = pam.PagedLayerSpec(HEAD_DIM, heads, kvh, BLOCK, DT.float16)
    req = pam.PagedAttentionDecodeRequest(q_dev, cache.kPoolBuffer, cache.vPoolBuffer, tables_dev, lens_dev, out_dev,
                                          BATCH, max_nb, layer)
    q_pin = torch.empty((BATCH, heads, HEAD_DIM), dtype=torch.float16, pin_memory=True)
    q_pin.copy_(q_dev)
    out_pin = torch.empty_like(q_pin, pin_memory=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # correctness guard on two sequences against the oracle (rank 0, its own heads)
    engine.decode(req)
    if rank == 0:
        from oracle import c_oracle as co
        chk = [int(np.argmin(lens)), 3]
        sub_tables, sub_lens = cache.batchTables(chk, max_nb)
        # gather the pages of the two sequences into a small pool for the oracle
        used = np.unique(np.concatenate([sub_tables[i, : (int(sub_lens[i]) + BLOCK - 1) // BLOCK] for i in range(2)]))
        remap = {int(b): i for i, b in enumerate(used)}
        pools = []
        for pb in (cache.kPoolBuffer, cache.vPoolBuffer):
            page_elems = kvh * BLOCK * HEAD_DIM
            small = np.empty((len(used), kvh, BLOCK, HEAD_DIM), np.float16)
            from pagedattentionmetal_b200._cabi import lib
            for i, b in enumerate(used):
                lib.pamc_memcpy(engine._ctx, small[i].ctypes.data, pb.ptr + int(b) * page_elems * 2, page_elems * 2, 1)
            pools.append(small)
        t2 = np.vectorize(lambda b: remap.get(int(b), 0))(sub_tables).astype(np.int32)
        ref = co.decode(q_dev[chk].cpu().numpy(), pools[0], pools[1], t2, sub_lens, kvh, BLOCK, 1)
        err = float(np.abs(out_dev[chk].float().cpu().numpy() - ref).max())
        assert err <= 2e-3, f"decode differs from the oracle by {err}"

    # ---- value: inputs resident in HBM, kernels only ----
    engine.setAsync(True)
    sampler = ClockSampler(local)
    sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        engine.decode(req)
    # keep the GPU busy for about half a second before timing, so that the
    # clock sampler sees the clocks the timed region runs at
    t_busy = time.perf_counter()
    while not args.profile and time.perf_counter() - t_busy < 0.5:
        for _ in range(10):
            engine.decode(req)
        torch.cuda.synchronize(dev)
        warm += 10
    barrier()
    launches0 = engine.kernelLaunches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        engine.decode(req)
    e1.record(stream)
    barrier()
    engine.synchronize()        # raises if a kernel of the timed region reported an error
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    engine.setAsync(False)

    # ---- e2e: the reference-shaped call with host buffers ----
    e2e_steps = 0 if args.profile else args.steps
    for _ in range(0 if args.profile else max(args.warmup, 3)):
        engine.decodeBatch(cache, ids, q_pin.data_ptr(), out_pin.data_ptr(), heads)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        engine.decodeBatch(cache, ids, q_pin.data_ptr(), out_pin.data_ptr(), heads)
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / max(e2e_steps, 1)
    launches = engine.kernelLaunches - launches0
    clocks = sampler.stop()
    if not args.profile:
        assert torch.equal(out_pin.to(dev), out_dev), "host-buffer path and device path disagree"

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        bytes_gpu = algorithmic_bytes(lens, heads, kvh)
        achieved = bytes_gpu / (ms_step * 1e-3) / 1e9
        cpu = time_cpu_path(lens, 90, 2) if world == 1 and not args.profile else None   # about 10 s of CPU work
        io_bytes = BATCH * heads * HEAD_DIM * 2
        line = {
            "metric": "paged decode tokens/s", "value": BATCH / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_dict(world),
            "kv_read_gbs_total": achieved * world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} copy bandwidth", "per": "GPU",
                         "kernel": "decodeSplitKernel (+ decodeMergeKernel, same timed step)",
                         "algorithmic_bytes_per_launch": bytes_gpu,
                         # DRAM read+write of one launch: 1.010 x algorithmic, from an ncu capture of the same
                         # kernel on a 64-sequence case (profiles/decode_split_f16_b64_full.md), scaled by tokens
                         "traffic": bytes_gpu * 1.010, "traffic_source": "ncu on batch 64, scaled by context tokens"},
            "e2e": {"value": BATCH / (e2e_ms * 1e-3) if e2e_steps else None, "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": io_bytes + tables_h.nbytes + lens_h.nbytes, "d2h_bytes_per_step": io_bytes,
                    "call": "pam_decode with pinned host q/out; block tables rebuilt and uploaded per call"},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    cache.close()
    engine.close()
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------- prefill workload (c3)

PF_SEQS, PF_LEN, PF_CHUNK, PF_PREFIX = 16, 2048, 512, 1024


def run_prefill(args):
    """Chunked causal prefill with prefix caching (`configs[3]`): 16 sequences x
    2048 prompt tokens in 512-token chunks, all sharing an identical 1024-token
    prefix (its pages are shared through the manager's prefix cache and written
    once), bf16, 32 q / 8 kv heads, head_dim 128, block 16.  A step is the four
    chunk launches (one launch per chunk for all 16 sequences); the metric is
    algorithmic TFLOP/s: 16 x 32 x (2048 x 2049 / 2) x 4 x 128 = 550.0 GFLOP per
    step, masked pairs and softmax not counted.  Tensor-bound."""
    import torch

    import pagedattentionmetal_b200 as pam

    DT = pam.PagedAttentionDataType
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    engine = pam.PagedAttentionEngine(0)
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    engine.setStream(stream.cuda_stream)
    nblk_seq = PF_LEN // BLOCK
    cache = pam.KVCacheManager(engine, PF_SEQS * nblk_seq + 64, BLOCK, HEAD_DIM, KV_HEADS, DT.bfloat16)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1003)
    prefix_kv = torch.randn((2, PF_PREFIX, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
    prefix_q = torch.randn((PF_PREFIX, HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
    qs = []
    hashes = list(range(PF_PREFIX // BLOCK))
    for sid in range(PF_SEQS):
        cache.allocateSequence(sid)
        cache.appendTokens(sid, PF_PREFIX, hashes)              # followers hit the leader's pages
        if sid == 0:
            engine.appendKV(cache, 0, prefix_kv[0].contiguous(), prefix_kv[1].contiguous(), 0, PF_PREFIX, HEADS)
        cache.appendTokens(sid, PF_LEN - PF_PREFIX)
        kv = torch.randn((2, PF_LEN - PF_PREFIX, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
        engine.appendKV(cache, sid, kv[0].contiguous(), kv[1].contiguous(), PF_PREFIX, PF_LEN - PF_PREFIX, HEADS)
        q_own = torch.randn((PF_LEN - PF_PREFIX, HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
        qs.append(torch.cat([prefix_q, q_own]))
    stats = cache.memoryStats()
    assert stats.sharedBlocks == PF_PREFIX // BLOCK and stats.prefixCacheHits == (PF_SEQS - 1) * (PF_PREFIX // BLOCK)
    tables_h, _ = cache.batchTables(list(range(PF_SEQS)), nblk_seq)
    tables = torch.from_numpy(tables_h).to(dev)
    layer = pam.PagedLayerSpec(HEAD_DIM, HEADS, KV_HEADS, BLOCK, DT.bfloat16)
    n_chunks = PF_LEN // PF_CHUNK
    q_chunks = [torch.cat([qs[s][c * PF_CHUNK:(c + 1) * PF_CHUNK] for s in range(PF_SEQS)]).contiguous() for c in range(n_chunks)]
    outs = [torch.empty_like(q_chunks[c]) for c in range(n_chunks)]

    def step():
        for c in range(n_chunks):
            engine.prefillBatch(q_chunks[c], cache.kPoolBuffer, cache.vPoolBuffer, tables, outs[c],
                                [(c + 1) * PF_CHUNK] * PF_SEQS, [c * PF_CHUNK] * PF_SEQS, [PF_CHUNK] * PF_SEQS,
                                nblk_seq, layer, True)

    # correctness guard: a few rows of one follower sequence against the oracle
    step()
    engine.synchronize()
    from oracle import c_oracle as co
    from oracle import paged_oracle as po
    gk, gv, _, _ = cache.readPools()
    sid, c, r0, n = min(5, PF_SEQS - 1), 2, 100, 8
    ref = co.prefill(qs[sid][c * PF_CHUNK + r0: c * PF_CHUNK + r0 + n].view(torch.uint16).cpu().numpy(), gk, gv,
                     tables_h[sid], (c + 1) * PF_CHUNK, KV_HEADS, BLOCK, 3, q_start=c * PF_CHUNK + r0)
    got = po.from_bf16_bits(outs[c][sid * PF_CHUNK + r0: sid * PF_CHUNK + r0 + n].view(torch.uint16).cpu().numpy())
    err = float(np.abs(got - ref).max())
    assert err <= 2e-3 + 2.0 ** -8, f"prefill differs from the oracle by {err}"
    tensor_path = engine.lastStats.operation == pam.Operation.prefillMMA

    engine.setAsync(True)
    sampler = ClockSampler(0)
    sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    t_busy = time.perf_counter()
    while not args.profile and time.perf_counter() - t_busy < 0.5:
        step()
        torch.cuda.synchronize(dev)
        warm += 1
    torch.cuda.synchronize(dev)
    launches0 = engine.kernelLaunches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    engine.synchronize()        # raises if a kernel of the timed region reported an error
    ms_step = e0.elapsed_time(e1) / args.steps
    launches = engine.kernelLaunches - launches0
    clocks = sampler.stop()
    flops = PF_SEQS * HEADS * (PF_LEN * (PF_LEN + 1) // 2) * 4 * HEAD_DIM
    tflops = flops / (ms_step * 1e-3) / 1e12

    # ---- e2e: the same four chunk calls with q and the output in pinned host memory ----
    engine.setAsync(False)
    q_pin = [q.cpu().pin_memory() for q in q_chunks]
    out_pin = [torch.empty_like(q).pin_memory() for q in q_pin]

    def step_host():
        for c in range(n_chunks):
            engine.prefillBatch(q_pin[c], cache.kPoolBuffer, cache.vPoolBuffer, tables, out_pin[c],
                                [(c + 1) * PF_CHUNK] * PF_SEQS, [c * PF_CHUNK] * PF_SEQS, [PF_CHUNK] * PF_SEQS,
                                nblk_seq, layer, True)

    e2e_ms, e2e_steps = None, 0 if args.profile else args.steps
    if e2e_steps:
        for _ in range(3):
            step_host()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_host()
        torch.cuda.synchronize(dev)
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        assert torch.equal(out_pin[n_chunks - 1].to(dev), outs[n_chunks - 1]), "host-buffer path and device path disagree"
    io_bytes = sum(q.numel() * 2 for q in q_pin)

    # ---- CPU baseline: the C oracle's prefill over the whole step (every row of all 16 sequences) ----
    cpu = None
    if not args.profile:
        t0 = time.perf_counter()
        for s_i in range(PF_SEQS):
            co.prefill(qs[s_i].view(torch.uint16).cpu().numpy(), gk, gv, tables_h[s_i], PF_LEN, KV_HEADS, BLOCK, 3, q_start=0)
        dt = time.perf_counter() - t0
        cpu = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": co.max_threads(), "kind": "port",
               "sample": f"the whole step once: 16 sequences x 2048 rows x 32 heads, causal ({dt:.1f} s): "
                         "oracle/paged_oracle.c orc_prefill, OpenMP over (row, head)"}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
            peak, kind = float(mp["bf16_tflops"]), "measured cuBLAS bf16 burst"
            sustained = float(mp.get("bf16_tflops_sustained", 0)) or None
    except Exception:
        peak, kind, sustained = 1590.0, "fallback", 1400.0
    line = {"metric": "prefill TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "prefill_c3: 16 seqs x 2048 tokens, chunks of 512, shared 1024-token prefix, bf16, "
                                   "32 q / 8 kv heads, head_dim 128, block 16", "seed": 1003},
            "tokens_per_s": PF_SEQS * PF_LEN / (ms_step * 1e-3),
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                         "peak_source": kind, "kernel": "prefillTcKernel" if tensor_path else "prefillGeneralKernel",
                         "algorithmic_flops_per_step": flops, "traffic": None,
                         # the step is timed inside a half-second loop of back-to-back steps: the fraction of the
                         # sustained cuBLAS figure is given beside the fraction of its burst figure
                         "frac_of_sustained": tflops / sustained if sustained else None, "peak_sustained": sustained},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12 if e2e_ms else None, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                    "call": "pamc_prefill_batch per chunk with pinned host q/out (block tables resident)"},
            "gpu_launches": int(launches), "clocks": clocks}
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    cache.close()
    engine.close()


# ------------------------------------------------ KV append + FP8 quantisation + CoW copy (c1)

C1_TOKENS, C1_BLOCKS, C1_COPIES = 4096, 4096, 512


def run_append(args):
    """`configs[1]`: 4096 new tokens (float16 K/V, 8 KV heads x 128) scattered by a slot
    mapping of random distinct slots into a pool of 4096 blocks x 16, once as float16 and
    once quantised to FP8 e4m3 with per-(block, kv_head) scales, plus the copy of 512
    random blocks (copy-on-write).  A step is the three calls; the working set is smaller
    than L2, so L2 is flushed (a 512 MB buffer is written) before every timed step and
    every step is timed with its own pair of CUDA events.  Metric: algorithmic GB/s."""
    import torch

    import pagedattentionmetal_b200 as pam

    DT = pam.PagedAttentionDataType
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    engine = pam.PagedAttentionEngine(0)
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    engine.setStream(stream.cuda_stream)
    rng = np.random.default_rng(1001)
    T, nblk = C1_TOKENS, C1_BLOCKS
    k_h = rng.standard_normal((T, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    v_h = rng.standard_normal((T, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
    slots_h = rng.choice(nblk * BLOCK, T, replace=False).astype(np.int64)
    perm = rng.permutation(nblk)
    src, dst = perm[:C1_COPIES].astype(np.int32), perm[C1_COPIES:2 * C1_COPIES].astype(np.int32)
    k, v, slots = torch.from_numpy(k_h).to(dev), torch.from_numpy(v_h).to(dev), torch.from_numpy(slots_h).to(dev)
    c16 = pam.KVCacheManager(engine, nblk, BLOCK, HEAD_DIM, KV_HEADS, DT.float16)
    c8 = pam.KVCacheManager(engine, nblk, BLOCK, HEAD_DIM, KV_HEADS, DT.float8)

    def step():
        engine.reshapeAndCache(c16, k, v, slots, T)
        engine.reshapeAndCache(c8, k, v, slots, T)
        engine.copyBlocks(c16, src, dst)

    # correctness guard: pools, codes and scales bit for bit against the oracle
    step()
    engine.synchronize()
    from oracle import c_oracle as co
    kp = np.zeros((nblk, KV_HEADS, BLOCK, HEAD_DIM), np.float16)
    vp = np.zeros_like(kp)
    co.reshape_and_cache(k_h, v_h, kp, vp, slots_h, BLOCK)
    co.copy_blocks(kp, vp, src, dst)
    gk, gv, _, _ = c16.readPools()
    assert np.array_equal(gk, kp) and np.array_equal(gv, vp), "float16 append or block copy differs from the oracle"
    kc = np.zeros((nblk, KV_HEADS, BLOCK, HEAD_DIM), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((nblk, KV_HEADS), np.float16)
    vs = np.zeros_like(ks)
    co.reshape_and_cache_fp8(k_h, v_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots_h, BLOCK)
    gk8, gv8, gks, gvs = c8.readPools()
    assert np.array_equal(gk8, kc) and np.array_equal(gv8, vc), "FP8 codes differ from the oracle"
    assert np.array_equal(gks, ks) and np.array_equal(gvs, vs), "FP8 scales differ from the oracle"

    engine.setAsync(True)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    sampler = ClockSampler(0)
    sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize(dev)
    launches0 = engine.kernelLaunches
    total_ms = 0.0
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        step()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        total_ms += e0.elapsed_time(e1)
    engine.synchronize()
    ms_step = total_ms / args.steps
    launches = engine.kernelLaunches - launches0
    clocks = sampler.stop()
    row = KV_HEADS * HEAD_DIM

    # ---- the same scatters with 16 times the tokens: 65 536 tokens that fill every slot of the
    # pool (a permutation of all slots), where the kernels run long enough for HBM to bound them
    x16 = None
    if not args.profile:
        T16 = nblk * BLOCK
        k16_h = rng.standard_normal((T16, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
        v16_h = rng.standard_normal((T16, KV_HEADS, HEAD_DIM), dtype=np.float32).astype(np.float16)
        slots16_h = rng.permutation(T16).astype(np.int64)
        k16, v16 = torch.from_numpy(k16_h).to(dev), torch.from_numpy(v16_h).to(dev)
        slots16 = torch.from_numpy(slots16_h).to(dev)

        def step16():
            engine.reshapeAndCache(c16, k16, v16, slots16, T16)
            engine.reshapeAndCache(c8, k16, v16, slots16, T16)

        step16()
        engine.synchronize()
        kp16 = np.zeros((nblk, KV_HEADS, BLOCK, HEAD_DIM), np.float16)
        vp16 = np.zeros_like(kp16)
        co.reshape_and_cache(k16_h, v16_h, kp16, vp16, slots16_h, BLOCK)
        gk, gv, _, _ = c16.readPools()
        assert np.array_equal(gk, kp16) and np.array_equal(gv, vp16), "x16 float16 append differs from the oracle"
        # the FP8 pool already holds codes and scales of the steps before: the oracle replays them
        for _ in range(warm + args.steps):
            co.reshape_and_cache_fp8(k_h, v_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots_h, BLOCK)
        co.reshape_and_cache_fp8(k16_h, v16_h, kc, vc, ks.view(np.uint16), vs.view(np.uint16), slots16_h, BLOCK)
        gk8, gv8, gks, gvs = c8.readPools()
        assert np.array_equal(gk8, kc) and np.array_equal(gv8, vc), "x16 FP8 codes differ from the oracle"
        assert np.array_equal(gks, ks) and np.array_equal(gvs, vs), "x16 FP8 scales differ from the oracle"
        for _ in range(3):
            step16()
        torch.cuda.synchronize(dev)
        t16 = 0.0
        for _ in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            step16()
            e1.record(stream)
            torch.cuda.synchronize(dev)
            t16 += e0.elapsed_time(e1)
        engine.synchronize()
        ms16 = t16 / args.steps
        bytes16 = 2 * (T16 * row * 2) * 2 + 2 * (T16 * row * 2) + 2 * (T16 * row) + 2 * 2 * nblk * KV_HEADS * 2 + T16 * 8 * 2
        peak16, _ = measured_hbm_peak()
        x16 = {"tokens": T16, "ms_per_step": ms16, "algorithmic_bytes": bytes16,
               "gbs": bytes16 / (ms16 * 1e-3) / 1e9, "frac": bytes16 / (ms16 * 1e-3) / 1e9 / peak16,
               "what": "float16 scatter + FP8 scatter of 65 536 tokens over all slots of the pool, no block copies"}
    block16 = KV_HEADS * BLOCK * HEAD_DIM * 2
    bytes_f16 = 2 * (T * row * 2) * 2                         # K and V: read + write
    bytes_fp8 = 2 * (T * row * 2) + 2 * (T * row) + 2 * 2 * T * KV_HEADS * 2   # read f16, write codes, scales (upper bound)
    bytes_cow = 2 * C1_COPIES * block16 * 2                   # K and V blocks: read + write
    total = bytes_f16 + bytes_fp8 + bytes_cow + T * 8 * 2
    peak, kind = measured_hbm_peak()
    achieved = total / (ms_step * 1e-3) / 1e9
    line = {"metric": "KV append GB/s", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 -> f16 / fp8-e4m3", "data": "synthetic",
            "config": {"workload": "append_c1: 4096 tokens x 8 kv heads x 128 scattered to random distinct slots of a "
                                   "4096-block pool as float16 and as FP8 e4m3 with (block, kv_head) scales, plus a copy of "
                                   "512 random blocks", "seed": 1001, "l2": "flushed before every timed step (512 MB written)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{kind} copy bandwidth",
                         "kernel": "reshapeAndCacheKernel, fp8AbsmaxKernel + fp8QuantizeKernel, copyBlocksKernel",
                         "algorithmic_bytes_per_launch": total, "traffic": None,
                         "note": "126 MB per step in 4 short kernels: launch latency, not HBM, bounds it"},
            "tokens_per_s": T / (ms_step * 1e-3), "gpu_launches": int(launches), "clocks": clocks}
    if x16 is not None:
        line["x16"] = x16
    print(json.dumps(line))
    c16.close()
    c8.close()
    engine.close()


# ------------------------------------------- long-context FP8 decode (c4)

C4_SEQS, C4_LO, C4_HI, C4_WINDOW, C4_HEADS, C4_CHUNK = 64, 32768, 131072, 4096, 64, 2048


def run_decode_fp8(args):
    """Decode part of `configs[4]`: 64 sequences with contexts uniform in
    [32768, 131072], sliding window 4096, FP8 e4m3 KV with per-(block, kv_head)
    scales, 64 query / 8 KV heads, head_dim 128, block 16.  Every block of every
    context is allocated through the manager (the pool holds all tokens, about
    10.7 GB, as the reference never frees out-of-window blocks); K/V is written
    (quantised by the append kernel) only for the tokens a decode can see, the
    rest of the pool is never read.  Metric: decode tokens/s; roofline: bytes of
    the visible window."""
    import torch

    import pagedattentionmetal_b200 as pam

    DT = pam.PagedAttentionDataType
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    engine = pam.PagedAttentionEngine(0)
    stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(stream)
    engine.setStream(stream.cuda_stream)
    rng = np.random.default_rng(1004)
    n_seq = min(C4_SEQS, args.batch) if args.batch != 256 else C4_SEQS
    lens = rng.integers(C4_LO, C4_HI + 1, size=n_seq).astype(np.int64)
    nblk = (lens + BLOCK - 1) // BLOCK
    cache = pam.KVCacheManager(engine, int(nblk.sum()) + 256 + C4_CHUNK // BLOCK, BLOCK, HEAD_DIM, KV_HEADS, DT.float8)
    gen = torch.Generator(device=dev)
    visible = 0
    for sid in range(n_seq):
        L = int(lens[sid])
        cache.allocateSequence(sid)
        cache.appendTokens(sid, L)
        first = ((L - C4_WINDOW) // BLOCK) * BLOCK                      # first token of the first visible block
        n = L - first
        visible += n
        gen.manual_seed(1004 * 1000 + sid)
        kv = torch.randn((2, n, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        engine.appendKV(cache, sid, kv[0].contiguous(), kv[1].contiguous(), first, n, C4_HEADS)
    max_nb = int(nblk.max())
    tables_h, lens_h = cache.batchTables(list(range(n_seq)), max_nb)
    tables = torch.from_numpy(tables_h).to(dev)
    lens_dev = torch.from_numpy(lens_h.view(np.int32)).to(dev)
    q = torch.randn((n_seq, C4_HEADS, HEAD_DIM), device=dev).to(torch.float16)
    out = torch.empty_like(q)
    layer = pam.PagedLayerSpec(HEAD_DIM, C4_HEADS, KV_HEADS, BLOCK, DT.float8, C4_WINDOW)
    req = pam.PagedAttentionDecodeRequest(q, cache.kPoolBuffer, cache.vPoolBuffer, tables, lens_dev, out, n_seq, max_nb,
                                          layer, cache.kScaleBuffer, cache.vScaleBuffer)
    engine.decode(req)
    # correctness guard: one sequence against the oracle (its visible pages only)
    from oracle import c_oracle as co
    from pagedattentionmetal_b200._cabi import lib
    sid = int(np.argmin(lens))
    L = int(lens[sid])
    first_blk = (L - C4_WINDOW) // BLOCK
    used = tables_h[sid, first_blk: (L + BLOCK - 1) // BLOCK]
    page = KV_HEADS * BLOCK * HEAD_DIM
    kc = np.zeros((len(used), KV_HEADS, BLOCK, HEAD_DIM), np.uint8)
    vc = np.zeros_like(kc)
    ks = np.zeros((len(used), KV_HEADS), np.float16)
    vs = np.zeros_like(ks)
    kp, vp, ksp, vsp = cache.kPoolBuffer.ptr, cache.vPoolBuffer.ptr, cache.kScaleBuffer.ptr, cache.vScaleBuffer.ptr
    for i, b in enumerate(used):
        lib.pamc_memcpy(engine._ctx, kc[i].ctypes.data, kp + int(b) * page, page, 1)
        lib.pamc_memcpy(engine._ctx, vc[i].ctypes.data, vp + int(b) * page, page, 1)
        lib.pamc_memcpy(engine._ctx, ks[i].ctypes.data, ksp + int(b) * KV_HEADS * 2, KV_HEADS * 2, 1)
        lib.pamc_memcpy(engine._ctx, vs[i].ctypes.data, vsp + int(b) * KV_HEADS * 2, KV_HEADS * 2, 1)
    t2 = np.zeros((1, (L + BLOCK - 1) // BLOCK), np.int32)
    t2[0, first_blk:] = np.arange(len(used))
    ref = co.decode(q[sid:sid + 1].cpu().numpy(), kc, vc, t2, np.array([L], np.uint32), KV_HEADS, BLOCK, 2,
                    window=C4_WINDOW, k_scale=ks.view(np.uint16), v_scale=vs.view(np.uint16))
    err = float(np.abs(out[sid:sid + 1].float().cpu().numpy() - ref).max())
    assert err <= 1e-2, f"FP8 decode differs from the oracle by {err}"

    # ---- the waiting sequence of the whole step (`step_c4`): its first 2048-token chunk is
    # appended (quantised to FP8) and prefilled in the same step as the 64 decodes
    whole = args.workload == "step_c4"
    step_tokens = n_seq
    decode_only = lambda: engine.decode(req)
    step = decode_only
    if whole:
        new_id = n_seq
        sched = pam.ContinuousBatchingScheduler(n_seq + 1, n_seq + 1)
        ids = [sched.addRequest(int(l), 1) for l in lens]
        for q_s in sched.step():
            sched.markPrefilled(q_s.id)
        wid = sched.addRequest(8192, 1)
        batch = [q_s.id for q_s in sched.step()]              # Scheduler.swift:78-114: waiting first, then running
        assert batch == [wid] + ids and sched.waitingCount == 0, "scheduler batch order"
        cache.allocateSequence(new_id)
        cache.appendTokens(new_id, C4_CHUNK)
        gen.manual_seed(1004 * 1000 + new_id)
        kv_new = torch.randn((2, C4_CHUNK, KV_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        k_new, v_new = kv_new[0].contiguous(), kv_new[1].contiguous()
        q_new = torch.randn((C4_CHUNK, C4_HEADS, HEAD_DIM), generator=gen, device=dev).to(torch.float16)
        o_new = torch.empty_like(q_new)
        t_new_h, _ = cache.batchTables([new_id], C4_CHUNK // BLOCK)
        t_new = torch.from_numpy(t_new_h).to(dev)

        def step():
            engine.appendKV(cache, new_id, k_new, v_new, 0, C4_CHUNK, C4_HEADS)
            engine.prefillBatch(q_new, cache.kPoolBuffer, cache.vPoolBuffer, t_new, o_new, [C4_CHUNK], [0], [C4_CHUNK],
                                C4_CHUNK // BLOCK, layer, True, cache.kScaleBuffer, cache.vScaleBuffer)
            engine.decode(req)

        step()
        engine.synchronize()
        prefill_tensor = None
        # correctness guard for the chunk: a few rows against the oracle on the quantised pages
        used_n = t_new_h[0]
        kc2 = np.zeros((len(used_n), KV_HEADS, BLOCK, HEAD_DIM), np.uint8)
        vc2 = np.zeros_like(kc2)
        ks2 = np.zeros((len(used_n), KV_HEADS), np.float16)
        vs2 = np.zeros_like(ks2)
        for i, b in enumerate(used_n):
            lib.pamc_memcpy(engine._ctx, kc2[i].ctypes.data, kp + int(b) * page, page, 1)
            lib.pamc_memcpy(engine._ctx, vc2[i].ctypes.data, vp + int(b) * page, page, 1)
            lib.pamc_memcpy(engine._ctx, ks2[i].ctypes.data, ksp + int(b) * KV_HEADS * 2, KV_HEADS * 2, 1)
            lib.pamc_memcpy(engine._ctx, vs2[i].ctypes.data, vsp + int(b) * KV_HEADS * 2, KV_HEADS * 2, 1)
        r0, nr = C4_CHUNK - 8, 8
        refp = co.prefill(q_new[r0:r0 + nr].cpu().numpy(), kc2, vc2, np.arange(len(used_n), dtype=np.int32), C4_CHUNK,
                          KV_HEADS, BLOCK, 2, q_start=r0, k_scale=ks2.view(np.uint16), v_scale=vs2.view(np.uint16))
        errp = float(np.abs(o_new[r0:r0 + nr].float().cpu().numpy() - refp).max())
        assert errp <= 1e-2, f"FP8 prefill chunk differs from the oracle by {errp}"
        step_tokens = n_seq + C4_CHUNK

    engine.setAsync(True)
    sampler = ClockSampler(0)
    sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    t_busy = time.perf_counter()
    while not args.profile and time.perf_counter() - t_busy < 0.5:
        for _ in range(10):
            step()
        torch.cuda.synchronize(dev)
        warm += 10
    torch.cuda.synchronize(dev)
    launches0 = engine.kernelLaunches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    engine.synchronize()        # raises if a kernel of the timed region reported an error
    ms_step = e0.elapsed_time(e1) / args.steps
    launches = engine.kernelLaunches - launches0
    ms_decode = ms_step
    if whole:
        # the decode launches alone, for the roofline of the HBM-bound kernel of the step
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record(stream)
        for _ in range(args.steps):
            engine.decode(req)
        d1.record(stream)
        torch.cuda.synchronize(dev)
        engine.synchronize()
        ms_decode = d0.elapsed_time(d1) / args.steps
    # The same decode launches replayed from a CUDA graph: the device time of the kernels
    # without the host's per-call work (request checks, launch calls), which is of the same
    # order as this short step.
    ms_graph = None
    try:
        if args.profile:
            raise RuntimeError("skipped under --profile")
        graph = torch.cuda.CUDAGraph()
        cap = torch.cuda.Stream(dev)
        cap.wait_stream(stream)
        engine.setStream(cap.cuda_stream)
        with torch.cuda.graph(graph, stream=cap):
            for _ in range(args.steps):
                engine.decode(req)
        engine.setStream(stream.cuda_stream)
        stream.wait_stream(cap)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(dev)
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        graph.replay()
        g1.record(stream)
        torch.cuda.synchronize(dev)
        engine.synchronize()
        ms_graph = g0.elapsed_time(g1) / args.steps
    except Exception as exc:           # capture refused: the eager figures stand alone
        engine.setStream(stream.cuda_stream)
        print(f"graph replay not measured: {exc}", file=sys.stderr)
    clocks = sampler.stop()
    # visible tokens per sequence: tokens in blocks >= floor((L - W) / 16); K and V codes, scales, q, out, tables
    nvis = np.array([int(l) - ((int(l) - C4_WINDOW) // BLOCK) * BLOCK for l in lens])
    bytes_step = int(nvis.sum()) * 2 * KV_HEADS * HEAD_DIM + int(((nvis + BLOCK - 1) // BLOCK).sum()) * (KV_HEADS * 4 + 4) \
        + 2 * n_seq * C4_HEADS * HEAD_DIM * 2 + n_seq * 4
    peak, kind = measured_hbm_peak()
    achieved = bytes_step / (ms_decode * 1e-3) / 1e9
    line = {"metric": "step tokens/s" if whole else "paged decode tokens/s", "value": step_tokens / (ms_step * 1e-3),
            "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8-e4m3 KV, f16 q/out", "data": "synthetic",
            "config": {"workload": ("step_c4: one scheduler step = append + prefill of a 2048-token chunk of a new "
                                    "sequence, and " if whole else "decode_c4: ") +
                                   f"{n_seq} seqs, context U[32768,131072], window 4096, FP8 e4m3 KV with "
                                   "(block, kv_head) scales, 64 q / 8 kv heads, head_dim 128, block 16", "seed": 1004,
                       "l2": "window bytes per step (0.54 GB) exceed L2; contexts are resident, only the window is read"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{kind} copy bandwidth", "kernel": "decodeSplitFp8Kernel (+ decodeMergeKernel)",
                         "algorithmic_bytes_per_launch": bytes_step, "traffic": None},
            "gpu_launches": int(launches), "clocks": clocks}
    if ms_graph is not None:
        line["graph_replay"] = {"decode_ms_per_step": ms_graph, "kv_read_gbs": bytes_step / (ms_graph * 1e-3) / 1e9,
                                "frac": bytes_step / (ms_graph * 1e-3) / 1e9 / peak}
    if whole:
        pf_flops = C4_HEADS * (C4_CHUNK * (C4_CHUNK + 1) // 2) * 4 * HEAD_DIM
        line["step_parts"] = {"decode_ms": ms_decode, "append_and_prefill_ms": ms_step - ms_decode,
                              "prefill_chunk_gflop": pf_flops / 1e9,
                              "prefill_path": "FP8 pages dequantised to float16 scratch, then prefillTcKernel"}
    print(json.dumps(line))
    cache.close()
    engine.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="number of sequences (default: the workload's 256; smaller values are for profiler captures)")
    ap.add_argument("--workload", default="decode_c2", choices=["decode_c2", "prefill_c3", "decode_c4", "step_c4", "append_c1"],
                    help="decode_c2 is the headline workload; prefill_c3 reports prefill TFLOP/s (1 GPU)")
    ap.add_argument("--profile", action="store_true",
                    help="profiler run: no clock-settling loop, no end-to-end leg, no CPU baseline")
    args = ap.parse_args()
    globals()["BATCH"] = args.batch
    if args.workload == "prefill_c3" and args.batch != 256:
        globals()["PF_SEQS"] = args.batch
    if args.workload == "prefill_c3" and args.impl == "ours":
        run_prefill(args)
    elif args.workload == "append_c1" and args.impl == "ours":
        run_append(args)
    elif args.workload in ("decode_c4", "step_c4") and args.impl == "ours":
        run_decode_fp8(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
