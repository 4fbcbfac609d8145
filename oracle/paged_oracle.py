"""CPU oracle for the paged-KV hot path (TEST INFRASTRUCTURE, not product code).

A numpy restatement of the reference's algorithms for block allocation, slot
mapping, FP8 e4m3 KV quantisation, copy-on-write block copies, paged decode and
paged prefill.  Only tests, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the product path never does.

Every function names the reference source it follows (paths are relative to
the reference project root):

* ``KVCM``  = Sources/PagedAttentionMetal/KVCacheManager.swift
* ``Sched`` = Sources/PagedAttentionMetal/Scheduler.swift
* ``Infer`` = Sources/PagedAttentionMetal/PagedAttentionInference.swift
* ``metal`` = Sources/PagedAttentionMetal/kernels.metal
* ``tests`` = Tests/PagedAttentionMetalTests/PagedAttentionMetalTests.swift
* ``sim``   = Reference/paged_attention_sim.py

Pinning: the attention functions are pinned against outputs of ``sim`` (the
reference's own numpy implementation) stored under tests/golden/, and the
allocator against the integer facts asserted by the reference's tests
(tests:599-604, 758-770, 799-807, 739-749).  The FP8 codec and the sliding
window have no golden vectors in the reference ("parity unpinned" for those
two): they follow the shader source text line by line.  ``OracleInference``
is likewise unpinned (the reference has no test of ``Infer``); it follows the
source and a run worked out by hand.

KV pool layout used here is the build's layout, ``[block][kv_head][slot][dim]``;
the reference stores ``[block][slot][kv_head][dim]`` (metal:1829-1832).  The two
address the same (block, slot, kv_head, dim) element, so results are identical.
"""
from __future__ import annotations

from collections import deque

import numpy as np

FIFO, LIFO, BEST_FIT = 0, 1, 2

DT_F32, DT_F16, DT_FP8, DT_BF16 = 0, 1, 2, 3


# --------------------------------------------------------------------------
# Errors (KVCM:6-11)
# --------------------------------------------------------------------------
class OutOfMemory(Exception):
    pass


class SequenceNotFound(Exception):
    pass


class SequenceAlreadyExists(Exception):
    pass


class InvalidRequest(Exception):
    pass


# --------------------------------------------------------------------------
# Block allocator (KVCM:47-379)
# --------------------------------------------------------------------------
class OracleKVCacheManager:
    """Host-side state machine of ``KVCacheManager`` (KVCM:47-379).

    ``cow_log`` records every copy-on-write as (src_block, dst_block) in the
    order it happened; the reference performs the byte copy at that point
    (KVCM:176-194).
    """

    def __init__(self, max_blocks: int, block_size: int = 16):
        self.max_blocks = max_blocks
        self.block_size = block_size
        # KVCM:101 -- Deque((0..<max).reversed()); allocate pops from the back.
        self.free = deque(range(max_blocks - 1, -1, -1))
        self.free_sizes: dict[int, int] = {}
        self.policy = FIFO
        self.sequences: dict[int, dict] = {}
        self.prefix_cache: dict[int, int] = {}
        self.refcounts = [0] * max_blocks
        self.prefix_hits = 0
        self.cow_log: list[tuple[int, int]] = []

    # KVCM:65-67, 267-283
    def set_policy(self, policy: int) -> None:
        self.policy = policy
        if policy in (FIFO, LIFO):
            self.free = deque(reversed(self.free))
            self.free_sizes.clear()
        else:
            for b in self.free:
                self.free_sizes.setdefault(b, self.block_size)
            # Swift's sort is not documented as stable, but its implementation
            # (a merge-based introsort replacement since 5.0) is; equal sizes
            # keep deque order.
            self.free = deque(sorted(self.free, key=lambda b: -self.free_sizes.get(b, 0)))

    # KVCM:106-113
    def allocate_sequence(self, sid: int) -> None:
        if sid in self.sequences:
            raise SequenceAlreadyExists()
        self.sequences[sid] = {"table": [], "len": 0}

    # KVCM:241-265
    def _allocate_block(self) -> int:
        if self.policy in (FIFO, LIFO):
            return self.free.pop()
        best_idx, best_delta = 0, None
        for i, b in enumerate(self.free):
            delta = abs(self.free_sizes.get(b, self.block_size) - self.block_size)
            if best_delta is None or delta < best_delta:
                best_delta, best_idx = delta, i
        b = self.free[best_idx]
        del self.free[best_idx]
        self.free_sizes.pop(b, None)
        return b

    # KVCM:176-194
    def _copy_on_write(self, block: int, index: int, seq: dict) -> None:
        if not self.free:
            raise OutOfMemory()
        new_block = self._allocate_block()
        self.cow_log.append((block, new_block))
        self.refcounts[block] -= 1
        self.refcounts[new_block] = 1
        seq["table"][index] = new_block

    # KVCM:115-174
    def append_tokens(self, sid: int, count: int, hashes=None) -> None:
        if count < 0:
            raise InvalidRequest("count must be non-negative")
        if count == 0:
            return
        if sid not in self.sequences:
            raise SequenceNotFound()
        # The reference works on a copy of the sequence and stores it back only
        # on success (KVCM:122, 173); a throw in CoW or the OOM guard leaves the
        # stored table untouched but keeps refcount/free-list side effects.
        stored = self.sequences[sid]
        seq = {"table": list(stored["table"]), "len": stored["len"]}
        bs = self.block_size
        cur = seq["len"]
        new_len = cur + count
        now = (cur + bs - 1) // bs
        after = (new_len + bs - 1) // bs
        additional = after - now
        if now > 0 and cur % bs != 0:
            last = seq["table"][now - 1]
            if self.refcounts[last] > 1:
                self._copy_on_write(last, now - 1, seq)
        if additional > 0:
            if len(self.free) < additional:
                raise OutOfMemory()
            for i in range(additional):
                if hashes is not None and i < len(hashes):
                    h = int(hashes[i])
                    if h in self.prefix_cache:
                        b = self.prefix_cache[h]
                        seq["table"].append(b)
                        self.refcounts[b] += 1
                        self.prefix_hits += 1
                        continue
                b = self._allocate_block()
                seq["table"].append(b)
                self.refcounts[b] = 1
                if hashes is not None and i < len(hashes):
                    self.prefix_cache[int(hashes[i])] = b
        seq["len"] = new_len
        self.sequences[sid] = seq

    # KVCM:196-198
    def register_block_hash(self, h: int, block: int) -> None:
        self.prefix_cache[int(h)] = block

    # KVCM:200-214
    def ensure_exclusive_access(self, sid: int, logical: int) -> None:
        if sid not in self.sequences:
            raise SequenceNotFound()
        stored = self.sequences[sid]
        seq = {"table": list(stored["table"]), "len": stored["len"]}
        if logical >= len(seq["table"]):
            raise InvalidRequest("block index out of range")
        b = seq["table"][logical]
        if self.refcounts[b] > 1:
            self._copy_on_write(b, logical, seq)
        self.sequences[sid] = seq

    # KVCM:216-239
    def free_sequence(self, sid: int) -> None:
        seq = self.sequences.pop(sid, None)
        if seq is None:
            return
        total = len(seq["table"])
        rem = seq["len"] % self.block_size
        last_tokens = self.block_size if rem == 0 else rem
        for i, b in enumerate(seq["table"]):
            self.refcounts[b] -= 1
            if self.refcounts[b] <= 0:
                if self.policy == FIFO:
                    self.free.appendleft(b)
                elif self.policy == LIFO:
                    self.free.append(b)
                else:
                    self.free_sizes[b] = self.block_size if i < total - 1 else last_tokens
                    self.free.append(b)

    def block_table(self, sid: int) -> list[int]:
        if sid not in self.sequences:
            raise SequenceNotFound()
        return list(self.sequences[sid]["table"])

    def sequence_length(self, sid: int) -> int:
        if sid not in self.sequences:
            raise SequenceNotFound()
        return self.sequences[sid]["len"]

    @property
    def available_blocks(self) -> int:
        return len(self.free)

    # KVCM:353-378 (bytes fields are left to the caller: they need the dtype)
    def memory_stats(self) -> dict:
        partially = sum(1 for s in self.sequences.values() if s["len"] % self.block_size > 0)
        return {
            "totalBlocks": self.max_blocks,
            "usedBlocks": self.max_blocks - len(self.free),
            "freeBlocks": len(self.free),
            "activeSequences": len(self.sequences),
            "partiallyFilledBlocks": partially,
            "fragmentationRatio": np.float32(partially) / np.float32(max(len(self.sequences), 1)),
            "prefixCacheHits": self.prefix_hits,
            "prefixCacheEntries": len(self.prefix_cache),
            "sharedBlocks": sum(1 for r in self.refcounts if r > 1),
            "evictionPolicy": self.policy,
        }

    # KVCM:661-703 / CABI:339-372 -- zero-padded [batch][max_num_blocks] table
    def batch_tables(self, ids, max_num_blocks: int):
        tables = np.zeros((len(ids), max_num_blocks), dtype=np.int32)
        lens = np.zeros(len(ids), dtype=np.uint32)
        for i, sid in enumerate(ids):
            if sid not in self.sequences:
                raise SequenceNotFound()
            t = self.sequences[sid]["table"]
            if len(t) > max_num_blocks:
                raise InvalidRequest("sequence needs more blocks than the table is wide")
            tables[i, : len(t)] = t
            lens[i] = self.sequences[sid]["len"]
        return tables, lens


# --------------------------------------------------------------------------
# Scheduler (Sched:42-177)
# --------------------------------------------------------------------------
WAITING, RUNNING, PAUSED, COMPLETED = 0, 1, 2, 3


class OracleScheduler:
    """``ContinuousBatchingScheduler`` (Sched:42-177)."""

    def __init__(self, max_batch_size: int, max_sequences: int = 128):
        self.max_batch_size = max_batch_size
        self.max_sequences = max_sequences
        self.seqs: dict[int, dict] = {}
        self.next_id = 0
        self.arrival = 0

    def add_request(self, prompt_tokens: int, max_new_tokens: int) -> int:  # Sched:59-70
        if len(self.seqs) >= self.max_sequences:
            return -1
        sid = self.next_id
        self.next_id += 1
        self.seqs[sid] = {"id": sid, "status": WAITING, "gen": 0, "max_new": max_new_tokens,
                          "prompt": prompt_tokens, "arrival": self.arrival}
        self.arrival += 1
        return sid

    def complete_sequence(self, sid: int) -> None:  # Sched:72-76
        if sid in self.seqs:
            self.seqs[sid]["status"] = COMPLETED

    def step(self) -> list[int]:  # Sched:78-114
        by_arrival = sorted(self.seqs.values(), key=lambda s: s["arrival"])
        waiting = [s for s in by_arrival if s["status"] == WAITING]
        running = [s for s in by_arrival if s["status"] == RUNNING and s["gen"] < s["max_new"]]
        paused = [s for s in by_arrival if s["status"] == PAUSED]
        batch = []
        for s in waiting[: min(len(waiting), self.max_batch_size)]:
            s["status"] = RUNNING
            batch.append(s["id"])
        rem = self.max_batch_size - len(batch)
        if rem > 0:
            batch.extend(s["id"] for s in running[:rem])
        rem = self.max_batch_size - len(batch)
        if rem > 0:
            for s in paused[:rem]:
                s["status"] = RUNNING
                batch.append(s["id"])
        return batch

    def mark_prefilled(self, sid: int) -> None:  # Sched:116-120
        if sid in self.seqs:
            self.seqs[sid]["status"] = RUNNING

    def mark_decoded(self, sid: int) -> None:  # Sched:122-126
        if sid in self.seqs:
            self.seqs[sid]["gen"] += 1

    def preempt_sequence(self, sid: int) -> None:  # Sched:128-132
        if sid in self.seqs:
            self.seqs[sid]["status"] = PAUSED

    def handle_memory_pressure(self, required: int, available) -> list[int]:  # Sched:134-152
        preempted = []
        while available() < required:
            cands = sorted((s for s in self.seqs.values() if s["status"] == RUNNING),
                           key=lambda s: -s["arrival"])
            if not cands:
                break
            cands[0]["status"] = PAUSED
            preempted.append(cands[0]["id"])
        return preempted

    def count(self, status: int) -> int:  # Sched:154-170
        return sum(1 for s in self.seqs.values() if s["status"] == status)


class OracleInference:
    """The bookkeeping of ``PagedAttentionInference`` (Infer:7-299) without the
    attention launches: which sequences a step prefills and decodes, the block
    tables, lengths and counters it leaves.  ``launches`` records, per step,
    ("prefill", id, seq_len, table) and ("decode", ids, lens, tables) in order."""

    def __init__(self, max_blocks: int, block_size: int, max_batch_size: int = 16, max_sequences: int = 128,
                 incremental_preemption: bool = False):
        self.cache = OracleKVCacheManager(max_blocks, block_size)
        self.sched = OracleScheduler(max_batch_size, max_sequences)
        self.block_size = block_size
        self.prefilled: set[int] = set()
        self.total_tokens = 0
        self.step_count = 0
        self.tokens: list[tuple[int, int]] = []        # onTokenGenerated calls
        self.launches: list[tuple] = []
        self.incremental = incremental_preemption

    def add_request(self, prompt_tokens: int, max_new_tokens: int) -> int:  # Infer:103-105
        return self.sched.add_request(prompt_tokens, max_new_tokens)

    def complete_sequence(self, sid: int) -> None:  # Infer:108-114
        self.sched.complete_sequence(sid)
        self.cache.free_sequence(sid)
        self.prefilled.discard(sid)

    def _ensure_blocks(self, needed: int) -> None:  # Infer:280-299
        if self.cache.available_blocks >= needed:
            return
        if not self.incremental:
            avail = self.cache.available_blocks       # read once: the victims are freed afterwards
            for pid in self.sched.handle_memory_pressure(needed, lambda: avail):
                self.cache.free_sequence(pid)
                self.prefilled.discard(pid)
        else:
            while self.cache.available_blocks < needed:
                calls = [0]

                def available():
                    calls[0] += 1
                    return self.cache.available_blocks if calls[0] == 1 else needed

                victims = self.sched.handle_memory_pressure(needed, available)
                if not victims:
                    break
                for pid in victims:
                    self.cache.free_sequence(pid)
                    self.prefilled.discard(pid)
        if self.cache.available_blocks < needed:
            raise OutOfMemory()

    def step(self) -> list[int]:  # Infer:119-148
        batch = self.sched.step()
        if not batch:
            return []
        prefill = [i for i in batch if i not in self.prefilled]
        decode = [i for i in batch if i in self.prefilled]
        bs = self.block_size
        for sid in prefill:  # Infer:169-220
            prompt = self.sched.seqs[sid]["prompt"]
            self._ensure_blocks((prompt + bs - 1) // bs)
            try:
                self.cache.allocate_sequence(sid)
            except SequenceAlreadyExists:
                self.cache.free_sequence(sid)
                self.cache.allocate_sequence(sid)
            self.cache.append_tokens(sid, prompt)
            self.launches.append(("prefill", sid, prompt, list(self.cache.block_table(sid))))
            self.sched.mark_prefilled(sid)
            self.prefilled.add(sid)
            self.total_tokens += prompt
        if decode:  # Infer:222-278
            extras = 0
            for sid in decode:
                try:
                    cur = self.cache.sequence_length(sid)
                except SequenceNotFound:
                    cur = self.sched.seqs[sid]["prompt"]
                extras += max(0, (cur + 1 + bs - 1) // bs - (cur + bs - 1) // bs)
            if extras > 0:
                self._ensure_blocks(extras)
            tables = [list(self.cache.block_table(sid)) for sid in decode]      # raises if a victim was in the batch
            lens = [self.cache.sequence_length(sid) for sid in decode]
            self.launches.append(("decode", list(decode), lens, tables))
            for sid in decode:
                self.cache.append_tokens(sid, 1)
                self.sched.mark_decoded(sid)
                self.total_tokens += 1
                self.tokens.append((sid, 0))
                sq = self.sched.seqs[sid]
                if sq["gen"] >= sq["max_new"]:
                    self.complete_sequence(sid)
        self.step_count += 1
        return batch

    def run_all(self) -> None:  # Infer:151-156
        while self.sched.count(WAITING) > 0 or self.sched.count(RUNNING) > 0:
            if not self.step():
                break


# --------------------------------------------------------------------------
# Slot mapping (metal:1823-1827)
# --------------------------------------------------------------------------
def slot_mapping(block_table, token_offset: int, num_tokens: int, block_size: int) -> np.ndarray:
    """slot(t) = table[(off+t)/bs]*bs + (off+t)%bs  (metal:1823-1827)."""
    pos = token_offset + np.arange(num_tokens, dtype=np.int64)
    table = np.asarray(block_table, dtype=np.int64)
    return table[pos // block_size] * block_size + pos % block_size


# --------------------------------------------------------------------------
# FP8 e4m3 software codec (metal:553-601) and scale rule (metal:1942-1954)
# --------------------------------------------------------------------------
def _round_half_away(x: np.ndarray) -> np.ndarray:
    """Metal ``round()`` on non-negative input; x is float64 holding an exact
    float32 product, so x + 0.5 is exact."""
    return np.floor(x + 0.5)


def quantize_fp8(value_f16: np.ndarray, scale_f16) -> np.ndarray:
    """``quantize_fp8`` (metal:564-601): f32 divide, clamp, round half away."""
    value = np.asarray(value_f16, dtype=np.float16).astype(np.float32)
    scale = np.asarray(scale_f16, dtype=np.float16).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (value / scale).astype(np.float32)                      # metal:565
    v = np.clip(v, np.float32(-448.0), np.float32(448.0))           # metal:566
    sign = (v < 0).astype(np.uint8)                                  # metal:568
    a = np.abs(v).astype(np.float64)
    out = np.zeros(a.shape, dtype=np.uint8)

    sub = (a < 2.0 ** -6) & (a != 0)                                 # metal:573-578
    m_sub = np.clip(_round_half_away(a * 512.0), 0, 7).astype(np.uint8)

    mant, exp = np.frexp(a)                                          # metal:580-583
    e = exp.astype(np.int64) - 1
    ebits = e + 7                                                    # metal:589
    m = _round_half_away((2.0 * mant - 1.0) * 8.0).astype(np.int64)  # metal:590-591
    carry = m > 7                                                    # metal:592
    m = np.where(carry, 0, m)
    ebits = np.where(carry, ebits + 1, ebits)
    sat = (e > 8) | (ebits > 15)                                     # metal:585, 593
    m = np.where((ebits == 15) & (m > 6), 6, m)                      # metal:596-598
    normal = ((sign.astype(np.int64) << 7) | (ebits << 3) | m)
    normal = np.where(sat, (sign.astype(np.int64) << 7) | 0x7E, normal)

    out = np.where(sub, (sign << 7) | m_sub, normal.astype(np.uint8)).astype(np.uint8)
    out = np.where(a == 0, np.uint8(0), out).astype(np.uint8)        # metal:571
    return out


def dequant_fp8(codes: np.ndarray, scale_f16) -> np.ndarray:
    """``dequant_fp8`` (metal:553-562): all-half arithmetic, left to right."""
    c = np.asarray(codes, dtype=np.uint8)
    scale = np.broadcast_to(np.asarray(scale_f16, dtype=np.float16), c.shape)
    sign = (c >> 7) & 1
    e = ((c >> 3) & 0xF).astype(np.int32)
    m = (c & 7).astype(np.float16)
    h = np.float16
    with np.errstate(over="ignore", under="ignore", invalid="ignore"):
        ss = np.where(sign == 1, -scale, scale).astype(h)            # (±1.0h) * scale
        frac = (m / h(8.0)).astype(h)
        normal = ((ss * (h(1.0) + frac).astype(h)).astype(h)
                  * np.ldexp(np.float32(1.0), e - 7).astype(h)).astype(h)
        subn = ((ss * frac).astype(h) * h(0.015625)).astype(h)
    out = np.where(e == 0, subn, normal).astype(h)
    out = np.where((e == 0) & ((c & 7) == 0), h(0.0), out).astype(h)  # metal:557 -> +0.0
    return out


def fp8_scale_update(amax_f32, old_scale_f16) -> np.ndarray:
    """New group scale (metal:1942-1954): max(new absmax, old*448)/448 as half,
    1.0 when the maximum is zero."""
    amax = np.asarray(amax_f32, dtype=np.float32)
    old = np.asarray(old_scale_f16, dtype=np.float16).astype(np.float32)
    mx = np.maximum(amax, (old * np.float32(448.0)).astype(np.float32))
    with np.errstate(over="ignore"):
        s = (mx / np.float32(448.0)).astype(np.float32).astype(np.float16)
    return np.where(mx > 0, s, np.float16(1.0)).astype(np.float16)


# --------------------------------------------------------------------------
# KV append ("reshape_and_cache") and copy-on-write block copies
# --------------------------------------------------------------------------
def reshape_and_cache(k_pool, v_pool, keys, values, slots, block_size: int) -> None:
    """Scatter new token rows into the pools (metal:1804-1874).

    pools: ``[blocks][kv_heads][block_size][head_dim]`` (any dtype, written in
    place); keys/values: ``[tokens][kv_heads][head_dim]`` of the pool dtype;
    slots: ``[tokens]`` physical slot = block*block_size + offset.
    """
    slots = np.asarray(slots, dtype=np.int64)
    blk, off = slots // block_size, slots % block_size
    k_pool[blk, :, off, :] = keys
    v_pool[blk, :, off, :] = values


def reshape_and_cache_fp8(k_codes, v_codes, k_scale, v_scale, keys_f16, values_f16, slots,
                          block_size: int) -> None:
    """FP8 append (metal:1876-1961) with the scale group narrowed from the
    reference's physical block to (block, kv_head).

    Pass 1 takes the absmax of the new tokens that land in each group
    (metal:1900-1904); pass 2 derives the group scale from it and the stored
    scale (metal:1942-1954), quantises the new tokens with it (metal:1956-1957)
    and stores the scale (metal:1959-1960).  Codes already in the block are
    left as they are.  k_scale/v_scale: ``[blocks][kv_heads]`` float16.
    """
    slots = np.asarray(slots, dtype=np.int64)
    blk, off = slots // block_size, slots % block_size
    kf = np.asarray(keys_f16, dtype=np.float16)
    vf = np.asarray(values_f16, dtype=np.float16)
    for src, codes, scales in ((kf, k_codes, k_scale), (vf, v_codes, v_scale)):
        amax = np.zeros(scales.shape, dtype=np.float32)
        tok_amax = np.abs(src.astype(np.float32)).max(axis=2)       # [T][KVH]
        np.maximum.at(amax, (blk[:, None], np.arange(src.shape[1])[None, :]), tok_amax)
        touched = np.zeros(scales.shape[0], dtype=bool)
        touched[blk] = True
        new_scale = fp8_scale_update(amax, scales)
        scales[touched] = new_scale[touched]
        tok_scale = scales[blk]                                      # [T][KVH]
        codes[blk, :, off, :] = quantize_fp8(src, tok_scale[:, :, None])


def copy_blocks(pools, src_blocks, dst_blocks) -> None:
    """Copy whole physical blocks (KVCM:176-194 does this with memcpy for K and
    V).  ``pools`` is any list of arrays indexed by block on axis 0 (K, V and,
    for FP8, their scale rows)."""
    src = np.asarray(src_blocks, dtype=np.int64)
    dst = np.asarray(dst_blocks, dtype=np.int64)
    for p in pools:
        p[dst] = p[src]


# --------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------
def _gather_kv(pool, table, kvh, n_tokens, block_size, scale_pool=None):
    nb = (n_tokens + block_size - 1) // block_size
    blocks = np.asarray(table[:nb], dtype=np.int64)
    if scale_pool is None:
        x = pool[blocks, kvh].astype(np.float32)
    else:
        x = dequant_fp8(pool[blocks, kvh], scale_pool[blocks, kvh][:, None, None]).astype(np.float32)
    return x.reshape(nb * block_size, -1)[:n_tokens]


def paged_decode(q, k_pool, v_pool, block_tables, seq_lens, num_kv_heads: int, block_size: int,
                 window: int = 0, k_scale=None, v_scale=None, online: bool = False) -> np.ndarray:
    """Batched paged decode (metal:1417-1482; FP8: metal:1551-1620).

    q: ``[batch][heads][dim]``; pools ``[blocks][kv_heads][block_size][dim]``;
    block_tables ``[batch][max_blocks]`` int32; seq_lens ``[batch]``.
    Window start per sequence is ``L - W`` when ``W > 0 and L > W``
    (metal:1442).  Sequences of length 0 give 0/0 in the reference; here the
    row is NaN as well.  With ``online=True`` the softmax is the token-by-token
    f32 recurrence of the shader (metal:1472-1477); otherwise it is the
    two-pass form in float64 (the same function, used for larger cases).
    Returns float32 ``[batch][heads][dim]``.
    """
    q = np.asarray(q)
    B, H, D = q.shape
    G = H // num_kv_heads
    max_nb = block_tables.shape[1]
    out = np.empty((B, H, D), dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(np.float32(D))                  # metal:1441
    for b in range(B):
        L = int(seq_lens[b])
        L_eff = min(L, max_nb * block_size)                          # metal:1451-1452
        ws = L - window if (window > 0 and L > window) else 0        # metal:1442
        for kvh in range(num_kv_heads):
            k = _gather_kv(k_pool, block_tables[b], kvh, L_eff, block_size, k_scale)[ws:]
            v = _gather_kv(v_pool, block_tables[b], kvh, L_eff, block_size, v_scale)[ws:]
            for g in range(G):
                h = kvh * G + g
                qv = q[b, h].astype(np.float32)
                if online:
                    m, l = np.float32(-np.inf), np.float32(0)
                    acc = np.zeros(D, dtype=np.float32)
                    for j in range(k.shape[0]):
                        s = np.float32(np.dot(qv, k[j])) * inv
                        m_old, m = m, max(m, s)
                        corr = np.exp(np.float32(m_old - m))
                        p = np.exp(np.float32(s - m))
                        l = l * corr + p
                        acc = acc * corr + p * v[j]
                    with np.errstate(invalid="ignore", divide="ignore"):
                        out[b, h] = acc / l
                else:
                    if k.shape[0] == 0:
                        out[b, h] = np.nan
                        continue
                    s = (k.astype(np.float64) @ qv.astype(np.float64)) * np.float64(inv)
                    p = np.exp(s - s.max())
                    out[b, h] = (p @ v.astype(np.float64) / p.sum()).astype(np.float32)
    return out


def paged_prefill(q, k_pool, v_pool, block_table, seq_len: int, num_kv_heads: int, block_size: int,
                  causal: bool = True, window_start: int = 0, q_start: int = 0, q_len=None,
                  k_scale=None, v_scale=None) -> np.ndarray:
    """Single-sequence paged prefill (metal:693-765; CPU loop tests:37-63 and
    GQA head map tests:128-148).

    q: ``[q_len][heads][dim]`` holding rows ``q_start .. q_start+q_len`` of the
    sequence; keys are tokens ``[window_start, seq_len)`` of the paged cache,
    key j visible to row i iff ``j <= i`` when causal (metal:745).  The
    reference takes ``window_start`` as one scalar for all rows
    (Engine.swift:802) and its chunk loop (Engine.swift:740-756) yields exactly
    the rows of a full prefill; ``q_start/q_len`` select those rows directly.
    Rows with no visible key are 0/0 in the reference; they are returned as
    NaN and are "don't care" for parity.  Returns float32.
    """
    q = np.asarray(q)
    if q_len is None:
        q_len = q.shape[0]
    H, D = q.shape[1], q.shape[2]
    G = H // num_kv_heads
    out = np.empty((q_len, H, D), dtype=np.float32)
    inv = np.float64(np.float32(1.0) / np.sqrt(np.float32(D)))
    rows = q_start + np.arange(q_len)
    keys_idx = np.arange(window_start, seq_len)
    for kvh in range(num_kv_heads):
        k = _gather_kv(k_pool, block_table, kvh, seq_len, block_size, k_scale)[window_start:].astype(np.float64)
        v = _gather_kv(v_pool, block_table, kvh, seq_len, block_size, v_scale)[window_start:].astype(np.float64)
        for g in range(G):
            h = kvh * G + g
            s = (q[:, h].astype(np.float64) @ k.T) * inv            # [q_len][keys]
            if causal:
                s = np.where(keys_idx[None, :] <= rows[:, None], s, -np.inf)
            with np.errstate(invalid="ignore", divide="ignore"):
                mx = s.max(axis=1, keepdims=True) if s.shape[1] else np.full((q_len, 1), -np.inf)
                p = np.exp(s - mx)
                out[:, h] = (p @ v / p.sum(axis=1, keepdims=True)).astype(np.float32)
    return out


def attention_stats(q, k_pool, block_table, seq_len: int, num_kv_heads: int, block_size: int,
                    window_start: int = 0):
    """The row maximum ``m`` and the row sum ``l`` of ``exp(s - m)`` over keys
    ``[window_start, seq_len)`` (no causal mask), float32 ``[seq_len][heads]``: what the
    backward kernel is handed beside the gradient (metal:1222-1223; the reference's
    forward kernels keep them in private buffers, Engine.swift:811-816)."""
    q = np.asarray(q)
    H, D = q.shape[1], q.shape[2]
    G = H // num_kv_heads
    inv = np.float64(np.float32(1.0) / np.sqrt(np.float32(D)))
    m = np.empty((seq_len, H), dtype=np.float32)
    l = np.empty((seq_len, H), dtype=np.float32)
    for kvh in range(num_kv_heads):
        k = _gather_kv(k_pool, block_table, kvh, seq_len, block_size)[window_start:].astype(np.float64)
        for g in range(G):
            h = kvh * G + g
            sc = (q[:seq_len, h].astype(np.float64) @ k.T) * inv
            mx = sc.max(axis=1)
            m[:, h] = mx
            l[:, h] = np.exp(sc - m[:, h].astype(np.float64)[:, None]).sum(axis=1)
    return m, l


def paged_backward(q, k_pool, v_pool, block_table, d_out, m, l, seq_len: int, num_kv_heads: int,
                   block_size: int, window_start: int = 0):
    """Gradients of paged attention (metal:1217-1315; float16: metal:1317-1415).

    Every row i of every head sees the keys ``[window_start, seq_len)`` (the kernel has no
    causal mask).  With ``P_ij = exp(q_i . k_j / sqrt(d) - m_i) / l_i`` (metal:1283),
    ``dP_ij = dO_i . v_j`` (metal:1284), ``rowsum_i = sum_j P_ij dP_ij`` (metal:1264) and
    ``dS_ij = P_ij (dP_ij - rowsum_i)`` (metal:1285):

        dQ_i  = sum_j dS_ij k_j / sqrt(d)                      (metal:1287, 1300)
        dK_j += sum over rows and the heads of the KV head of dS_ij q_i / sqrt(d)   (metal:1289-1291)
        dV_j += sum over rows and heads of P_ij dO_i           (metal:1293-1295)

    Returns ``(dQ [seq_len][heads][dim], dK, dV)`` with dK, dV shaped like the pools
    ``[blocks][kv_heads][block_size][dim]`` and holding only the contributions (the kernel
    adds them to what the gradient pools hold), all float64.  The reference accumulates the
    pool gradients with float (half) atomics in an order that is not defined; this is the
    exact sum.
    """
    q = np.asarray(q)
    d_out = np.asarray(d_out)
    H, D = q.shape[1], q.shape[2]
    G = H // num_kv_heads
    inv = np.float64(np.float32(1.0) / np.sqrt(np.float32(D)))
    dq = np.zeros((seq_len, H, D), dtype=np.float64)
    dk = np.zeros(k_pool.shape, dtype=np.float64)
    dv = np.zeros(v_pool.shape, dtype=np.float64)
    nkeys = seq_len - window_start
    toks = np.arange(window_start, seq_len)
    blocks = np.asarray(block_table, dtype=np.int64)[toks // block_size]
    slots = toks % block_size
    for kvh in range(num_kv_heads):
        k = _gather_kv(k_pool, block_table, kvh, seq_len, block_size)[window_start:].astype(np.float64)
        v = _gather_kv(v_pool, block_table, kvh, seq_len, block_size)[window_start:].astype(np.float64)
        dk_acc = np.zeros((nkeys, D))
        dv_acc = np.zeros((nkeys, D))
        for g in range(G):
            h = kvh * G + g
            qh = q[:seq_len, h].astype(np.float64)
            doh = d_out[:seq_len, h].astype(np.float64)
            sc = (qh @ k.T) * inv
            p = np.exp(sc - m[:seq_len, h].astype(np.float64)[:, None]) / l[:seq_len, h].astype(np.float64)[:, None]
            dp = doh @ v.T
            rowsum = (p * dp).sum(axis=1, keepdims=True)
            ds = p * (dp - rowsum)
            dq[:, h] = (ds @ k) * inv
            dk_acc += (ds.T @ qh) * inv
            dv_acc += p.T @ doh
        np.add.at(dk, (blocks, kvh, slots), dk_acc)
        np.add.at(dv, (blocks, kvh, slots), dv_acc)
    return dq, dk, dv


# --------------------------------------------------------------------------
# Seeded workload generators (shapes of the five benchmark configurations)
# --------------------------------------------------------------------------
def round_to(x: np.ndarray, dtype: int) -> np.ndarray:
    """Round float32 data once to the storage dtype and widen back."""
    if dtype == DT_F32:
        return x.astype(np.float32)
    if dtype == DT_F16:
        return x.astype(np.float16).astype(np.float32)
    if dtype == DT_BF16:
        u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000               # round to nearest even
        return u.astype(np.uint32).view(np.float32)
    raise ValueError(dtype)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    return (round_to(x, DT_BF16).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(u: np.ndarray) -> np.ndarray:
    return (np.asarray(u, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_decode_case(seed: int, batch: int, len_lo: int, len_hi: int, heads: int, kv_heads: int,
                     head_dim: int = 128, block_size: int = 16, spare_blocks: int = 0,
                     pool_blocks=None):
    """Lengths ~ U{lo..hi}; block tables are consecutive slices of one random
    permutation of the pool (non-contiguous pages).  Returns lens, tables
    (zero padded), number of pool blocks."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(len_lo, len_hi + 1, size=batch).astype(np.uint32)
    nblk = (lens.astype(np.int64) + block_size - 1) // block_size
    total = int(nblk.sum())
    n_pool = pool_blocks if pool_blocks is not None else total + spare_blocks
    assert n_pool >= total
    perm = rng.permutation(n_pool).astype(np.int32)
    max_nb = int(nblk.max())
    tables = np.zeros((batch, max_nb), dtype=np.int32)
    o = 0
    for i in range(batch):
        tables[i, : nblk[i]] = perm[o: o + nblk[i]]
        o += int(nblk[i])
    return rng, lens, tables, n_pool
