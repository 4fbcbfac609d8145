"""KVCacheManager and ContinuousBatchingScheduler through the C ABI against
the oracle state machines and the integer facts the reference's tests assert.
Bookkeeping-only managers: no GPU needed."""
import random

import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from oracle import paged_oracle as po


def new_manager(max_blocks, block_size):
    return pam.KVCacheManager(None, max_blocks, block_size)


def test_reference_cabi_lifecycle_facts():
    # Tests/PagedAttentionMetalTests.swift:599-604: 8 blocks of 4, 5 tokens -> 6 free, free -> 8
    m = new_manager(8, 4)
    m.allocateSequence(7)
    m.appendTokens(7, 5)
    assert m.availableBlocks == 6 and m.getSequenceLength(7) == 5
    m.freeSequence(7)
    assert m.availableBlocks == 8


def test_reference_allocate_then_free_facts():
    # Tests:758-770: 4 blocks; 16 tokens -> 3 free; free -> 4; then 32 tokens take 2 blocks
    m = new_manager(4, 16)
    m.allocateSequence(1)
    m.appendTokens(1, 16)
    assert m.availableBlocks == 3
    m.freeSequence(1)
    assert m.availableBlocks == 4
    m.allocateSequence(2)
    m.appendTokens(2, 32)
    assert m.getNumBlocks(2) == 2


def test_reference_block_boundary_facts():
    # Tests:799-807: 55 tokens -> 4 blocks, +32 -> 6 blocks, length 87
    m = new_manager(16, 16)
    m.allocateSequence(1)
    m.appendTokens(1, 55)
    assert m.getNumBlocks(1) == 4
    m.appendTokens(1, 32)
    assert m.getNumBlocks(1) == 6 and m.getSequenceLength(1) == 87


def test_reference_out_of_memory_fact():
    # Tests:739-749: pool exhausted -> outOfMemory
    m = new_manager(2, 16)
    m.allocateSequence(1)
    m.appendTokens(1, 32)
    m.allocateSequence(2)
    with pytest.raises(pam.KVCacheError) as e:
        m.appendTokens(2, 1)
    assert e.value.case == "outOfMemory"


def test_errors_match_reference_cases():
    m = new_manager(4, 4)
    m.allocateSequence(1)
    with pytest.raises(pam.KVCacheError) as e:
        m.allocateSequence(1)
    assert e.value.case == "sequenceAlreadyExists"
    with pytest.raises(pam.KVCacheError) as e:
        m.appendTokens(1, -1)
    assert e.value.case == "invalidRequest"
    m.appendTokens(5, 0)                                        # count 0 returns before the lookup (KVCM:121)
    with pytest.raises(pam.KVCacheError) as e:
        m.appendTokens(5, 1)
    assert e.value.case == "sequenceNotFound"
    with pytest.raises(pam.KVCacheError) as e:
        m.ensureExclusiveAccess(1, 0)
    assert e.value.case == "invalidRequest"
    m.freeSequence(99)                                          # unknown id is a no-op (KVCM:219)


def test_fresh_manager_hands_out_ascending_blocks():
    m = new_manager(6, 2)
    m.allocateSequence(0)
    m.appendTokens(0, 7)
    assert m.getBlockTable(0) == [0, 1, 2, 3]                   # KVCM:101, 244


def test_prefix_sharing_and_copy_on_write():
    bs = 4
    m, o = new_manager(32, bs), po.OracleKVCacheManager(32, bs)
    for x in (m, o):
        pass
    hashes = [100, 101, 102]
    m.allocateSequence(0); o.allocate_sequence(0)
    m.appendTokens(0, 10, hashes); o.append_tokens(0, 10, hashes)      # 3 blocks, last one holds 2 tokens
    m.allocateSequence(1); o.allocate_sequence(1)
    m.appendTokens(1, 10, hashes); o.append_tokens(1, 10, hashes)      # all three hit
    assert m.getBlockTable(1) == m.getBlockTable(0) == o.block_table(0)
    st = m.memoryStats()
    assert st.prefixCacheHits == 3 and st.sharedBlocks == 3 and st.prefixCacheEntries == 3
    # first divergent write into the shared, partially filled block copies it
    m.appendTokens(1, 1); o.append_tokens(1, 1)
    assert m.getBlockTable(1) == o.block_table(1)
    assert m.getBlockTable(1)[:2] == m.getBlockTable(0)[:2] and m.getBlockTable(1)[2] != m.getBlockTable(0)[2]
    assert m.drainCopyOnWriteLog() == o.cow_log == [(2, 3)]
    assert m.memoryStats().sharedBlocks == 2
    # ensureExclusiveAccess on a still-shared full block
    m.ensureExclusiveAccess(0, 0); o.ensure_exclusive_access(0, 0)
    assert m.getBlockTable(0) == o.block_table(0)
    assert m.drainCopyOnWriteLog() == [(0, 4)]


def _stats_equal(m, o):
    a, b = m.memoryStats(), o.memory_stats()
    assert (a.totalBlocks, a.usedBlocks, a.freeBlocks, a.activeSequences) == \
           (b["totalBlocks"], b["usedBlocks"], b["freeBlocks"], b["activeSequences"])
    assert a.partiallyFilledBlocks == b["partiallyFilledBlocks"]
    assert np.float32(a.fragmentationRatio) == np.float32(b["fragmentationRatio"])
    assert (a.prefixCacheHits, a.prefixCacheEntries, a.sharedBlocks) == \
           (b["prefixCacheHits"], b["prefixCacheEntries"], b["sharedBlocks"])
    assert int(a.evictionPolicy) == b["evictionPolicy"]


@pytest.mark.parametrize("seed", range(6))
def test_random_operations_match_oracle_bit_exactly(seed):
    rnd = random.Random(seed)
    bs = rnd.choice([1, 4, 16])
    nblk = rnd.choice([8, 24, 64])
    m, o = new_manager(nblk, bs), po.OracleKVCacheManager(nblk, bs)
    live = []
    for step in range(400):
        op = rnd.random()
        err_m = err_o = None
        if op < 0.15 or not live:
            sid = rnd.randrange(12)
            try: m.allocateSequence(sid)
            except pam.KVCacheError as e: err_m = e.case
            try: o.allocate_sequence(sid)
            except po.SequenceAlreadyExists: err_o = "sequenceAlreadyExists"
            if err_m is None and sid not in live: live.append(sid)
        elif op < 0.65:
            sid = rnd.choice(live + [99])
            count = rnd.choice([0, 1, 1, 2, bs, bs + 1, 3 * bs, 40])
            hashes = None
            if rnd.random() < 0.5:
                hashes = [rnd.randrange(10) for _ in range(rnd.randrange(0, 5))]
            try: m.appendTokens(sid, count, hashes)
            except pam.KVCacheError as e: err_m = e.case
            try: o.append_tokens(sid, count, hashes)
            except po.OutOfMemory: err_o = "outOfMemory"
            except po.SequenceNotFound: err_o = "sequenceNotFound"
        elif op < 0.80:
            sid = rnd.choice(live)
            m.freeSequence(sid); o.free_sequence(sid)
            live.remove(sid)
        elif op < 0.88:
            sid = rnd.choice(live)
            idx = rnd.randrange(0, 6)
            try: m.ensureExclusiveAccess(sid, idx)
            except pam.KVCacheError as e: err_m = e.case
            try: o.ensure_exclusive_access(sid, idx)
            except po.OutOfMemory: err_o = "outOfMemory"
            except po.InvalidRequest: err_o = "invalidRequest"
        elif op < 0.94:
            pol = rnd.choice([0, 1, 2])
            m.evictionPolicy = pol; o.set_policy(pol)
        else:
            h, b = rnd.randrange(10), rnd.randrange(nblk)
            m.registerBlockHash(h, b); o.register_block_hash(h, b)
        assert err_m == err_o, (step, err_m, err_o)
        assert m.availableBlocks == o.available_blocks
        for sid in live:
            assert m.getBlockTable(sid) == o.block_table(sid), (step, sid)
            assert m.getSequenceLength(sid) == o.sequence_length(sid)
        assert m.drainCopyOnWriteLog() == o.cow_log
        o.cow_log.clear()
    _stats_equal(m, o)


def test_eviction_policies_order():
    # fifo: freed blocks are reused last; lifo: reused next (KVCM:227-235)
    for policy, expect_first in ((pam.BlockEvictionPolicy.fifo, 2), (pam.BlockEvictionPolicy.lifo, 1)):
        m, o = new_manager(4, 1), po.OracleKVCacheManager(4, 1)
        if policy != pam.BlockEvictionPolicy.fifo:
            m.evictionPolicy = policy; o.set_policy(int(policy))
            # the setter reverses the free list (KVCM:267-274); undo to compare like with like
            m.evictionPolicy = policy; o.set_policy(int(policy))
        m.allocateSequence(0); o.allocate_sequence(0)
        m.appendTokens(0, 2); o.append_tokens(0, 2)
        m.freeSequence(0); o.free_sequence(0)
        m.allocateSequence(1); o.allocate_sequence(1)
        m.appendTokens(1, 1); o.append_tokens(1, 1)
        assert m.getBlockTable(1) == o.block_table(1) == [expect_first]


def test_batch_tables_zero_padded():
    m = new_manager(16, 4)
    for sid, n in ((3, 9), (5, 1), (8, 0)):
        m.allocateSequence(sid)
        m.appendTokens(sid, n)
    tables, lens = m.batchTables([5, 3, 8], 4)
    assert tables.tolist() == [[3, 0, 0, 0], [0, 1, 2, 0], [0, 0, 0, 0]]      # CABI.swift:353-364
    assert lens.tolist() == [1, 9, 0]
    with pytest.raises(pam.KVCacheError):
        m.batchTables([3], 2)                                                  # KVCM:675-677
    assert m.slotMapping(3, 2, 5).tolist() == po.slot_mapping([0, 1, 2], 2, 5, 4).tolist()


# ---- scheduler ----

def test_scheduler_step_order_and_limits():
    s, o = pam.ContinuousBatchingScheduler(3, 5), po.OracleScheduler(3, 5)
    ids = [s.addRequest(10, 2) for _ in range(5)]
    assert ids == [o.add_request(10, 2) for _ in range(5)] == [0, 1, 2, 3, 4]
    assert s.addRequest(1, 1) == -1 == o.add_request(1, 1)                     # Sched:62
    assert [x.id for x in s.step()] == o.step() == [0, 1, 2]
    assert s.runningCount == 3 and s.waitingCount == 2
    # waiting sequences come first, running ones fill what is left (Sched:88-100)
    assert [x.id for x in s.step()] == o.step() == [3, 4, 0]
    s.preemptSequence(1); o.preempt_sequence(1)
    for i in (0, 0):
        s.markDecoded(i); o.mark_decoded(i)
    # sequence 0 is done: it stays "running" but leaves the batch (Sched:83)
    assert [x.id for x in s.step()] == o.step() == [2, 3, 4]
    s.completeSequence(0); o.complete_sequence(0)
    s.completeSequence(2); o.complete_sequence(2)
    assert [x.id for x in s.step()] == o.step() == [3, 4, 1]                   # paused resumes last
    assert s.completedCount == 2 and s.totalSequencesProcessed == 5
    seq = s.sequence(0)
    assert seq.isDone and seq.currentLength == 12 and seq.status == pam.SequenceStatus.completed


def test_scheduler_memory_pressure_victims():
    s, o = pam.ContinuousBatchingScheduler(8), po.OracleScheduler(8)
    for _ in range(4):
        s.addRequest(4, 4); o.add_request(4, 4)
    s.step(); o.step()
    avail = {"n": 0}
    def available():
        return avail["n"]
    # nothing frees blocks while the loop runs: every running sequence is paused, newest first (Sched:139-147)
    assert s.handleMemoryPressure(2, available) == o.handle_memory_pressure(2, available) == [3, 2, 1, 0]
    assert s.runningCount == 0
    s2 = pam.ContinuousBatchingScheduler(8)
    for _ in range(3):
        s2.addRequest(4, 4)
    s2.step()
    calls = {"n": 0}
    def grows():
        calls["n"] += 1
        return calls["n"]                                                      # 1, 2, 3 ...
    assert s2.handleMemoryPressure(3, grows) == [2, 1]


@pytest.mark.parametrize("seed", range(4))
def test_scheduler_random_matches_oracle(seed):
    rnd = random.Random(seed)
    mb = rnd.choice([1, 2, 5])
    s, o = pam.ContinuousBatchingScheduler(mb, 20), po.OracleScheduler(mb, 20)
    for _ in range(300):
        r = rnd.random()
        if r < 0.2:
            a, b = rnd.randrange(1, 50), rnd.randrange(0, 4)
            assert s.addRequest(a, b) == o.add_request(a, b)
        elif r < 0.5:
            assert [x.id for x in s.step()] == o.step()
        else:
            sid = rnd.randrange(22)
            f = rnd.choice(["d", "p", "c", "f"])
            if f == "d": s.markDecoded(sid); o.mark_decoded(sid)
            elif f == "p": s.preemptSequence(sid); o.preempt_sequence(sid)
            elif f == "c": s.completeSequence(sid); o.complete_sequence(sid)
            else: s.markPrefilled(sid); o.mark_prefilled(sid)
        for st in range(4):
            assert lib_count(s, st) == o.count(st)


def lib_count(s, status):
    from pagedattentionmetal_b200._cabi import lib
    return lib.pamc_sched_count(s._h, status)


# ---- the two fixes of reference behaviour behind pamc_cache_set_hygiene (default: off)

def test_stale_prefix_hash_is_kept_by_default_and_dropped_with_hygiene():
    # KVCacheManager.swift:216-239 frees blocks without touching the prefix map, so a later
    # appendTokens with the same hash is handed a block that now belongs to someone else.
    for hygiene in (False, True):
        m = new_manager(4, 16)
        m.setHygiene(hygiene)
        m.allocateSequence(1)
        m.appendTokens(1, 16, [111])
        shared = m.getBlockTable(1)[0]
        m.freeSequence(1)
        assert m.memoryStats().prefixCacheEntries == (0 if hygiene else 1)
        m.allocateSequence(2)
        m.appendTokens(2, 64)                              # takes every block, the freed one included
        assert shared in m.getBlockTable(2)
        m.allocateSequence(3)
        if hygiene:
            with pytest.raises(pam.KVCacheError) as e:     # no hit: it needs a block and there is none
                m.appendTokens(3, 16, [111])
            assert e.value.case == "outOfMemory"
        else:
            # the reference's OOM check comes before the hit is looked up (:142-146)
            with pytest.raises(pam.KVCacheError):
                m.appendTokens(3, 16, [111])
            m.freeSequence(2)
            m.allocateSequence(4)
            m.appendTokens(4, 16)                          # block `shared` may be handed out again ...
            m.appendTokens(3, 16, [111])                   # ... and the stale hash still points at it
            assert m.memoryStats().prefixCacheHits == 1


def test_hygiene_keeps_hashes_of_blocks_that_are_still_referenced():
    m = new_manager(8, 16)
    m.setHygiene(True)
    for sid in (1, 2):
        m.allocateSequence(sid)
        m.appendTokens(sid, 32, [5, 6])
    assert m.getBlockTable(1) == m.getBlockTable(2) and m.memoryStats().prefixCacheHits == 2
    m.freeSequence(1)                                      # sequence 2 still holds both blocks
    assert m.memoryStats().prefixCacheEntries == 2
    m.allocateSequence(3)
    m.appendTokens(3, 32, [5, 6])
    assert m.getBlockTable(3) == m.getBlockTable(2)
    m.freeSequence(2)
    m.freeSequence(3)
    assert m.memoryStats().prefixCacheEntries == 0 and m.availableBlocks == 8


def test_append_that_runs_out_of_blocks_after_copy_on_write():
    # A shared, partly filled last block plus an append the pool cannot hold.  The reference
    # copies the block first and fails afterwards (KVCacheManager.swift:134-146): the fresh
    # block is lost and the shared block loses a reference.  With hygiene nothing changes.
    for hygiene in (False, True):
        m = new_manager(3, 16)
        m.setHygiene(hygiene)
        m.allocateSequence(1)
        m.appendTokens(1, 8, [9])                          # block 0, half full, hashed
        m.allocateSequence(2)
        m.appendTokens(2, 8, [9])                          # shares block 0
        assert m.memoryStats().sharedBlocks == 1 and m.availableBlocks == 2
        with pytest.raises(pam.KVCacheError) as e:
            m.appendTokens(2, 8 + 3 * 16)                  # copy of block 0 + three more blocks: too many
        assert e.value.case == "outOfMemory"
        assert m.getBlockTable(2) == [0] and m.getSequenceLength(2) == 8
        if hygiene:
            assert m.availableBlocks == 2 and m.memoryStats().sharedBlocks == 1
            assert m.drainCopyOnWriteLog() == []
        else:
            assert m.availableBlocks == 1 and m.memoryStats().sharedBlocks == 0
            assert m.drainCopyOnWriteLog() == [(0, 1)]


def test_block_hashes_chain_over_the_prefix():
    a = list(range(100, 164))
    b = a[:32] + [7] + a[33:]
    ha, hb = pam.KVCacheManager.blockHashes(a, 16), pam.KVCacheManager.blockHashes(b, 16)
    assert len(ha) == 4 and len(set(ha)) == 4
    assert ha[:2] == hb[:2] and ha[2] != hb[2] and ha[3] != hb[3]      # a change reaches every later block
    assert pam.KVCacheManager.blockHashes(a[:47], 16) == ha[:2]        # only full blocks are hashed
    assert pam.KVCacheManager.blockHashes(a, 16, seed=1)[0] != ha[0]
    # usable as blockHashes: the second sequence shares the common prefix's blocks
    m = new_manager(16, 16)
    m.allocateSequence(1)
    m.appendTokens(1, 64, ha)
    m.allocateSequence(2)
    m.appendTokens(2, 64, hb)
    assert m.getBlockTable(1)[:2] == m.getBlockTable(2)[:2] and m.getBlockTable(1)[2:] != m.getBlockTable(2)[2:]
    assert m.memoryStats().prefixCacheHits == 2
