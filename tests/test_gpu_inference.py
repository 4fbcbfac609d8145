"""PagedAttentionInference (PagedAttentionInference.swift:7-299) on the GPU: the
library's step loop against the oracle's restatement of the same state machine
(batches, block tables, lengths, counters, token callbacks), with the attention
launches of every step really made."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT
from oracle import paged_oracle as po

pytestmark = pytest.mark.gpu

LAYERS = [pam.PagedLayerSpec(128, 8, 2, 16, DT.float16), pam.PagedLayerSpec(128, 4, 2, 16, DT.float16)]


def _pair(engine, max_blocks, max_batch, incremental=False, layers=LAYERS):
    inf = pam.PagedAttentionInference(max_blocks, 16, layers, max_batch, 128, engine=engine)
    ora = po.OracleInference(max_blocks, 16, max_batch, 128, incremental)
    if incremental:
        inf.setIncrementalPreemption(True)
    return inf, ora


def _same_state(inf, ora, ids):
    assert inf.cache.availableBlocks == ora.cache.available_blocks
    assert inf.totalTokensGenerated == ora.total_tokens
    assert inf.stepCount == ora.step_count
    for status, name in ((po.WAITING, "waitingCount"), (po.RUNNING, "runningCount"), (po.COMPLETED, "completedCount")):
        assert getattr(inf, name) == ora.sched.count(status)
    for sid in ids:
        sq = inf.scheduler.sequence(sid)
        o = ora.sched.seqs[sid]
        assert (int(sq.status), sq.numGeneratedTokens) == (o["status"], o["gen"])
        if sid in ora.cache.sequences:
            assert inf.cache.getBlockTable(sid) == list(ora.cache.block_table(sid))
            assert inf.cache.getSequenceLength(sid) == ora.cache.sequence_length(sid)
        else:
            with pytest.raises(pam.KVCacheError):
                inf.cache.getBlockTable(sid)


def test_step_by_step_matches_the_oracle(engine):
    inf, ora = _pair(engine, 64, 3)
    tokens = []
    inf.onTokenGenerated = lambda sid, tok: tokens.append((sid, tok))
    ids = []
    for prompt, new in ((40, 3), (17, 1), (100, 5), (5, 2), (64, 4)):
        a, b = inf.addRequest(prompt, new), ora.add_request(prompt, new)
        assert a == b
        ids.append(a)
    launches_before = engine.kernelLaunches
    for _ in range(40):
        got = [s.id for s in inf.step()]
        want = ora.step()
        assert got == want
        _same_state(inf, ora, ids)
        if not want:
            break
    assert tokens == ora.tokens and len(tokens) == 3 + 1 + 5 + 2 + 4
    assert inf.completedCount == 5 and inf.runningCount == 0
    assert inf.cache.availableBlocks == 64
    assert engine.kernelLaunches > launches_before          # the attention of every step really ran
    assert engine.lastStats.operation == pam.Operation.decode
    inf.close()


def test_run_all_and_late_requests(engine):
    inf, ora = _pair(engine, 128, 4)
    for prompt, new in ((33, 2), (70, 6), (9, 1)):
        inf.addRequest(prompt, new), ora.add_request(prompt, new)
    inf.runAll(), ora.run_all()
    _same_state(inf, ora, range(3))
    for prompt, new in ((200, 3), (16, 16)):
        assert inf.addRequest(prompt, new) == ora.add_request(prompt, new)
    inf.runAll(), ora.run_all()
    _same_state(inf, ora, range(5))
    assert inf.totalTokensGenerated == 33 + 70 + 9 + 200 + 16 + 2 + 6 + 1 + 3 + 16
    inf.close()


@pytest.mark.parametrize("incremental", [False, True])
def test_memory_pressure_preemption(engine, incremental):
    """14 blocks of 16 tokens: three running sequences hold 12, the fourth prompt needs 6.
    The reference pauses every running sequence (the free count it passes does not move while
    victims are chosen); with incremental preemption only as many as needed.  Either way a
    victim that was part of the same batch makes the step fail like the reference's
    (its block table is gone when the decode tables are built)."""
    inf, ora = _pair(engine, 14, 4, incremental)
    for prompt, new in ((48, 8), (48, 8), (48, 8)):
        inf.addRequest(prompt, new), ora.add_request(prompt, new)
    assert [s.id for s in inf.step()] == ora.step()
    assert [s.id for s in inf.step()] == ora.step()
    inf.addRequest(90, 2), ora.add_request(90, 2)
    with pytest.raises(po.SequenceNotFound):
        ora.step()
    with pytest.raises(pam.KVCacheError) as e:
        inf.step()
    assert e.value.case == "sequenceNotFound"
    _same_state(inf, ora, range(4))
    n_paused = sum(1 for i in range(3) if inf.scheduler.sequence(i).status == pam.SequenceStatus.paused)
    # (the newest running sequence is the new one itself, promoted by the scheduler's step
    # before its prefill: it is the first victim in both modes and is prefilled all the same)
    assert n_paused == (1 if incremental else 3)
    # from here on the two must keep agreeing, failing steps included
    for _ in range(80):
        err = None
        try:
            want = ora.step()
        except po.SequenceNotFound:
            err = "sequenceNotFound"
        except po.OutOfMemory:
            err = "outOfMemory"
        if err:
            with pytest.raises(pam.KVCacheError) as e:
                inf.step()
            assert e.value.case == err
        else:
            assert [s.id for s in inf.step()] == want
        _same_state(inf, ora, range(4))
        if not err and not want:
            break
    assert inf.completedCount == ora.sched.count(po.COMPLETED)
    # pausing everything under pressure never lets this workload finish (the resumed sequences
    # evict one another's pages step after step); pausing one victim at a time does
    assert inf.completedCount == (4 if incremental else 0)
    inf.close()


def test_out_of_memory_and_errors(engine):
    inf, ora = _pair(engine, 4, 2)
    inf.addRequest(200, 1), ora.add_request(200, 1)
    with pytest.raises(po.OutOfMemory):
        ora.step()
    with pytest.raises(pam.KVCacheError) as e:
        inf.step()
    assert e.value.case == "outOfMemory"
    inf.close()
    with pytest.raises(pam.PagedAttentionError, match="at least one layer spec required"):
        pam.PagedAttentionInference(8, 16, [], 2, 8, engine=engine)


def test_fp8_layers(engine):
    layers = [pam.PagedLayerSpec(128, 8, 2, 16, DT.float8)] * 2
    inf, ora = _pair(engine, 32, 2, layers=layers)
    for prompt, new in ((50, 2), (31, 3)):
        inf.addRequest(prompt, new), ora.add_request(prompt, new)
    inf.runAll(), ora.run_all()
    _same_state(inf, ora, range(2))
    assert inf.completedCount == 2
    inf.close()


def _run_pair(inf, ora, ids, steps=120, must_finish=True):
    for _ in range(steps):
        err = None
        try:
            want = ora.step()
        except po.SequenceNotFound:
            err = "sequenceNotFound"
        except po.OutOfMemory:
            err = "outOfMemory"
        if err:
            with pytest.raises(pam.KVCacheError) as e:
                inf.step()
            assert e.value.case == err
        else:
            assert [s.id for s in inf.step()] == want
        _same_state(inf, ora, ids)
        if not err and not want:
            return
    # (pausing every running sequence under pressure never lets the 14-block workload finish,
    # in the reference's loop as here: the resumed sequences evict one another step after step)
    assert not must_finish, "did not finish"


@pytest.mark.parametrize("blocks", [64, 14])
def test_batched_prefill_leaves_the_reference_state(engine, blocks):
    """With pamc_infer_set_batched_prefill the prompts of a step are prefilled by one launch
    per layer; batches, block tables, lengths, statuses and counters stay those of the
    reference's one-sequence-per-dispatch loop, step by step, under memory pressure too."""
    inf, ora = _pair(engine, blocks, 4)
    inf.setBatchedPrefill(True)
    plain, _ = _pair(engine, blocks, 4)
    requests = ((40, 3), (17, 1), (48, 5), (5, 2)) if blocks == 64 else ((48, 8), (48, 8), (48, 8))
    for prompt, new in requests:
        assert inf.addRequest(prompt, new) == ora.add_request(prompt, new)
        plain.addRequest(prompt, new)
    ids = list(range(len(requests)))
    assert [s.id for s in inf.step()] == ora.step()
    plain.step()
    _same_state(inf, ora, ids)
    # one launch set for the whole step instead of one per prompt
    assert inf.prefillLaunchSets == 1 and plain.prefillLaunchSets == len(requests)
    if blocks == 14:
        assert [s.id for s in inf.step()] == ora.step()
        inf.addRequest(90, 2), ora.add_request(90, 2)
        ids.append(3)
    _run_pair(inf, ora, ids, steps=80, must_finish=blocks == 64)
    inf.close()
    plain.close()


def test_prefill_token_budget_spreads_prompts_over_steps(engine):
    """A budget of 64 prompt rows per step: a 150-token prompt takes three steps, the prompts
    behind it wait, nothing decodes before its whole prompt is done, and the run ends with
    the same totals as without a budget."""
    inf, _ = _pair(engine, 64, 8)
    inf.setBatchedPrefill(True, 64)
    prompts = ((150, 2), (20, 3), (70, 1), (10, 2))
    for prompt, new in prompts:
        inf.addRequest(prompt, new)
    tokens = []
    inf.onTokenGenerated = lambda sid, tok: tokens.append(sid)
    seen_first_token_at = {}
    for step in range(40):
        before, decoded = inf.totalTokensGenerated, len(tokens)
        batch = inf.step()
        if not batch:
            break
        for sid in tokens:
            seen_first_token_at.setdefault(sid, step)
        # prompt tokens are counted when a prompt completes (:216): the prompts completed in
        # one step are the ones whose last chunk fitted the budget of 64 rows
        completed_prompt_tokens = inf.totalTokensGenerated - before - (len(tokens) - decoded)
        sums = {0}
        for pr, _ in prompts:
            sums |= {x + pr for x in sums}
        assert completed_prompt_tokens in sums
    assert inf.completedCount == 4 and inf.cache.availableBlocks == 64
    assert inf.totalTokensGenerated == sum(p + n for p, n in prompts)
    # 150 rows at 64 per step: the first sequence cannot decode before the fourth step
    assert seen_first_token_at[0] >= 3
    # prompts 1 and 2 share the budget left over behind it, in arrival order
    assert seen_first_token_at[1] <= seen_first_token_at[2] <= seen_first_token_at[3] + 1
    assert inf.prefillLaunchSets >= 4
    inf.close()
