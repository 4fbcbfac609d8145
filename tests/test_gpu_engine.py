"""Engine behaviour around the kernels: validation and error texts, retry,
circuit breaker and zero-fill with host-injected failures, statistics."""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, DecodeCase, max_abs

pytestmark = pytest.mark.gpu


def _decode_request(engine, case, **over):
    out = np.zeros(case.q.shape, np.float16)
    kp, vp = engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool)
    args = dict(q=case.q, kPool=kp, vPool=vp, blockTables=case.tables, seqLengths=case.lens, output=out,
                batchSize=len(case.lens), maxNumBlocks=case.tables.shape[1], layer=case.layer())
    args.update(over)
    return pam.PagedAttentionDecodeRequest(**args), out


def test_validation_errors_match_reference(engine):
    case = DecodeCase(41, 3, 10, 60, 8, 2, 128, 16, DT.float16)
    req, _ = _decode_request(engine, case, output=np.zeros(10, np.float16))
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decode(req)
    # PagedAttentionTypes.swift:44-45 and the name used at PagedAttentionEngine.swift:1930
    assert e.value.case == "bufferTooSmall"
    assert str(e.value) == f"output buffer is too small: expected at least {3 * 8 * 128 * 2} bytes, got 20."
    assert engine.lastError == str(e.value)
    for name, over, text in (
        ("batchSize", dict(batchSize=0), "batchSize must be positive."),
        ("maxNumBlocks", dict(maxNumBlocks=0), "maxNumBlocks must be positive."),
        ("capacity", dict(maxNumBlocks=999), "maxNumBlocks exceeds blockTables buffer capacity"),
    ):
        req, _ = _decode_request(engine, case, **over)
        with pytest.raises(pam.PagedAttentionError) as e:
            engine.decode(req)
        assert e.value.case == "invalidConfiguration" and text in str(e.value)
    bad = pam.PagedLayerSpec(128, 7, 2, 16, DT.float16)
    req, _ = _decode_request(engine, case, layer=bad)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decode(req)
    assert "numHeads must be divisible by numKVHeads" in str(e.value)      # PagedAttentionTypes.swift:137
    # a good call clears the error (CABI.swift:32-37)
    req, out = _decode_request(engine, case)
    engine.decode(req)
    assert engine.lastError is None
    assert max_abs(out.astype(np.float32), case.oracle()) <= 2e-3


def test_unknown_dtype_and_bad_cache_config(engine):
    from pagedattentionmetal_b200._cabi import lib
    from pagedattentionmetal_b200.engine import _raise
    assert lib.pam_create_cache(engine._ctx, 4, 16, 64, 2, 9) is None
    with pytest.raises(pam.PagedAttentionError) as e:
        _raise(engine._ctx)
    assert e.value.case == "invalidConfiguration" and "unknown dtype 9" in str(e.value)   # CABI.swift:66
    with pytest.raises(pam.PagedAttentionError) as e:
        pam.KVCacheManager(engine, 0, 16, 64, 2, DT.float16)
    assert "maxBlocks must be positive" in str(e.value)                      # CABI.swift:116
    with pytest.raises(pam.PagedAttentionError) as e:
        pam.KVCacheManager(engine, 4, 16, 0, 2, DT.float16)
    assert "headDim must be positive." in str(e.value)                       # PagedAttentionTypes.swift:128


def test_append_and_prefill_validation(engine):
    cache = pam.KVCacheManager(engine, 4, 16, 64, 2, DT.float16)
    cache.allocateSequence(1)
    cache.appendTokens(1, 10)
    k = np.zeros((10, 2, 64), np.float16)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.appendKV(cache, 1, k, k, 0, 0, 2)
    assert "numNewTokens must be positive." in str(e.value)                  # PagedAttentionEngine.swift:1940
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.appendKV(cache, 1, k, k, -1, 4, 2)
    assert "tokenOffset must be non-negative." in str(e.value)               # PagedAttentionEngine.swift:1937
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.appendKV(cache, 1, k, k, 10, 10, 2)                           # 20 tokens need 2 blocks, table has 1
    assert e.value.case == "bufferTooSmall" and str(e.value).startswith("blockTable buffer is too small")
    with pytest.raises(pam.KVCacheError) as e:
        engine.appendKV(cache, 77, k, k, 0, 4, 2)
    assert e.value.case == "sequenceNotFound"
    q = np.zeros((10, 2, 64), np.float16)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.prefillSequence(cache, 1, q, q.copy(), 0, 2)
    assert "seqLen must be positive." in str(e.value)                        # PagedAttentionEngine.swift:1899
    with pytest.raises(pam.PagedAttentionError):
        engine.decodeBatch(cache, [], q, q.copy(), 2)                        # empty batch must throw (Tests:774-792)
    cache.close()


def test_retry_breaker_and_zero_fill_with_injected_failures():
    """PagedAttentionEngine.swift:375-414.  Failures are injected on the host:
    the launch wrapper reports an error without touching the GPU."""
    engine = pam.PagedAttentionEngine()
    case = DecodeCase(42, 2, 10, 40, 8, 2, 128, 16, DT.float16)
    ref = case.oracle()
    # two failures, third attempt succeeds: result is correct
    engine.enableGracefulDegradation = False
    engine.injectLaunchFailures(2)
    req, out = _decode_request(engine, case)
    engine.decode(req)
    assert max_abs(out.astype(np.float32), ref) <= 2e-3
    # three failures exhaust maxRetries = 3: the last error is thrown
    engine.injectLaunchFailures(3)
    req, out = _decode_request(engine, case)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decode(req)
    assert e.value.case == "commandExecutionFailed"
    # three more consecutive failures reach 2 * maxRetries: circuit breaker
    engine.injectLaunchFailures(3)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decode(req)
    assert e.value.case == "recurringError" and "decodeFlat" in str(e.value) and "6 attempts" in str(e.value)
    engine.injectLaunchFailures(0)
    # graceful degradation (the default): the error is swallowed and the output zero-filled
    engine.enableGracefulDegradation = True
    engine.injectLaunchFailures(3)
    req, out = _decode_request(engine, case)
    out[:] = 1
    engine.decode(req)
    assert np.all(out == 0)
    engine.injectLaunchFailures(0)
    req, out = _decode_request(engine, case)
    engine.decode(req)                                                       # a success resets the failure count
    assert max_abs(out.astype(np.float32), ref) <= 2e-3
    engine.maxRetries = 1
    engine.injectLaunchFailures(1)
    req, out = _decode_request(engine, case)
    out[:] = 1
    engine.decode(req)
    assert np.all(out == 0)
    engine.close()


def test_stats_and_recommended_blocks(engine):
    case = DecodeCase(43, 3, 10, 60, 8, 2, 128, 16, DT.float16)
    before = engine.kernelLaunches
    req, _ = _decode_request(engine, case)
    engine.decode(req)
    st = engine.lastStats
    assert st.operation == pam.Operation.decode and st.batchSize == 3 and st.numBlocks == case.tables.shape[1]
    assert st.elapsedMs > 0 and engine.kernelLaunches > before
    n = engine.recommendedMaxBlocks(16, 8, 128, DT.float16, 0.5, 2)          # PagedAttentionEngine.swift:201-217
    assert n >= 1
    n8 = engine.recommendedMaxBlocks(16, 8, 128, DT.float8, 0.5, 2)
    assert abs(n8 - 2 * n) <= 2


def test_batch_manager_slabs(engine):
    m = pam.BatchKVCacheManager(engine, 4, 6, 32, 16, 64, 2, DT.float16)
    for sid, n in ((1, 40), (2, 5)):
        m.allocateSequence(sid)
        m.appendTokens(sid, n)
    t = m.getBatchBlockTableBuffer([2, 1]).download(np.int32, (4, 6))
    l = m.getSeqLengthsBuffer([2, 1]).download(np.uint32, (4,))
    assert t[0].tolist() == [3, 0, 0, 0, 0, 0] and t[1].tolist() == [0, 1, 2, 0, 0, 0]   # KVCacheManager.swift:661-688
    assert l[:2].tolist() == [5, 40]
    with pytest.raises(pam.KVCacheError):
        m.getBatchBlockTableBuffer([1, 2, 1, 2, 1])                          # more than maxBatchSize (KVCM:664-666)
    m.close()


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """Every wait inside the tensor-core prefill kernel is bounded.  With the wait limit set
    to about a millisecond and the test switch that keeps each CTA's first value tile from
    being fetched, the wait for that tile runs out: the kernel returns through its error exit
    (nothing spins, nothing faults), the call fails with the site of the wait, the retry loop
    and the zero fill of graceful degradation take over as for any failed launch, and the
    next prefill on the same context is correct."""
    from test_gpu_prefill import PrefillCase
    from gpu_helpers import assert_close
    engine = pam.PagedAttentionEngine()
    case = PrefillCase(61, 300, 8, 2, 128, 16, DT.float16)
    ref = case.oracle()
    engine.setWaitLimit(2_000_000)                       # about 1 ms of SM clock cycles
    # one starved launch: the first attempt fails, the retry succeeds (PagedAttentionEngine.swift:375-400)
    engine.testStarvePrefill(1)
    before = engine.kernelLaunches
    assert_close(case.run(engine), ref, DT.float16)
    assert engine.lastStats.operation == pam.Operation.prefillMMA and engine.kernelLaunches - before == 2
    # every attempt starved, errors reported: the message names the wait that gave up
    engine.enableGracefulDegradation = False
    engine.testStarvePrefill(3)
    with pytest.raises(pam.PagedAttentionError) as e:
        case.run(engine)
    assert e.value.case == "commandExecutionFailed"
    assert "a kernel's bounded wait ran out (site " in str(e.value)
    assert engine.lastError == str(e.value)
    # the same with graceful degradation: no error, the output is zero-filled (:408-414)
    engine.enableGracefulDegradation = True
    engine.testStarvePrefill(3)
    assert np.all(case.run(engine) == 0)
    assert engine.lastError is None
    # and the context works as before, with the default limit as well
    assert_close(case.run(engine), ref, DT.float16)
    engine.setWaitLimit(0)
    assert_close(case.run(engine, q_start=100, q_len=150), case.oracle(q_start=100, q_len=150), DT.float16)
    engine.close()


def test_allgather_heads_single_rank(engine):
    """One rank: the gathered tensor is the local one (the NCCL path needs a GPU per rank
    and is exercised by the multi-GPU benchmark)."""
    try:
        comm = engine.joinComm(pam.PagedAttentionEngine.makeCommId(), 0, 1)
    except pam.PagedAttentionError:
        pytest.skip("NCCL is not loadable here")
    local = np.random.default_rng(62).standard_normal((5, 4, 128)).astype(np.float16)
    src, dst = engine.makeBufferFrom(local), engine.makeBuffer(local.nbytes)
    engine.allGatherHeads(comm, src, dst, 5, 4, 128, DT.float16)
    assert np.array_equal(dst.download(np.float16, local.shape), local)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.allGatherHeads(comm, src, dst, 5, 1, 4, DT.float16)       # an 8-byte slice
    assert e.value.case == "unsupported" and "multiple of 16" in str(e.value)
    pam.PagedAttentionEngine.leaveComm(comm)
