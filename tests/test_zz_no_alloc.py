"""pamc_decode_noalloc: the decode for callers that must not allocate device
memory (work being recorded for replay, a server that gave all free memory to
the KV pools, a host that only receives pointers from another allocator).

It must give what pamc_decode gives.  Both run the same kernel; the no-allocation
variant keeps the partial results of shared sequences in the library's fixed
array, which can hold fewer records than the context's arena, so it may launch
fewer warps: the list of tiles is then cut into other pieces, the two sum in a
different order and agree to rounding.  The outputs are compared within the
tolerance of the other decode tests (and with each other far inside it), on
two calls in a row that share the fixed array (the second with other data and
another shape, so stale partial results of the first would
show).  Collected last on purpose.
"""
import numpy as np
import pytest

import pagedattentionmetal_b200 as pam
from gpu_helpers import DT, DecodeCase, assert_close, from_io, io_numpy_dtype

pytestmark = pytest.mark.gpu


def _device_request(engine, case, window=0):
    out = engine.makeBuffer(case.q.nbytes)
    req = pam.PagedAttentionDecodeRequest(
        engine.makeBufferFrom(case.q), engine.makeBufferFrom(case.k_pool), engine.makeBufferFrom(case.v_pool),
        engine.makeBufferFrom(case.tables), engine.makeBufferFrom(case.lens), out, len(case.lens),
        case.tables.shape[1], case.layer(window))
    return req, out


def _download(out, case):
    return out.download(io_numpy_dtype(case.dtype), case.q.shape)


def test_noalloc_decode_matches_decode_on_two_calls_in_a_row():
    engine = pam.PagedAttentionEngine()
    # few long sequences: the plan splits each context, so the scratch array is really used
    cases = [DecodeCase(51, 3, 3000, 6000, 8, 2, 128, 16, DT.float16),
             DecodeCase(52, 2, 2000, 5000, 16, 2, 128, 16, DT.bfloat16)]
    for case in cases:
        req, out = _device_request(engine, case)
        engine.decode(req)
        assert engine.lastStats.temporaryBytes > 0, "the case must need records for shared sequences"
        expected = _download(out, case)
        req2, out2 = _device_request(engine, case)
        engine.decodeNoAlloc(req2)
        assert 0 < engine.lastStats.temporaryBytes <= 8 << 20
        got = _download(out2, case)
        assert_close(from_io(got, case.dtype), from_io(expected, case.dtype), case.dtype)
        # same products, another order of the final sum: a few units in the last place at most
        assert np.abs(from_io(got, case.dtype) - from_io(expected, case.dtype)).max() <= 2.0 ** -8
        assert_close(from_io(got, case.dtype), case.oracle(), case.dtype)
    # a windowed call through the same array
    req3, out3 = _device_request(engine, cases[0], window=1500)
    engine.decodeNoAlloc(req3)
    assert_close(from_io(_download(out3, cases[0]), DT.float16), cases[0].oracle(window=1500), DT.float16)
    engine.close()


def test_noalloc_decode_rejects_what_it_cannot_hold():
    engine = pam.PagedAttentionEngine()
    engine.enableGracefulDegradation = False
    # The built-in arrays hold one arrival word per (sequence, kv head) pair, 65 536 of them:
    # 70 000 single-head sequences are refused before any launch, so small buffers that only
    # satisfy the argument checks are enough.
    B, H, KVH, D, bs, max_nb = 70000, 1, 1, 128, 16, 1
    pool = engine.makeBuffer(max_nb * bs * KVH * D * 2)
    q = engine.makeBuffer(B * H * D * 2)
    out = engine.makeBuffer(B * H * D * 2)
    tables = engine.makeBufferFrom(np.zeros((B, max_nb), np.int32))
    lens = engine.makeBufferFrom(np.full(B, max_nb * bs, np.uint32))
    layer = pam.PagedLayerSpec(D, H, KVH, bs, DT.float16)
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decodeNoAlloc(pam.PagedAttentionDecodeRequest(q, pool, pool, tables, lens, out, B, max_nb, layer))
    assert e.value.case == "resourceExhausted"
    assert str(8 << 20) in str(e.value) and "65536" in str(e.value) and "pamc_decode" in str(e.value)
    # the same batch is fine for pamc_decode, which takes what it needs from the context
    engine.decode(pam.PagedAttentionDecodeRequest(q, pool, pool, tables, lens, out, B, max_nb, layer))
    # host buffers would need staging memory: refused as well
    with pytest.raises(pam.PagedAttentionError) as e:
        engine.decodeNoAlloc(pam.PagedAttentionDecodeRequest(np.zeros((1, H, D), np.float16), pool, pool, tables, lens,
                                                             out, 1, max_nb, layer))
    assert "device memory only" in str(e.value)
    engine.close()


def test_noalloc_decode_allocates_nothing_and_can_be_recorded():
    """Free device memory and the context's arena stay as they were across the call, and a
    call made while the stream is being captured only records its launches (no wait, no
    retry loop): the replayed graph gives the bits of the eager call, every time."""
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    engine = pam.PagedAttentionEngine(0)
    case = DecodeCase(53, 3, 3000, 6000, 8, 2, 128, 16, DT.float16)
    req, out = _device_request(engine, case)
    engine.decode(req)
    expected = _download(out, case)
    req2, out2 = _device_request(engine, case)
    engine.decodeNoAlloc(req2)                    # the first call on this GPU looks the scratch array up
    torch.cuda.synchronize(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]
    for _ in range(3):
        engine.decodeNoAlloc(req2)
    torch.cuda.synchronize(dev)
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    eager = _download(out2, case)
    assert_close(from_io(eager, case.dtype), from_io(expected, case.dtype), case.dtype)
    # recorded into a graph on a capturing stream, then replayed
    req3, out3 = _device_request(engine, case)
    stream = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    engine.setStream(stream.cuda_stream)
    launches = engine.kernelLaunches
    with torch.cuda.graph(graph, stream=stream):
        engine.decodeNoAlloc(req3)
    assert engine.kernelLaunches > launches
    engine.setStream(None)
    graph.replay()
    torch.cuda.synchronize(dev)
    assert np.array_equal(_download(out3, case).view(np.uint16), eager.view(np.uint16))
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize(dev)
    assert np.array_equal(_download(out3, case).view(np.uint16), eager.view(np.uint16))
    engine.close()
