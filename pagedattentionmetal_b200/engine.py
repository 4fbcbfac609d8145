"""Python face of the library: PagedAttentionEngine, KVCacheManager,
BatchKVCacheManager and ContinuousBatchingScheduler with the reference's method
names and error behaviour, each a thin veneer over the C ABI (all logic and all
kernels live in libpam_cuda.so; nothing here computes).

Buffers may be numpy arrays (host memory; staged by the library inside the
call, like the reference's host-visible MTLBuffers), ``DeviceBuffer`` objects,
torch CUDA tensors, or raw device addresses.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Iterable, Optional, Sequence

import numpy as np

from . import _cabi
from ._cabi import lib
from .api_types import (BlockEvictionPolicy, KVCacheError, KVCacheMemoryStats, LogicalSequence,
                        Operation, PagedAttentionDataType, PagedAttentionDecodeRequest,
                        PagedAttentionError, PagedAttentionFusedPrefillRequest, PagedAttentionPrefillRequest,
                        PagedAttentionStats,
                        PagedKVAppendRequest, PagedLayerSpec, SchedulerSequence, SequenceStatus)


def _raise(ctx) -> None:
    code = lib.pamc_last_error_code(ctx)
    msg = lib.pam_last_error(ctx)
    text = msg.decode() if msg else "unknown error"
    if 20 <= code < 30:
        raise KVCacheError(code, text)
    raise PagedAttentionError(code, text)


def _check(ctx, rc: int) -> None:
    if rc != 0:
        _raise(ctx)


def _layer(spec: PagedLayerSpec) -> _cabi.PamLayerSpec:
    return _cabi.PamLayerSpec(spec.headDim, spec.numHeads, spec.numKVHeads, spec.blockSize,
                              int(spec.dataType), spec.windowSize)


class DeviceBuffer:
    """Device memory owned by the library (stands where the reference has an
    MTLBuffer): address + length, upload/download through the context."""

    def __init__(self, engine: "PagedAttentionEngine", nbytes: int):
        self._engine = engine
        self.nbytes = int(nbytes)
        self.ptr = lib.pamc_buffer_alloc(engine._ctx, self.nbytes)
        if not self.ptr:
            raise PagedAttentionError(10, f"GPU resource exhausted: cannot allocate {nbytes} bytes")

    @property
    def length(self) -> int:
        return self.nbytes

    def data_ptr(self) -> int:
        return self.ptr

    def upload(self, array: np.ndarray, offset: int = 0) -> "DeviceBuffer":
        a = np.ascontiguousarray(array)
        assert offset + a.nbytes <= self.nbytes
        _check(self._engine._ctx, lib.pamc_memcpy(self._engine._ctx, self.ptr + offset, a.ctypes.data, a.nbytes, 0))
        return self

    def download(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert offset + out.nbytes <= self.nbytes
        _check(self._engine._ctx, lib.pamc_memcpy(self._engine._ctx, out.ctypes.data, self.ptr + offset, out.nbytes, 1))
        return out

    def free(self) -> None:
        if self.ptr:
            lib.pamc_buffer_free(self._engine._ctx, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _buf(x) -> _cabi.PamBuffer:
    if x is None:
        return _cabi.PamBuffer(None, 0)
    if isinstance(x, DeviceBuffer):
        return _cabi.PamBuffer(x.ptr, x.nbytes)
    return _cabi.buffer(x)


class PagedAttentionEngine:
    """PagedAttentionEngine (PagedAttentionEngine.swift:82): prefill, decode and
    appendToCache over paged KV pools, with the reference's validation, retry,
    graceful-degradation and statistics behaviour."""

    def __init__(self, device: Optional[int] = None):
        if lib.pamc_device_count() <= 0:
            raise PagedAttentionError(1, "Metal device or command queue could not be initialized.")
        self._ctx = lib.pamc_create_context_on(device) if device is not None else lib.pam_create_context()
        if not self._ctx:
            raise PagedAttentionError(1, "Metal device or command queue could not be initialized.")
        self._splitThreshold, self._defaultWindowSize, self._defaultChunkSize = 1024, 0, 0
        self._maxRetries, self._graceful = 3, True
        self._dependents = weakref.WeakSet()      # objects whose native side refers to this context

    def close(self) -> None:
        for d in list(getattr(self, "_dependents", ())):
            d.close()                             # they must go before the context they point at
        if getattr(self, "_ctx", None):
            lib.pam_destroy_context(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- properties (PagedAttentionEngine.swift:116-129) --
    splitThreshold = property(lambda s: s._splitThreshold)
    defaultWindowSize = property(lambda s: s._defaultWindowSize)
    defaultChunkSize = property(lambda s: s._defaultChunkSize)
    maxRetries = property(lambda s: s._maxRetries)
    enableGracefulDegradation = property(lambda s: s._graceful)

    @splitThreshold.setter
    def splitThreshold(self, v):
        self._splitThreshold = int(v)
        lib.pamc_set_split_threshold(self._ctx, int(v))

    @defaultWindowSize.setter
    def defaultWindowSize(self, v):
        self._defaultWindowSize = int(v)
        lib.pamc_set_default_window(self._ctx, int(v))

    @defaultChunkSize.setter
    def defaultChunkSize(self, v):
        self._defaultChunkSize = int(v)
        lib.pamc_set_default_chunk(self._ctx, int(v))

    @maxRetries.setter
    def maxRetries(self, v):
        self._maxRetries = int(v)
        lib.pamc_set_max_retries(self._ctx, int(v))

    @enableGracefulDegradation.setter
    def enableGracefulDegradation(self, v):
        self._graceful = bool(v)
        lib.pamc_set_graceful_degradation(self._ctx, 1 if v else 0)

    @property
    def lastStats(self) -> PagedAttentionStats:      # PagedAttentionEngine.swift:137-141
        s = _cabi.PamStats()
        lib.pamc_last_stats(self._ctx, C.byref(s))
        return PagedAttentionStats(Operation(s.operation), s.batch_size, s.sequence_length, s.num_blocks,
                                   s.temporary_bytes, bool(s.used_split_pass), s.elapsed_ms)

    @property
    def lastError(self) -> Optional[str]:            # PagedAttentionEngine.swift:144-148
        m = lib.pam_last_error(self._ctx)
        return m.decode() if m else None

    @property
    def kernelLaunches(self) -> int:
        return int(lib.pamc_kernel_launches(self._ctx))

    def recommendedMaxBlocks(self, blockSize, numKVHeads, headDim, dataType, memoryFraction=0.75, layerCount=1) -> int:
        """PagedAttentionEngine.swift:201-217"""
        return int(lib.pamc_recommended_max_blocks(self._ctx, blockSize, numKVHeads, headDim, int(dataType),
                                                   memoryFraction, layerCount))

    def makeBuffer(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def makeBufferFrom(self, array: np.ndarray) -> DeviceBuffer:
        a = np.ascontiguousarray(array)
        return DeviceBuffer(self, max(a.nbytes, 1)).upload(a) if a.nbytes else DeviceBuffer(self, 1)

    def setStream(self, cuda_stream: Optional[int]) -> None:
        _check(self._ctx, lib.pamc_set_stream(self._ctx, cuda_stream))

    def setAsync(self, enabled: bool) -> None:
        lib.pamc_set_async(self._ctx, 1 if enabled else 0)

    def synchronize(self) -> None:
        _check(self._ctx, lib.pamc_synchronize(self._ctx))

    def setPrefillTensorPath(self, on: bool) -> None:
        lib.pamc_set_prefill_tensor_path(self._ctx, 1 if on else 0)

    def setPrefillExactWeights(self, mode: int) -> None:
        """0 / 1 / 2, see pamc_set_prefill_exact_weights."""
        lib.pamc_set_prefill_exact_weights(self._ctx, mode)

    def injectLaunchFailures(self, n: int) -> None:
        lib.pamc_inject_launch_failures(self._ctx, n)

    def setWaitLimit(self, smCycles: int) -> None:
        """Bound of every wait inside the tensor-core prefill kernel, in SM clock
        cycles (0: the default, about 0.2 s); see pamc_set_wait_limit."""
        _check(self._ctx, lib.pamc_set_wait_limit(self._ctx, int(smCycles)))

    def testStarvePrefill(self, launches: int) -> None:
        """The next `launches` tensor-core prefill launches never fetch their first
        value tile, so the wait for it runs out (see pamc_test_starve_prefill)."""
        _check(self._ctx, lib.pamc_test_starve_prefill(self._ctx, int(launches)))

    @staticmethod
    def decodePath(request: PagedAttentionDecodeRequest) -> int:
        """1: the stream kernel would run this request, 0: the general kernel
        (pamc_decode_path; nothing is launched)."""
        r = _cabi.PamDecodeRequest(_buf(request.q), _buf(request.kPool), _buf(request.vPool),
                                   _buf(request.blockTables), _buf(request.seqLengths), _buf(request.output),
                                   request.batchSize, request.maxNumBlocks, _layer(request.layer),
                                   _buf(request.kScaleBuffer), _buf(request.vScaleBuffer))
        return int(lib.pamc_decode_path(C.byref(r)))

    # -- outputs of a cache sharded by KV head over several GPUs (no reference counterpart) --
    @staticmethod
    def makeCommId() -> bytes:
        """128 bytes that rank 0 makes and every rank passes to joinComm."""
        raw = C.create_string_buffer(128)
        if lib.pamc_comm_unique_id(raw) != 0:
            raise PagedAttentionError(1, "NCCL could not be loaded")
        return raw.raw

    def joinComm(self, commId: bytes, rank: int, numRanks: int):
        raw = C.create_string_buffer(bytes(commId), 128)
        h = lib.pamc_comm_create(self._ctx, raw, rank, numRanks)
        if not h:
            _raise(self._ctx)
        return h

    @staticmethod
    def leaveComm(comm) -> None:
        lib.pamc_comm_destroy(comm)

    def allGatherHeads(self, comm, local, full, rows: int, headsLocal: int, headDim: int, dataType) -> None:
        """[rows][headsLocal][headDim] of every rank into [rows][headsLocal * ranks][headDim]
        on every rank (pamc_allgather_heads; a collective call)."""
        _check(self._ctx, lib.pamc_allgather_heads(self._ctx, comm, _cabi.address(local), _cabi.address(full), rows,
                                                    headsLocal, headDim, int(dataType)))

    # -- operations --
    def prefill(self, request: PagedAttentionPrefillRequest, chunkSize: int = 0) -> None:
        """PagedAttentionEngine.swift:405-418 (request form) and :713-768 (chunk loop)."""
        r = _cabi.PamPrefillRequest(_buf(request.q), _buf(request.kPool), _buf(request.vPool),
                                    _buf(request.blockTable), _buf(request.output), request.seqLen,
                                    _layer(request.layer), 1 if request.causal else 0,
                                    _buf(request.kScaleBuffer), _buf(request.vScaleBuffer),
                                    request.qStart, request.qLen)
        _check(self._ctx, lib.pamc_prefill(self._ctx, C.byref(r), chunkSize))

    def fusedPrefill(self, request: PagedAttentionFusedPrefillRequest, cache: Optional["KVCacheManager"] = None) -> None:
        """PagedAttentionEngine.swift:633-710: the raw keys and values of tokens
        [0, seqLen) go into the pages and the prefill of the same rows runs over
        them.  cache is the manager that owns the pools (required for FP8)."""
        r = _cabi.PamFusedPrefillRequest(_buf(request.q), _buf(request.rawK), _buf(request.rawV),
                                         _buf(request.blockTable), _buf(request.kPool), _buf(request.vPool),
                                         _buf(request.output), request.seqLen, _layer(request.layer),
                                         1 if request.causal else 0, _buf(request.kScaleBuffer),
                                         _buf(request.vScaleBuffer))
        _check(self._ctx, lib.pamc_fused_prefill(self._ctx, C.byref(r), cache._h if cache is not None else None))

    def backward(self, q, kPool, vPool, blockTable, dO, m, l, dQ, dKPool, dVPool, seqLen: int, headDim: int,
                 numHeads: int, numKVHeads: int, blockSize: int,
                 dataType: PagedAttentionDataType = PagedAttentionDataType.float32, windowSize: int = 0) -> None:
        """PagedAttentionEngine.swift:1341-1395: gradients with respect to the queries (dQ,
        written) and the paged keys and values (dKPool, dVPool, added to) of the attention of
        rows [0, seqLen) over keys [windowStart, seqLen), no causal mask; m and l are the row
        maximum and row sum of the forward pass, float32 [seqLen][numHeads]."""
        layer = _cabi.PamLayerSpec(headDim, numHeads, numKVHeads, blockSize, int(dataType), windowSize)
        r = _cabi.PamBackwardRequest(_buf(q), _buf(kPool), _buf(vPool), _buf(blockTable), _buf(dO), _buf(m), _buf(l),
                                     _buf(dQ), _buf(dKPool), _buf(dVPool), seqLen, layer)
        _check(self._ctx, lib.pamc_backward(self._ctx, C.byref(r)))

    def prefillBatch(self, q, kPool, vPool, blockTables, output, seqLens: Sequence[int], qStarts: Sequence[int],
                     qLens: Sequence[int], maxNumBlocks: int, layer: PagedLayerSpec, causal: bool = True,
                     kScaleBuffer=None, vScaleBuffer=None) -> None:
        """One launch for the same chunk of several sequences (no counterpart in
        the reference, whose prefill takes one sequence per dispatch)."""
        n = len(seqLens)
        arr = lambda v: (C.c_int32 * n)(*[int(x) for x in v])
        sl, qs, ql = arr(seqLens), arr(qStarts), arr(qLens)
        r = _cabi.PamBatchPrefillRequest(_buf(q), _buf(kPool), _buf(vPool), _buf(blockTables), _buf(output),
                                         sl, qs, ql, n, maxNumBlocks, _layer(layer), 1 if causal else 0,
                                         _buf(kScaleBuffer), _buf(vScaleBuffer))
        _check(self._ctx, lib.pamc_prefill_batch(self._ctx, C.byref(r)))

    def decode(self, request: PagedAttentionDecodeRequest) -> None:
        """PagedAttentionEngine.swift:533-546"""
        r = _cabi.PamDecodeRequest(_buf(request.q), _buf(request.kPool), _buf(request.vPool),
                                   _buf(request.blockTables), _buf(request.seqLengths), _buf(request.output),
                                   request.batchSize, request.maxNumBlocks, _layer(request.layer),
                                   _buf(request.kScaleBuffer), _buf(request.vScaleBuffer))
        _check(self._ctx, lib.pamc_decode(self._ctx, C.byref(r)))

    def decodeNoAlloc(self, request: PagedAttentionDecodeRequest) -> None:
        """The same decode for callers that must not allocate device memory
        (see pamc_decode_noalloc in include/pam_cuda.h): device buffers only,
        partial results of shared sequences in the library's fixed 8 MiB array."""
        r = _cabi.PamDecodeRequest(_buf(request.q), _buf(request.kPool), _buf(request.vPool),
                                   _buf(request.blockTables), _buf(request.seqLengths), _buf(request.output),
                                   request.batchSize, request.maxNumBlocks, _layer(request.layer),
                                   _buf(request.kScaleBuffer), _buf(request.vScaleBuffer))
        _check(self._ctx, lib.pamc_decode_noalloc(self._ctx, C.byref(r)))

    def appendToCache(self, request: PagedKVAppendRequest) -> None:
        """PagedAttentionEngine.swift:585-597"""
        r = _cabi.PamAppendRequest(_buf(request.keys), _buf(request.values), _buf(request.kPool),
                                   _buf(request.vPool), _buf(request.blockTable), request.tokenOffset,
                                   request.numNewTokens, _layer(request.layer), _buf(request.kScaleBuffer),
                                   _buf(request.vScaleBuffer))
        _check(self._ctx, lib.pamc_append_to_cache(self._ctx, C.byref(r)))

    # -- batched-layer calls (PagedAttentionEngine.swift:1433-1895) --
    @staticmethod
    def _perLayer(x, n: int, what: str) -> list:
        """A buffer shared by all layers (the reference's kPool / vPool) or one per layer."""
        if isinstance(x, (list, tuple)):
            if len(x) != n:
                raise PagedAttentionError(4, f"Invalid paged attention configuration: {what} count must match layers count")
            return list(x)
        return [x] * n

    @staticmethod
    def _layerCounts(n: int, *lists) -> None:
        if n == 0 or any(len(x) != n for x in lists):       # :1445-1447, :1652-1654, :1757-1759
            raise PagedAttentionError(4, "Invalid paged attention configuration: buffer/layer count mismatch")

    def prefillLayers(self, qBuffers, kPool, vPool, blockTable, outputBuffers, seqLen: int,
                      layers: Sequence[PagedLayerSpec], causal: bool = True, windowSize: int = 0,
                      kScaleBuffers=None, vScaleBuffers=None) -> None:
        """PagedAttentionEngine.swift:1433-1639: the prefill of every layer, one wait."""
        n = len(layers)
        self._layerCounts(n, qBuffers, outputBuffers)
        kp, vp = self._perLayer(kPool, n, "kPool"), self._perLayer(vPool, n, "vPool")
        ks, vs = self._perLayer(kScaleBuffers, n, "kScaleBuffers"), self._perLayer(vScaleBuffers, n, "vScaleBuffers")
        arr = (_cabi.PamPrefillRequest * n)()
        for i, spec in enumerate(layers):
            arr[i] = _cabi.PamPrefillRequest(_buf(qBuffers[i]), _buf(kp[i]), _buf(vp[i]), _buf(blockTable),
                                             _buf(outputBuffers[i]), seqLen, _layer(self._windowed(spec, windowSize)),
                                             1 if causal else 0, _buf(ks[i]), _buf(vs[i]), 0, 0)
        _check(self._ctx, lib.pamc_prefill_layers(self._ctx, arr, n))

    def decodeLayers(self, qBuffers, kPool, vPool, blockTables, seqLengths, outputBuffers, batchSize: int,
                     maxNumBlocks: int, layers: Sequence[PagedLayerSpec], windowSize: int = 0,
                     kScaleBuffers=None, vScaleBuffers=None) -> None:
        """PagedAttentionEngine.swift:1641-1742: the decode of every layer, one wait."""
        n = len(layers)
        self._layerCounts(n, qBuffers, outputBuffers)
        kp, vp = self._perLayer(kPool, n, "kPool"), self._perLayer(vPool, n, "vPool")
        ks, vs = self._perLayer(kScaleBuffers, n, "kScaleBuffers"), self._perLayer(vScaleBuffers, n, "vScaleBuffers")
        arr = (_cabi.PamDecodeRequest * n)()
        for i, spec in enumerate(layers):
            arr[i] = _cabi.PamDecodeRequest(_buf(qBuffers[i]), _buf(kp[i]), _buf(vp[i]), _buf(blockTables),
                                            _buf(seqLengths), _buf(outputBuffers[i]), batchSize, maxNumBlocks,
                                            _layer(self._windowed(spec, windowSize)), _buf(ks[i]), _buf(vs[i]))
        _check(self._ctx, lib.pamc_decode_layers(self._ctx, arr, n))

    def appendLayers(self, keys, values, kPool, vPool, blockTable, tokenOffset: int, numNewTokens: int,
                     layers: Sequence[PagedLayerSpec], kScaleBuffers=None, vScaleBuffers=None, caches=None) -> None:
        """PagedAttentionEngine.swift:1744-1895: the append of every layer, one wait.
        caches: the managers that own the pools, one per layer (required for FP8 layers)."""
        n = len(layers)
        self._layerCounts(n, keys, values)
        kp, vp = self._perLayer(kPool, n, "kPool"), self._perLayer(vPool, n, "vPool")
        ks, vs = self._perLayer(kScaleBuffers, n, "kScaleBuffers"), self._perLayer(vScaleBuffers, n, "vScaleBuffers")
        cs = self._perLayer(caches, n, "caches")
        arr = (_cabi.PamAppendRequest * n)()
        for i, spec in enumerate(layers):
            arr[i] = _cabi.PamAppendRequest(_buf(keys[i]), _buf(values[i]), _buf(kp[i]), _buf(vp[i]), _buf(blockTable),
                                            tokenOffset, numNewTokens, _layer(spec), _buf(ks[i]), _buf(vs[i]))
        handles = (C.c_void_p * n)(*[c._h if c is not None else None for c in cs])
        _check(self._ctx, lib.pamc_append_layers(self._ctx, arr, n, handles))

    @staticmethod
    def _windowed(spec: PagedLayerSpec, windowSize: int) -> PagedLayerSpec:
        """An explicit window wins over the layer's own (PagedAttentionEngine.swift:1466, 1673)."""
        if windowSize > 0 and windowSize != spec.windowSize:
            return PagedLayerSpec(spec.headDim, spec.numHeads, spec.numKVHeads, spec.blockSize, spec.dataType, windowSize)
        return spec

    # -- cache-handle forms (the reference's C ABI, PagedAttentionCABI.swift:203-337) --
    def appendKV(self, cache: "KVCacheManager", sequenceId: int, keys, values, tokenOffset: int,
                 numNewTokens: int, numHeads: int) -> None:
        _check(self._ctx, lib.pam_append_kv(self._ctx, cache._h, sequenceId, _cabi.address(keys),
                                            _cabi.address(values), tokenOffset, numNewTokens, numHeads))

    def prefillSequence(self, cache: "KVCacheManager", sequenceId: int, q, output, seqLen: int, numHeads: int,
                        causal: bool = True) -> None:
        _check(self._ctx, lib.pam_prefill(self._ctx, cache._h, sequenceId, _cabi.address(q),
                                          _cabi.address(output), seqLen, numHeads, causal))

    def decodeBatch(self, cache: "KVCacheManager", ids: Sequence[int], q, output, numHeads: int) -> None:
        arr = (C.c_int64 * len(ids))(*[int(i) for i in ids])
        _check(self._ctx, lib.pam_decode(self._ctx, cache._h, arr, len(ids), _cabi.address(q),
                                         _cabi.address(output), numHeads))

    def reshapeAndCache(self, cache: "KVCacheManager", keys, values, slotMapping, numTokens: int) -> None:
        _check(self._ctx, lib.pamc_reshape_and_cache(self._ctx, cache._h, _cabi.address(keys),
                                                     _cabi.address(values), _cabi.address(slotMapping), numTokens))

    def copyBlocks(self, cache: "KVCacheManager", src: Iterable[int], dst: Iterable[int]) -> None:
        s = np.ascontiguousarray(list(src), dtype=np.int32)
        d = np.ascontiguousarray(list(dst), dtype=np.int32)
        assert len(s) == len(d)
        _check(self._ctx, lib.pamc_copy_blocks(self._ctx, cache._h, s.ctypes.data_as(C.POINTER(C.c_int32)),
                                               d.ctypes.data_as(C.POINTER(C.c_int32)), len(s)))


class KVCacheManager:
    """KVCacheManager (KVCacheManager.swift:47-379).  With ``engine=None`` the
    manager only keeps the books (no pools, no GPU)."""

    def __init__(self, engine: Optional[PagedAttentionEngine], maxBlocks: int, blockSize: int = 16,
                 headDim: int = 0, numKVHeads: int = 0,
                 dataType: PagedAttentionDataType = PagedAttentionDataType.float16):
        self.engine = engine
        self.maxBlocks, self.blockSize, self.headDim, self.numKVHeads = maxBlocks, blockSize, headDim, numKVHeads
        self.dataType = PagedAttentionDataType(dataType)
        self._ownCtx = None
        if engine is None:
            self._h = lib.pamc_cache_create_bookkeeping(maxBlocks, blockSize)
            if not self._h:
                raise PagedAttentionError(4, "Invalid paged attention configuration: maxBlocks must be positive")
            # errors of a manager without an engine are kept in a context-free holder
            self._ctx = None
        else:
            self._ctx = engine._ctx
            self._h = lib.pam_create_cache(self._ctx, maxBlocks, blockSize, headDim, numKVHeads, int(dataType))
            if not self._h:
                _raise(self._ctx)
        self._policy = BlockEvictionPolicy.fifo

    def _context(self):
        if self._ctx is None:
            raise PagedAttentionError(12, "Invalid engine state: this manager has no engine")
        return self._ctx

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.pam_destroy_cache(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # pools (KVCacheManager.swift:59-60)
    def _pools(self):
        k, v, ks, vs = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        pb, sb = C.c_size_t(), C.c_size_t()
        lib.pamc_cache_pools(self._h, C.byref(k), C.byref(v), C.byref(ks), C.byref(vs), C.byref(pb), C.byref(sb))
        return k.value, v.value, ks.value, vs.value, pb.value, sb.value

    @property
    def kPoolBuffer(self) -> _cabi.PamBuffer:
        p = self._pools()
        return _cabi.PamBuffer(p[0], p[4])

    @property
    def vPoolBuffer(self) -> _cabi.PamBuffer:
        p = self._pools()
        return _cabi.PamBuffer(p[1], p[4])

    @property
    def kScaleBuffer(self) -> Optional[_cabi.PamBuffer]:
        p = self._pools()
        return _cabi.PamBuffer(p[2], p[5]) if p[2] else None

    @property
    def vScaleBuffer(self) -> Optional[_cabi.PamBuffer]:
        p = self._pools()
        return _cabi.PamBuffer(p[3], p[5]) if p[3] else None

    def readPools(self):
        """Download K/V pools as arrays [blocks][kv_heads][block_size][head_dim]
        (and FP8 scales [blocks][kv_heads] float16, else None)."""
        k, v, ks, vs, pb, sb = self._pools()
        dt = {0: np.float32, 1: np.float16, 2: np.uint8, 3: np.uint16}[int(self.dataType)]
        shape = (self.maxBlocks, self.numKVHeads, self.blockSize, self.headDim)
        ctx = self._context()
        kp, vp = np.empty(shape, dtype=dt), np.empty(shape, dtype=dt)
        _check(ctx, lib.pamc_memcpy(ctx, kp.ctypes.data, k, pb, 1))
        _check(ctx, lib.pamc_memcpy(ctx, vp.ctypes.data, v, pb, 1))
        ksc = vsc = None
        if ks:
            ksc = np.empty((self.maxBlocks, self.numKVHeads), dtype=np.float16)
            vsc = np.empty((self.maxBlocks, self.numKVHeads), dtype=np.float16)
            _check(ctx, lib.pamc_memcpy(ctx, ksc.ctypes.data, ks, sb, 1))
            _check(ctx, lib.pamc_memcpy(ctx, vsc.ctypes.data, vs, sb, 1))
        return kp, vp, ksc, vsc

    # -- bookkeeping --
    def _kv(self, rc: int):
        if rc < 0:
            if self._ctx is None:
                raise KVCacheError(0, "KVCacheError")
            _raise(self._ctx)
        return rc

    def _ctx_or_scratch(self):
        if self._ctx is None:
            if self._ownCtx is None:
                self._ownCtx = _ErrorHolder()
            return self._ownCtx.ctx
        return self._ctx

    def allocateSequence(self, id: int) -> None:                       # KVCacheManager.swift:106-113
        ctx = self._ctx_or_scratch()
        _check(ctx, lib.pam_reserve_sequence(ctx, self._h, id))

    def appendTokens(self, toSequence: int, count: int, blockHashes: Optional[Sequence[int]] = None) -> None:
        """KVCacheManager.swift:115-174"""
        ctx = self._ctx_or_scratch()
        if blockHashes is None:
            _check(ctx, lib.pamc_cache_append_tokens(ctx, self._h, toSequence, count, None, 0))
        else:
            n = len(blockHashes)
            arr = (C.c_uint64 * max(n, 1))(*[int(h) for h in blockHashes])
            _check(ctx, lib.pamc_cache_append_tokens(ctx, self._h, toSequence, count, arr, n))

    def registerBlockHash(self, hash: int, physicalBlock: int) -> None:   # KVCacheManager.swift:196-198
        lib.pamc_cache_register_block_hash(self._h, hash, physicalBlock)

    def ensureExclusiveAccess(self, sequenceId: int, logicalBlockIndex: int) -> None:   # :200-214
        ctx = self._ctx_or_scratch()
        _check(ctx, lib.pamc_cache_ensure_exclusive(ctx, self._h, sequenceId, logicalBlockIndex))

    def freeSequence(self, id: int) -> None:                           # KVCacheManager.swift:216-239
        lib.pam_free_sequence(self._h, id)

    def getBlockTable(self, forSequence: int) -> list:                  # KVCacheManager.swift:299-303
        ctx = self._ctx_or_scratch()
        n = lib.pamc_cache_block_table(ctx, self._h, forSequence, None, 0)
        if n < 0:
            _raise(ctx)
        out = (C.c_int32 * max(n, 1))()
        lib.pamc_cache_block_table(ctx, self._h, forSequence, out, n)
        return list(out[:n])

    def getSequence(self, id: int) -> LogicalSequence:                  # KVCacheManager.swift:323-327
        return LogicalSequence(id, self.getBlockTable(id), self.getSequenceLength(id))

    def getSequenceLength(self, id: int) -> int:                        # KVCacheManager.swift:329-333
        ctx = self._ctx_or_scratch()
        n = lib.pam_sequence_length(ctx, self._h, id)
        if n < 0:
            _raise(ctx)
        return n

    def getNumBlocks(self, forSequence: int) -> int:                    # KVCacheManager.swift:335-339
        ctx = self._ctx_or_scratch()
        n = lib.pamc_cache_num_blocks(ctx, self._h, forSequence)
        if n < 0:
            _raise(ctx)
        return n

    @property
    def availableBlocks(self) -> int:                                   # KVCacheManager.swift:341-345
        return lib.pam_available_blocks(self._h)

    @property
    def activeSequenceCount(self) -> int:                               # KVCacheManager.swift:347-351
        return lib.pamc_cache_active_sequences(self._h)

    @property
    def evictionPolicy(self) -> BlockEvictionPolicy:
        return self._policy

    @evictionPolicy.setter
    def evictionPolicy(self, p) -> None:                                # KVCacheManager.swift:65-67
        self._policy = BlockEvictionPolicy(p)
        lib.pamc_cache_set_eviction_policy(self._h, int(self._policy))

    def memoryStats(self) -> KVCacheMemoryStats:                        # KVCacheManager.swift:353-378
        s = _cabi.PamMemoryStats()
        lib.pamc_cache_memory_stats(self._h, C.byref(s))
        return KVCacheMemoryStats(s.total_blocks, s.used_blocks, s.free_blocks, s.active_sequences,
                                  s.total_memory_bytes, s.used_memory_bytes, s.partially_filled_blocks,
                                  s.fragmentation_ratio, s.prefix_cache_hits, s.prefix_cache_entries,
                                  s.shared_blocks, BlockEvictionPolicy(s.eviction_policy))

    def setHygiene(self, on: bool) -> None:
        """Forget a block's prefix hashes when it is freed, and make an append that
        runs out of blocks change nothing (see pamc_cache_set_hygiene).  Off by
        default: the reference does neither."""
        lib.pamc_cache_set_hygiene(self._h, 1 if on else 0)

    @staticmethod
    def blockHashes(tokenIds: Sequence[int], blockSize: int, seed: int = 0) -> list:
        """Chained content hashes of the full blocks of a token sequence, usable as
        appendTokens' blockHashes (see pamc_block_hashes)."""
        n = len(tokenIds)
        ids = (C.c_int32 * max(n, 1))(*[int(t) for t in tokenIds])
        full = n // blockSize
        out = (C.c_uint64 * max(full, 1))()
        got = lib.pamc_block_hashes(ids, n, blockSize, seed, out, full)
        return [int(out[i]) for i in range(got)]

    def drainCopyOnWriteLog(self) -> list:
        out = (C.c_int32 * 2048)()
        n = lib.pamc_cache_drain_cow_log(self._h, out, 1024)
        return [(out[2 * i], out[2 * i + 1]) for i in range(n)]

    def slotMapping(self, id: int, tokenOffset: int, numTokens: int) -> np.ndarray:
        ctx = self._ctx_or_scratch()
        out = np.empty(numTokens, dtype=np.int64)
        _check(ctx, lib.pamc_cache_slot_mapping(ctx, self._h, id, tokenOffset, numTokens,
                                                out.ctypes.data_as(C.POINTER(C.c_int64))))
        return out

    def batchTables(self, ids: Sequence[int], maxNumBlocks: int):
        """Zero-padded [n][maxNumBlocks] int32 tables and [n] uint32 lengths
        (KVCacheManager.swift:661-703), as host arrays."""
        ctx = self._ctx_or_scratch()
        n = len(ids)
        tables = np.zeros((n, maxNumBlocks), dtype=np.int32)
        lens = np.zeros(n, dtype=np.uint32)
        arr = (C.c_int64 * max(n, 1))(*[int(i) for i in ids])
        _check(ctx, lib.pamc_cache_batch_tables(ctx, self._h, arr, n, maxNumBlocks, tables.ctypes.data, lens.ctypes.data))
        return tables, lens


class _ErrorHolder:
    """A manager without an engine still needs a place for its last error; the
    C ABI keeps that in a context.  A host-only context needs no GPU."""

    def __init__(self):
        self.ctx = lib.pamc_create_host_context()

    def __del__(self):
        try:
            if self.ctx:
                lib.pam_destroy_context(self.ctx)
                self.ctx = None
        except Exception:
            pass


class BatchKVCacheManager(KVCacheManager):
    """BatchKVCacheManager (KVCacheManager.swift:382-739): adds device slabs for
    block tables and lengths that getBatchBlockTableBuffer/getSeqLengthsBuffer
    overwrite on every call."""

    def __init__(self, engine: PagedAttentionEngine, maxBatchSize: int, maxSequenceBlocks: int, maxBlocks: int,
                 blockSize: int = 16, headDim: int = 0, numKVHeads: int = 0,
                 dataType: PagedAttentionDataType = PagedAttentionDataType.float16):
        super().__init__(engine, maxBlocks, blockSize, headDim, numKVHeads, dataType)
        self.maxBatchSize, self.maxSequenceBlocks = maxBatchSize, maxSequenceBlocks
        self.blockTablesSlab = engine.makeBuffer(maxBatchSize * maxSequenceBlocks * 4)   # KVCacheManager.swift:446
        self.seqLengthsSlab = engine.makeBuffer(maxBatchSize * 4)

    def getBatchBlockTableBuffer(self, forBatch: Sequence[int]) -> DeviceBuffer:   # KVCacheManager.swift:661-688
        if len(forBatch) > self.maxBatchSize:
            raise KVCacheError(20, "KVCacheError.outOfMemory")
        n = len(forBatch)
        arr = (C.c_int64 * max(n, 1))(*[int(i) for i in forBatch])
        _check(self._ctx, lib.pamc_cache_batch_tables(self._ctx, self._h, arr, n, self.maxSequenceBlocks,
                                                      self.blockTablesSlab.ptr, None))
        return self.blockTablesSlab

    def getSeqLengthsBuffer(self, forBatch: Sequence[int]) -> DeviceBuffer:        # KVCacheManager.swift:690-703
        n = len(forBatch)
        arr = (C.c_int64 * max(n, 1))(*[int(i) for i in forBatch])
        _check(self._ctx, lib.pamc_cache_batch_tables(self._ctx, self._h, arr, n, self.maxSequenceBlocks,
                                                      None, self.seqLengthsSlab.ptr))
        return self.seqLengthsSlab


class ContinuousBatchingScheduler:
    """ContinuousBatchingScheduler (Scheduler.swift:42-177)."""

    def __init__(self, maxBatchSize: int, maxSequences: int = 128):
        self.maxBatchSize, self.maxSequences = maxBatchSize, maxSequences
        self._h = lib.pamc_sched_create(maxBatchSize, maxSequences)

    def __del__(self):
        try:
            if self._h:
                lib.pamc_sched_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def _get(self, id: int) -> Optional[SchedulerSequence]:
        s = _cabi.PamSchedSequence()
        if lib.pamc_sched_get(self._h, id, C.byref(s)) != 0:
            return None
        return SchedulerSequence(s.id, SequenceStatus(s.status), s.num_generated_tokens, s.max_new_tokens,
                                 s.prompt_length, s.arrival_order)

    def addRequest(self, promptTokenCount: int, maxNewTokens: int) -> int:          # Scheduler.swift:58-70
        return int(lib.pamc_sched_add_request(self._h, promptTokenCount, maxNewTokens))

    def completeSequence(self, id: int) -> None:                                    # Scheduler.swift:72-76
        lib.pamc_sched_complete(self._h, id)

    def step(self) -> list:                                                         # Scheduler.swift:78-114
        cap = max(self.maxBatchSize, 1)
        out = (C.c_int64 * cap)()
        n = lib.pamc_sched_step(self._h, out, cap)
        return [self._get(out[i]) for i in range(min(n, cap))]

    def markPrefilled(self, id: int) -> None:                                       # Scheduler.swift:116-120
        lib.pamc_sched_mark_prefilled(self._h, id)

    def markDecoded(self, id: int) -> None:                                         # Scheduler.swift:122-126
        lib.pamc_sched_mark_decoded(self._h, id)

    def preemptSequence(self, id: int) -> None:                                     # Scheduler.swift:128-132
        lib.pamc_sched_preempt(self._h, id)

    def handleMemoryPressure(self, requiredBlocks: int, availableBlocks) -> list:   # Scheduler.swift:134-152
        fn = _cabi.AVAILABLE_FN(lambda _user: int(availableBlocks()))
        cap = max(self.maxSequences, 1)
        out = (C.c_int64 * cap)()
        n = lib.pamc_sched_handle_memory_pressure(self._h, requiredBlocks, fn, None, out, cap)
        return [int(out[i]) for i in range(min(n, cap))]

    def sequence(self, id: int) -> Optional[SchedulerSequence]:
        return self._get(id)

    @property
    def waitingCount(self) -> int:                                                  # Scheduler.swift:154-158
        return lib.pamc_sched_count(self._h, int(SequenceStatus.waiting))

    @property
    def runningCount(self) -> int:                                                  # Scheduler.swift:160-164
        return lib.pamc_sched_count(self._h, int(SequenceStatus.running))

    @property
    def completedCount(self) -> int:                                                # Scheduler.swift:166-170
        return lib.pamc_sched_count(self._h, int(SequenceStatus.completed))

    @property
    def totalSequencesProcessed(self) -> int:                                       # Scheduler.swift:172-176
        return lib.pamc_sched_total(self._h)


class PagedAttentionInference:
    """PagedAttentionInference (PagedAttentionInference.swift:7-299): engine,
    cache and scheduler driven step by step.  The state machine lives in the
    library (pamc_infer_*); ``cache`` and ``scheduler`` are views of the handles
    it owns."""

    def __init__(self, maxBlocks: int, blockSize: int = 16, layerSpecs: Sequence[PagedLayerSpec] = (),
                 maxBatchSize: int = 16, maxSequences: int = 128, engine: Optional[PagedAttentionEngine] = None):
        self.engine = engine if engine is not None else PagedAttentionEngine()
        self.layerSpecs = list(layerSpecs)
        self.maxBatchSize, self.numLayers = maxBatchSize, len(self.layerSpecs)
        specs = (_cabi.PamLayerSpec * max(self.numLayers, 1))(*[_layer(s) for s in self.layerSpecs])
        self._h = lib.pamc_infer_create(self.engine._ctx, maxBlocks, blockSize, specs, self.numLayers, maxBatchSize,
                                        maxSequences)
        if not self._h:
            _raise(self.engine._ctx)
        first = self.layerSpecs[0]
        # views of the handles the library object owns (never destroyed from here)
        cache = object.__new__(BatchKVCacheManager)
        cache.engine, cache._ctx, cache._ownCtx = self.engine, self.engine._ctx, None
        cache.maxBlocks, cache.blockSize, cache.headDim, cache.numKVHeads = maxBlocks, blockSize, first.headDim, first.numKVHeads
        cache.dataType = PagedAttentionDataType(first.dataType)
        cache._policy = BlockEvictionPolicy.fifo
        cache.maxBatchSize, cache.maxSequenceBlocks = maxBatchSize, maxBlocks            # :75
        cache._h = lib.pamc_infer_cache(self._h)
        cache.close = lambda: None
        cache.blockTablesSlab = cache.seqLengthsSlab = None
        self.cache = cache
        self.scheduler = _BorrowedScheduler(lib.pamc_infer_scheduler(self._h), maxBatchSize, maxSequences)
        self._callback = None
        self._onTokenGenerated = None
        self.engine._dependents.add(self)         # closed before the engine's context goes away

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.cache._h = None
            lib.pamc_infer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def onTokenGenerated(self):
        return self._onTokenGenerated

    @onTokenGenerated.setter
    def onTokenGenerated(self, fn) -> None:                                  # :27
        self._onTokenGenerated = fn
        self._callback = _cabi.TOKEN_FN(lambda user, seq, tok: fn(int(seq), int(tok))) if fn else _cabi.TOKEN_FN(0)
        lib.pamc_infer_set_token_callback(self._h, self._callback, None)

    def setIncrementalPreemption(self, on: bool) -> None:
        """Pause one victim at a time under memory pressure instead of every
        running sequence (see pamc_infer_set_incremental_preemption)."""
        lib.pamc_infer_set_incremental_preemption(self._h, 1 if on else 0)

    def setBatchedPrefill(self, on: bool, tokenBudget: int = 0) -> None:
        """One prefill launch per layer and step for all prompts of the step, with an
        optional bound on the prompt rows per step (see pamc_infer_set_batched_prefill)."""
        lib.pamc_infer_set_batched_prefill(self._h, 1 if on else 0, int(tokenBudget))

    @property
    def prefillLaunchSets(self) -> int:
        return int(lib.pamc_infer_prefill_launch_sets(self._h))

    def addRequest(self, promptTokenCount: int, maxNewTokens: int) -> int:   # :103-105
        return int(lib.pamc_infer_add_request(self._h, promptTokenCount, maxNewTokens))

    def completeSequence(self, id: int) -> None:                             # :108-114
        lib.pamc_infer_complete_sequence(self._h, id)

    def step(self) -> list:                                                  # :119-148
        cap = max(self.maxBatchSize, 1)
        out = (C.c_int64 * cap)()
        n = lib.pamc_infer_step(self._h, out, cap)
        if n < 0:
            _raise(self.engine._ctx)
        return [self.scheduler._get(out[i]) for i in range(min(n, cap))]

    def runAll(self) -> None:                                                # :151-156
        _check(self.engine._ctx, lib.pamc_infer_run_all(self._h))

    @property
    def waitingCount(self) -> int:
        return self.scheduler.waitingCount

    @property
    def runningCount(self) -> int:
        return self.scheduler.runningCount

    @property
    def completedCount(self) -> int:
        return self.scheduler.completedCount

    @property
    def totalTokensGenerated(self) -> int:                                   # :166-170
        return int(lib.pamc_infer_total_tokens(self._h))

    @property
    def stepCount(self) -> int:                                              # :34
        return int(lib.pamc_infer_step_count(self._h))


class _BorrowedScheduler(ContinuousBatchingScheduler):
    """The scheduler a PagedAttentionInference owns: same methods, not destroyed here."""

    def __init__(self, handle, maxBatchSize: int, maxSequences: int):
        self.maxBatchSize, self.maxSequences = maxBatchSize, maxSequences
        self._h = handle

    def __del__(self):
        self._h = None
