"""Value types of the reference's public API (PagedAttentionTypes.swift,
KVCacheManager.swift:6-44, Scheduler.swift:5-40), spelled as in the reference.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Optional


class PagedAttentionError(Exception):
    """PagedAttentionError (PagedAttentionTypes.swift:5-64).  ``case`` names the
    Swift enum case, ``code`` is the library's PAM_ERR_* value."""

    CASES = {1: "deviceInitializationFailed", 4: "invalidConfiguration", 5: "bufferTooSmall",
             6: "commandEncodingFailed", 7: "commandExecutionFailed", 8: "unsupported",
             10: "resourceExhausted", 12: "invalidState", 13: "recurringError", 30: "nullHandle"}

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.case = self.CASES.get(code, "unknown")
        self.description = message


class KVCacheError(Exception):
    """KVCacheError (KVCacheManager.swift:6-11)."""

    CASES = {20: "outOfMemory", 21: "sequenceNotFound", 22: "sequenceAlreadyExists", 23: "invalidRequest"}

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.case = self.CASES.get(code, "unknown")


class PagedAttentionDataType(enum.IntEnum):
    """PagedAttentionTypes.swift:67-91; bfloat16 is an addition."""
    float32 = 0
    float16 = 1
    float8 = 2
    bfloat16 = 3

    @property
    def byteWidth(self) -> int:
        return {0: 4, 1: 2, 2: 1, 3: 2}[int(self)]

    @property
    def isQuantized(self) -> bool:
        return self == PagedAttentionDataType.float8

    @property
    def ioByteWidth(self) -> int:
        """Bytes per element of queries, new K/V rows and outputs."""
        return 4 if self == PagedAttentionDataType.float32 else 2


class BlockEvictionPolicy(enum.IntEnum):
    """KVCacheManager.swift:13-17"""
    fifo = 0
    lifo = 1
    bestFit = 2


class SequenceStatus(enum.IntEnum):
    """Scheduler.swift:5-10"""
    waiting = 0
    running = 1
    paused = 2
    completed = 3


class Operation(enum.IntEnum):
    """PagedAttentionStats.Operation (PagedAttentionTypes.swift:171-180)"""
    none = 0
    prefillSinglePass = 1
    prefillMMA = 2
    prefillFlash = 3
    prefillTiledPass = 4
    decode = 5
    append = 6
    backward = 7


@dataclass
class PagedLayerSpec:
    """PagedAttentionTypes.swift:94-152"""
    headDim: int
    numHeads: int
    numKVHeads: int
    blockSize: int = 16
    dataType: PagedAttentionDataType = PagedAttentionDataType.float16
    windowSize: int = 0

    @property
    def qElementsPerToken(self) -> int:
        return self.numHeads * self.headDim

    @property
    def kvElementsPerToken(self) -> int:
        return self.numKVHeads * self.headDim


@dataclass
class PagedAttentionStats:
    """PagedAttentionTypes.swift:169-207"""
    operation: Operation = Operation.none
    batchSize: int = 0
    sequenceLength: int = 0
    numBlocks: int = 0
    temporaryBytes: int = 0
    usedSplitPass: bool = False
    elapsedMs: float = 0.0


@dataclass
class KVCacheMemoryStats:
    """KVCacheManager.swift:19-32"""
    totalBlocks: int
    usedBlocks: int
    freeBlocks: int
    activeSequences: int
    totalMemoryBytes: int
    usedMemoryBytes: int
    partiallyFilledBlocks: int
    fragmentationRatio: float
    prefixCacheHits: int
    prefixCacheEntries: int
    sharedBlocks: int
    evictionPolicy: BlockEvictionPolicy


@dataclass
class LogicalSequence:
    """KVCacheManager.swift:34-44"""
    id: int
    blockTable: list = field(default_factory=list)
    sequenceLength: int = 0


@dataclass
class SchedulerSequence:
    """Scheduler.swift:24-40"""
    id: int
    status: SequenceStatus
    numGeneratedTokens: int
    maxNewTokens: int
    promptLength: int
    arrivalOrder: int

    @property
    def currentLength(self) -> int:
        return self.promptLength + self.numGeneratedTokens

    @property
    def isDone(self) -> bool:
        return self.numGeneratedTokens >= self.maxNewTokens


@dataclass
class PagedAttentionPrefillRequest:
    """PagedAttentionTypes.swift:210-256; qStart/qLen select the rows of one chunk."""
    q: Any
    kPool: Any
    vPool: Any
    blockTable: Any
    output: Any
    seqLen: int
    layer: PagedLayerSpec
    causal: bool = True
    kScaleBuffer: Optional[Any] = None
    vScaleBuffer: Optional[Any] = None
    qStart: int = 0
    qLen: int = 0


@dataclass
class PagedAttentionFusedPrefillRequest:
    """PagedAttentionTypes.swift:367-421"""
    q: Any
    rawK: Any
    rawV: Any
    blockTable: Any
    kPool: Any
    vPool: Any
    output: Any
    seqLen: int
    layer: PagedLayerSpec
    causal: bool = True
    kScaleBuffer: Optional[Any] = None
    vScaleBuffer: Optional[Any] = None


@dataclass
class PagedAttentionDecodeRequest:
    """PagedAttentionTypes.swift:259-315"""
    q: Any
    kPool: Any
    vPool: Any
    blockTables: Any
    seqLengths: Any
    output: Any
    batchSize: int
    maxNumBlocks: int
    layer: PagedLayerSpec
    kScaleBuffer: Optional[Any] = None
    vScaleBuffer: Optional[Any] = None


@dataclass
class PagedKVAppendRequest:
    """PagedAttentionTypes.swift:318-364"""
    keys: Any
    values: Any
    kPool: Any
    vPool: Any
    blockTable: Any
    tokenOffset: int
    numNewTokens: int
    layer: PagedLayerSpec
    kScaleBuffer: Optional[Any] = None
    vScaleBuffer: Optional[Any] = None
