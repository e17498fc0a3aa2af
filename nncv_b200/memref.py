"""Host-side mirror of nncv's runtime types for the compiled-forward boundary.

Follows the reference byte for byte (paths relative to the nncv tree):
  * ``MemRefDescriptor<T,N>``  include/libnncv/DataType.hpp:129-136
  * ``MemRefIndexer``          include/libnncv/DataType.hpp:144-151  (224 bytes)
  * ``MemRefMagicHead``        include/libnncv/DataType.hpp:158-162  (24 bytes, magic 0x42)
  * ``MemRefFlatArray``        include/libnncv/DataType.hpp:164-196, src/libnncv/DataType.cpp:9-123

File layout of the split-params container ("model.bin"): head, then ``numMemRefIndex``
indexer records, then the tensors back to back with no padding.  ``dataOffset`` of each
indexer is the byte offset of its tensor from the start of the file.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

MAGIC = 0x42
NAME_LEN = 128
MAX_DIMS = 8


def memref_descriptor(rank: int):
    """ctypes struct equal to ``MemRefDescriptor<T, rank>`` (strides count elements)."""

    class _Desc(ctypes.Structure):
        _fields_ = [
            ("allocated", ctypes.c_void_p),
            ("aligned", ctypes.c_void_p),
            ("offset", ctypes.c_ssize_t),
            ("sizes", ctypes.c_ssize_t * rank),
            ("strides", ctypes.c_ssize_t * rank),
        ]

    _Desc.__name__ = f"MemRefDescriptor{rank}"
    return _Desc


MemRefDescriptor1 = memref_descriptor(1)
MemRefDescriptor2 = memref_descriptor(2)
MemRefDescriptor4 = memref_descriptor(4)


def make_descriptor(ptr: int, sizes: Sequence[int], strides: Sequence[int] | None = None):
    """Dense row-major descriptor over the memory at ``ptr`` (host or device address)."""
    rank = len(sizes)
    cls = {1: MemRefDescriptor1, 2: MemRefDescriptor2, 4: MemRefDescriptor4}.get(rank) or memref_descriptor(rank)
    if strides is None:
        strides = [1] * rank
        for i in range(rank - 2, -1, -1):
            strides[i] = strides[i + 1] * int(sizes[i + 1])
    d = cls()
    d.allocated = ptr
    d.aligned = ptr
    d.offset = 0
    for i in range(rank):
        d.sizes[i] = int(sizes[i])
        d.strides[i] = int(strides[i])
    return d


class MemRefIndexer(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * NAME_LEN),
        ("dims", ctypes.c_size_t),
        ("shape", ctypes.c_size_t * MAX_DIMS),
        ("eleWidth", ctypes.c_size_t),
        ("aligned", ctypes.c_size_t),
        ("dataOffset", ctypes.c_size_t),
    ]


class MemRefMagicHead(ctypes.Structure):
    _fields_ = [
        ("magicNumber", ctypes.c_int64),
        ("memRefIndexStartOffset", ctypes.c_size_t),
        ("numMemRefIndex", ctypes.c_size_t),
    ]


assert ctypes.sizeof(MemRefIndexer) == 224 and ctypes.sizeof(MemRefMagicHead) == 24


@dataclass
class FlatTensor:
    name: str
    shape: Tuple[int, ...]
    data: np.ndarray  # float32 or float16 (bf16 carried as uint16)


class FlatArrayError(ValueError):
    pass


class MemRefFlatArray:
    """Reader/writer of the split-params container, same bytes as the reference's."""

    def __init__(self, ele_width: int = 4):
        if ele_width not in (2, 4):
            raise FlatArrayError("eleWidth must be 2 or 4")
        self.ele_width = ele_width
        self.tensors: List[FlatTensor] = []

    def add(self, name: str, array: np.ndarray) -> None:
        if array.itemsize != self.ele_width:
            raise FlatArrayError(f"{name}: itemsize {array.itemsize} != eleWidth {self.ele_width}")
        if array.ndim > MAX_DIMS:
            raise FlatArrayError(f"{name}: rank {array.ndim} > {MAX_DIMS}")
        if len(name.encode()) >= NAME_LEN:
            raise FlatArrayError(f"{name}: name longer than {NAME_LEN - 1} bytes")
        self.tensors.append(FlatTensor(name, tuple(array.shape), np.ascontiguousarray(array)))

    # -- writer: MemRefFlatArray::write, DataType.cpp:9-43 --------------------------------
    def tobytes(self) -> bytes:
        n = len(self.tensors)
        head = MemRefMagicHead(MAGIC, ctypes.sizeof(MemRefMagicHead), n)
        out = [bytes(head)]
        off = ctypes.sizeof(MemRefMagicHead) + n * ctypes.sizeof(MemRefIndexer)
        for t in self.tensors:
            idx = MemRefIndexer()
            idx.name = t.name.encode()
            idx.dims = len(t.shape)
            for i, s in enumerate(t.shape):
                idx.shape[i] = s
            idx.eleWidth = self.ele_width
            idx.aligned = 64
            idx.dataOffset = off
            out.append(bytes(idx))
            off += int(np.prod(t.shape, dtype=np.int64)) * self.ele_width
        for t in self.tensors:
            out.append(t.data.tobytes())
        return b"".join(out)

    def write(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.tobytes())

    # -- reader: MemRefFlatArray::read, DataType.cpp:48-87 ---------------------------------
    @classmethod
    def frombytes(cls, buf: bytes, dtype=None) -> "MemRefFlatArray":
        hs, isz = ctypes.sizeof(MemRefMagicHead), ctypes.sizeof(MemRefIndexer)
        if len(buf) < hs:
            raise FlatArrayError("file shorter than the magic head")
        head = MemRefMagicHead.from_buffer_copy(buf[:hs])
        if head.magicNumber != MAGIC:
            raise FlatArrayError("bad magic number")
        n = head.numMemRefIndex
        start = head.memRefIndexStartOffset
        if start < hs or n > (len(buf) - start) // isz:
            raise FlatArrayError("indexer table runs past the end of the file")
        idxs = [MemRefIndexer.from_buffer_copy(buf[start + i * isz: start + (i + 1) * isz]) for i in range(n)]
        width = idxs[0].eleWidth if n else 4
        arr = cls(int(width))
        off = start + n * isz
        for idx in idxs:
            if idx.eleWidth != width or idx.dims > MAX_DIMS:
                raise FlatArrayError("mixed element widths or rank > 8")
            shape = tuple(int(idx.shape[i]) for i in range(idx.dims))
            nbytes = int(np.prod(shape, dtype=np.int64)) * int(width)
            if off + nbytes > len(buf):
                raise FlatArrayError("tensor data runs past the end of the file")
            dt = dtype or (np.float32 if width == 4 else np.float16)
            data = np.frombuffer(buf, dtype=dt, count=nbytes // int(width), offset=off).reshape(shape)
            arr.tensors.append(FlatTensor(idx.name.decode(), shape, data))
            off += nbytes
        return arr

    @classmethod
    def read(cls, path: str, dtype=None) -> "MemRefFlatArray":
        with open(path, "rb") as f:
            return cls.frombytes(f.read(), dtype)

    # -- MemRefFlatArray::wrap, DataType.cpp:89-119: one rank-1 view over every tensor ------
    def blob(self) -> np.ndarray:
        if not self.tensors:
            return np.zeros(0, np.float32 if self.ele_width == 4 else np.float16)
        return np.concatenate([t.data.reshape(-1) for t in self.tensors])

    def total_elements(self) -> int:
        return sum(int(np.prod(t.shape, dtype=np.int64)) for t in self.tensors)
