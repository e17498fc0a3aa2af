"""The split-params container: our Python and C++ readers/writers against the reference's own
MemRefFlatArray (compiled from the nncv tree into oracle/_ref when that tree is present) and against
a file that the reference's writer produced (tests/golden/kat0_two_params.bin)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import binding as ob
from nncv_b200 import _lib
from nncv_b200.memref import (FlatArrayError, MemRefDescriptor1, MemRefDescriptor2, MemRefDescriptor4,
                              MemRefFlatArray, MemRefIndexer, MemRefMagicHead, make_descriptor)


def _sample(width=4):
    g = np.random.default_rng(0)
    dt = np.float32 if width == 4 else np.float16
    arr = MemRefFlatArray(width)
    arr.add("fc.bias", g.standard_normal(10).astype(dt))
    arr.add("layer1.0.conv1.weight", g.standard_normal((4, 3, 3, 3)).astype(dt))
    arr.add("bn.scalar_like", g.standard_normal((1,)).astype(dt))
    return arr


def test_record_sizes_match_reference_layout():
    assert ctypes.sizeof(MemRefMagicHead) == 24 and ctypes.sizeof(MemRefIndexer) == 224
    assert (ctypes.sizeof(MemRefDescriptor1), ctypes.sizeof(MemRefDescriptor2), ctypes.sizeof(MemRefDescriptor4)) == (40, 56, 88)
    ref = ob.ref_lib()
    if ref is not None:
        assert ref.ref_sizeof_head() == 24 and ref.ref_sizeof_indexer() == 224
        assert (ref.ref_sizeof_desc1(), ref.ref_sizeof_desc2(), ref.ref_sizeof_desc4()) == (40, 56, 88)


def test_reads_file_written_by_reference(golden_dir):
    arr = MemRefFlatArray.read(os.path.join(golden_dir, "kat0_two_params.bin"))
    assert [t.name for t in arr.tensors] == ["__constant_1x1x5x5xf32", "__constant_1x3x3x3xf32"]
    assert np.array_equal(arr.tensors[0].data[0, 0], np.eye(5, dtype=np.float32))
    assert arr.total_elements() == 52 and arr.blob().shape == (52,)


def test_python_writer_is_byte_identical_to_reference_writer(golden_dir):
    gold = open(os.path.join(golden_dir, "kat0_two_params.bin"), "rb").read()
    src = MemRefFlatArray.frombytes(gold)
    out = MemRefFlatArray(4)
    for t in src.tensors:
        out.add(t.name, t.data)
    assert out.tobytes() == gold


@pytest.mark.parametrize("width", [4, 2])
def test_round_trip_through_reference_reader(tmp_path, width):
    ref = ob.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built (the nncv tree is absent)")
    arr = _sample(width)
    path = str(tmp_path / "m.bin")
    arr.write(path)
    total = ctypes.c_long(0)
    buf = np.zeros(arr.total_elements(), arr.blob().dtype)
    assert ref.ref_flat_array_read(path.encode(), width, ctypes.byref(total), buf.ctypes.data, buf.nbytes) == 0
    assert total.value == arr.total_elements()
    assert np.array_equal(buf.view(np.uint8), arr.blob().view(np.uint8))


@pytest.mark.parametrize("width", [4, 2])
def test_c_reader_and_writer(tmp_path, width):
    """nncv_flat_array_read / _write of libnncv_b200.so (host-only code, runs without a GPU)."""
    L = _lib.lib()
    arr = _sample(width)
    path = str(tmp_path / "m.bin")
    arr.write(path)
    h = L.nncv_flat_array_read(path.encode())
    assert h, L.nncv_b200_last_error()
    try:
        assert L.nncv_flat_array_count(h) == 3
        for i, t in enumerate(arr.tensors):
            idx = L.nncv_flat_array_indexer(h, i).contents
            assert idx.name.decode() == t.name and idx.dims == len(t.shape) and idx.eleWidth == width
            assert tuple(idx.shape[d] for d in range(idx.dims)) == t.shape
            n = int(np.prod(t.shape))
            got = np.ctypeslib.as_array(ctypes.cast(L.nncv_flat_array_data(h, i), ctypes.POINTER(ctypes.c_uint8)), (n * width,))
            assert np.array_equal(got, t.data.reshape(-1).view(np.uint8))
        w = L.nncv_flat_array_wrapped(h).contents
        assert w.sizes[0] == arr.total_elements() and w.strides[0] == 1 and w.offset == 0
        # write it back with the C writer: identical bytes
        n = 3
        idxs = (MemRefIndexer * n)(*[L.nncv_flat_array_indexer(h, i).contents for i in range(n)])
        ptrs = (ctypes.c_void_p * n)(*[L.nncv_flat_array_data(h, i) for i in range(n)])
        path2 = str(tmp_path / "m2.bin")
        assert L.nncv_flat_array_write(path2.encode(), n, idxs, ptrs) == 0
        assert open(path2, "rb").read() == open(path, "rb").read()
    finally:
        L.nncv_flat_array_free(h)


def test_bad_files_are_rejected(tmp_path):
    L = _lib.lib()
    good = _sample().tobytes()
    cases = {
        "magic": b"\x43" + good[1:],
        "short_head": good[:10],
        "truncated_index": good[:24 + 100],
        "truncated_data": good[:-8],
        "huge_count": good[:16] + (2 ** 40).to_bytes(8, "little") + good[24:],
    }
    for name, data in cases.items():
        with pytest.raises(FlatArrayError):
            MemRefFlatArray.frombytes(data)
        p = str(tmp_path / f"{name}.bin")
        open(p, "wb").write(data)
        assert not L.nncv_flat_array_read(p.encode()), name
        assert L.nncv_b200_last_status() == 2  # NNCV_B200_EIO
    assert not L.nncv_flat_array_read(str(tmp_path / "missing.bin").encode())
    assert MemRefFlatArray.frombytes(MemRefFlatArray(4).tobytes()).tensors == []


def test_make_descriptor_strides():
    d = make_descriptor(0x1000, (2, 3, 8, 8))
    assert list(d.sizes) == [2, 3, 8, 8] and list(d.strides) == [192, 64, 8, 1] and d.aligned == 0x1000
