// C shim over the reference's own MemRefFlatArray (nncv: include/libnncv/DataType.hpp:164-196,
// src/libnncv/DataType.cpp:9-123).  TEST INFRASTRUCTURE: compiled together with the reference
// source file where it lies (never copied into this repository) into oracle/_ref/, and used
// only by the tests as the format oracle for the split-params container.
#include <cstring>
#include <string>

#include "libnncv/DataType.hpp"

using namespace nncv::rt;

extern "C" {

// Write a container holding `n` tensors with the reference's writer.
// shapes: n rows of 8 entries; dims[i] entries of row i are used.
int ref_flat_array_write(const char* path, int n, const char* const* names, const size_t* dims,
                         const size_t* shapes, size_t ele_width, void* const* data) {
  // Heap-allocated and never destroyed: the reference's destructor frees m_binaryData, which
  // stays uninitialised when only write() was used (DataType.cpp:121-123).
  auto& arr = *new MemRefFlatArray(ele_width == 2 ? dataType::kFloat16 : dataType::kFloat32);
  for (int i = 0; i < n; ++i) {
    MemRefIndexer idx;
    std::memset(&idx, 0, sizeof(idx));
    std::strncpy(idx.name, names[i], sizeof(idx.name) - 1);
    idx.dims = dims[i];
    for (size_t d = 0; d < dims[i]; ++d) idx.shape[d] = shapes[(size_t)i * 8 + d];
    idx.eleWidth = ele_width;
    idx.aligned = 64;
    arr.addMemRefIndexer(idx, data[i]);
  }
  return arr.write(path) ? 0 : 1;
}

// Read a container with the reference's reader; copies out the total element count and up to
// `cap` bytes of the blob the wrapped rank-1 descriptor points at.
int ref_flat_array_read(const char* path, size_t ele_width, long* total_elems, void* out,
                        size_t cap) {
  auto* arr = new MemRefFlatArray(ele_width == 2 ? dataType::kFloat16 : dataType::kFloat32);
  if (!arr->read(path)) return 1;  // (the reference's destructor frees an uninitialised
                                   //  pointer when read() fails early, so `arr` is leaked)
  if (ele_width == 2) {
    auto* d = arr->getWrapedData<MemRefDescriptor<nncvFloat16, 1>>();
    *total_elems = d->sizes[0];
    std::memcpy(out, d->aligned, std::min(cap, (size_t)d->sizes[0] * 2));
  } else {
    auto* d = arr->getWrapedData<MemRefDescriptor<nncvFloat32, 1>>();
    *total_elems = d->sizes[0];
    std::memcpy(out, d->aligned, std::min(cap, (size_t)d->sizes[0] * 4));
  }
  delete arr;
  return 0;
}

size_t ref_sizeof_head() { return sizeof(MemRefMagicHead); }
size_t ref_sizeof_indexer() { return sizeof(MemRefIndexer); }
size_t ref_sizeof_desc1() { return sizeof(MemRefDescriptor<float, 1>); }
size_t ref_sizeof_desc2() { return sizeof(MemRefDescriptor<float, 2>); }
size_t ref_sizeof_desc4() { return sizeof(MemRefDescriptor<float, 4>); }
}
