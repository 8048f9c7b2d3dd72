// Host side of TMA: encoding CUtensorMap objects without linking libcuda
// (the driver entry point is fetched through the runtime).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mvpa_common.cuh"

namespace mvpa {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A tensor map is a pure function of these arguments, and a model calls the operator with the same
// buffers layer after layer, step after step: a small per-thread table (direct-mapped on a hash of the
// arguments) returns the 128-byte object again instead of asking the driver to encode it.
struct TensorMapKey {
  const void* base;
  int rank;
  uint64_t dims[5], strides[4];
  uint32_t box[5];
};
inline bool same_key(const TensorMapKey& a, const TensorMapKey& b) {
  if (a.base != b.base || a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i) {
    if (a.dims[i] != b.dims[i] || a.box[i] != b.box[i]) return false;
    if (i > 0 && a.strides[i - 1] != b.strides[i - 1]) return false;
  }
  return true;
}
struct TensorMapSlot {
  TensorMapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTensorMapSlots = 64;

inline int encode_bf16_sw128_uncached(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                      const uint64_t* strides_bytes, const uint32_t* box);

// bf16 tensor of `rank` dims (dims[0] innermost, contiguous), byte strides for dims 1..rank-1,
// box of `box` elements, 128-byte swizzle, zero fill outside the tensor.
inline int encode_bf16_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes, const uint32_t* box) {
  static thread_local TensorMapSlot table[kTensorMapSlots] = {};
  TensorMapKey key = {};
  key.base = base;
  key.rank = rank;
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull + (uint64_t)rank;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
    h = (h ^ dims[i] ^ ((uint64_t)box[i] << 40) ^ (i > 0 ? strides_bytes[i - 1] << 7 : 0)) * 0x9E3779B97F4A7C15ull;
  }
  TensorMapSlot& slot = table[(h >> 32) % kTensorMapSlots];
  if (slot.used && same_key(slot.key, key)) {
    *map = slot.map;
    return MVPA_OK;
  }
  const int rc = encode_bf16_sw128_uncached(map, base, rank, dims, strides_bytes, box);
  if (rc == MVPA_OK) {
    slot.key = key;
    slot.map = *map;
    slot.used = true;
  }
  return rc;
}

inline int encode_bf16_sw128_uncached(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                      const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return MVPA_ERR_CUDA;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr,
                  bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu %llu %llu, box %u %u %u)",
              (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1],
              (unsigned long long)(rank > 2 ? dims[2] : 0), box[0], box[1], rank > 2 ? box[2] : 0);
    return MVPA_ERR_CUDA;
  }
  return MVPA_OK;
}

}  // namespace mvpa
