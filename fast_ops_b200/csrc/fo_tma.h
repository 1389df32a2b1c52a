// Host-side construction of the TMA tensor maps used by the attention kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "flash_attn_common.cuh"
#include "fo_host.h"

namespace fo {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled comes from the driver; resolving it through the runtime avoids
// linking against libcuda.
inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map over a (B, H, S, D) tensor with element strides (sb, sh, ss, 1): dimensions are
// listed innermost first, the box is one [box_rows x 64 columns] swizzled tile (128 rows, or 64
// for the half tiles of the short-sequence kernel), and reads past S are filled with zeros.
inline int encode_tensor_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int S, int D,
                             const int64_t strides[3], const char* name, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fo::fail(FO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  FO_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "%s must be 16-byte aligned", name);
  // A dimension of extent 1 never uses its stride; give it a harmless one.
  int64_t sb = B > 1 ? strides[0] : static_cast<int64_t>(H) * S * D;
  int64_t sh = H > 1 ? strides[1] : static_cast<int64_t>(S) * D;
  int64_t ss = S > 1 ? strides[2] : D;
  FO_REQUIRE(sb > 0 && sh > 0 && ss >= D, "%s: strides must be positive and rows must not overlap", name);
  FO_REQUIRE(sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0, "%s: strides must be multiples of 8 elements", name);
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t gstrides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh) * 2,
                                  static_cast<cuuint64_t>(sb) * 2};
  const cuuint32_t box[4] = {kBoxCols, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == FO_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, gstrides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fo::fail(FO_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", name, (int)r);
  return FO_OK;
}

// The same through a small per-thread cache: a tensor map depends only on the base address, the
// element type and the geometry, never on the tensor's contents, and a training or serving loop
// presents the same few (address, shape, strides) combinations call after call.  A hit costs a
// scan of at most kTensorMapCacheSize keys instead of a driver call.
constexpr int kTensorMapCacheSize = 16;

struct TensorMapKey {
  const void* base;
  int64_t strides[3];
  int dtype, B, H, S, D, box_rows;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && strides[0] == o.strides[0] && strides[1] == o.strides[1] && strides[2] == o.strides[2] &&
           dtype == o.dtype && B == o.B && H == o.H && S == o.S && D == o.D && box_rows == o.box_rows;
  }
};

struct TensorMapCache {
  TensorMapKey keys[kTensorMapCacheSize];
  alignas(64) CUtensorMap maps[kTensorMapCacheSize];
  int used = 0, next = 0;  // entries in use; slot the next miss overwrites (round robin)
};

inline int make_tensor_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int S, int D,
                           const int64_t strides[3], const char* name, int box_rows = kBlockN) {
  thread_local TensorMapCache cache;
  const TensorMapKey key{base, {strides[0], strides[1], strides[2]}, dtype, B, H, S, D, box_rows};
  for (int i = 0; i < cache.used; ++i)
    if (cache.keys[i] == key) {
      *map = cache.maps[i];
      return FO_OK;
    }
  if (int rc = encode_tensor_map(map, base, dtype, B, H, S, D, strides, name, box_rows)) return rc;
  const int slot = cache.next;
  cache.keys[slot] = key;
  cache.maps[slot] = *map;
  cache.next = (slot + 1) % kTensorMapCacheSize;
  if (cache.used < kTensorMapCacheSize) ++cache.used;
  return FO_OK;
}

// Tensor map over the fp32 dQ accumulation buffer (B*H, Sq, D), dense: box = 128 rows x 32
// floats (128 bytes, one swizzle span), used as the destination of tiled reduce-adds.
inline int make_dq_accum_map(CUtensorMap* map, float* base, int64_t BH, int Sq, int D) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fo::fail(FO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(Sq), static_cast<cuuint64_t>(BH)};
  const cuuint64_t gstrides[2] = {static_cast<cuuint64_t>(D) * 4, static_cast<cuuint64_t>(Sq) * D * 4};
  const cuuint32_t box[3] = {32, kBlockM, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, gstrides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fo::fail(FO_ERR_CUDA, "cuTensorMapEncodeTiled(dq_accum) failed with CUresult %d", (int)r);
  return FO_OK;
}

}  // namespace fo
