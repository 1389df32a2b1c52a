// Pieces shared by the attention kernels: tile geometry, kernel parameters, operand
// descriptors of the three tile kinds (Q, K as K-major; V as N-major) and small numeric helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fo_ptx.cuh"

namespace fo {

constexpr int kBlockM = 128;  // query rows per tile (one tensor-memory lane per row)
constexpr int kBlockN = 128;  // key/value rows per tile
constexpr int kBoxCols = 64;  // elements per TMA box row: 128 bytes, one swizzle span
constexpr int kBoxBytes = kBlockN * kBoxCols * 2;  // 16 KiB: a [128 x 64] 16-bit box

struct AttnParams {
  void* o;
  float* lse;  // may be null
  int64_t o_stride_b, o_stride_h, o_stride_s;  // elements
  int B, H, Sq, Sk;
  int causal;
  float scale_log2;  // softmax_scale * log2(e)
  int* device_status;
  int num_q_tiles;
  int head_group;  // heads per scheduling group (>= 1)
  int kv_head_bcast;  // 1: K and V have one head shared by all query heads (multi-query attention)
  // Optional timeline of CTA 0 (debug): [role][key tile][event] SM clock values, or null.
  unsigned long long* trace;
};

constexpr int kTraceRoles = 3;   // softmax tile 0, softmax tile 1, MMA issuer
constexpr int kTraceIters = 160;
constexpr int kTraceEvents = 6;

__device__ __forceinline__ void trace_event(const AttnParams& prm, int role, int j, int ev) {
  if (prm.trace != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && j < kTraceIters)
    prm.trace[(role * kTraceIters + j) * kTraceEvents + ev] = clock64();
}

// Descriptor of the kk-th K=16 slice of a K-major [128 x D] tile stored as D/64 boxes.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile_smem, int kk) {
  return smem_desc(tile_smem + (kk >> 2) * kBoxBytes + (kk & 3) * 32, 16, 1024);
}

// Descriptor of the kk-th K=16 slice (16 key rows) of V stored as D/64 boxes of [128 x 64]:
// N (head_dim) is the contiguous direction, consecutive 64-wide column blocks are kBoxBytes apart.
__device__ __forceinline__ uint64_t nmajor_desc(uint32_t tile_smem, int kk) {
  return smem_desc(tile_smem + kk * 2048, kBoxBytes, 1024);
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low 16 bits), .y = hi
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

}  // namespace fo
