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

// Optional additive bias and dropout of the extended entry points (all zero: plain attention).
struct AttnExtras {
  const void* bias;  // null: none; element (b, h, i, j) at bias + b*stride_b + h*stride_h + i*stride_q + j
  int64_t bias_stride_b, bias_stride_h, bias_stride_q;  // elements; 0 along a broadcast dimension
  int bias_f32;   // 1: fp32 bias, 0: the 16-bit type of Q
  int bias_vec;   // 1: every bias row starts on a 16-byte boundary (vector loads allowed)
  int dropout;    // 1: dropout on
  uint32_t drop_threshold;  // an element is kept iff dropout_hash(index, seed) > threshold
  uint32_t drop_seed;
  uint32_t drop_base;       // low 32 bits of the generator offset
  float drop_rescale;       // 1 / (1 - p), or 1 when dropout is off
};

// Keep/drop decision of element `idx` (fast_ops/flash_attention/flash_attention_triton.py:38-50:
// an integer hash in place of a Philox draw; all arithmetic modulo 2^32).
__device__ __forceinline__ uint32_t dropout_hash(uint32_t idx, uint32_t seed) {
  uint32_t a = idx ^ seed;
  a ^= a >> 4;
  a = (a ^ 0xDEADBEEFu) + (a << 5);
  a ^= a >> 11;
  return a;
}

// out[i] = log2(e) * bias[col0 + i] for the 32 columns col0.. of one bias row (`rowp` points at
// column 0 of the row, or is null for a row past the end); columns >= Sk give 0.
template <bool kBf16>
__device__ __forceinline__ void load_bias32(const AttnExtras& ex, const uint8_t* rowp, int col0, int Sk,
                                            float (&out)[32]) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (rowp == nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = 0.f;
    return;
  }
  const bool full = ex.bias_vec && (col0 + 32 <= Sk);
  if (ex.bias_f32) {
    const float* p = reinterpret_cast<const float*>(rowp) + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p + i));
        out[i] = v.x * kLog2e; out[i + 1] = v.y * kLog2e; out[i + 2] = v.z * kLog2e; out[i + 3] = v.w * kLog2e;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = (col0 + i < Sk) ? __ldg(p + i) * kLog2e : 0.f;
    }
  } else {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(rowp) + col0;
    auto cvt = [](uint16_t h) -> float {
      if constexpr (kBf16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
      else return __half2float(__ushort_as_half(h));
    };
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p + i));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          out[i + 2 * t] = cvt(static_cast<uint16_t>(w[t] & 0xffffu)) * kLog2e;
          out[i + 2 * t + 1] = cvt(static_cast<uint16_t>(w[t] >> 16)) * kLog2e;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = (col0 + i < Sk) ? cvt(__ldg(p + i)) * kLog2e : 0.f;
    }
  }
}

struct AttnParams {
  void* o;
  float* lse;  // may be null
  int64_t o_stride_b, o_stride_h, o_stride_s;  // elements
  int B, H, Sq, Sk;
  // head_dim of the tensors; the kernels are built for 64 and 128, smaller multiples of 8 run in
  // the next larger one: TMA fills the missing columns of Q, K, V with zeros (they add nothing
  // to Q K^T and give zero columns of O), and only d_real columns are written back
  int d_real;
  int causal;
  float scale_log2;  // softmax_scale * log2(e)
  int* device_status;
  int num_q_tiles;
  int head_group;  // heads per scheduling group (>= 1)
  int kv_head_bcast;  // 1: K and V have one head shared by all query heads (multi-query attention)
  // Optional timeline of CTA 0 (debug): [role][key tile][event] SM clock values, or null.
  unsigned long long* trace;
  AttnExtras ex;  // read only by the kernel variants built for bias / dropout
  int ping_pong;  // 64-key-step kernel: the two query tiles take turns on the ex2 units (1) or not (0)
  int device;     // device index of the launch (host side only)
  int num_sms;    // multiprocessors of that device: the size of a persistent grid
  // Persistent kernels: two words in global memory, zero at launch, that the launch's CTAs use to
  // hand out work items ([0]) and to find the last CTA, which zeroes them again ([1]).
  int* sched;
};

// One element of a bias row as log2(e) * value; `base` points at column 0 of the row.
template <bool kBf16>
__device__ __forceinline__ float load_bias1(const AttnExtras& ex, const uint8_t* base, int col) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (ex.bias_f32) return __ldg(reinterpret_cast<const float*>(base) + col) * kLog2e;
  const uint16_t h = __ldg(reinterpret_cast<const uint16_t*>(base) + col);
  if constexpr (kBf16) return __uint_as_float(static_cast<uint32_t>(h) << 16) * kLog2e;
  else return __half2float(__ushort_as_half(h)) * kLog2e;
}

// L2 prefetch of the `ncols` bias elements of a row starting at column col0 (row pointer non-null,
// columns clamped to Sk by the caller).
__device__ __forceinline__ void prefetch_bias(const AttnExtras& ex, const uint8_t* rowp, int col0, int ncols) {
  const int esize = ex.bias_f32 ? 4 : 2;
  const uint8_t* p = rowp + static_cast<int64_t>(col0) * esize;
  for (int off = 0; off < ncols * esize; off += 128) prefetch_l2(p + off);
}

constexpr int kTraceRoles = 3;   // softmax tile 0, softmax tile 1, MMA issuer
constexpr int kTraceIters = 160;
constexpr int kTraceEvents = 6;

// The timeline hook is compiled in only with -DFO_ATTN_TRACE=1 (a tuning build): the test of
// prm.trace sits inside loops whose warps issue in order, so the default build carries none of it.
#ifndef FO_ATTN_TRACE
#define FO_ATTN_TRACE 0
#endif

__device__ __forceinline__ void trace_event(const AttnParams& prm, int role, int j, int ev) {
#if FO_ATTN_TRACE
  if (FO_ATTN_TRACE == 2 && (role == 2 || (ev != 0 && ev != 2))) return;  // light: softmax turn / exponentials done only
  if (prm.trace != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && j < kTraceIters)
    prm.trace[(role * kTraceIters + j) * kTraceEvents + ev] = clock64();
#else
  (void)prm; (void)role; (void)j; (void)ev;
#endif
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
