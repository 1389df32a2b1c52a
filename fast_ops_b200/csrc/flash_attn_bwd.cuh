// Attention backward for sm_100a: dQ, dK, dV from dO, Q, K, V and the forward's LSE.
//
// The reference's CUDA path has no backward (fast_ops/flash_attention/flash_attention.py:41-45
// raises); the semantics follow its complete implementation
// (fast_ops/flash_attention/flash_attention_triton.py:273-315 for delta = rowsum(O o dO),
// :322-638 for the main loop): one CTA owns a 128-key tile, keeps dK and dV for it in tensor
// memory, walks the query tiles that see those keys, and adds its share of dQ into an fp32
// buffer (the reference uses scalar atomics, :610; here each tile goes through shared memory and
// tiled bulk reduce-adds, cp.reduce.async.bulk.tensor).
//
// The scores are held transposed (key rows in the tensor-memory lanes, query columns).  With
// query rows in the lanes, P and dS would both have to go through shared memory to be transposed
// for dV += P^T dO and dK += dS^T Q, and the shared-memory port (128 bytes per clock for
// tensor-core operands, thread stores and bulk copies together) would carry about 576 KB per query
// tile at head_dim 128: 4600 cycles against 2560 of arithmetic.  Per query tile, five tcgen05
// MMAs (all fp32 accumulation in tensor memory):
//   S^T  = K Q^T          (K, Q K-major from shared memory; key rows in the lanes)
//   dP^T = V dO^T         (V, dO K-major)
//   -- threads: P^T = exp2(S^T*scale - LSE[query]), written over S^T in tensor memory as 16-bit;
//      dS^T = P^T o (dP^T - delta[query]) * scale, written over dP^T in tensor memory as 16-bit
//      and to shared memory as a [key row][query] tile --
//   dV += P^T dO          (P^T read from tensor memory, dO as the N-major B operand)
//   dK += dS^T Q          (dS^T read from tensor memory, Q N-major)
//   dQ  = dS K            (dS^T tile of shared memory as the M-major A operand, K N-major)
// so P never touches shared memory and two of the five matmuls read one operand from tensor memory.
// dQ is written over dP^T / dS^T (not over S^T), and Q has two shared-memory slots, so the S^T
// matmul of the next query tile is issued right behind this tile's dV matmul: the exponentials of
// tile i+1 run while the tensor core does dK and dQ of tile i, and only dP^T of tile i+1 waits for
// dQ of tile i to leave tensor memory.  Matmuls that overwrite tensor-memory columns an earlier
// matmul reads (S^T of the next tile over P^T, dQ over dS^T) rely on the tensor core executing one
// thread's tcgen05.mma in issue order.
//
// Warps 0-7: two threads per key row, each taking 64 of the tile's 128 query columns; in the
// epilogue one thread per key row for dK (warps 0-3) and dV (warps 4-7).  Warps 8-11: one thread
// per query row takes dQ out of tensor memory (all of it at once, so the columns are free again
// after one load), then stages it 64 columns at a time in a 32 KB area of its own and adds it into
// the fp32 buffer with tiled bulk reductions (cp.reduce.async.bulk.tensor).  Warp 12 issues the
// MMAs, warp 13 the TMA loads, warp 14 brings LSE and delta of the next query tile into shared
// memory (they vary along the columns, so every thread needs all 128 of them).
#pragma once

#include "flash_attn_common.cuh"
#include "fo_host.h"

namespace fo {

struct AttnBwdParams {
  const float* lse;    // (B, H, Sq) natural-log LSE of the forward
  const float* delta;  // (B, H, Sq) rowsum(O o dO)
  float* dq_accum;     // (B, H, Sq, D) fp32, zeroed before the launch
  void* dk;
  void* dv;
  int64_t dk_stride_b, dk_stride_h, dk_stride_s;
  int64_t dv_stride_b, dv_stride_h, dv_stride_s;
  int B, H, Sq, Sk;
  int d_real;  // head_dim of the tensors (<= the kernel's D; the missing columns are zero-filled by TMA)
  int causal;
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  int* device_status;
  unsigned long long* trace;  // optional timeline of CTA (0,0) (debug), or null
  int device;  // device index of the launch (host side only)
  AttnExtras ex;  // bias / dropout of the forward; read only by the kernel variants built for them
};

__device__ __forceinline__ void bwd_trace(const AttnBwdParams& prm, int role, int it, int ev) {
#if FO_ATTN_TRACE
  if (prm.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && it < kTraceIters)
    prm.trace[(role * kTraceIters + it) * kTraceEvents + ev] = clock64();
#else
  (void)prm; (void)role; (void)it; (void)ev;
#endif
}

// Writes 8 consecutive 16-bit values (one 16-byte unit) of row `r`, unit `u` (0..15 over 128
// columns) of a [128 x 128] tile stored as two [128 x 64] boxes with the 128-byte swizzle.
__device__ __forceinline__ void store_swizzled_unit(uint8_t* tile, int r, int u, uint4 v) {
  const int box = u >> 3;
  const int slot = (u & 7) ^ (r & 7);
  *reinterpret_cast<uint4*>(tile + box * kBoxBytes + r * 128 + slot * 16) = v;
}


template <int D>
struct BwdConfig {
  static constexpr int kTileBytes = kBlockM * D * 2;      // Q, dO, K, V tiles
  static constexpr int kDSBytes = kBlockN * kBlockM * 2;  // dS^T: [128 key rows][128 queries] 16-bit
  static constexpr int kStageBytes = kBlockM * 64 * 4;    // dQ, 64 columns at a time: two swizzled boxes of [128 rows][32 floats]
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTileBytes;
  static constexpr int kOffQ = 2 * kTileBytes;  // two slots
  static constexpr int kOffDO = 4 * kTileBytes;
  static constexpr int kOffDS = 5 * kTileBytes;
  static constexpr int kOffStage = kOffDS + kDSBytes;
  static constexpr int kOffBars = kOffStage + kStageBytes;
  static constexpr int kNumBars = 15;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  // [128] float each: -LSE*log2(e) and -delta*scale of the query tile; read as float4
  static constexpr int kOffNegLse = (kOffMisc + 64 + 15) & ~15;
  static constexpr int kOffNegDelta = kOffNegLse + 128 * 4;
  static constexpr int kSmemBytes = kOffNegDelta + 128 * 4 + 1024;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColDK = 0, kColDV = D, kColS = 256, kColDP = 384;  // dQ reuses kColDP
  static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

template <int N> __device__ __forceinline__ void tma_store_wait_read_n() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// grid = (key tiles, B*H); block = 512.
template <int D, bool kBf16, int kExt>
__global__ void __launch_bounds__(512, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_dq, const AttnBwdParams prm) {
  using Cfg = BwdConfig<D>;
  constexpr int kTileBytes = Cfg::kTileBytes;
  constexpr int kBoxes = D / kBoxCols;
  constexpr int kHalves = D / 64;  // dQ is staged in pieces of 64 columns (two boxes of 32 floats)

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem + Cfg::kOffK;
  uint8_t* sV = smem + Cfg::kOffV;
  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sDO = smem + Cfg::kOffDO;
  uint8_t* sDS = smem + Cfg::kOffDS;
  uint8_t* sStage = smem + Cfg::kOffStage;
  float* sNegLse = reinterpret_cast<float*>(smem + Cfg::kOffNegLse);
  float* sNegDelta = reinterpret_cast<float*>(smem + Cfg::kOffNegDelta);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* bar_kv = bars + 0;        // TMA -> MMA: K and V of this CTA are in shared memory
  uint64_t* bar_q_full = bars + 1;    // [2] TMA -> MMA: Q_i loaded into slot i % 2
  uint64_t* bar_q_empty = bars + 3;   // [2] MMA -> TMA: the matmuls reading that slot (S^T, dK) have completed
  uint64_t* bar_do_full = bars + 5;   // TMA -> MMA: dO_i loaded
  uint64_t* bar_do_empty = bars + 6;  // MMA -> TMA: the matmuls reading dO_i (dP^T, dV) have completed
  uint64_t* bar_s_full = bars + 7;    // MMA -> threads: S^T is in tensor memory
  uint64_t* bar_dp_full = bars + 8;   // MMA -> threads: dP^T is in tensor memory
  uint64_t* bar_p_full = bars + 9;    // threads -> MMA: P^T is in tensor memory (256 arrivals)
  uint64_t* bar_ds_full = bars + 10;  // threads -> MMA, row loader: dS^T is in tensor and shared memory (256 arrivals)
  uint64_t* bar_dq_full = bars + 11;  // MMA -> dQ warps: dQ tile (and dK, dV so far) complete
  uint64_t* bar_dp_free = bars + 12;  // dQ warps -> MMA: dQ read, the dP^T columns are reusable (128 arrivals)
  uint64_t* bar_lse_full = bars + 13;    // row loader -> threads: -LSE of the query tile's rows is in shared memory
  uint64_t* bar_delta_full = bars + 14;  // row loader -> threads: -delta of the query tile's rows is in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip = cta_abort + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int j = blockIdx.x;  // key tile
  const int bh = blockIdx.y;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int k0 = j * kBlockN;
  const int n_q_tiles = (prm.Sq + kBlockM - 1) / kBlockM;
  // query tiles that see this key tile: all of them, or with a causal mask those whose last
  // row is not above the tile's first key
  const int i0 = prm.causal ? min(j, n_q_tiles) : 0;
  const int n_iter = n_q_tiles - i0;
  int* const dstat = prm.device_status;

  if (tid == 0) {
    *cta_abort = 0;
    *skip = *reinterpret_cast<volatile int*>(prm.device_status);
    mbar_init(bar_kv, 1);
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar_q_full + x, 1);
      mbar_init(bar_q_empty + x, 1);
    }
    mbar_init(bar_do_full, 1);
    mbar_init(bar_do_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_p_full, 256);
    mbar_init(bar_ds_full, 256);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dp_free, 128);
    mbar_init(bar_lse_full, 1);
    mbar_init(bar_delta_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_do);
    prefetch_tensormap(&tm_dq);
  }
  __syncthreads();
  if (*skip) return;
  // K, V and the first Q / dO need only the barriers: requested here, under the tensor-memory allocation
  if (warp == 13 && lane == 0) {
    mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
    for (int c = 0; c < kBoxes; ++c) tma_load_4d(sK + c * kBoxBytes, &tm_k, bar_kv, c * kBoxCols, k0, h, b);
    for (int c = 0; c < kBoxes; ++c) tma_load_4d(sV + c * kBoxBytes, &tm_v, bar_kv, c * kBoxCols, k0, h, b);
    for (int t = 0; t < min(n_iter, 2); ++t) {
      mbar_arrive_expect_tx(bar_q_full + t, kTileBytes);
      for (int c = 0; c < kBoxes; ++c)
        tma_load_4d(sQ + t * kTileBytes + c * kBoxBytes, &tm_q, bar_q_full + t, c * kBoxCols, (i0 + t) * kBlockM, h, b);
    }
    if (n_iter > 0) {
      mbar_arrive_expect_tx(bar_do_full, kTileBytes);
      for (int c = 0; c < kBoxes; ++c) tma_load_4d(sDO + c * kBoxBytes, &tm_do, bar_do_full, c * kBoxCols, i0 * kBlockM, h, b);
    }
  }
  if (warp == 12) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // ================================ compute threads ================================
    reg_alloc<152>();
    const int r = (warp & 3) * 32 + lane;  // key row of the tile (tensor-memory lane)
    const int half = warp >> 2;            // which 64 query columns this thread takes
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // this thread's 64 fp32 columns of S^T / dP^T; its 16-bit results go over the first 32 of them
    const uint32_t tS = tmem_base + Cfg::kColS + lane_base + half * 64;
    const uint32_t tDP = tmem_base + Cfg::kColDP + lane_base + half * 64;
    constexpr bool has_bias = (kExt & 1) != 0;
    constexpr bool has_drop = (kExt & 2) != 0;
    // with dropout dP arrives without the 1 / (1 - p) factor of the kept elements
    const float dp_scale = kExt ? prm.scale * prm.ex.drop_rescale : prm.scale;
    const int key = k0 + r;
    const bool key_ok = key < prm.Sk;
    // A bias that is the same for every query row depends only on this thread's key: one register.
    const bool vec_bias = has_bias && prm.ex.bias_stride_q == 0;
    float bias_key = 0.f;
    const uint8_t* bias_bh = nullptr;
    if constexpr (kExt) {
      if (has_bias) {
        bias_bh = static_cast<const uint8_t*>(prm.ex.bias) +
                  (b * prm.ex.bias_stride_b + h * prm.ex.bias_stride_h) * (prm.ex.bias_f32 ? 4 : 2);
        if (vec_bias && key_ok) bias_key = load_bias1<kBf16>(prm.ex, bias_bh, key);
      }
    }
    for (int it = 0; it < n_iter; ++it) {
      const int i = i0 + it;
      const int q0 = i * kBlockM;
      const int qc0 = q0 + half * 64;  // first query of this thread's columns
      // masks are rare (diagonal tiles, a ragged last key tile); rows past Sq have -LSE = -inf
      const bool need_mask = !key_ok || (prm.causal && k0 + kBlockN - 1 > q0);
      mbar_wait(bar_lse_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
      mbar_wait(bar_s_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      if (warp == 0) bwd_trace(prm, 0, it, 0);
      // ---- P^T = exp2(S^T * scale - LSE) of this thread's 64 columns, fp32 in registers; the dP^T matmul runs meanwhile ----
      uint32_t sr[2][32];
      tmem_ld32(tS, sr[0]);
      tmem_ld32(tS + 32, sr[1]);
      uint32_t keep[2] = {0xffffffffu, 0xffffffffu};  // dropout: bit x of keep[cc] = element kept
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const float* nl = sNegLse + half * 64 + cc * 32;
        tmem_ld_wait(sr[cc]);
        if constexpr (has_bias) {
          if (vec_bias) {
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
              const float4 t = *reinterpret_cast<const float4*>(nl + x);  // broadcast read
              sr[cc][x + 0] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 0]), prm.scale_log2, bias_key) + t.x));
              sr[cc][x + 1] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 1]), prm.scale_log2, bias_key) + t.y));
              sr[cc][x + 2] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 2]), prm.scale_log2, bias_key) + t.z));
              sr[cc][x + 3] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 3]), prm.scale_log2, bias_key) + t.w));
            }
          } else {
            // matrix bias: element (query, key) of a row-major matrix; consecutive lanes read consecutive keys
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              const int q = qc0 + cc * 32 + x;
              float bv = 0.f;
              if (key_ok && q < prm.Sq)
                bv = load_bias1<kBf16>(prm.ex, bias_bh + static_cast<int64_t>(q) * prm.ex.bias_stride_q * (prm.ex.bias_f32 ? 4 : 2), key);
              sr[cc][x] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x]), prm.scale_log2, bv) + nl[x]));
            }
          }
        } else {
#pragma unroll
          for (int x = 0; x < 32; x += 4) {
            const float4 t = *reinterpret_cast<const float4*>(nl + x);  // broadcast read
            sr[cc][x + 0] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 0]), prm.scale_log2, t.x)));
            sr[cc][x + 1] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 1]), prm.scale_log2, t.y)));
            sr[cc][x + 2] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 2]), prm.scale_log2, t.z)));
            sr[cc][x + 3] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 3]), prm.scale_log2, t.w)));
          }
        }
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const int q = qc0 + cc * 32 + x;
            if (!key_ok || (prm.causal && key > q)) sr[cc][x] = 0u;
          }
        }
        if constexpr (has_drop) {
          uint32_t kb = 0;
          const uint32_t base = prm.ex.drop_base + static_cast<uint32_t>(bh) * static_cast<uint32_t>(prm.Sq) * static_cast<uint32_t>(prm.Sk) +
                                static_cast<uint32_t>(key);
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const uint32_t idx = base + static_cast<uint32_t>(qc0 + cc * 32 + x) * static_cast<uint32_t>(prm.Sk);
            if (dropout_hash(idx, prm.ex.drop_seed) > prm.ex.drop_threshold) kb |= 1u << x;
          }
          keep[cc] = kb;
        }
      }
      if (warp == 0) bwd_trace(prm, 0, it, 4);
      // ---- P^T (zero where the forward dropped the element), 16-bit, over the first 32 of this thread's S^T columns ----
      {
        uint32_t pp[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float z0 = __uint_as_float(sr[cc][x]), z1 = __uint_as_float(sr[cc][x + 1]);
            if constexpr (has_drop) {
              if (!((keep[cc] >> x) & 1u)) z0 = 0.f;
              if (!((keep[cc] >> (x + 1)) & 1u)) z1 = 0.f;
            }
            pp[cc * 16 + (x >> 1)] = pack2<kBf16>(z0, z1);
          }
        }
        tmem_st32(tS, pp);
      }
      tcgen05_wait_st();
      tcgen05_fence_before_sync();
      mbar_arrive(bar_p_full);  // the dV matmul may start
      if (warp == 0) bwd_trace(prm, 0, it, 5);

      // ---- dS^T = P^T o (dP^T - delta) * scale, dP = 0 for a dropped element ----
      mbar_wait(bar_delta_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
      mbar_wait(bar_dp_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      {
        uint32_t dd[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const float* nd = sNegDelta + half * 64 + cc * 32;
          uint32_t dpr[32];
          tmem_ld32(tDP + cc * 32, dpr);
          tmem_ld_wait(dpr);
#pragma unroll
          for (int x = 0; x < 32; x += 4) {
            const float4 t = *reinterpret_cast<const float4*>(nd + x);  // broadcast read
            const float ndv[4] = {t.x, t.y, t.z, t.w};
            float dsv[4];
#pragma unroll
            for (int y = 0; y < 4; ++y) {
              float g = __uint_as_float(dpr[x + y]);
              if constexpr (has_drop) {
                if (!((keep[cc] >> (x + y)) & 1u)) g = 0.f;
              }
              dsv[y] = __uint_as_float(sr[cc][x + y]) * fmaf(g, dp_scale, ndv[y]);
            }
            dd[cc * 16 + (x >> 1)] = pack2<kBf16>(dsv[0], dsv[1]);
            dd[cc * 16 + (x >> 1) + 1] = pack2<kBf16>(dsv[2], dsv[3]);
          }
        }
        // The shared-memory tile was last read by the dQ matmul of the previous query tile, which
        // completed before this tile's dP^T matmul was issued (the MMA warp waits for the dQ warps,
        // who wait for that matmul), so it may be overwritten here.
        tmem_st32(tDP, dd);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          store_swizzled_unit(sDS, r, half * 8 + u, make_uint4(dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]));
      }
      tcgen05_wait_st();
      fence_proxy_async_smem();  // shared-memory writes of these threads must be visible to the tensor core's reads
      tcgen05_fence_before_sync();
      mbar_arrive(bar_ds_full);
      if (warp == 0) bwd_trace(prm, 0, it, 1);
    }

    // ---- epilogue: key row (k0 + r); warps 0-3 write dK, warps 4-7 write dV ----
    uint16_t* dk_row = static_cast<uint16_t*>(prm.dk) + b * prm.dk_stride_b + h * prm.dk_stride_h +
                       static_cast<int64_t>(key) * prm.dk_stride_s;
    uint16_t* dv_row = static_cast<uint16_t*>(prm.dv) + b * prm.dv_stride_b + h * prm.dv_stride_h +
                       static_cast<int64_t>(key) * prm.dv_stride_s;
    if (n_iter > 0) {
      mbar_wait(bar_dq_full, (n_iter - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);  // every matmul has completed
      tcgen05_fence_after_sync();
    }
    {
      const int which = half;
      const uint32_t tAcc = tmem_base + (which ? Cfg::kColDV : Cfg::kColDK) + lane_base;
      uint16_t* out_row = which ? dv_row : dk_row;
      // dV was accumulated from the kept P without the dropout factor
      const float out_scale = (kExt && which) ? prm.ex.drop_rescale : 1.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ar[32];
        if (n_iter > 0) {
          tmem_ld32(tAcc + c * 32, ar);
          tmem_ld_wait(ar);
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) ar[x] = 0;  // no query tile sees these keys
        }
        if (key_ok) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 v;
            if constexpr (kExt != 0) {
#pragma unroll
              for (int y = 0; y < 8; ++y) ar[x + y] = __float_as_uint(__uint_as_float(ar[x + y]) * out_scale);
            }
            v.x = pack2<kBf16>(__uint_as_float(ar[x + 0]), __uint_as_float(ar[x + 1]));
            v.y = pack2<kBf16>(__uint_as_float(ar[x + 2]), __uint_as_float(ar[x + 3]));
            v.z = pack2<kBf16>(__uint_as_float(ar[x + 4]), __uint_as_float(ar[x + 5]));
            v.w = pack2<kBf16>(__uint_as_float(ar[x + 6]), __uint_as_float(ar[x + 7]));
            if (c * 32 + x < prm.d_real) *reinterpret_cast<uint4*>(out_row + c * 32 + x) = v;
          }
        }
      }
    }
  } else if (warp < 12) {
    // ================================ dQ warps ================================
    // Query row r of the tile: all of its dQ out of tensor memory, which frees the columns for the
    // next tile's dP^T; then 64 columns at a time through the staging area (two swizzled boxes of
    // [128 rows x 32 floats]) into the fp32 accumulation buffer with tiled bulk reductions (rows
    // past Sq are dropped by the hardware).  One thread issues every reduction, so the bulk groups
    // it waits for are its own.
    reg_alloc<152>();
    const int r = (warp & 3) * 32 + lane;
    const uint32_t tQ = tmem_base + Cfg::kColDP + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const bool issuer = tid == 8 * 32;
    for (int it = 0; it < n_iter; ++it) {
      const int q0 = (i0 + it) * kBlockM;
      mbar_wait(bar_dq_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      if (warp == 8) bwd_trace(prm, 1, it, 0);
      uint32_t qr[D / 32][32];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld32(tQ + c * 32, qr[c]);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_wait(qr[c]);
      tcgen05_fence_before_sync();
      mbar_arrive(bar_dp_free);  // the next query tile's dP^T may be written
      if (warp == 8) bwd_trace(prm, 1, it, 1);
#pragma unroll
      for (int hh = 0; hh < kHalves; ++hh) {
        // the reduction that last read the staging area must have finished reading
        if (issuer) tma_store_wait_read();
        named_barrier_sync(1, 128);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint8_t* box = sStage + cc * kBoxBytes;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(box + r * 128 + ((u ^ (r & 7)) * 16)) =
                make_uint4(qr[hh * 2 + cc][4 * u], qr[hh * 2 + cc][4 * u + 1], qr[hh * 2 + cc][4 * u + 2], qr[hh * 2 + cc][4 * u + 3]);
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (issuer) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = hh * 2 + cc;
            if (c * 32 < prm.d_real) tma_reduce_add_3d(&tm_dq, sStage + cc * kBoxBytes, c * 32, q0, bh);
          }
          tma_store_commit();
        }
      }
      if (warp == 8) bwd_trace(prm, 1, it, 2);
    }
    if (issuer) tma_store_wait_all();  // the reductions must have landed before the CTA ends
  } else {
    reg_dealloc<56>();
    if (warp == 12) {
      // ================================ MMA issuer ================================
      constexpr uint32_t idesc_s = make_idesc(kBf16, kBlockN, kBlockM, 0, 0);  // S^T, dP^T: both K-major
      constexpr uint32_t idesc_a = make_idesc(kBf16, kBlockN, D, 0, 1);        // dV, dK: A from tensor memory, B N-major
      constexpr uint32_t idesc_q = make_idesc(kBf16, kBlockM, D, 1, 1);        // dQ: A M-major, B N-major
      constexpr uint32_t kBoxStep = kBoxBytes >> 4;
      const uint32_t q_k = desc_lo(smem_u32(sQ), 16), do_k = desc_lo(smem_u32(sDO), 16);
      const uint32_t k_k = desc_lo(smem_u32(sK), 16), v_k = desc_lo(smem_u32(sV), 16);
      const uint32_t q_n = desc_lo(smem_u32(sQ), kBoxBytes), do_n = desc_lo(smem_u32(sDO), kBoxBytes);
      const uint32_t k_n = desc_lo(smem_u32(sK), kBoxBytes);
      const uint32_t ds_m = desc_lo(smem_u32(sDS), kBoxBytes);
      const uint32_t tDK = tmem_base + Cfg::kColDK, tDV = tmem_base + Cfg::kColDV;
      const uint32_t tS = tmem_base + Cfg::kColS, tDP = tmem_base + Cfg::kColDP;

      auto issue_st = [&](int t) {  // S^T = K Q^T of query tile t  (K = head_dim)
        mbar_wait(bar_q_full + (t & 1), (t >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        tcgen05_fence_after_sync();
        const uint32_t qs = q_k + (t & 1) * (kTileBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
          umma_ss_lo_elect(tS, k_k + off, qs + off, idesc_s, kk > 0 ? 1u : 0u);
        }
        tcgen05_commit_elect(bar_s_full);
      };
      auto issue_dpt = [&](int t) {  // dP^T = V dO^T of query tile t
        mbar_wait(bar_do_full, t & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        tcgen05_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
          umma_ss_lo_elect(tDP, v_k + off, do_k + off, idesc_s, kk > 0 ? 1u : 0u);
        }
        tcgen05_commit_elect(bar_dp_full);
      };
      mbar_wait(bar_kv, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
      if (n_iter > 0) {
        issue_st(0);
        issue_dpt(0);
      }
      for (int it = 0; it < n_iter; ++it) {
        bwd_trace(prm, 2, it, 0);
        // 16 queries per step; the two column halves' 16-bit results sit at columns 0-31 and 64-95
        mbar_wait(bar_p_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        tcgen05_fence_after_sync();
        bwd_trace(prm, 2, it, 1);
#pragma unroll
        for (int kk = 0; kk < kBlockM / 16; ++kk)  // dV += P^T dO
          umma_ts_lo_elect(tDV, tS + (kk >> 2) * 64 + (kk & 3) * 8, do_n + kk * 128, idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
        tcgen05_commit_elect(bar_do_empty);  // dO_i has no reader after this point
        if (it + 1 < n_iter) issue_st(it + 1);  // over P^T, behind the matmul that reads it
        mbar_wait(bar_ds_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        tcgen05_fence_after_sync();
        bwd_trace(prm, 2, it, 2);
        const uint32_t qn = q_n + (it & 1) * (kTileBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kBlockM / 16; ++kk)  // dK += dS^T Q
          umma_ts_lo_elect(tDK, tDP + (kk >> 2) * 64 + (kk & 3) * 8, qn + kk * 128, idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
        tcgen05_commit_elect(bar_q_empty + (it & 1));  // this Q slot has no reader after this point
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk)  // dQ = dS K  (K = 16 keys per step), over dS^T, behind the matmul that reads it
          umma_ss_lo_elect(tDP, ds_m + kk * 128, k_n + kk * 128, idesc_q, kk > 0 ? 1u : 0u);
        tcgen05_commit_elect(bar_dq_full);
        bwd_trace(prm, 2, it, 3);
        if (it + 1 < n_iter) {
          mbar_wait(bar_dp_free, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
          issue_dpt(it + 1);
        }
      }
    } else if (warp == 13) {
      // ================================ TMA producer ================================
      const bool issuer = lane == 0;
      for (int it = 1; it < n_iter; ++it) {  // Q of tiles 0 and 1 and dO of tile 0 went out before the allocation
        const int q0 = (i0 + it) * kBlockM;
        if (it >= 2) {
          mbar_wait(bar_q_empty + (it & 1), ((it >> 1) - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
          if (issuer) {
            mbar_arrive_expect_tx(bar_q_full + (it & 1), kTileBytes);
            for (int c = 0; c < kBoxes; ++c)
              tma_load_4d(sQ + (it & 1) * kTileBytes + c * kBoxBytes, &tm_q, bar_q_full + (it & 1), c * kBoxCols, q0, h, b);
          }
        }
        mbar_wait(bar_do_empty, (it - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
        if (issuer) {
          mbar_arrive_expect_tx(bar_do_full, kTileBytes);
          for (int c = 0; c < kBoxes; ++c) tma_load_4d(sDO + c * kBoxBytes, &tm_do, bar_do_full, c * kBoxCols, q0, h, b);
        }
        __syncwarp();
      }
      if (n_iter == 0) mbar_wait(bar_kv, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);  // drain the K/V load before exit
    } else if (warp == 14) {
      // ================================ row loader ================================
      // -LSE * log2(e) and -delta * scale of the query tile's 128 rows, four per lane.  A row past
      // the end, or one whose keys are all masked (LSE = -inf), gets -inf, so that its P and dS are 0.
      const float* const lse_bh = prm.lse + static_cast<int64_t>(bh) * prm.Sq;
      const float* const delta_bh = prm.delta + static_cast<int64_t>(bh) * prm.Sq;
      for (int it = 0; it < n_iter; ++it) {
        const int row0 = (i0 + it) * kBlockM + lane * 4;
        float nl[4], nd[4];
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          const bool ok = row0 + y < prm.Sq;
          const float l = ok ? lse_bh[row0 + y] : -INFINITY;
          nl[y] = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
          nd[y] = ok ? -delta_bh[row0 + y] * prm.scale : 0.f;
        }
        // -LSE is read during the exponentials (until P^T is complete), -delta until dS^T is complete
        if (it > 0) mbar_wait(bar_p_full, (it - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        *reinterpret_cast<float4*>(sNegLse + lane * 4) = make_float4(nl[0], nl[1], nl[2], nl[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_lse_full);
        if (it > 0) mbar_wait(bar_ds_full, (it - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        *reinterpret_cast<float4*>(sNegDelta + lane * 4) = make_float4(nd[0], nd[1], nd[2], nd[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_delta_full);
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fo
