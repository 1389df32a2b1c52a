// Attention backward for sm_100a: dQ, dK, dV from dO, Q, K, V and the forward's LSE.
//
// The reference's CUDA path has no backward (fast_ops/flash_attention/flash_attention.py:41-45
// raises); the semantics follow its complete implementation
// (fast_ops/flash_attention/flash_attention_triton.py:273-315 for delta = rowsum(O o dO),
// :322-638 for the main loop): one CTA owns a 128-key tile, keeps dK and dV for it in tensor
// memory, walks the query tiles that see those keys, and adds its share of dQ into an fp32
// buffer (the reference uses scalar atomics, :610; here each tile goes through shared memory and
// one tiled bulk reduce-add, cp.reduce.async.bulk.tensor).
//
// Per query tile, five tcgen05 MMAs (all fp32 accumulation in tensor memory):
//   S  = Q K^T          (Q, K K-major from shared memory)
//   dP = dO V^T         (dO, V K-major)
//   -- threads: P = exp2(S*scale - LSE), dS = P o (dP - delta) * scale, both written to shared
//      memory as 16-bit [query row][key] tiles in the 128-byte-swizzled layout --
//   dV += P^T dO        (P as the M-major A operand, dO as the N-major B operand)
//   dK += dS^T Q        (dS M-major A, Q N-major B)
//   dQ  = dS K          (dS K-major A, K N-major B), read back and reduce-added to the fp32 dQ buffer
//
// Warps 0-7: two threads per query row, each taking half of the tile's columns (no reduction
// across a row is needed in the backward), and in the epilogue one thread per key row for dK
// (warps 0-3) and dV (warps 4-7); warp 8 issues the MMAs; warp 9 issues the TMA loads.
//
// The hand-offs of one query tile are split so that each side works while the other does:
// S and dP are committed separately (the exponentials of S run under the dP matmul), P and dS are
// handed over separately (the dV matmul runs while dS is formed and stored), and the S / dP columns
// are released as soon as dQ sits in registers (the S matmul of the next tile runs while dQ is
// staged and reduced).  The load of the next Q / dO tile and the drain of the previous dQ reduction
// overlap the rest.
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

template <int D>
struct BwdConfig {
  static constexpr int kTileBytes = kBlockM * D * 2;  // Q, dO, K, V tiles
  static constexpr int kPBytes = kBlockM * kBlockN * 2;  // P and dS: [128 rows][128 keys] 16-bit
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTileBytes;
  static constexpr int kOffQ = 2 * kTileBytes;
  static constexpr int kOffDO = 3 * kTileBytes;
  static constexpr int kOffP = 4 * kTileBytes;
  static constexpr int kOffDS = kOffP + kPBytes;
  static constexpr int kOffBars = kOffDS + kPBytes;
  static constexpr int kNumBars = 9;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  // [128] float: a row-independent bias of this key tile; read as float4, so 16-byte aligned
  static constexpr int kOffBias = (kOffMisc + 64 + 15) & ~15;
  static constexpr int kSmemBytes = kOffBias + 128 * 4 + 1024;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColDK = 0, kColDV = D, kColS = 256, kColDP = 384;  // dQ reuses kColS
};

// Writes 8 consecutive 16-bit values (one 16-byte unit) of row `r`, unit `u` (0..15 over 128
// columns) of a [128 x 128] tile stored as two [128 x 64] boxes with the 128-byte swizzle.
__device__ __forceinline__ void store_swizzled_unit(uint8_t* tile, int r, int u, uint4 v) {
  const int box = u >> 3;
  const int slot = (u & 7) ^ (r & 7);
  *reinterpret_cast<uint4*>(tile + box * kBoxBytes + r * 128 + slot * 16) = v;
}

// grid = (key tiles, B*H); block = 320.
static_assert(BwdConfig<128>::kOffBias % 16 == 0 && BwdConfig<64>::kOffBias % 16 == 0, "float4 reads");

template <int D, bool kBf16, int kExt>
__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, const AttnBwdParams prm) {
  using Cfg = BwdConfig<D>;
  constexpr int kTileBytes = Cfg::kTileBytes;
  constexpr int kBoxes = D / kBoxCols;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem + Cfg::kOffK;
  uint8_t* sV = smem + Cfg::kOffV;
  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sDO = smem + Cfg::kOffDO;
  uint8_t* sP = smem + Cfg::kOffP;
  uint8_t* sDS = smem + Cfg::kOffDS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* bar_kv = bars + 0;        // TMA -> MMA: K and V of this CTA are in shared memory
  uint64_t* bar_q_full = bars + 1;    // TMA -> MMA: Q_i and dO_i loaded
  uint64_t* bar_q_empty = bars + 2;   // MMA -> TMA: every MMA reading Q_i / dO_i has completed
  uint64_t* bar_s_full = bars + 3;    // MMA -> threads: S is in tensor memory
  uint64_t* bar_dp_full = bars + 4;   // MMA -> threads: dP is in tensor memory
  uint64_t* bar_p_full = bars + 5;    // threads -> MMA: P is in shared memory (256 arrivals)
  uint64_t* bar_ds_full = bars + 6;   // threads -> MMA: dS is in shared memory, dP has been read (256 arrivals)
  uint64_t* bar_dq_full = bars + 7;   // MMA -> threads: dQ tile (and dK, dV so far) complete
  uint64_t* bar_s_free = bars + 8;    // threads -> MMA: dQ read, S / dP columns reusable (256 arrivals)
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
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_p_full, 256);
    mbar_init(bar_ds_full, 256);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_s_free, 256);
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_do);
    prefetch_tensormap(&tm_dq);
  }
  __syncthreads();
  if (*skip) return;
  // K, V and the first Q / dO need only the barriers: requested here, under the tensor-memory
  // allocation, instead of after it
  if (warp == 9 && lane == 0) {
    mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
    for (int c = 0; c < kBoxes; ++c) tma_load_4d(sK + c * kBoxBytes, &tm_k, bar_kv, c * kBoxCols, k0, h, b);
    for (int c = 0; c < kBoxes; ++c) tma_load_4d(sV + c * kBoxBytes, &tm_v, bar_kv, c * kBoxCols, k0, h, b);
    if (n_iter > 0) {
      const int q0 = i0 * kBlockM;
      mbar_arrive_expect_tx(bar_q_full, 2 * kTileBytes);
      for (int c = 0; c < kBoxes; ++c) tma_load_4d(sQ + c * kBoxBytes, &tm_q, bar_q_full, c * kBoxCols, q0, h, b);
      for (int c = 0; c < kBoxes; ++c) tma_load_4d(sDO + c * kBoxBytes, &tm_do, bar_q_full, c * kBoxCols, q0, h, b);
    }
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // ================================ compute threads ================================
    const int r = (warp & 3) * 32 + lane;  // row of the tile (tensor-memory lane)
    const int half = warp >> 2;            // which half of the columns this thread takes
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + Cfg::kColS + lane_base;
    const uint32_t tDP = tmem_base + Cfg::kColDP + lane_base;
    constexpr bool has_bias = (kExt & 1) != 0;
    constexpr bool has_drop = (kExt & 2) != 0;
    // with dropout dP arrives without the 1 / (1 - p) factor of the kept elements
    const float dp_scale = kExt ? prm.scale * prm.ex.drop_rescale : prm.scale;
    // A bias that is the same for every query row is the same for every query tile of this CTA
    // (its key tile is fixed): fetched once into shared memory.
    const bool vec_bias = has_bias && prm.ex.bias_stride_q == 0;
    float* sb = reinterpret_cast<float*>(smem + Cfg::kOffBias);
    if constexpr (kExt) {
      if (vec_bias) {
        if (tid < kBlockN) {
          const uint8_t* base = static_cast<const uint8_t*>(prm.ex.bias) +
                                (b * prm.ex.bias_stride_b + h * prm.ex.bias_stride_h) * (prm.ex.bias_f32 ? 4 : 2);
          sb[tid] = (k0 + tid < prm.Sk) ? load_bias1<kBf16>(prm.ex, base, k0 + tid) : 0.f;
        }
        named_barrier_sync(1, 256);
      }
    }
    // LSE and delta of a row are fetched one query tile ahead, so that their latency is not in the tile's chain
    const float* const lse_bh = prm.lse + static_cast<int64_t>(bh) * prm.Sq;
    const float* const delta_bh = prm.delta + static_cast<int64_t>(bh) * prm.Sq;
    float lse_next = INFINITY, delta_next = 0.f;
    if (n_iter > 0 && i0 * kBlockM + r < prm.Sq) {
      lse_next = lse_bh[i0 * kBlockM + r];
      delta_next = delta_bh[i0 * kBlockM + r];
    }
    for (int it = 0; it < n_iter; ++it) {
      const int i = i0 + it;
      const int q0 = i * kBlockM;
      const int row = q0 + r;
      const bool row_ok = row < prm.Sq;
      // a row past the end, or one whose keys are all masked (LSE = -inf), gets LSE = +inf, so
      // that its P and dS are exactly 0
      const float lse_nat = lse_next;
      const float delta = delta_next;
      if (it + 1 < n_iter && row + kBlockM < prm.Sq) {
        lse_next = lse_bh[row + kBlockM];
        delta_next = delta_bh[row + kBlockM];
      } else {
        lse_next = INFINITY;
        delta_next = 0.f;
      }
      const float lse2 = (lse_nat == -INFINITY) ? INFINITY : lse_nat * 1.4426950408889634f;
      const uint8_t* bias_row = nullptr;
      uint32_t drop_row = 0;
      if constexpr (kExt) {
        if (has_bias && row_ok)
          bias_row = static_cast<const uint8_t*>(prm.ex.bias) +
                     (b * prm.ex.bias_stride_b + h * prm.ex.bias_stride_h + static_cast<int64_t>(row) * prm.ex.bias_stride_q) *
                         (prm.ex.bias_f32 ? 4 : 2);
        drop_row = prm.ex.drop_base + static_cast<uint32_t>(bh) * static_cast<uint32_t>(prm.Sq) * static_cast<uint32_t>(prm.Sk) +
                   static_cast<uint32_t>(row) * static_cast<uint32_t>(prm.Sk);
      }
      const bool need_mask = (k0 + kBlockN > prm.Sk) || (prm.causal && k0 + kBlockN - 1 > q0);
      if constexpr (kExt) {
        // matrix bias: ask for this thread's 64 columns of the next query tile's row now
        if (has_bias && !vec_bias && it + 1 < n_iter && row + kBlockM < prm.Sq) {
          const int c0 = k0 + half * 64;
          if (c0 < prm.Sk)
            prefetch_bias(prm.ex, bias_row + static_cast<int64_t>(kBlockM) * prm.ex.bias_stride_q * (prm.ex.bias_f32 ? 4 : 2),
                          c0, min(64, prm.Sk - c0));
        }
      }
      mbar_wait(bar_s_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      if (warp == 0) bwd_trace(prm, 0, it, 0);
      // ---- P = exp2(S * scale - LSE) of this thread's 64 columns, in fp32 registers; the dP matmul runs meanwhile ----
      uint32_t sr[2][32];
      tmem_ld32(tS + (half * 2) * 32, sr[0]);
      tmem_ld32(tS + (half * 2 + 1) * 32, sr[1]);
      uint32_t keep[2] = {0xffffffffu, 0xffffffffu};  // dropout: bit x of keep[cc] = element kept
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        float bb[kExt ? 32 : 1];  // matrix bias only: fetched while the tensor-memory loads fly
        if constexpr (kExt) {
          if (has_bias && !vec_bias) load_bias32<kBf16>(prm.ex, bias_row, k0 + c * 32, prm.Sk, bb);
        }
        tmem_ld_wait(sr[cc]);
        // the mask (rare: diagonal and ragged tiles) is a separate, warp-uniform branch so that
        // full tiles pay nothing for it
        bool plain = true;
        if constexpr (kExt) {
          if (vec_bias) {
            plain = false;
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
              const float4 t = *reinterpret_cast<const float4*>(sb + c * 32 + x);  // broadcast read
              sr[cc][x + 0] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 0]), prm.scale_log2, t.x) - lse2));
              sr[cc][x + 1] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 1]), prm.scale_log2, t.y) - lse2));
              sr[cc][x + 2] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 2]), prm.scale_log2, t.z) - lse2));
              sr[cc][x + 3] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x + 3]), prm.scale_log2, t.w) - lse2));
            }
          } else if (has_bias) {
            plain = false;
#pragma unroll
            for (int x = 0; x < 32; ++x)
              sr[cc][x] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x]), prm.scale_log2, bb[x]) - lse2));
          }
        }
        if (plain) {
#pragma unroll
          for (int x = 0; x < 32; ++x)
            sr[cc][x] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(sr[cc][x]), prm.scale_log2, -lse2)));
        }
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const int col = k0 + c * 32 + x;
            if (col >= prm.Sk || (prm.causal && col > row)) sr[cc][x] = 0u;
          }
        }
        if constexpr (kExt) {
          if (has_drop) {
            uint32_t kb = 0;
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              const uint32_t idx = drop_row + static_cast<uint32_t>(k0 + c * 32 + x);
              if (dropout_hash(idx, prm.ex.drop_seed) > prm.ex.drop_threshold) kb |= 1u << x;
            }
            keep[cc] = kb;
          }
        }
      }
      if (warp == 0) bwd_trace(prm, 0, it, 4);
      // ---- P (zero where the forward dropped the element) and dS = P o (dP - delta) * scale (dP = 0 for a
      // dropped element), packed to 16 bits in registers ----
      uint32_t pp[2][16], dd[2][16];
      mbar_wait(bar_dp_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      const float neg_delta_scale = -delta * prm.scale;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t dpr[32];
        tmem_ld32(tDP + (half * 2 + cc) * 32, dpr);
        tmem_ld_wait(dpr);
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float p0 = __uint_as_float(sr[cc][x]), p1 = __uint_as_float(sr[cc][x + 1]);
          float z0 = p0, z1 = p1;
          float g0 = __uint_as_float(dpr[x]), g1 = __uint_as_float(dpr[x + 1]);
          if constexpr (kExt) {
            if (has_drop) {
              if (!((keep[cc] >> x) & 1u)) { z0 = 0.f; g0 = 0.f; }
              if (!((keep[cc] >> (x + 1)) & 1u)) { z1 = 0.f; g1 = 0.f; }
            }
          }
          pp[cc][x >> 1] = pack2<kBf16>(z0, z1);
          dd[cc][x >> 1] = pack2<kBf16>(p0 * fmaf(g0, dp_scale, neg_delta_scale), p1 * fmaf(g1, dp_scale, neg_delta_scale));
        }
      }
      tcgen05_fence_before_sync();  // the dP loads above precede the next tile's dP matmul
      // The P / dS buffers double as the staging area of the previous tile's dQ reduction, whose
      // shared-memory reads take about 2800 cycles: they must have finished before the buffers are
      // overwritten, which is why all of the arithmetic above runs first.
      if (it > 0) {
        if (tid == 0) tma_store_wait_read();
        named_barrier_sync(1, 256);
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          store_swizzled_unit(sP, r, c * 4 + u,
                              make_uint4(pp[cc][4 * u], pp[cc][4 * u + 1], pp[cc][4 * u + 2], pp[cc][4 * u + 3]));
      }
      fence_proxy_async_smem();  // shared-memory writes of these threads must be visible to the tensor core's reads
      mbar_arrive(bar_p_full);   // the dV matmul runs while dS is stored
      if (warp == 0) bwd_trace(prm, 0, it, 5);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          store_swizzled_unit(sDS, r, c * 4 + u,
                              make_uint4(dd[cc][4 * u], dd[cc][4 * u + 1], dd[cc][4 * u + 2], dd[cc][4 * u + 3]));
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_ds_full);
      if (warp == 0) bwd_trace(prm, 0, it, 1);

      // dQ tile of this (query tile, key tile) pair -> fp32 accumulation buffer
      mbar_wait(bar_dq_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      if (warp == 0) bwd_trace(prm, 0, it, 2);
      // dQ into registers first: the S / dP columns are then free for the next tile's matmuls, which
      // run while this tile is staged in shared memory (over P and dS, which the MMAs have finished
      // reading) as D/32 swizzled boxes of [128 rows x 32 floats] and added into the global
      // accumulation buffer with tiled bulk reductions; rows past Sq are dropped by the hardware
      uint32_t qr[D / 64][32];
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) tmem_ld32(tS + (half * (D / 64) + cc) * 32, qr[cc]);
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) tmem_ld_wait(qr[cc]);
      tcgen05_fence_before_sync();
      mbar_arrive(bar_s_free);
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(sP + c * kBoxBytes + r * 128 + ((u ^ (r & 7)) * 16)) =
              make_uint4(qr[cc][4 * u], qr[cc][4 * u + 1], qr[cc][4 * u + 2], qr[cc][4 * u + 3]);
      }
      fence_proxy_async_smem();
      if (warp == 0) bwd_trace(prm, 0, it, 3);
      named_barrier_sync(1, 256);
      if (tid == 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          if (c * 32 < prm.d_real) tma_reduce_add_3d(&tm_dq, sP + c * kBoxBytes, c * 32, q0, bh);
        tma_store_commit();
      }
    }
    if (tid == 0) tma_store_wait_all();  // the reductions must have landed before the CTA ends

    // ---- epilogue: key row (k0 + r); warps 0-3 write dK, warps 4-7 write dV ----
    const int kv_row = k0 + r;
    const bool kv_ok = kv_row < prm.Sk;
    uint16_t* dk_row = static_cast<uint16_t*>(prm.dk) + b * prm.dk_stride_b + h * prm.dk_stride_h +
                       static_cast<int64_t>(kv_row) * prm.dk_stride_s;
    uint16_t* dv_row = static_cast<uint16_t*>(prm.dv) + b * prm.dv_stride_b + h * prm.dv_stride_h +
                       static_cast<int64_t>(kv_row) * prm.dv_stride_s;
    if (n_iter > 0) tcgen05_fence_after_sync();
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
        if (kv_ok) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 v;
            if constexpr (kExt) {
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
  } else if (warp == 8) {
    // ================================ MMA issuer ================================
    constexpr uint32_t idesc_s = make_idesc(kBf16, kBlockM, kBlockN, 0, 0);  // S, dP: both K-major
    constexpr uint32_t idesc_t = make_idesc(kBf16, kBlockM, D, 1, 1);        // dV, dK: A M-major, B N-major
    constexpr uint32_t idesc_q = make_idesc(kBf16, kBlockM, D, 0, 1);        // dQ: A K-major, B N-major
    constexpr uint32_t kBoxStep = kBoxBytes >> 4;
    const uint32_t q_k = desc_lo(smem_u32(sQ), 16), do_k = desc_lo(smem_u32(sDO), 16);
    const uint32_t k_k = desc_lo(smem_u32(sK), 16), v_k = desc_lo(smem_u32(sV), 16);
    const uint32_t q_n = desc_lo(smem_u32(sQ), kBoxBytes), do_n = desc_lo(smem_u32(sDO), kBoxBytes);
    const uint32_t k_n = desc_lo(smem_u32(sK), kBoxBytes);
    const uint32_t p_m = desc_lo(smem_u32(sP), kBoxBytes), ds_m = desc_lo(smem_u32(sDS), kBoxBytes);
    const uint32_t ds_k = desc_lo(smem_u32(sDS), 16);
    const uint32_t tDK = tmem_base + Cfg::kColDK, tDV = tmem_base + Cfg::kColDV;
    const uint32_t tS = tmem_base + Cfg::kColS, tDP = tmem_base + Cfg::kColDP;

    mbar_wait(bar_kv, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
    for (int it = 0; it < n_iter; ++it) {
      mbar_wait(bar_q_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
      bwd_trace(prm, 2, it, 0);
      if (it > 0) mbar_wait(bar_s_free, (it - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
      tcgen05_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {  // S = Q K^T  (K = head_dim)
        const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
        umma_ss_lo_elect(tS, q_k + off, k_k + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      tcgen05_commit_elect(bar_s_full);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {  // dP = dO V^T
        const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
        umma_ss_lo_elect(tDP, do_k + off, v_k + off, idesc_s, kk > 0 ? 1u : 0u);
      }
      tcgen05_commit_elect(bar_dp_full);
      bwd_trace(prm, 2, it, 1);

      mbar_wait(bar_p_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
      tcgen05_fence_after_sync();
      bwd_trace(prm, 2, it, 2);
#pragma unroll
      for (int kk = 0; kk < kBlockM / 16; ++kk)  // dV += P^T dO  (K = 16 query rows per step: 2048 bytes)
        umma_ss_lo_elect(tDV, p_m + kk * 128, do_n + kk * 128, idesc_t, (it > 0 || kk > 0) ? 1u : 0u);
      mbar_wait(bar_ds_full, it & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
      tcgen05_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < kBlockM / 16; ++kk)  // dK += dS^T Q
        umma_ss_lo_elect(tDK, ds_m + kk * 128, q_n + kk * 128, idesc_t, (it > 0 || kk > 0) ? 1u : 0u);
      // Q_i and dO_i have no reader after this point: let the next tile's load start under dQ
      tcgen05_commit_elect(bar_q_empty);
#pragma unroll
      for (int kk = 0; kk < kBlockN / 16; ++kk) {  // dQ = dS K  (K = 16 keys per step), over the S columns
        const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
        umma_ss_lo_elect(tS, ds_k + off, k_n + kk * 128, idesc_q, kk > 0 ? 1u : 0u);
      }
      tcgen05_commit_elect(bar_dq_full);
      bwd_trace(prm, 2, it, 3);
    }
  } else {
    // ================================ TMA producer ================================
    const bool issuer = lane == 0;
    for (int it = 1; it < n_iter; ++it) {  // tile 0 went out before the allocation
      mbar_wait(bar_q_empty, (it - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      if (issuer) {
        const int q0 = (i0 + it) * kBlockM;
        mbar_arrive_expect_tx(bar_q_full, 2 * kTileBytes);
        for (int c = 0; c < kBoxes; ++c) tma_load_4d(sQ + c * kBoxBytes, &tm_q, bar_q_full, c * kBoxCols, q0, h, b);
        for (int c = 0; c < kBoxes; ++c) tma_load_4d(sDO + c * kBoxBytes, &tm_do, bar_q_full, c * kBoxCols, q0, h, b);
      }
      __syncwarp();
    }
    if (n_iter == 0) mbar_wait(bar_kv, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);  // drain the K/V load before exit
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

}  // namespace fo
