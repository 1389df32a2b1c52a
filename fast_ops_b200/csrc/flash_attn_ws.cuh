// Attention forward, warp-specialised kernel for sm_100a.
//
// One CTA owns TWO consecutive 128-row query tiles of one (batch, head) and walks the key/value
// tiles once for both.  Sixteen warps, four roles:
//
//   warps  0-3   softmax of query tile 0      (one thread per row: tcgen05.ld S, max, exp2,
//   warps  4-7   softmax of query tile 1       pack to 16 bit, tcgen05.st P over S)
//   warps  8-11  correction: rescales the O accumulators in tensor memory when a row maximum
//                moved, and at the end divides by the row sum and writes O and LSE
//   warp   12    MMA issuer: S = Q K^T (operands in shared memory) and O += P V (P from tensor
//                memory, V from shared memory), accumulators in tensor memory
//   warp   13    TMA producer: Q once, then K0 V0 K1 V1 ... through a ring of shared-memory stages
//   warps 14-15  idle (they give their registers to the softmax warps)
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1; P_s overwrites the first 64 columns of S_s.
// While the softmax warps of one tile work on S_j, the tensor core runs the other tile's PV and
// next QK^T, so MMA and exponentials overlap.  With a causal mask only key tiles at or below
// the diagonal are visited; tile 1 has one more than tile 0.
#pragma once

#include "flash_attn_common.cuh"
#include "fo_host.h"

namespace fo {

template <int D>
struct WsConfig {
  static constexpr int kTileBytes = kBlockM * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 6;
  static constexpr int kBoxes = D / kBoxCols;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = 2 * kTileBytes;
  static constexpr int kOffAlpha = kOffKV + kStages * kTileBytes;  // [2 tiles][2 buffers][128] float
  static constexpr int kOffFinal = kOffAlpha + 2 * 2 * 128 * 4;    // [2 tiles][l, m][128] float
  static constexpr int kOffBias = kOffFinal + 2 * 2 * 128 * 4;     // [2 tiles][2 buffers][128] float
  static constexpr int kOffBars = kOffBias + 2 * 2 * 128 * 4;
  static constexpr int kNumBars = 1 + 2 * kStages + 2 * 6;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 64 + 1024 /* alignment slack */;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColO0 = 256;
};

static_assert(WsConfig<128>::kOffBias % 16 == 0 && WsConfig<64>::kOffBias % 16 == 0, "float4 reads");

// A row keeps its reference maximum until the true maximum exceeds it by this much (log2
// units): exp2 arguments then stay below 8, P stays below 256, and most key tiles need no
// rescaling of O at all.
constexpr float kRescaleThreshold = 8.0f;




// grid = (num_q_pairs * B * H); block = 512.  Consecutive blocks sweep a group of heads whose K
// and V fit in L2 together, so the query tiles of those heads re-read K/V from L2 rather than
// from HBM; within the group the pairs with the most key tiles (causal mask) start first.
// kExt selects what is compiled in besides plain attention: bit 0 the additive bias, bit 1
// dropout (both described by prm.ex).  They are compile-time choices because a uniform run-time
// test inside the unrolled loops gets if-converted, and the unused path then still costs issue
// slots.
template <int D, bool kBf16, int kExt>
__global__ void __launch_bounds__(512, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnParams prm) {
  using Cfg = WsConfig<D>;
  constexpr int kTileBytes = Cfg::kTileBytes;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBoxes = Cfg::kBoxes;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + Cfg::kOffQ;    // two tiles
  uint8_t* sKV = smem + Cfg::kOffKV;  // kStages tiles
  float* s_alpha = reinterpret_cast<float*>(smem + Cfg::kOffAlpha);
  float* s_final = reinterpret_cast<float*>(smem + Cfg::kOffFinal);
  float* s_bias = reinterpret_cast<float*>(smem + Cfg::kOffBias);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* bar_q_full = bars;                  // TMA -> MMA
  uint64_t* bar_kv_full = bars + 1;             // [kStages] TMA -> MMA
  uint64_t* bar_kv_empty = bar_kv_full + kStages;  // [kStages] MMA -> TMA
  uint64_t* bar_s_full = bar_kv_empty + kStages;   // [2] MMA -> softmax
  uint64_t* bar_p_full = bar_s_full + 2;           // [2] softmax -> MMA (128 arrivals)
  uint64_t* bar_o_full = bar_p_full + 2;           // [2] MMA -> correction
  uint64_t* bar_corr = bar_o_full + 2;             // [2] softmax -> correction (128 arrivals)
  uint64_t* bar_o_scaled = bar_corr + 2;           // [2] correction -> MMA (128 arrivals)
  // [2] softmax -> correction, once: final row sum and maximum are in shared memory.  A barrier
  // of its own, because a fast softmax thread reaches this hand-off while a slower one has not
  // yet arrived on bar_corr for the last key tile.
  uint64_t* bar_final = bar_o_scaled + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip = cta_abort + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh_count = prm.B * prm.H;
  const int num_pairs = (prm.num_q_tiles + 1) >> 1;
  // Heads are taken in groups of prm.head_group (chosen on the host so that a group's K and V
  // fit in L2); inside a group the blocks go pair-major, heaviest pairs of all its heads first.
  const int group_blocks = prm.head_group * num_pairs;
  const int group = static_cast<int>(blockIdx.x) / group_blocks;
  const int in_group = static_cast<int>(blockIdx.x) - group * group_blocks;
  const int heads_here = min(prm.head_group, bh_count - group * prm.head_group);
  const int pair = num_pairs - 1 - in_group / heads_here;
  const int bh = group * prm.head_group + in_group % heads_here;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int hk = prm.kv_head_bcast ? 0 : h;  // head coordinate of K and V
  const int n_kv_total = (prm.Sk + kBlockN - 1) / kBlockN;
  // key tiles visited by query tile 0 / 1 of this pair; n1 >= n0 >= 1
  const int n0 = prm.causal ? min(n_kv_total, 2 * pair + 1) : n_kv_total;
  const int n1 = prm.causal ? min(n_kv_total, 2 * pair + 2) : n_kv_total;

  if (tid == 0) {
    *cta_abort = 0;
    *skip = *reinterpret_cast<volatile int*>(prm.device_status);
    mbar_init(bar_q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kv_full + i, 1);
      mbar_init(bar_kv_empty + i, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_s_full + s, 1);
      mbar_init(bar_p_full + s, 128);
      mbar_init(bar_o_full + s, 1);
      mbar_init(bar_corr + s, 128);
      mbar_init(bar_o_scaled + s, 128);
      mbar_init(bar_final + s, 128);
    }
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*skip) return;  // another CTA already timed out: do nothing

  if (warp == 12) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int* const dstat = prm.device_status;

  if (warp < 8) {
    // ================================ softmax ================================
    reg_alloc<192>();
    const int s = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int q0 = (2 * pair + s) * kBlockM;
    const int row = q0 + r;
    const int n_s = s ? n1 : n0;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + Cfg::kColS0 + s * kBlockN + lane_base;
    float* alpha_slot = s_alpha + s * 256 + r;
    float m_run = -INFINITY, l_run = 0.f;
    // bias row of this thread (null: no bias, or a row past the end) and the dropout index of
    // its column 0; with a bias the scores are scaled when the bias is added, not in the exponent
    constexpr bool has_bias = (kExt & 1) != 0;
    constexpr bool has_drop = (kExt & 2) != 0;
    const uint8_t* bias_row = nullptr;
    uint32_t drop_row = 0;
    if constexpr (kExt) {
      if (has_bias && row < prm.Sq)
        bias_row = static_cast<const uint8_t*>(prm.ex.bias) +
                   (b * prm.ex.bias_stride_b + h * prm.ex.bias_stride_h + static_cast<int64_t>(row) * prm.ex.bias_stride_q) *
                       (prm.ex.bias_f32 ? 4 : 2);
      drop_row = prm.ex.drop_base + static_cast<uint32_t>(bh) * static_cast<uint32_t>(prm.Sq) * static_cast<uint32_t>(prm.Sk) +
                 static_cast<uint32_t>(row) * static_cast<uint32_t>(prm.Sk);
    }
    const float exp_scale = has_bias ? 1.f : prm.scale_log2;
    // A bias that is the same for every query row ("vector") is staged through shared memory,
    // one key tile ahead: thread r fetches column r of the next tile while this tile is computed.
    const bool vec_bias = has_bias && prm.ex.bias_stride_q == 0;
    const uint8_t* bias_vec = nullptr;
    float* sb = s_bias + s * 256;
    float bias_next = 0.f;
    if constexpr (kExt) {
      if (vec_bias) {
        bias_vec = static_cast<const uint8_t*>(prm.ex.bias) +
                   (b * prm.ex.bias_stride_b + h * prm.ex.bias_stride_h) * (prm.ex.bias_f32 ? 4 : 2);
        bias_next = (r < prm.Sk) ? load_bias1<kBf16>(prm.ex, bias_vec, r) : 0.f;
      }
    }

    for (int j = 0; j < n_s; ++j) {
      const int k0 = j * kBlockN;
      if constexpr (kExt) {
        if (vec_bias) {
          sb[(j & 1) * 128 + r] = bias_next;
          const int col = k0 + kBlockN + r;
          bias_next = (j + 1 < n_s && col < prm.Sk) ? load_bias1<kBf16>(prm.ex, bias_vec, col) : 0.f;
          // the 128 threads of this tile; a buffer is rewritten two tiles later, behind the
          // barrier of the tile in between
          named_barrier_sync(1 + s, 128);
        } else if (bias_row != nullptr && j + 1 < n_s) {
          const int c0 = k0 + kBlockN;
          prefetch_bias(prm.ex, bias_row, c0, min(kBlockN, prm.Sk - c0));
        }
      }
      mbar_wait(bar_s_full + s, j & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      if ((warp & 3) == 0) trace_event(prm, s, j, 0);
      const bool need_mask = (k0 + kBlockN > prm.Sk) || (prm.causal && k0 + kBlockN - 1 > q0);
      uint32_t sr[4][32];
      float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
      // Tensor-memory loads are software-pipelined against the row maximum: chunk c+1 is in
      // flight while chunk c is reduced.
      tmem_ld32(tS, sr[0]);
      tmem_ld_wait(sr[0]);
      if ((warp & 3) == 0) trace_event(prm, s, j, 4);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c + 1 < 4) tmem_ld32(tS + (c + 1) * 32, sr[c + 1]);
        if constexpr (kExt) {
          if (vec_bias) {
            const float4* bv = reinterpret_cast<const float4*>(sb + (j & 1) * 128 + c * 32);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 t = bv[i >> 2];  // the same address in every thread: a broadcast
              sr[c][i + 0] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 0]), prm.scale_log2, t.x));
              sr[c][i + 1] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 1]), prm.scale_log2, t.y));
              sr[c][i + 2] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 2]), prm.scale_log2, t.z));
              sr[c][i + 3] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 3]), prm.scale_log2, t.w));
            }
          } else if (has_bias) {
            float bb[32];
            load_bias32<kBf16>(prm.ex, bias_row, k0 + c * 32, prm.Sk, bb);
#pragma unroll
            for (int i = 0; i < 32; ++i)
              sr[c][i] = __float_as_uint(fmaf(__uint_as_float(sr[c][i]), prm.scale_log2, bb[i]));
          }
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0 + c * 32 + i;
            if (col >= prm.Sk || (prm.causal && col > row)) sr[c][i] = 0xff800000u;  // -inf
          }
        }
        // four independent accumulators (and 3-input max) keep the dependency chain short
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          mxa = max3(mxa, __uint_as_float(sr[c][i + 0]), __uint_as_float(sr[c][i + 1]));
          mxb = max3(mxb, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
          mxc = max3(mxc, __uint_as_float(sr[c][i + 4]), __uint_as_float(sr[c][i + 5]));
          mxd = max3(mxd, __uint_as_float(sr[c][i + 6]), __uint_as_float(sr[c][i + 7]));
        }
        if (c + 1 < 4) tmem_ld_wait(sr[c + 1]);
      }
      const float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
      if ((warp & 3) == 0) trace_event(prm, s, j, 5);
      const float m_cand = fmaxf(m_run, mx * exp_scale);
      const float m_new = (m_cand - m_run > kRescaleThreshold) ? m_cand : m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_new == m_run) ? 1.f : fast_exp2(m_run - m_use);
      // P = exp2(S * scale - m): packed fp32 pairs for the multiply-add and the row sum, one
      // unrolled block over the whole tile so that ex2 latencies overlap across chunks.
      const float2 sc2 = make_float2(exp_scale, exp_scale);
      const float2 nm2 = make_float2(-m_use, -m_use);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
      uint32_t pr[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int q = 0; q < 16; ++q) {  // column pair q of the chunk
          float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c][2 * q]), __uint_as_float(sr[c][2 * q + 1])), sc2, nm2);
          x.x = fast_exp2(x.x);
          x.y = fast_exp2(x.y);
          if (q & 1) acc1 = __fadd2_rn(acc1, x); else acc0 = __fadd2_rn(acc0, x);
          if constexpr (kExt) {
            // dropped elements leave the row sum untouched and enter P V as zeros; the factor
            // 1 / (1 - p) is applied once, to O, in the epilogue
            if (has_drop) {
              const uint32_t idx = drop_row + static_cast<uint32_t>(k0 + c * 32 + 2 * q);
              if (dropout_hash(idx, prm.ex.drop_seed) <= prm.ex.drop_threshold) x.x = 0.f;
              if (dropout_hash(idx + 1u, prm.ex.drop_seed) <= prm.ex.drop_threshold) x.y = 0.f;
            }
          }
          pr[c][q] = pack2<kBf16>(x.x, x.y);
        }
        if (c == 0) {
          // hand the rescale factor to the correction warps once the first exponentials are in
          // flight (it is off this thread's critical path)
          alpha_slot[(j & 1) * 128] = alpha;
          mbar_arrive(bar_corr + s);
          if ((warp & 3) == 0) trace_event(prm, s, j, 1);
        }
      }
      if ((warp & 3) == 0) trace_event(prm, s, j, 2);
      // P (two 16-bit values per column) over the first 64 columns of S
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st16(tS + c * 16, pr[c]);
      tcgen05_wait_st();
      tcgen05_fence_before_sync();
      mbar_arrive(bar_p_full + s);
      if ((warp & 3) == 0) trace_event(prm, s, j, 3);
      const float rsum = (acc0.x + acc0.y) + (acc1.x + acc1.y);
      l_run = l_run * alpha + rsum;
      m_run = m_new;
    }
    s_final[s * 256 + r] = l_run;
    s_final[s * 256 + 128 + r] = m_run;
    mbar_arrive(bar_final + s);
  } else if (warp < 12) {
    // ================================ correction + epilogue ================================
    reg_dealloc<80>();
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int j = 0; j < n1; ++j) {
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (j >= (s ? n1 : n0)) continue;
        mbar_wait(bar_corr + s, j & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        const float alpha = s_alpha[s * 256 + (j & 1) * 128 + r];
        if (j > 0) {
          mbar_wait(bar_o_full + s, (j - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
          tcgen05_fence_after_sync();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            const uint32_t tO = tmem_base + Cfg::kColO0 + s * D + lane_base;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t orr[32];
              tmem_ld32(tO + c * 32, orr);
              tmem_ld_wait(orr);
#pragma unroll
              for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
              tmem_st32(tO + c * 32, orr);
            }
            tcgen05_wait_st();
          }
          tcgen05_fence_before_sync();
        }
        mbar_arrive(bar_o_scaled + s);
      }
    }
    // epilogue: O / l and LSE
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int n_s = s ? n1 : n0;
      mbar_wait(bar_final + s, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
      mbar_wait(bar_o_full + s, (n_s - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      const float l_run = s_final[s * 256 + r];
      const float m_run = s_final[s * 256 + 128 + r];
      const float o_scale = kExt ? prm.ex.drop_rescale : 1.f;
      const float inv_l = (l_run > 0.f) ? o_scale / l_run : 0.f;
      const int row = (2 * pair + s) * kBlockM + r;
      const bool row_ok = row < prm.Sq;
      uint16_t* orow = static_cast<uint16_t*>(prm.o) + b * prm.o_stride_b + h * prm.o_stride_h +
                       static_cast<int64_t>(row) * prm.o_stride_s;
      const uint32_t tO = tmem_base + Cfg::kColO0 + s * D + lane_base;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld32(tO + c * 32, orr);
        tmem_ld_wait(orr);
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack2<kBf16>(__uint_as_float(orr[i + 0]) * inv_l, __uint_as_float(orr[i + 1]) * inv_l);
            v.y = pack2<kBf16>(__uint_as_float(orr[i + 2]) * inv_l, __uint_as_float(orr[i + 3]) * inv_l);
            v.z = pack2<kBf16>(__uint_as_float(orr[i + 4]) * inv_l, __uint_as_float(orr[i + 5]) * inv_l);
            v.w = pack2<kBf16>(__uint_as_float(orr[i + 6]) * inv_l, __uint_as_float(orr[i + 7]) * inv_l);
            if (c * 32 + i < prm.d_real) *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
          }
        }
      }
      if (row_ok && prm.lse != nullptr) {
        prm.lse[static_cast<int64_t>(bh) * prm.Sq + row] =
            (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  } else {
    reg_dealloc<48>();
    if (warp == 12) {
      // ================================ MMA issuer ================================
      constexpr uint32_t idesc_qk = make_idesc(kBf16, kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, kBlockM, D, 0, 1);
      // Everything below is warp-uniform; only the tcgen05 instructions themselves are issued by
      // one elected lane.  Descriptors are kept as 32-bit low halves: per instruction one add.
      const uint32_t q_lo0 = desc_lo(smem_u32(sQ), 16);
      const uint32_t q_lo1 = desc_lo(smem_u32(sQ) + kTileBytes, 16);
      const uint32_t kv_k_lo = desc_lo(smem_u32(sKV), 16);         // K tiles: K-major
      const uint32_t kv_v_lo = desc_lo(smem_u32(sKV), kBoxBytes);  // V tiles: N-major
      constexpr uint32_t kStageStep = kTileBytes >> 4;
      const uint32_t tS0 = tmem_base + Cfg::kColS0;
      const uint32_t tO0 = tmem_base + Cfg::kColO0;
      // S_s = Q_s K^T over the K tile in ring slot `stage`
      auto issue_s = [&](int s, int stage) {
        const uint32_t a_lo = s ? q_lo1 : q_lo0;
        const uint32_t b_lo = kv_k_lo + stage * kStageStep;
        const uint32_t tS = tS0 + s * kBlockN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // k-slice kk: box kk/4, 32 bytes per slice inside the 128-byte swizzle span
          constexpr uint32_t kBoxStep = kBoxBytes >> 4;
          const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
          umma_ss_lo_elect(tS, a_lo + off, b_lo + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      // O_s (+)= P_s V over the V tile in ring slot `stage`
      auto issue_pv = [&](int s, int stage, bool acc) {
        const uint32_t tP = tS0 + s * kBlockN;
        const uint32_t tO = tO0 + s * D;
        const uint32_t b_lo = kv_v_lo + stage * kStageStep;
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          // 16 key rows per slice: 2048 bytes of V, 8 packed columns of P
          umma_ts_lo_elect(tO, tP + kk * 8, b_lo + kk * 128, idesc_pv, (acc || kk > 0) ? 1u : 0u);
        }
      };
      // waits for P_s of key tile j (and for O_s to have been rescaled) and issues PV; the caller commits
      auto pv_tile = [&](int s, int stage, int j) {
        mbar_wait(bar_o_scaled + s, j & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        mbar_wait(bar_p_full + s, j & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        tcgen05_fence_after_sync();
        issue_pv(s, stage, j > 0);
      };

      mbar_wait(bar_q_full, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
      mbar_wait(bar_kv_full + 0, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);  // K_0 is ring slot 0
      tcgen05_fence_after_sync();
      issue_s(0, 0);
      tcgen05_commit_elect(bar_s_full + 0);
      issue_s(1, 0);
      tcgen05_commit_elect(bar_s_full + 1);
      tcgen05_commit_elect(bar_kv_empty + 0);
      for (int j = 0; j < n1; ++j) {
        const int iv = 2 * j + 1;  // ring index of V_j; K_{j+1} is iv + 1
        const int st_v = iv % kStages;
        const int st_k = (iv + 1) % kStages;
        const bool more = j + 1 < n1;
        mbar_wait(bar_kv_full + st_v, (iv / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        if (more) mbar_wait(bar_kv_full + st_k, ((iv + 1) / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        trace_event(prm, 2, j, 0);
        if (j < n0) {
          pv_tile(0, st_v, j);
          trace_event(prm, 2, j, 1);
          tcgen05_commit_elect(bar_o_full + 0);
          if (j + 1 < n0) {
            issue_s(0, st_k);
            tcgen05_commit_elect(bar_s_full + 0);
          }
        }
        trace_event(prm, 2, j, 2);
        pv_tile(1, st_v, j);
        trace_event(prm, 2, j, 3);
        tcgen05_commit_elect(bar_o_full + 1);
        tcgen05_commit_elect(bar_kv_empty + st_v);
        if (more) {
          issue_s(1, st_k);
          tcgen05_commit_elect(bar_s_full + 1);
          tcgen05_commit_elect(bar_kv_empty + st_k);
        }
      }
    } else if (warp == 13) {
      // ================================ TMA producer ================================
      const bool issuer = lane == 0;
      if (issuer) {
        mbar_arrive_expect_tx(bar_q_full, 2 * kTileBytes);
        for (int s = 0; s < 2; ++s)
          for (int c = 0; c < kBoxes; ++c)
            tma_load_4d(sQ + s * kTileBytes + c * kBoxBytes, &tm_q, bar_q_full, c * kBoxCols,
                        (2 * pair + s) * kBlockM, h, b);
      }
      __syncwarp();
      for (int i = 0; i < 2 * n1; ++i) {
        const int st = i % kStages;
        mbar_wait(bar_kv_empty + st, ((i / kStages) & 1) ^ 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
        if (issuer) {
          mbar_arrive_expect_tx(bar_kv_full + st, kTileBytes);
          const CUtensorMap* map = (i & 1) ? &tm_v : &tm_k;
          for (int c = 0; c < kBoxes; ++c)
            tma_load_4d(sKV + st * kTileBytes + c * kBoxBytes, map, bar_kv_full + st, c * kBoxCols,
                        (i >> 1) * kBlockN, hk, b);
        }
        __syncwarp();
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D, bool kBf16, int kExt>
int launch_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& prm,
              cudaStream_t stream) {
  auto kernel = attn_fwd_ws_kernel<D, kBf16, kExt>;
  constexpr int smem = WsConfig<D>::kSmemBytes;
  cudaError_t ea = ensure_dynamic_smem<attn_fwd_ws_kernel<D, kBf16, kExt>>(smem, prm.device);
  if (ea != cudaSuccess)
    return fail(FO_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", smem, cudaGetErrorString(ea));
  const int num_pairs = (prm.num_q_tiles + 1) / 2;
  const int64_t blocks = static_cast<int64_t>(num_pairs) * prm.B * prm.H;
  if (blocks > 0x7fffffffLL) return fail(FO_ERR_INVALID_ARGUMENT, "too many query tiles for one launch");
  kernel<<<static_cast<unsigned>(blocks), 512, smem, stream>>>(tq, tk, tv, prm);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}

}  // namespace fo
