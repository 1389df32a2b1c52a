// Attention forward: the 64-key-step kernel of flash_attn_ws64.cuh as a PERSISTENT grid.
//
// Same roles, tensor-memory layout (S0a | S0b | S1a | S1b | O0 | O1), K/V ring and softmax
// arithmetic.  The differences:
//
//  * One CTA per SM works through items (an item = two consecutive 128-row query tiles of one
//    (batch, head)) that it draws from a counter in global memory, heaviest items first, heads
//    grouped so that their K and V stay in L2: the order in which the non-persistent kernel's
//    CTAs are started.  Warp 13 is scheduler and TMA producer: it publishes each item to the other
//    roles through a two-slot ring in shared memory.
//  * Barriers and tensor memory are set up once per CTA.  The K/V ring, the step buffers and
//    every barrier phase run on across items: the loads of the next item are in flight, and its
//    first two Q K^T steps are computed, while the current item's last steps and its epilogue
//    drain.  Steps are numbered globally per query tile (g = steps of earlier items + t): a step's
//    S / P buffer and barrier are chosen by g & 1 and its barrier phase by (g >> 1) & 1, whatever
//    item it belongs to.  Three barriers are new: q_empty (the item's Q K^T are done, Q may be
//    overwritten), o_free (the epilogue has read O and the row statistics) and the item ring's.
//  * The two query tiles' turns on the ex2 units are tied to shared-memory accesses (turn_wait /
//    turn_pass), so that the assembler cannot move the exponentials across the barriers.
//
// Measured against the non-persistent kernel on the same GPU (bf16, causal, D = 128): S = 1024
// 627 against 606 TFLOP/s, S = 2048 823 against 857, S = 4096 955 against 1035, S = 16384 1006
// against 1136.  The set-up that the persistent grid saves is visible at S = 1024 only; per step
// its softmax loop runs about a tenth slower (the same source compiled into a different
// instruction order), so it is not the default.  Plain attention only (no bias, no dropout).
#pragma once

#include "flash_attn_common.cuh"
#include "flash_attn_ws.cuh"
#include "flash_attn_ws64.cuh"
#include "fo_host.h"

namespace fo {


template <int D>
struct Ws64pConfig : WsConfig<D> {
  // barriers: q_full, q_empty, kv_full/empty per stage, then s_full[2][2], p_full[2][2],
  // o_full[2], corr[2][2], final[2], o_done[2], o_free[2], item_full[2], item_empty[2]
  static constexpr int kNumBars = 2 + 2 * WsConfig<D>::kStages + 4 + 4 + 2 + 4 + 2 + 2 + 2 + 2 + 2;
  static constexpr int kOffMisc = WsConfig<D>::kOffBars + kNumBars * 8;
  static constexpr int kOffTurn = kOffMisc + 64;  // [256] float slots of the turn hand-off, then one word of 0.0f
  static constexpr int kSmemBytes = kOffTurn + 257 * 4 + 12 + 1024 /* alignment slack */;
};

// What an item index means: items are numbered group by group (a group = head_group heads whose
// K and V fit in L2 together), inside a group pair-major with the heaviest query-tile pair first.
struct Ws64pItem {
  int pair, bh, b, h, hk;
  int T0, T1;  // 64-key steps of query tile 0 / 1 (T1 >= T0 >= 1)
  int n1;      // 128-key tiles of K (and of V) the item walks
};

__device__ __forceinline__ Ws64pItem ws64p_decode(const AttnParams& prm, int it) {
  Ws64pItem w;
  const int bh_count = prm.B * prm.H;
  const int num_pairs = (prm.num_q_tiles + 1) >> 1;
  const int group_blocks = prm.head_group * num_pairs;
  const int group = it / group_blocks;
  const int in_group = it - group * group_blocks;
  const int heads_here = min(prm.head_group, bh_count - group * prm.head_group);
  w.pair = num_pairs - 1 - in_group / heads_here;
  w.bh = group * prm.head_group + in_group % heads_here;
  w.b = w.bh / prm.H;
  w.h = w.bh - w.b * prm.H;
  w.hk = prm.kv_head_bcast ? 0 : w.h;  // head coordinate of K and V
  // keys visible to query tile 0 / 1 of this pair
  const int vis0 = prm.causal ? min(prm.Sk, (2 * w.pair + 1) * kBlockM) : prm.Sk;
  const int vis1 = prm.causal ? min(prm.Sk, (2 * w.pair + 2) * kBlockM) : prm.Sk;
  w.T0 = (vis0 + kStepN - 1) / kStepN;
  w.T1 = (vis1 + kStepN - 1) / kStepN;
  w.n1 = (w.T1 + 1) >> 1;
  return w;
}

template <int D, bool kBf16, int kExt>
__global__ void __launch_bounds__(512, 1)
attn_fwd_ws64p_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const AttnParams prm) {
  using Cfg = Ws64pConfig<D>;
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
  uint64_t* bar_q_full = bars;                     // TMA -> MMA, once per item
  uint64_t* bar_q_empty = bars + 1;                // MMA -> TMA, once per item: every Q K^T of the item has run
  uint64_t* bar_kv_full = bars + 2;                // [kStages] TMA -> MMA
  uint64_t* bar_kv_empty = bar_kv_full + kStages;  // [kStages] MMA -> TMA
  uint64_t* bar_s_full = bar_kv_empty + kStages;   // [2 tiles][2 buffers] MMA -> softmax
  // [2][2] softmax and correction -> MMA (256 arrivals): P of the step is in tensor memory (128
  // softmax threads) and O has been rescaled if the step needed it (128 correction threads).
  // One barrier for both, because every wait on the issuing warp's path costs about 200 cycles
  // even when the phase completed long ago.  The correction threads arrive as soon as they have
  // the step's rescale factors, unless a factor differs from 1: only then do they wait for the
  // previous P V and rescale O first.
  uint64_t* bar_p_full = bar_s_full + 4;
  uint64_t* bar_o_full = bar_p_full + 4;           // [2] MMA -> correction, once per P V
  // [2][2] softmax -> correction (128 arrivals), one barrier per step parity: the softmax
  // threads can be two steps ahead of the correction warps, which a single barrier's phase
  // bit could not tell from zero steps ahead
  uint64_t* bar_corr = bar_o_full + 2;
  uint64_t* bar_final = bar_corr + 4;              // [2] softmax -> correction, once per item
  // [2] MMA -> epilogue, once per item: every P V of the tile has finished.  bar_o_full cannot
  // serve: by then nobody may have waited on it for many steps, and its phase bit alone does not
  // say whether the last P V is the one that completed.
  uint64_t* bar_o_done = bar_final + 2;
  // [2] epilogue -> MMA and softmax (128 arrivals), once per item: O of the tile has been read out
  // of tensor memory (the next item's first P V may overwrite it) and the tile's row sums and
  // maxima have been read out of shared memory (the softmax threads may write the next ones).
  uint64_t* bar_o_free = bar_o_done + 2;
  // [2 slots] scheduler -> everybody / everybody -> scheduler: the item ring
  uint64_t* bar_item_full = bar_o_free + 2;
  uint64_t* bar_item_empty = bar_item_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip = cta_abort + 1;
  volatile int* s_item = skip + 1;  // [2] item index of ring slot, or -1: no more items
  float* s_turn = reinterpret_cast<float*>(smem + Cfg::kOffTurn);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_items = ((prm.num_q_tiles + 1) >> 1) * prm.B * prm.H;
  // arrivals that free an item slot: every softmax and correction thread, one lane of each MMA warp
  constexpr int kItemReaders = 256 + 128 + 2;

  if (tid == 0) {
    *cta_abort = 0;
    *skip = *reinterpret_cast<volatile int*>(prm.device_status);
    s_turn[256] = 0.f;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 2);  // one commit from each MMA-issuing warp
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kv_full + i, 1);
      mbar_init(bar_kv_empty + i, 2);  // one commit from each MMA-issuing warp
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_s_full + i, 1);
      mbar_init(bar_p_full + i, 256);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_o_full + s, 1);
      mbar_init(bar_corr + 2 * s, 128);
      mbar_init(bar_corr + 2 * s + 1, 128);
      mbar_init(bar_final + s, 128);
      mbar_init(bar_o_done + s, 1);
      mbar_init(bar_o_free + s, 128);
      mbar_init(bar_item_full + s, 1);
      mbar_init(bar_item_empty + s, kItemReaders);
    }
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  const bool live = *skip == 0;  // false: another launch's CTA timed out earlier and nobody reset the word
  int* const dstat = prm.device_status;
  uint32_t tmem_base = 0;
  if (live) {
    if (warp == 12) {
      tmem_alloc(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    tmem_base = *tmem_slot;
  }

  // Every consumer role takes the next item from the ring the same way.
  auto next_item = [&](int k) -> int {
    const int slot = k & 1;
    mbar_wait(bar_item_full + slot, (k >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_EPILOGUE);
    const int it = *cta_abort ? -1 : s_item[slot];  // an aborted CTA stops at once
    return it;
  };

  if (!live) {
    // nothing to do
  } else if (warp < 8) {
    // ================================ softmax ================================
    reg_alloc<184>();
    const int s = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS_tile = tmem_base + Cfg::kColS0 + s * kBlockN + lane_base;
    constexpr bool has_bias = (kExt & 1) != 0;
    constexpr bool has_drop = (kExt & 2) != 0;
    // with a bias the scores are scaled when the bias is added, not in the exponent
    const float exp_scale = has_bias ? 1.f : prm.scale_log2;
    // a row-independent bias goes through shared memory, fetched one 128-key tile ahead
    const bool vec_bias = has_bias && prm.ex.bias_stride_q == 0;
    float* sb = s_bias + s * 256;
    // The two tiles' softmax warps share the ex2 units.  Left alone they fall into lockstep: both
    // reduce maxima at the same time (ex2 idle), then both exponentiate (ex2 contended).  The
    // exponentials of the two tiles are therefore made to alternate with a pair of named barriers
    // (tile 0 goes first): while one tile exponentiates, the other loads S and stores P.  In every
    // item both tiles take T0 turns; the steps that only tile 1 has (two, under a causal mask) run
    // without one.  Tile 1's last arrival of an item is what lets tile 0 into the next item.
    constexpr int kTurn0 = 3, kTurn1 = 4, kTurnCount = 256;  // named barriers: "tile 0 may exponentiate", "tile 1 may"
    const bool ping_pong = prm.ping_pong != 0;
    if (ping_pong && s == 1) named_barrier_arrive(kTurn0, kTurnCount);

    int g = 0;  // steps of this tile in earlier items
    for (int k = 0;; ++k) {
      const int it = next_item(k);
      mbar_arrive(bar_item_empty + (k & 1));
      if (it < 0) break;
      const Ws64pItem w = ws64p_decode(prm, it);
      const int T_s = s ? w.T1 : w.T0;
      const int q0 = (2 * w.pair + s) * kBlockM;
      const int row = q0 + r;
      float m_run = -INFINITY, l_run = 0.f;
      const uint8_t* bias_row = nullptr;
      uint32_t drop_row = 0;
      const uint8_t* bias_vec = nullptr;
      float bias_next = 0.f;
      if constexpr (kExt != 0) {
        if (has_bias && row < prm.Sq)
          bias_row = static_cast<const uint8_t*>(prm.ex.bias) +
                     (w.b * prm.ex.bias_stride_b + w.h * prm.ex.bias_stride_h +
                      static_cast<int64_t>(row) * prm.ex.bias_stride_q) * (prm.ex.bias_f32 ? 4 : 2);
        drop_row = prm.ex.drop_base +
                   static_cast<uint32_t>(w.bh) * static_cast<uint32_t>(prm.Sq) * static_cast<uint32_t>(prm.Sk) +
                   static_cast<uint32_t>(row) * static_cast<uint32_t>(prm.Sk);
        if (vec_bias) {
          bias_vec = static_cast<const uint8_t*>(prm.ex.bias) +
                     (w.b * prm.ex.bias_stride_b + w.h * prm.ex.bias_stride_h) * (prm.ex.bias_f32 ? 4 : 2);
          bias_next = (r < prm.Sk) ? load_bias1<kBf16>(prm.ex, bias_vec, r) : 0.f;
        }
      }

      if constexpr (kExt != 0) {
        // the bias staging buffers are about to be rewritten: every thread of the tile must be
        // done reading the previous item's
        if (vec_bias && k > 0) named_barrier_sync(1 + s, 128);
      }

      uint32_t sr[2][32];  // scores of the current step (scaled and biased already when there is a bias)

      // Stages the row-independent bias of the key tile that step `tn` (even) starts.
      auto stage_vec_bias = [&](int tn) {
        const int j = tn >> 1;
        sb[(j & 1) * 128 + r] = bias_next;
        const int col = tn * kStepN + kBlockN + r;
        bias_next = (col < prm.Sk) ? load_bias1<kBf16>(prm.ex, bias_vec, col) : 0.f;
        // a buffer is rewritten two key tiles later, behind the barrier of the tile between
        named_barrier_sync(1 + s, 128);
      };
      // Issues the tensor-memory loads of step tn's scores (S must be complete).
      auto issue_load = [&](int tn, int c) {
        const uint32_t tSn = tS_tile + ((g + tn) & 1) * kStepN;
        tmem_ld32(tSn + c * 32, sr[c]);
      };
      // Waits for those loads and applies bias and masks in place.
      auto prep_loads = [&](int tn) {
        const int k0n = tn * kStepN;
        const bool need_mask = (k0n + kStepN > prm.Sk) || (prm.causal && k0n + kStepN - 1 > q0);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tmem_ld_wait(sr[c]);
          if ((warp & 3) == 0 && tn > 0) trace_event(prm, s, tn - 1, c == 0 ? 1 : 4);  // loads in
          if constexpr (kExt != 0) {
            if (vec_bias) {
              const float4* bv = reinterpret_cast<const float4*>(sb + ((tn >> 1) & 1) * 128 + (tn & 1) * kStepN + c * 32);
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 v4 = bv[i >> 2];  // the same address in every thread: a broadcast
                sr[c][i + 0] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 0]), prm.scale_log2, v4.x));
                sr[c][i + 1] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 1]), prm.scale_log2, v4.y));
                sr[c][i + 2] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 2]), prm.scale_log2, v4.z));
                sr[c][i + 3] = __float_as_uint(fmaf(__uint_as_float(sr[c][i + 3]), prm.scale_log2, v4.w));
              }
            } else if (has_bias) {
              float bb[32];
              load_bias32<kBf16>(prm.ex, bias_row, k0n + c * 32, prm.Sk, bb);
#pragma unroll
              for (int i = 0; i < 32; ++i)
                sr[c][i] = __float_as_uint(fmaf(__uint_as_float(sr[c][i]), prm.scale_log2, bb[i]));
            }
          }
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = k0n + c * 32 + i;
              if (col >= prm.Sk || (prm.causal && col > row)) sr[c][i] = 0xff800000u;  // -inf
            }
          }
        }
      };
      // Row maximum of the scores in sr: four independent accumulators (and 3-input max) keep the
      // dependency chain short.
      auto row_max = [&]() {
        float mxa = -INFINITY, mxb = -INFINITY, mxc = -INFINITY, mxd = -INFINITY;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            mxa = max3(mxa, __uint_as_float(sr[c][i + 0]), __uint_as_float(sr[c][i + 1]));
            mxb = max3(mxb, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
            mxc = max3(mxc, __uint_as_float(sr[c][i + 4]), __uint_as_float(sr[c][i + 5]));
            mxd = max3(mxd, __uint_as_float(sr[c][i + 6]), __uint_as_float(sr[c][i + 7]));
          }
        }
        return fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
      };

      // prologue: scores of step 0; their row maximum is the first reference maximum
      if constexpr (kExt != 0) {
        if (vec_bias) stage_vec_bias(0);
      }
      mbar_wait(bar_s_full + 2 * s + (g & 1), (g >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      tcgen05_fence_after_sync();
      issue_load(0, 0);
      issue_load(0, 1);
      prep_loads(0);
      m_run = row_max() * exp_scale;

      // The exponentials of a step do not wait for the step's own row maximum: they are taken
      // against the reference maximum the row already has (lazy rescaling moves it only when the
      // true maximum exceeds it by kRescaleThreshold), and the maximum is reduced alongside them,
      // its instructions filling issue slots that the ex2 unit's rate leaves empty.  Only if a row
      // of the warp turns out to need a new reference (rare after the first steps) are the step's
      // exponentials taken again.  Each iteration then fetches step t + 1 (whose S the tensor core
      // finished meanwhile) behind the P stores, so that the latencies of the loads, of the P store
      // and of the barriers overlap instead of adding up.
      for (int t = 0; t < T_s; ++t) {
        const int gt = g + t;
        const int ub = gt & 1;                 // S / P buffer, barrier and rescale-factor slot of the step
        const uint32_t ph = (gt >> 1) & 1;     // phase of those barriers
        const uint32_t ph_next = ((gt + 1) >> 1) & 1;
        const int k0 = t * kStepN;
        const uint32_t tS = tS_tile + ub * kStepN;
        const bool turn = ping_pong && t < w.T0;
        float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
        if (turn) neg_m += turn_wait(s ? kTurn1 : kTurn0, kTurnCount, s_turn + 256);  // exponentials start after this
        if ((warp & 3) == 0) trace_event(prm, s, t, 0);  // turn taken
        const float2 sc2 = make_float2(exp_scale, exp_scale);
        float2 acc0, acc1;
        uint32_t pr[2][16];
        const bool more = t + 1 < T_s;
        bool s_next_ready = false;
        float mxa = -INFINITY, mxb = -INFINITY;
        // P = exp2(S * scale - reference) for the whole step; `first` is the pass that also passes
        // the turn on, polls the next S and reduces the row maximum
        auto exp_pass = [&](float neg_ref, const bool first) {
          const float2 nm2 = make_float2(neg_ref, neg_ref);
          acc0 = make_float2(0.f, 0.f);
          acc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            // one non-blocking look at S of step t + 1 (as a rule complete by now); the answer is
            // needed only after the exponentials, so its latency is hidden
            if (first && c == 1 && more) s_next_ready = mbar_test_wait(bar_s_full + 2 * s + (ub ^ 1), ph_next);
            // The turn is passed on after the first half (the partial row sums depend on all of its
            // exponentials): the other tile's first half then shares the ex2 units with this tile's
            // second half, two warps per scheduler, which hides the latencies a lone warp exposes.
            // (Measured: handing over after three quarters, or after all of them, is slower.)
            float2 nm2c = nm2;
            if (first && c == 1 && turn)
              turn_pass(s ? kTurn0 : kTurn1, kTurnCount, s_turn + tid, (acc0.x + acc0.y) + (acc1.x + acc1.y));
#pragma unroll
            for (int q = 0; q < 16; ++q) {  // column pair q of the chunk
              const float a = __uint_as_float(sr[c][2 * q]), b = __uint_as_float(sr[c][2 * q + 1]);
              float2 x = __ffma2_rn(make_float2(a, b), sc2, nm2c);
              x.x = fast_exp2(x.x);
              x.y = fast_exp2(x.y);
              if (q & 1) acc1 = __fadd2_rn(acc1, x); else acc0 = __fadd2_rn(acc0, x);
              if (first) {
                if (q & 1) mxb = max3(mxb, a, b); else mxa = max3(mxa, a, b);
              }
              if constexpr (kExt != 0) {
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
          }
        };
        exp_pass(neg_m, true);
        // did a row outgrow its reference?
        const float m_cand = fmaxf(m_run, fmaxf(mxa, mxb) * exp_scale);
        const bool grow = m_cand - m_run > kRescaleThreshold;  // false when both are -inf (NaN)
        float alpha = 1.f;
        if (__any_sync(0xffffffffu, grow)) {
          // new reference for the rows that need one; the others repeat what they had
          const float m_new = grow ? m_cand : m_run;
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          alpha = grow ? fast_exp2(m_run - m_use) : 1.f;
          m_run = m_new;
          exp_pass(-m_use, false);
        }
        // hand the rescale factor to the correction warps
        s_alpha[s * 256 + ub * 128 + r] = alpha;
        mbar_arrive(bar_corr + 2 * s + ub);
        if ((warp & 3) == 0) trace_event(prm, s, t, 2);
        // P (two 16-bit values per column) over the first 32 columns of this step's buffer
        tmem_st16(tS, pr[0]);
        tmem_st16(tS + 16, pr[1]);
        if (more) {
          // S of step t + 1 was issued when P of step t - 1 was handed over: complete by now as a
          // rule.  Its loads go out behind the P stores; the score registers are free, everything
          // of step t is in pr.
          if constexpr (kExt != 0) {
            if (vec_bias && (t & 1) == 1) stage_vec_bias(t + 1);
            if (!vec_bias && bias_row != nullptr) {
              const int c0 = k0 + kStepN;
              prefetch_bias(prm.ex, bias_row, c0, min(kStepN, prm.Sk - c0));
            }
          }
          if (!s_next_ready)
            mbar_wait(bar_s_full + 2 * s + (ub ^ 1), ph_next, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
          tcgen05_fence_after_sync();
          issue_load(t + 1, 0);
          issue_load(t + 1, 1);
        }
        tcgen05_wait_st();
        tcgen05_fence_before_sync();
        mbar_arrive(bar_p_full + 2 * s + ub);
        if ((warp & 3) == 0) trace_event(prm, s, t, 3);
        const float rsum = (acc0.x + acc0.y) + (acc1.x + acc1.y);
        l_run = l_run * alpha + rsum;
        if (more) prep_loads(t + 1);
        if ((warp & 3) == 0) trace_event(prm, s, t, 5);
      }
      // The epilogue of the previous item must have read that item's row sums before these
      // replace them (it has, long ago, unless this item is only a step or two long).
      if (k > 0) mbar_wait(bar_o_free + s, (k - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_EPILOGUE);
      s_final[s * 256 + r] = l_run;
      s_final[s * 256 + 128 + r] = m_run;
      mbar_arrive(bar_final + s);
      g += T_s;
    }
  } else if (warp < 12) {
    // ================================ correction + epilogue ================================
    reg_dealloc<80>();
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    int g0 = 0, g1 = 0;  // steps of tile 0 / 1 in earlier items
    for (int k = 0;; ++k) {
      const int it = next_item(k);
      mbar_arrive(bar_item_empty + (k & 1));
      if (it < 0) break;
      const Ws64pItem w = ws64p_decode(prm, it);
      // epilogue of one query tile: O / l and LSE
      auto epilogue = [&](int s) {
        mbar_wait(bar_final + s, k & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
        mbar_wait(bar_o_done + s, k & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
        tcgen05_fence_after_sync();
        const float l_run = s_final[s * 256 + r];
        const float m_run = s_final[s * 256 + 128 + r];
        const float o_scale = (kExt != 0) ? prm.ex.drop_rescale : 1.f;
        const float inv_l = (l_run > 0.f) ? o_scale / l_run : 0.f;
        const int row = (2 * w.pair + s) * kBlockM + r;
        const bool row_ok = row < prm.Sq;
        uint16_t* orow = static_cast<uint16_t*>(prm.o) + w.b * prm.o_stride_b + w.h * prm.o_stride_h +
                         static_cast<int64_t>(row) * prm.o_stride_s;
        const uint32_t tO = tmem_base + Cfg::kColO0 + s * D + lane_base;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld32(tO + c * 32, orr);
          tmem_ld_wait(orr);
          if (c == D / 32 - 1) {
            // O and the row statistics are in registers: the tile's tensor memory and its slots in
            // shared memory may be reused
            tcgen05_fence_before_sync();
            mbar_arrive(bar_o_free + s);
          }
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
          prm.lse[static_cast<int64_t>(w.bh) * prm.Sq + row] =
              (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
        }
      };
      for (int t = 0; t < w.T1; ++t) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (t >= (s ? w.T1 : w.T0)) continue;
          const int gt = (s ? g1 : g0) + t;
          const int ub = gt & 1;
          mbar_wait(bar_corr + 2 * s + ub, (gt >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
          const float alpha = s_alpha[s * 256 + ub * 128 + r];
          if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
            // this step's P V is not issued before this warp arrives below; O is complete up to
            // the previous step once that step's P V has finished.  (The P V two steps back is
            // known to have finished, since S of this step exists: the phase bit is unambiguous.)
            mbar_wait(bar_o_full + s, (gt - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
            tcgen05_fence_after_sync();
            {
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
          mbar_arrive(bar_p_full + 2 * s + ub);
        }
        // With a causal mask tile 0 has two steps fewer than tile 1: its epilogue runs here, between
        // two arrivals for tile 1, instead of at the item's tail.
        if (t == w.T0 && w.T0 < w.T1) epilogue(0);
      }
      if (w.T0 == w.T1) epilogue(0);
      epilogue(1);
      g0 += w.T0;
      g1 += w.T1;
    }
  } else {
    reg_dealloc<64>();
    if (warp == 12 || warp == 14) {
      // ================================ MMA issuers ================================
      // One warp per query tile (12: tile 0, 14: tile 1).  The tensor core's instruction queue
      // is short: whenever the issuing warp is not issuing (a barrier wait costs it about 200
      // cycles even on a completed phase) the pipe runs dry.  With two issuers one tile's waits
      // hide behind the other tile's instructions.  Nothing orders the two streams against each
      // other, and nothing has to: each tile owns its S / P buffers and its O accumulator, and a
      // K/V ring slot is released by both warps (bar_kv_empty counts two arrivals).
      const int s = (warp == 14) ? 1 : 0;
      constexpr uint32_t idesc_qk = make_idesc(kBf16, kBlockM, kStepN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, kBlockM, D, 0, 1);
      // Everything below is warp-uniform; only the tcgen05 instructions themselves are issued by
      // one elected lane.  Descriptors are kept as 32-bit low halves: per instruction one add.
      const uint32_t q_lo = desc_lo(smem_u32(sQ) + s * kTileBytes, 16);
      const uint32_t kv_k_lo = desc_lo(smem_u32(sKV), 16);         // K tiles: K-major
      const uint32_t kv_v_lo = desc_lo(smem_u32(sKV), kBoxBytes);  // V tiles: N-major
      constexpr uint32_t kStageStep = kTileBytes >> 4;
      constexpr uint32_t kBoxStep = kBoxBytes >> 4;
      const uint32_t tS_tile = tmem_base + Cfg::kColS0 + s * kBlockN;
      const uint32_t tO = tmem_base + Cfg::kColO0 + s * D;
      // S into buffer `ub` = Q_s K^T over keys [64 uk, 64 uk + 64) of the K tile in ring slot `stage`:
      // 64 rows of a K-major box are 64 * 128 bytes further on
      auto issue_s = [&](int ub, int uk, int stage) {
        const uint32_t b_lo = kv_k_lo + stage * kStageStep + uk * ((kStepN * 128) >> 4);
        const uint32_t tS = tS_tile + ub * kStepN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // k-slice kk: box kk/4, 32 bytes per slice inside the 128-byte swizzle span
          const uint32_t off = (kk >> 2) * kBoxStep + (kk & 3) * 2;
          umma_ss_lo_elect(tS, q_lo + off, b_lo + off, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      // O_s (+)= P (buffer `ub`) V over key rows [64 uk, 64 uk + 64) of the V tile in ring slot `stage`
      auto issue_pv = [&](int ub, int uk, int stage, bool acc) {
        const uint32_t tP = tS_tile + ub * kStepN;
        const uint32_t b_lo = kv_v_lo + stage * kStageStep + uk * (kStepN / 16) * 128;
#pragma unroll
        for (int kk = 0; kk < kStepN / 16; ++kk) {
          // 16 key rows per slice: 2048 bytes of V, 8 packed columns of P
          umma_ts_lo_elect(tO, tP + kk * 8, b_lo + kk * 128, idesc_pv, (acc || kk > 0) ? 1u : 0u);
        }
      };

      int g = 0;   // steps of this tile in earlier items
      int ri = 0;  // K/V ring entries of earlier items
      for (int k = 0;; ++k) {
        const int it = next_item(k);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_item_empty + (k & 1));
        if (it < 0) break;
        const Ws64pItem w = ws64p_decode(prm, it);
        const int T_s = s ? w.T1 : w.T0;
        const int T1 = w.T1, n1 = w.n1;
        const int st0 = ri % kStages;  // K_0 of the item
        mbar_wait(bar_q_full, k & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        mbar_wait(bar_kv_full + st0, (ri / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
        tcgen05_fence_after_sync();
        // prologue: the first two steps, both on K_0.  Their buffers are free: the tensor core
        // runs one thread's instructions in order, and the P V that last read them was issued in
        // the previous item.
        issue_s(g & 1, 0, st0);
        tcgen05_commit_elect(bar_s_full + 2 * s + (g & 1));
        if (T_s > 1) {
          issue_s((g + 1) & 1, 1, st0);
          tcgen05_commit_elect(bar_s_full + 2 * s + ((g + 1) & 1));
        }
        tcgen05_commit_elect(bar_kv_empty + st0);
        if (T_s <= 2) tcgen05_commit_elect(bar_q_empty);  // this tile's last Q K^T has been issued
        // Barriers are polled (without blocking) one iteration ahead and waited on only if the
        // poll failed.
        bool p_ready = false, kv_ready = false;
        for (int t = 0; t < T1; ++t) {  // both warps walk all key tiles: the ring needs both
          const int j = t >> 1, uk = t & 1;
          const int iv = ri + 2 * j + 1;  // ring index of V_j; K_{j+1} is iv + 1
          const int st_v = iv % kStages;
          const int st_k = (iv + 1) % kStages;
          const bool k_next = j + 1 < n1;  // K_{j+1} exists
          if (uk == 0 && !kv_ready) {
            mbar_wait(bar_kv_full + st_v, (iv / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
            if (k_next) mbar_wait(bar_kv_full + st_k, ((iv + 1) / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
          }
          if (s == 0) trace_event(prm, 2, t, 0);
          kv_ready = false;
          if (t < T_s) {
            const int gt = g + t;
            const int ub = gt & 1;
            if (!p_ready)
              mbar_wait(bar_p_full + 2 * s + ub, (gt >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
            // the first P V of an item overwrites O: the previous item's epilogue must have read it
            if (t == 0 && k > 0) mbar_wait(bar_o_free + s, (k - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_EPILOGUE);
            tcgen05_fence_after_sync();
            if (s == 0) trace_event(prm, 2, t, 1);
            issue_pv(ub, uk, st_v, t > 0);
            tcgen05_commit_elect(bar_o_full + s);
            if (t + 1 == T_s) tcgen05_commit_elect(bar_o_done + s);
            if (s == 0) trace_event(prm, 2, t, 2);
            // step t + 2 goes into the buffer that P of step t is being read from; the tensor core
            // runs one thread's instructions in order, so the read comes first
            if (t + 2 < T_s) {
              issue_s(ub, uk, st_k);
              tcgen05_commit_elect(bar_s_full + 2 * s + ub);
              if (t + 3 == T_s) tcgen05_commit_elect(bar_q_empty);  // that was this tile's last Q K^T
            }
            if (s == 0) trace_event(prm, 2, t, 3);
            p_ready = (t + 1 < T_s) && mbar_test_wait(bar_p_full + 2 * s + (ub ^ 1), ((gt + 1) >> 1) & 1);
          }
          if (uk == 1 || t + 1 == T1) {
            // this warp's readers of V_j (and of K_{j+1}) have all been issued
            tcgen05_commit_elect(bar_kv_empty + st_v);
            if (k_next) tcgen05_commit_elect(bar_kv_empty + st_k);
            if (t + 1 < T1) {
              const int iv2 = iv + 2;
              kv_ready = mbar_test_wait(bar_kv_full + iv2 % kStages, (iv2 / kStages) & 1) &&
                         (!(j + 2 < n1) || mbar_test_wait(bar_kv_full + (iv2 + 1) % kStages, ((iv2 + 1) / kStages) & 1));
            }
          }
        }
        g += T_s;
        ri += 2 * n1;
      }
    } else if (warp == 13) {
      // ================================ scheduler + TMA producer ================================
      // Lane 0 does the work: it draws items, publishes each one to the other roles through a
      // two-slot ring in shared memory, and issues the item's loads: Q once the previous item's
      // Q K^T are done, K0 V0 K1 V1 ... as ring slots are released.  The first item is the CTA's
      // index; the others come from a counter in global memory.
      if (lane == 0) {
        const int G = static_cast<int>(gridDim.x);
        int it = static_cast<int>(blockIdx.x);
        int ri = 0;
        for (int k = 0;; ++k) {
          const int slot = k & 1;
          // every reader of the item that used this slot two items ago has taken it
          mbar_wait(bar_item_empty + slot, ((k >> 1) & 1) ^ 1, cta_abort, dstat, FO_STATUS_TIMEOUT_EPILOGUE);
          const bool valid = it < n_items && !*cta_abort;
          s_item[slot] = valid ? it : -1;
          mbar_arrive(bar_item_full + slot);
          if (!valid) break;
          const Ws64pItem w = ws64p_decode(prm, it);
          if (k > 0) mbar_wait(bar_q_empty, (k - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
          mbar_arrive_expect_tx(bar_q_full, 2 * kTileBytes);
          for (int s = 0; s < 2; ++s)
            for (int c = 0; c < kBoxes; ++c)
              tma_load_4d(sQ + s * kTileBytes + c * kBoxBytes, &tm_q, bar_q_full, c * kBoxCols,
                          (2 * w.pair + s) * kBlockM, w.h, w.b);
          for (int i = 0; i < 2 * w.n1; ++i) {  // ring entry: K_{i/2} (even) or V_{i/2} (odd)
            const int e = ri + i;
            const int st = e % kStages;
            mbar_wait(bar_kv_empty + st, ((e / kStages) & 1) ^ 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
            mbar_arrive_expect_tx(bar_kv_full + st, kTileBytes);
            const CUtensorMap* map = (i & 1) ? &tm_v : &tm_k;
            for (int c = 0; c < kBoxes; ++c)
              tma_load_4d(sKV + st * kTileBytes + c * kBoxBytes, map, bar_kv_full + st, c * kBoxCols,
                          (i >> 1) * kBlockN, w.hk, w.b);
          }
          ri += 2 * w.n1;
          // Drawn only now, when this item's loads are all on their way (a few steps before its
          // end): drawing earlier hands the second round of items to the CTAs that hold the
          // heaviest first-round items.
          it = G + atomicAdd(prm.sched, 1);
        }
      }
      __syncwarp();
    }
  }

  if (live) {
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  // The last CTA to finish puts the launch's scheduling words back to zero for the next launch
  // that is given them.
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(prm.sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      prm.sched[0] = 0;
      prm.sched[1] = 0;
      __threadfence();
    }
  }
}

template <int D, bool kBf16, int kExt>
int launch_ws64p(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& prm,
                cudaStream_t stream) {
  auto kernel = attn_fwd_ws64p_kernel<D, kBf16, kExt>;
  constexpr int smem = Ws64pConfig<D>::kSmemBytes;
  cudaError_t ea = ensure_dynamic_smem<attn_fwd_ws64p_kernel<D, kBf16, kExt>>(smem, prm.device);
  if (ea != cudaSuccess)
    return fail(FO_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", smem, cudaGetErrorString(ea));
  const int num_pairs = (prm.num_q_tiles + 1) / 2;
  const int64_t items = static_cast<int64_t>(num_pairs) * prm.B * prm.H;
  if (items > 0x3fffffffLL) return fail(FO_ERR_INVALID_ARGUMENT, "too many query tiles for one launch");
  // one CTA per SM (shared memory and tensor memory allow no second one), never more than items
  const int64_t ctas = items < prm.num_sms ? items : prm.num_sms;
  kernel<<<static_cast<unsigned>(ctas), 512, smem, stream>>>(tq, tk, tv, prm);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}

}  // namespace fo
