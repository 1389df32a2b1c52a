// Attention forward for short sequences: the 64-key-step pipeline of flash_attn_ws64.cuh with ONE
// 128-row query tile per CTA and TWO CTAs per SM.
//
// The kernel in flash_attn_ws64.cuh gives an SM one CTA that interleaves two query tiles; whatever
// a CTA does before its first and after its last step (barrier and tensor-memory set-up, the first
// loads' latency, the ramp of the pipeline, the epilogue) is time in which that SM computes
// nothing, and at a sequence length of 1024 to 2048 that is a third to a half of a CTA's life.
// Here the two tiles that share an SM are two independent CTAs: one's set-up and epilogue run
// under the other's steady state, and the two need no turn-taking protocol, since nothing ties
// their steps together.  The price is that each CTA loads K and V for its own tile (twice the
// shared-memory fill of the paired kernel), which is why the launcher uses this kernel only where
// a CTA's life is short.
//
// Per CTA (192 threads): warps 0-3 softmax, one thread per query row, which also rescale O on the
// rare steps whose reference maximum moves and write O and LSE at the end (there is no correction
// warpgroup); warp 4 issues the MMAs; warp 5 issues the TMA loads.  Tensor memory (256 columns):
// Sa | Sb | O.  Shared memory: Q (128 x D) and a ring of kStages HALF tiles (64 keys x D) of K and
// V in the order the MMA warp consumes them: K(0) K(1) V(0) K(2) V(1) K(3) ... (step t's P V
// needs V(t), and S of step t + 2 is issued right behind it); a slot is released as soon as the
// instruction that reads it has been issued, so four slots of 16 KB keep about two steps of loads in
// flight.  Plain attention only (no bias, no dropout).  No register reallocation between the roles
// (setmaxnreg): the CTA's six warps do not make whole warpgroups, and a version that used it did
// not return; the softmax code fits the 168 registers of the launch bound with 84 bytes of spills.
#pragma once

#include "flash_attn_common.cuh"
#include "flash_attn_ws.cuh"
#include "flash_attn_ws64.cuh"
#include "fo_host.h"

namespace fo {

template <int D>
struct Ws64sConfig {
  static constexpr int kQBytes = kBlockM * D * 2;     // one query tile
  static constexpr int kHalfBytes = kStepN * D * 2;   // 64 keys of K or of V
  static constexpr int kHalfBoxBytes = kStepN * kBoxCols * 2;  // a [64 rows x 64 columns] box: 8 KiB
  static constexpr int kStages = (D == 128) ? 4 : 8;  // five 16 KiB slots would put two CTAs 140 bytes over the SM
  static constexpr int kBoxes = D / kBoxCols;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kQBytes;
  static constexpr int kOffBars = kOffKV + kStages * kHalfBytes;
  // barriers: q_full, kv_full/empty per stage, s_full[2], p_full[2], o_full, o_done
  static constexpr int kNumBars = 1 + 2 * kStages + 2 + 2 + 1 + 1;
  static constexpr int kOffMisc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffMisc + 32 + 1024 /* alignment slack */;
  static constexpr uint32_t kTmemCols = 256;
  static constexpr uint32_t kColS = 0, kColO = 128;
};
// two CTAs per SM: 2 x (dynamic + 1 KiB reserved) must fit in the SM's 228 KiB
static_assert(2 * (Ws64sConfig<128>::kSmemBytes + 1024) <= 228 * 1024, "two CTAs of the D=128 kernel per SM");

// grid = num_q_tiles * B * H; block = 192.  Blocks sweep heads in L2-sized groups, inside a group
// tile-major with the last query tile (the most keys under a causal mask) first.
template <int D, bool kBf16>
__global__ void __launch_bounds__(192, 2)
attn_fwd_ws64s_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams prm) {
  using Cfg = Ws64sConfig<D>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBoxes = Cfg::kBoxes;
  constexpr int kHalfBytes = Cfg::kHalfBytes;
  constexpr int kHalfBoxBytes = Cfg::kHalfBoxBytes;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sKV = smem + Cfg::kOffKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* bar_q_full = bars;                     // TMA -> MMA
  uint64_t* bar_kv_full = bars + 1;                // [kStages] TMA -> MMA
  uint64_t* bar_kv_empty = bar_kv_full + kStages;  // [kStages] MMA -> TMA
  uint64_t* bar_s_full = bar_kv_empty + kStages;   // [2 buffers] MMA -> softmax
  uint64_t* bar_p_full = bar_s_full + 2;           // [2 buffers] softmax -> MMA (128 arrivals)
  uint64_t* bar_o_full = bar_p_full + 2;           // MMA -> softmax, once per P V (waited on only to rescale O)
  uint64_t* bar_o_done = bar_o_full + 1;           // MMA -> softmax, once: every P V has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffMisc);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip = cta_abort + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh_count = prm.B * prm.H;
  const int group_blocks = prm.head_group * prm.num_q_tiles;
  const int group = static_cast<int>(blockIdx.x) / group_blocks;
  const int in_group = static_cast<int>(blockIdx.x) - group * group_blocks;
  const int heads_here = min(prm.head_group, bh_count - group * prm.head_group);
  const int q_tile = prm.num_q_tiles - 1 - in_group / heads_here;
  const int bh = group * prm.head_group + in_group % heads_here;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int hk = prm.kv_head_bcast ? 0 : h;  // head coordinate of K and V
  const int q0 = q_tile * kBlockM;
  const int vis = prm.causal ? min(prm.Sk, q0 + kBlockM) : prm.Sk;  // keys this tile sees
  const int T = (vis + kStepN - 1) / kStepN;                       // 64-key steps, >= 1
  // ring entries: K(0), K(1) if it exists, then per step t: V(t), K(t + 2) if it exists
  const int n_entries = 2 * T;

  if (tid == 0) {
    *cta_abort = 0;
    *skip = *reinterpret_cast<volatile int*>(prm.device_status);
    mbar_init(bar_q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kv_full + i, 1);
      mbar_init(bar_kv_empty + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + i, 1);
      mbar_init(bar_p_full + i, 128);
    }
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_done, 1);
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*skip) return;  // another CTA already timed out: do nothing

  // Ring entry e holds 64 keys of K or of V: which, and which 64, in consumption order:
  // K(0), K(1), then pairs (V(t), K(t + 2)) while K(t + 2) exists, then the V's that are left.
  auto entry_of = [&](int e, bool& is_v, int& half) {
    // K(0), K(1) lead (only K(0) if T == 1)
    const int lead = T > 1 ? 2 : 1;
    if (e < lead) { is_v = false; half = e; return; }
    const int r = e - lead;            // position after the lead
    const int pairs = T - lead;        // steps t for which K(t + 2) exists: t = 0 .. T - 3 (T - lead of them)
    if (r < 2 * pairs) { is_v = (r & 1) == 0; half = is_v ? (r >> 1) : (r >> 1) + 2; return; }
    is_v = true;                       // the remaining V's: t = pairs .. T - 1
    half = pairs + (r - 2 * pairs);
  };
  auto load_entry = [&](int e) {
    bool is_v; int half;
    entry_of(e, is_v, half);
    const int st = e % kStages;
    mbar_arrive_expect_tx(bar_kv_full + st, kHalfBytes);
    const CUtensorMap* map = is_v ? &tm_v : &tm_k;
    for (int c = 0; c < kBoxes; ++c)
      tma_load_4d(sKV + st * kHalfBytes + c * kHalfBoxBytes, map, bar_kv_full + st, c * kBoxCols, half * kStepN, hk, b);
  };
  // The first loads need only the barriers: they go out under the tensor-memory allocation.
  const int first_fill = min(kStages, n_entries);
  if (warp == 5 && lane == 0) {
    mbar_arrive_expect_tx(bar_q_full, Cfg::kQBytes);
    for (int c = 0; c < kBoxes; ++c)
      tma_load_4d(sQ + c * kBoxBytes, &tm_q, bar_q_full, c * kBoxCols, q0, h, b);
    for (int e = 0; e < first_fill; ++e) load_entry(e);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int* const dstat = prm.device_status;

  if (warp < 4) {
    // ================================ softmax, rescale, epilogue ================================
    const int r = warp * 32 + lane;
    const int row = q0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tS_tile = tmem_base + Cfg::kColS + lane_base;
    const uint32_t tO = tmem_base + Cfg::kColO + lane_base;
    const float exp_scale = prm.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t sr[2][32];  // scores of the current step

    auto issue_load = [&](int tn, int c) { tmem_ld32(tS_tile + (tn & 1) * kStepN + c * 32, sr[c]); };
    // Waits for those loads and applies the masks in place.
    auto prep_loads = [&](int tn) {
      const int k0n = tn * kStepN;
      const bool need_mask = (k0n + kStepN > prm.Sk) || (prm.causal && k0n + kStepN - 1 > q0);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld_wait(sr[c]);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0n + c * 32 + i;
            if (col >= prm.Sk || (prm.causal && col > row)) sr[c][i] = 0xff800000u;  // -inf
          }
        }
      }
    };

    // prologue: scores of step 0; their row maximum is the first reference maximum
    mbar_wait(bar_s_full + 0, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
    tcgen05_fence_after_sync();
    issue_load(0, 0);
    issue_load(0, 1);
    prep_loads(0);
    {
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
      m_run = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd)) * exp_scale;
    }

    // As in flash_attn_ws64.cuh: a step's exponentials are taken against the reference maximum the
    // row already has, its own maximum is reduced alongside, and only a row that outgrows its
    // reference (by kRescaleThreshold) makes the warp take the step's exponentials again.
    for (int t = 0; t < T; ++t) {
      const int u = t & 1;
      const uint32_t tS = tS_tile + u * kStepN;
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      const float2 sc2 = make_float2(exp_scale, exp_scale);
      float2 acc0, acc1;
      uint32_t pr[2][16];
      const bool more = t + 1 < T;
      bool s_next_ready = false;
      float mxa = -INFINITY, mxb = -INFINITY;
      auto exp_pass = [&](float neg_ref, const bool first) {
        const float2 nm2 = make_float2(neg_ref, neg_ref);
        acc0 = make_float2(0.f, 0.f);
        acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // one non-blocking look at S of step t + 1; the answer is needed only after the exponentials
          if (first && c == 1 && more) s_next_ready = mbar_test_wait(bar_s_full + (u ^ 1), ((t + 1) >> 1) & 1);
#pragma unroll
          for (int q = 0; q < 16; ++q) {  // column pair q of the chunk
            const float a = __uint_as_float(sr[c][2 * q]), bb = __uint_as_float(sr[c][2 * q + 1]);
            float2 x = __ffma2_rn(make_float2(a, bb), sc2, nm2);
            x.x = fast_exp2(x.x);
            x.y = fast_exp2(x.y);
            if (q & 1) acc1 = __fadd2_rn(acc1, x); else acc0 = __fadd2_rn(acc0, x);
            if (first) {
              if (q & 1) mxb = max3(mxb, a, bb); else mxa = max3(mxa, a, bb);
            }
            pr[c][q] = pack2<kBf16>(x.x, x.y);
          }
        }
      };
      exp_pass(neg_m, true);
      const float m_cand = fmaxf(m_run, fmaxf(mxa, mxb) * exp_scale);
      const bool grow = m_cand - m_run > kRescaleThreshold;  // false when both are -inf (NaN)
      float alpha = 1.f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? m_cand : m_run;
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha = grow ? fast_exp2(m_run - m_use) : 1.f;
        m_run = m_new;
        exp_pass(-m_use, false);
        if (t > 0) {
          // O holds the sum up to step t - 1 once that step's P V has finished (the P V two steps
          // back is known to have finished, since S of this step exists: the phase is unambiguous);
          // this step's P V is not issued before this warp arrives on p_full below.
          mbar_wait(bar_o_full, (t - 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
          tcgen05_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld32(tO + c * 32, orr);
            tmem_ld_wait(orr);
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(tO + c * 32, orr);
          }
        }
      }
      // P (two 16-bit values per column) over the first 32 columns of this step's buffer
      tmem_st16(tS, pr[0]);
      tmem_st16(tS + 16, pr[1]);
      if (more) {
        if (!s_next_ready)
          mbar_wait(bar_s_full + (u ^ 1), ((t + 1) >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
        tcgen05_fence_after_sync();
        issue_load(t + 1, 0);
        issue_load(t + 1, 1);
      }
      tcgen05_wait_st();
      tcgen05_fence_before_sync();
      mbar_arrive(bar_p_full + u);
      const float rsum = (acc0.x + acc0.y) + (acc1.x + acc1.y);
      l_run = l_run * alpha + rsum;
      if (more) prep_loads(t + 1);
    }

    // epilogue: O / l and LSE, when every P V has finished
    mbar_wait(bar_o_done, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
    tcgen05_fence_after_sync();
    const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
    const bool row_ok = row < prm.Sq;
    uint16_t* orow = static_cast<uint16_t*>(prm.o) + b * prm.o_stride_b + h * prm.o_stride_h +
                     static_cast<int64_t>(row) * prm.o_stride_s;
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
  } else if (warp == 4) {
    // ================================ MMA issuer ================================
    constexpr uint32_t idesc_qk = make_idesc(kBf16, kBlockM, kStepN, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(kBf16, kBlockM, D, 0, 1);
    const uint32_t q_lo = desc_lo(smem_u32(sQ), 16);
    const uint32_t kv_k_lo = desc_lo(smem_u32(sKV), 16);             // K halves: K-major
    const uint32_t kv_v_lo = desc_lo(smem_u32(sKV), kHalfBoxBytes);  // V halves: N-major, 64-column blocks 8 KiB apart
    constexpr uint32_t kStageStep = kHalfBytes >> 4;
    constexpr uint32_t kQBoxStep = kBoxBytes >> 4;
    constexpr uint32_t kHalfBoxStep = kHalfBoxBytes >> 4;
    const uint32_t tS_tile = tmem_base + Cfg::kColS;
    const uint32_t tO = tmem_base + Cfg::kColO;
    // S into buffer u = Q K^T over the 64 keys in ring slot `stage`
    auto issue_s = [&](int u, int stage) {
      const uint32_t b_lo = kv_k_lo + stage * kStageStep;
      const uint32_t tS = tS_tile + u * kStepN;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        // k-slice kk: box kk/4 of Q (16 KiB boxes) and of the K half (8 KiB boxes), 32 bytes per slice
        umma_ss_lo_elect(tS, q_lo + (kk >> 2) * kQBoxStep + (kk & 3) * 2, b_lo + (kk >> 2) * kHalfBoxStep + (kk & 3) * 2,
                         idesc_qk, kk > 0 ? 1u : 0u);
      }
    };
    // O (+)= P (buffer u) V over the 64 keys in ring slot `stage`
    auto issue_pv = [&](int u, int stage, bool acc) {
      const uint32_t tP = tS_tile + u * kStepN;
      const uint32_t b_lo = kv_v_lo + stage * kStageStep;
#pragma unroll
      for (int kk = 0; kk < kStepN / 16; ++kk)  // 16 key rows per slice: 2048 bytes of V, 8 packed columns of P
        umma_ts_lo_elect(tO, tP + kk * 8, b_lo + kk * 128, idesc_pv, (acc || kk > 0) ? 1u : 0u);
    };
    auto wait_entry = [&](int e) {
      mbar_wait(bar_kv_full + e % kStages, (e / kStages) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
    };

    mbar_wait(bar_q_full, 0, cta_abort, dstat, FO_STATUS_TIMEOUT_TMA);
    int e = 0;  // next ring entry, in the order of entry_of
    wait_entry(e);
    tcgen05_fence_after_sync();
    issue_s(0, e % kStages);
    tcgen05_commit_elect(bar_s_full + 0);
    tcgen05_commit_elect(bar_kv_empty + e % kStages);
    ++e;
    if (T > 1) {
      wait_entry(e);
      tcgen05_fence_after_sync();
      issue_s(1, e % kStages);
      tcgen05_commit_elect(bar_s_full + 1);
      tcgen05_commit_elect(bar_kv_empty + e % kStages);
      ++e;
    }
    bool p_ready = false;
    for (int t = 0; t < T; ++t) {
      const int u = t & 1;
      wait_entry(e);  // V(t)
      if (!p_ready) mbar_wait(bar_p_full + u, (t >> 1) & 1, cta_abort, dstat, FO_STATUS_TIMEOUT_SOFTMAX);
      tcgen05_fence_after_sync();
      issue_pv(u, e % kStages, t > 0);
      tcgen05_commit_elect(bar_o_full);
      if (t + 1 == T) tcgen05_commit_elect(bar_o_done);
      tcgen05_commit_elect(bar_kv_empty + e % kStages);
      ++e;
      // step t + 2 goes into the buffer that P of step t is being read from; the tensor core runs
      // one thread's instructions in order, so the read comes first
      if (t + 2 < T) {
        wait_entry(e);  // K(t + 2)
        tcgen05_fence_after_sync();
        issue_s(u, e % kStages);
        tcgen05_commit_elect(bar_s_full + u);
        tcgen05_commit_elect(bar_kv_empty + e % kStages);
        ++e;
      }
      p_ready = (t + 1 < T) && mbar_test_wait(bar_p_full + (u ^ 1), ((t + 1) >> 1) & 1);
    }
  } else {
    // ================================ TMA producer ================================
    const bool issuer = lane == 0;
    for (int e = first_fill; e < n_entries; ++e) {  // the rest of the ring, as slots are released
      mbar_wait(bar_kv_empty + e % kStages, ((e / kStages) & 1) ^ 1, cta_abort, dstat, FO_STATUS_TIMEOUT_MMA);
      if (issuer) load_entry(e);
      __syncwarp();
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D, bool kBf16>
int launch_ws64s(const CUtensorMap& tq, const CUtensorMap& tk_half, const CUtensorMap& tv_half, const AttnParams& prm,
                 cudaStream_t stream) {
  auto kernel = attn_fwd_ws64s_kernel<D, kBf16>;
  constexpr int smem = Ws64sConfig<D>::kSmemBytes;
  cudaError_t ea = ensure_dynamic_smem<attn_fwd_ws64s_kernel<D, kBf16>>(smem, prm.device);
  if (ea != cudaSuccess)
    return fail(FO_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", smem, cudaGetErrorString(ea));
  const int64_t blocks = static_cast<int64_t>(prm.num_q_tiles) * prm.B * prm.H;
  if (blocks > 0x7fffffffLL) return fail(FO_ERR_INVALID_ARGUMENT, "too many query tiles for one launch");
  kernel<<<static_cast<unsigned>(blocks), 192, smem, stream>>>(tq, tk_half, tv_half, prm);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}

}  // namespace fo
