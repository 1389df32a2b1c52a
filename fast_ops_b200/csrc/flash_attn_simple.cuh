// Attention forward, bring-up kernel: one 128-row query tile per CTA, four warps, every step
// in program order (TMA load -> QK^T MMA -> softmax -> PV MMA).  It exercises the same
// descriptors, tensor-memory layout and softmax arithmetic as the pipelined kernel, with no
// overlap inside a CTA (two CTAs share an SM and cover some of each other's latency).  Kept as
// the always-available path and as the cross-check of the pipelined kernel.
#pragma once

#include "flash_attn_common.cuh"
#include "fo_host.h"

namespace fo {

template <int D>
constexpr int simple_smem_bytes() {
  return 3 * kBlockM * D * 2 + 1024 /* alignment slack */ + 128 /* barriers, slots */;
}

// grid = (num_q_tiles, B*H); block = 128.  blockIdx.x = 0 is the LAST query tile: with a
// causal mask it has the most key tiles, so the heavy tiles start first.
template <int D, bool kBf16>
__global__ void __launch_bounds__(128)
attn_fwd_simple_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const AttnParams prm) {
  constexpr int kTileBytes = kBlockM * D * 2;
  constexpr int kBoxes = D / kBoxCols;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColP = 0, kColO = 128;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes);
  uint64_t* bar_kv = bar_q + 1;
  uint64_t* bar_mma = bar_q + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 3);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip = cta_abort + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int q_tile = prm.num_q_tiles - 1 - static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int hk = prm.kv_head_bcast ? 0 : h;  // head coordinate of K and V
  const int q0 = q_tile * kBlockM;

  if (tid == 0) {
    *cta_abort = 0;
    // A CTA that starts after another one has timed out does no work at all.
    *skip = *reinterpret_cast<volatile int*>(prm.device_status);
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_mma, 1);
    fence_mbar_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  __syncthreads();
  if (*skip) return;

  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base + kColS;
  const uint32_t tP = tmem_base + kColP;
  const uint32_t tO = tmem_base + kColO;

  int n_kv = (prm.Sk + kBlockN - 1) / kBlockN;
  if (prm.causal && q_tile + 1 < n_kv) n_kv = q_tile + 1;

  constexpr uint32_t idesc_qk = make_idesc(kBf16, kBlockM, kBlockN, 0, 0);
  constexpr uint32_t idesc_pv = make_idesc(kBf16, kBlockM, D, 0, 1);

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_q, kTileBytes);
    for (int c = 0; c < kBoxes; ++c) tma_load_4d(sQ + c * kBoxBytes, &tm_q, bar_q, c * kBoxCols, q0, h, b);
  }

  const int row = q0 + tid;  // this thread's query row (tensor-memory lane tid)
  float m_run = -INFINITY;   // running row maximum, in the log2 domain (already scaled)
  float l_run = 0.f;         // running row sum of exp2(s - m_run)
  uint32_t phase_kv = 0, phase_mma = 0;

  mbar_wait(bar_q, 0, cta_abort, prm.device_status, FO_STATUS_TIMEOUT_TMA);

  for (int j = 0; j < n_kv; ++j) {
    const int k0 = j * kBlockN;
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
      for (int c = 0; c < kBoxes; ++c) tma_load_4d(sK + c * kBoxBytes, &tm_k, bar_kv, c * kBoxCols, k0, hk, b);
      for (int c = 0; c < kBoxes; ++c) tma_load_4d(sV + c * kBoxBytes, &tm_v, bar_kv, c * kBoxCols, k0, hk, b);
    }
    mbar_wait(bar_kv, phase_kv, cta_abort, prm.device_status, FO_STATUS_TIMEOUT_TMA);
    phase_kv ^= 1;

    // S = Q K^T  (128 x 128, K = D)
    if (tid == 0) {
      tcgen05_fence_after_sync();
      const uint32_t aq = smem_u32(sQ), ak = smem_u32(sK);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        umma_ss(tS, kmajor_desc(aq, kk), kmajor_desc(ak, kk), idesc_qk, kk > 0 ? 1u : 0u);
      tcgen05_commit(bar_mma);
    }
    mbar_wait(bar_mma, phase_mma, cta_abort, prm.device_status, FO_STATUS_TIMEOUT_MMA);
    phase_mma ^= 1;
    tcgen05_fence_after_sync();

    // ---- online softmax on this thread's row -------------------------------------------
    uint32_t sr[4][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld32(tS + lane_base + c * 32, sr[c]);
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld_wait(sr[c]);

    const bool need_mask = (k0 + kBlockN > prm.Sk) || (prm.causal && k0 + kBlockN - 1 > q0);
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float s = __uint_as_float(sr[c][i]);
        if (need_mask) {
          const int col = k0 + c * 32 + i;
          if (col >= prm.Sk || (prm.causal && col > row)) s = -INFINITY;
          sr[c][i] = __float_as_uint(s);
        }
        mx = fmaxf(mx, s);
      }
    }
    const float m_new = fmaxf(m_run, mx * prm.scale_log2);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // a fully masked row stays all-zero
    const float alpha = fast_exp2(m_run - m_use);
    float rsum = 0.f;
    uint32_t pr[2][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c][i]), prm.scale_log2, -m_use));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c][i + 1]), prm.scale_log2, -m_use));
        rsum += p0 + p1;
        pr[c >> 1][(c & 1) * 16 + (i >> 1)] = pack2<kBf16>(p0, p1);
      }
    }
    l_run = l_run * alpha + rsum;
    m_run = m_new;

    // O *= alpha (skipped by a warp none of whose rows moved its maximum)
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld32(tO + lane_base + c * 32, orr);
        tmem_ld_wait(orr);
#pragma unroll
        for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
        tmem_st32(tO + lane_base + c * 32, orr);
      }
    }
    // P (16-bit, two per column) over the first 64 columns of S
    tmem_st32(tP + lane_base, pr[0]);
    tmem_st32(tP + lane_base + 32, pr[1]);
    tcgen05_wait_st();
    tcgen05_fence_before_sync();
    __syncthreads();

    // O += P V  (128 x D, K = 128 key rows)
    if (tid == 0) {
      tcgen05_fence_after_sync();
      const uint32_t av = smem_u32(sV);
#pragma unroll
      for (int kk = 0; kk < kBlockN / 16; ++kk)
        umma_ts(tO, tP + kk * 8, nmajor_desc(av, kk), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
      tcgen05_commit(bar_mma);
    }
    mbar_wait(bar_mma, phase_mma, cta_abort, prm.device_status, FO_STATUS_TIMEOUT_MMA);
    phase_mma ^= 1;
    tcgen05_fence_after_sync();
  }

  // ---- epilogue: O / l -> global, LSE ---------------------------------------------------
  const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
  const bool row_ok = row < prm.Sq;
  uint16_t* orow = static_cast<uint16_t*>(prm.o) + b * prm.o_stride_b + h * prm.o_stride_h +
                   static_cast<int64_t>(row) * prm.o_stride_s;
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t orr[32];
    if (n_kv > 0) {
      tmem_ld32(tO + lane_base + c * 32, orr);
      tmem_ld_wait(orr);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) orr[i] = 0;
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
    const float lse = (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    prm.lse[(static_cast<int64_t>(bh)) * prm.Sq + row] = lse;
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace fo
