// FlashAttention forward for sm_100a: host launcher behind fo_flash_attn_fwd, the tensor-map
// (TMA descriptor) construction, and the one-tile self-test of the tensor-core building blocks.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "flash_attn_simple.cuh"
#include "flash_attn_ws.cuh"
#include "flash_attn_ws64.cuh"
#include "flash_attn_ws64p.cuh"
#include "flash_attn_ws64s.cuh"
#include "fo_host.h"
#include "fo_tma.h"

namespace fo {
// Debug timeline buffer handed to the next attention launches (null = off).
unsigned long long* g_attn_trace = nullptr;
AttnOptions g_attn_options;
}  // namespace fo

namespace {

// Scheduling words of the persistent forward kernel: every launch is given one pair (round robin),
// which its last CTA zeroes again.  Launches that run at the same time (different streams) thus
// use different pairs unless more than kSchedSlots of them are in flight at once.
constexpr int kSchedSlots = 1024;
__device__ int g_attn_sched[kSchedSlots][2];
std::atomic<unsigned> g_sched_next{0};

struct DeviceInfo {
  int* sched = nullptr;  // device address of g_attn_sched
  int num_sms = 0;
};

// Per-device facts a launch needs, looked up once (with the device current).
const DeviceInfo* device_info(int device) {
  static std::mutex mu;
  static DeviceInfo info[64];
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = info[device];
  if (d.sched == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_attn_sched) != cudaSuccess || p == nullptr) return nullptr;
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return nullptr;
    d.num_sms = n;
    d.sched = static_cast<int*>(p);
  }
  return &d;
}

using fo::AttnParams;
using fo::g_attn_trace;
using fo::kBlockM;
using fo::kBlockN;
using fo::kBoxCols;

using fo::make_tensor_map;

// ---- one-tile self-test ------------------------------------------------------------------------
// mode 0: C = A B^T, A (128 x K) and B (N x K) K-major through TMA (the QK^T path).
// mode 1: C = A B, A (128 x K) placed in tensor memory by the threads as packed 16-bit pairs,
//         B (K x N) with N contiguous through TMA (the PV path).
template <bool kBf16>
__global__ void __launch_bounds__(128)
umma_tile_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const uint16_t* __restrict__ a_global, float* __restrict__ c, int N, int K, int mode,
                 int* device_status) {
  using namespace fo;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sA = smem;               // up to 2 boxes
  uint8_t* sB = smem + 2 * kBoxBytes;  // up to 2 boxes
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + 4 * kBoxBytes);
  uint64_t* bar_mma = bar_tma + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    *cta_abort = 0;
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tC = tmem_base;        // N fp32 columns
  const uint32_t tA = tmem_base + 128;  // K/2 packed columns (mode 1)

  if (mode == 0) {
    // A: rows 0..127, K columns -> K/64 boxes; B: rows 0..N-1 (box is 128 rows; rows >= N are
    // zero-filled), K columns.
    if (tid == 0) {
      const int boxes = K / kBoxCols;
      mbar_arrive_expect_tx(bar_tma, 2 * boxes * kBoxBytes);
      for (int cb = 0; cb < boxes; ++cb) tma_load_4d(sA + cb * kBoxBytes, &tm_a, bar_tma, cb * kBoxCols, 0, 0, 0);
      for (int cb = 0; cb < boxes; ++cb) tma_load_4d(sB + cb * kBoxBytes, &tm_b, bar_tma, cb * kBoxCols, 0, 0, 0);
    }
    mbar_wait(bar_tma, 0, cta_abort, device_status, FO_STATUS_TIMEOUT_TMA);
    if (tid == 0) {
      tcgen05_fence_after_sync();
      const uint32_t idesc = make_idesc(kBf16, 128, N, 0, 0);
      for (int kk = 0; kk < K / 16; ++kk)
        umma_ss(tC, kmajor_desc(smem_u32(sA), kk), kmajor_desc(smem_u32(sB), kk), idesc, kk > 0 ? 1u : 0u);
      tcgen05_commit(bar_mma);
    }
  } else {
    // B: K rows (box: 128 rows, rows >= K zero-filled), N columns -> N/64 boxes.
    if (tid == 0) {
      const int boxes = N / kBoxCols;
      mbar_arrive_expect_tx(bar_tma, boxes * kBoxBytes);
      for (int cb = 0; cb < boxes; ++cb) tma_load_4d(sB + cb * kBoxBytes, &tm_b, bar_tma, cb * kBoxCols, 0, 0, 0);
    }
    // A: thread t writes row t as packed pairs (element 2c in the low half of column c).
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(a_global + static_cast<size_t>(tid) * K);
    for (int cb = 0; cb < K / 2; cb += 32) {
      uint32_t regs[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) regs[i] = arow[cb + i];
      tmem_st32(tA + lane_base + cb, regs);
    }
    tcgen05_wait_st();
    tcgen05_fence_before_sync();
    mbar_wait(bar_tma, 0, cta_abort, device_status, FO_STATUS_TIMEOUT_TMA);
    __syncthreads();
    if (tid == 0) {
      tcgen05_fence_after_sync();
      const uint32_t idesc = make_idesc(kBf16, 128, N, 0, 1);
      for (int kk = 0; kk < K / 16; ++kk)
        umma_ts(tC, tA + kk * 8, nmajor_desc(smem_u32(sB), kk), idesc, kk > 0 ? 1u : 0u);
      tcgen05_commit(bar_mma);
    }
  }
  mbar_wait(bar_mma, 0, cta_abort, device_status, FO_STATUS_TIMEOUT_MMA);
  tcgen05_fence_after_sync();
  for (int cb = 0; cb < N; cb += 32) {
    uint32_t regs[32];
    tmem_ld32(tC + lane_base + cb, regs);
    tmem_ld_wait(regs);
#pragma unroll
    for (int i = 0; i < 32; ++i) c[static_cast<size_t>(tid) * N + cb + i] = __uint_as_float(regs[i]);
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

enum class AttnImpl { kAuto = 0, kSimple = 1, kWarpSpecialized = 2, kWarpSpecialized64 = 3, kPersistent64 = 4, kShort64 = 5 };

template <int D, bool kBf16>
int launch_simple(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& prm,
                  cudaStream_t stream) {
  auto kernel = fo::attn_fwd_simple_kernel<D, kBf16>;
  constexpr int smem = fo::simple_smem_bytes<D>();
  FO_CUDA_CHECK((fo::ensure_dynamic_smem<fo::attn_fwd_simple_kernel<D, kBf16>>(smem, prm.device)));
  dim3 grid(prm.num_q_tiles, prm.B * prm.H);
  kernel<<<grid, 128, smem, stream>>>(tq, tk, tv, prm);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

}  // namespace

namespace fo {

// Validates the optional bias / dropout arguments of the extended entry points and fills `ex`.
int make_attn_extras(AttnExtras* ex, const void* bias, const int64_t* bias_strides, int bias_dtype, int dtype,
                     float dropout_p, uint64_t rng_seed, uint64_t rng_offset) {
  std::memset(ex, 0, sizeof(*ex));
  ex->drop_rescale = 1.f;
  if (bias != nullptr) {
    FO_REQUIRE(bias_strides != nullptr, "bias given without strides");
    FO_REQUIRE(bias_dtype == FO_F32 || bias_dtype == dtype,
               "bias must be fp32 or have the dtype of q (got dtype %d)", bias_dtype);
    for (int i = 0; i < 3; ++i) FO_REQUIRE(bias_strides[i] >= 0, "bias: strides must be non-negative");
    ex->bias = bias;
    ex->bias_stride_b = bias_strides[0];
    ex->bias_stride_h = bias_strides[1];
    ex->bias_stride_q = bias_strides[2];
    ex->bias_f32 = bias_dtype == FO_F32;
    const int per16 = ex->bias_f32 ? 4 : 8;  // elements per 16 bytes
    ex->bias_vec = (reinterpret_cast<uintptr_t>(bias) & 15) == 0 && bias_strides[0] % per16 == 0 &&
                   bias_strides[1] % per16 == 0 && bias_strides[2] % per16 == 0;
  }
  FO_REQUIRE(dropout_p >= 0.f && dropout_p < 1.f, "dropout_p must be in [0, 1) (got %g)", (double)dropout_p);
  if (dropout_p > 0.f) {
    ex->dropout = 1;
    // fast_ops/flash_attention/flash_attention_triton.py:50: keep iff hash > uint32(p * 4294967295),
    // the product formed in fp32 (where 4294967295 rounds to 2^32) and truncated
    const float prod = dropout_p * 4294967296.f;
    ex->drop_threshold = prod >= 4294967296.f ? 0xffffffffu : static_cast<uint32_t>(prod);
    ex->drop_seed = static_cast<uint32_t>(rng_seed);
    ex->drop_base = static_cast<uint32_t>(rng_offset);
    ex->drop_rescale = 1.f / (1.f - dropout_p);
  }
  return FO_OK;
}

}  // namespace fo

static int attn_fwd_impl(const void* q, const void* k, const void* v, void* o, float* lse,
                         int B, int H, int Sq, int Sk, int D,
                         const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t o_strides[3],
                         int dtype, int causal, float softmax_scale, const fo::AttnExtras* ex,
                         int device, void* stream) {
  FO_REQUIRE(q && k && v && o, "null tensor pointer");
  FO_REQUIRE(q_strides && k_strides && v_strides && o_strides, "null stride array");
  FO_REQUIRE(dtype == FO_F16 || dtype == FO_BF16, "attention inputs must be fp16 or bf16 (got dtype %d)", dtype);
  FO_REQUIRE(B > 0 && H > 0 && Sq > 0 && Sk > 0, "B, H, Sq, Sk must be positive (got %d %d %d %d)", B, H, Sq, Sk);
  FO_REQUIRE(static_cast<int64_t>(B) * H <= 65535, "B*H must be <= 65535 (got %lld)", (long long)B * H);
  if (D <= 0 || D > 128 || D % 8 != 0)
    return fo::fail(FO_ERR_INVALID_ARGUMENT, "head_dim must be a multiple of 8 and <= 128 (got %d)", D);
  const int Dk = D <= 64 ? 64 : 128;  // head_dim the kernel is built for
  FO_REQUIRE(softmax_scale > 0.f && std::isfinite(softmax_scale), "softmax_scale must be positive and finite");
  FO_REQUIRE((reinterpret_cast<uintptr_t>(o) & 15) == 0, "o must be 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    FO_REQUIRE(o_strides[i] % 8 == 0 && o_strides[i] >= 0, "o: strides must be non-negative multiples of 8 elements");

  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  int* status = fo::device_status_ptr(device);
  if (!status) return fo::fail(FO_ERR_CUDA, "cannot resolve the status word of device %d", device);

  CUtensorMap tq, tk, tv;
  if (int rc = make_tensor_map(&tq, q, dtype, B, H, Sq, D, q_strides, "q")) return rc;
  // Multi-query attention: K and V expanded over the head dimension with stride 0 (one shared
  // head, as the reference's tests build it, tests/test_flash_attention_triton.py:71-73) are
  // described to TMA as single-head tensors and every query head reads head 0.
  const bool kv_bcast = H > 1 && k_strides[1] == 0 && v_strides[1] == 0;
  FO_REQUIRE(kv_bcast || H == 1 || (k_strides[1] != 0 && v_strides[1] != 0),
             "k and v must both have a head stride, or both be expanded with head stride 0");
  const int Hkv = kv_bcast ? 1 : H;
  if (int rc = make_tensor_map(&tk, k, dtype, B, Hkv, Sk, D, k_strides, "k")) return rc;
  if (int rc = make_tensor_map(&tv, v, dtype, B, Hkv, Sk, D, v_strides, "v")) return rc;

  AttnParams prm;
  prm.o = o;
  prm.lse = lse;
  prm.o_stride_b = o_strides[0];
  prm.o_stride_h = o_strides[1];
  prm.o_stride_s = o_strides[2];
  prm.B = B;
  prm.H = H;
  prm.Sq = Sq;
  prm.Sk = Sk;
  prm.d_real = D;
  prm.causal = causal ? 1 : 0;
  prm.scale_log2 = softmax_scale * 1.4426950408889634f;
  prm.device_status = status;
  prm.num_q_tiles = (Sq + kBlockM - 1) / kBlockM;
  prm.trace = g_attn_trace;
  prm.kv_head_bcast = kv_bcast ? 1 : 0;
  prm.ping_pong = fo::g_attn_options.ping_pong.load(std::memory_order_relaxed);
  prm.device = device;
  const DeviceInfo* info = device_info(device);
  if (!info) return fo::fail(FO_ERR_CUDA, "cannot look up device %d", device);
  prm.num_sms = info->num_sms;
  prm.sched = info->sched + 2 * (g_sched_next.fetch_add(1, std::memory_order_relaxed) % kSchedSlots);
  std::memset(&prm.ex, 0, sizeof(prm.ex));
  prm.ex.drop_rescale = 1.f;
  const bool ext = ex != nullptr && (ex->bias != nullptr || ex->dropout);
  if (ext) prm.ex = *ex;
  {
    // as many heads per group as keep their K and V (2 * Sk * D * 2 bytes each) within about a
    // third of the 126 MB L2, leaving room for Q, O and the other traffic
    const int64_t kv_bytes = 4LL * Sk * D;
    int64_t g = (40LL << 20) / kv_bytes;
    const int forced = fo::g_attn_options.head_group.load(std::memory_order_relaxed);
    if (forced > 0) g = forced;
    if (g < 1) g = 1;
    if (g > static_cast<int64_t>(B) * H) g = static_cast<int64_t>(B) * H;
    prm.head_group = static_cast<int>(g);
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == FO_BF16;
  AttnImpl impl = static_cast<AttnImpl>(fo::g_attn_options.impl.load(std::memory_order_relaxed));
  if (impl == AttnImpl::kAuto) {
    // The 64-key-step kernel is the faster one at every shape measured (same box, hot loop, bf16
    // causal: S=16384 1.11 against 1.02 PFLOP/s, S=4096 0.98 against 0.82, GPT-2-small shape
    // 0.29 against 0.21); the 128-key kernel stays selectable.
    impl = AttnImpl::kWarpSpecialized64;
    // one exception, also measured: with a bias and no dropout, over a long key range, the
    // 128-key kernel is about 7 % ahead (0.79 against 0.73 PFLOP/s at S=16384)
    const int n_kv = (Sk + kBlockN - 1) / kBlockN;
    const bool bias_only = ext && ex->bias != nullptr && !ex->dropout;
    if (bias_only && (causal ? (n_kv + 1) / 2 : n_kv) > 48) impl = AttnImpl::kWarpSpecialized;
    // Plain attention where a CTA's life is short or the grid is small runs one query tile per CTA
    // and two CTAs per SM (measured, bf16 causal, same box: D=64 8 to 28 % ahead at every length
    // from 512 to 8192; D=128 3 % ahead at S=1024, 5 % behind at S=2048, 10 % behind at S=16384,
    // and 7 to 12 % ahead when the query-tile pairs would not fill the SMs once).
    if (!ext) {
      const int64_t pair_items = static_cast<int64_t>((prm.num_q_tiles + 1) / 2) * B * H;
      if (Dk == 64 || Sk <= 1024 || pair_items <= info->num_sms) impl = AttnImpl::kShort64;
    }
  }
  const int mode = ext ? ((prm.ex.bias != nullptr ? 1 : 0) | (prm.ex.dropout ? 2 : 0)) : 0;
  // bias and dropout exist in the warp-specialised kernels only
#define FO_WS_MODE(LAUNCH, M)                                                                          \
  if (mode == M) {                                                                                     \
    if (Dk == 128) return bf16 ? fo::LAUNCH<128, true, M>(tq, tk, tv, prm, s) : fo::LAUNCH<128, false, M>(tq, tk, tv, prm, s); \
    return bf16 ? fo::LAUNCH<64, true, M>(tq, tk, tv, prm, s) : fo::LAUNCH<64, false, M>(tq, tk, tv, prm, s);                 \
  }
  if (impl == AttnImpl::kShort64 && mode == 0) {
    // one query tile per CTA, two CTAs per SM: K and V are loaded in 64-key halves
    CUtensorMap tkh, tvh;
    if (int rc = make_tensor_map(&tkh, k, dtype, B, Hkv, Sk, D, k_strides, "k", fo::kStepN)) return rc;
    if (int rc = make_tensor_map(&tvh, v, dtype, B, Hkv, Sk, D, v_strides, "v", fo::kStepN)) return rc;
    if (Dk == 128) return bf16 ? fo::launch_ws64s<128, true>(tq, tkh, tvh, prm, s) : fo::launch_ws64s<128, false>(tq, tkh, tvh, prm, s);
    return bf16 ? fo::launch_ws64s<64, true>(tq, tkh, tvh, prm, s) : fo::launch_ws64s<64, false>(tq, tkh, tvh, prm, s);
  }
  if (impl == AttnImpl::kShort64) impl = AttnImpl::kWarpSpecialized64;  // bias and dropout: the paired kernel
  if (impl == AttnImpl::kPersistent64) {
    FO_WS_MODE(launch_ws64p, 0)  // plain attention only; bias and dropout run in the 64-key kernel
    impl = AttnImpl::kWarpSpecialized64;
  }
  if (impl == AttnImpl::kWarpSpecialized64) {
    FO_WS_MODE(launch_ws64, 0)
    FO_WS_MODE(launch_ws64, 1)
    FO_WS_MODE(launch_ws64, 2)
    FO_WS_MODE(launch_ws64, 3)
  }
  if (impl != AttnImpl::kSimple || mode != 0) {
    FO_WS_MODE(launch_ws, 0)
    FO_WS_MODE(launch_ws, 1)
    FO_WS_MODE(launch_ws, 2)
    FO_WS_MODE(launch_ws, 3)
  }
#undef FO_WS_MODE
  if (Dk == 128) return bf16 ? launch_simple<128, true>(tq, tk, tv, prm, s) : launch_simple<128, false>(tq, tk, tv, prm, s);
  return bf16 ? launch_simple<64, true>(tq, tk, tv, prm, s) : launch_simple<64, false>(tq, tk, tv, prm, s);
}

extern "C" int fo_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                                 int B, int H, int Sq, int Sk, int D,
                                 const int64_t q_strides[3], const int64_t k_strides[3],
                                 const int64_t v_strides[3], const int64_t o_strides[3],
                                 int dtype, int causal, float softmax_scale, int device, void* stream) {
  fo::clear_error();
  return attn_fwd_impl(q, k, v, o, lse, B, H, Sq, Sk, D, q_strides, k_strides, v_strides, o_strides, dtype, causal,
                       softmax_scale, nullptr, device, stream);
}

extern "C" int fo_flash_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse,
                                    int B, int H, int Sq, int Sk, int D,
                                    const int64_t q_strides[3], const int64_t k_strides[3],
                                    const int64_t v_strides[3], const int64_t o_strides[3],
                                    int dtype, int causal, float softmax_scale,
                                    const void* bias, const int64_t bias_strides[3], int bias_dtype,
                                    float dropout_p, uint64_t rng_seed, uint64_t rng_offset,
                                    int device, void* stream) {
  fo::clear_error();
  FO_REQUIRE(dtype == FO_F16 || dtype == FO_BF16, "attention inputs must be fp16 or bf16 (got dtype %d)", dtype);
  fo::AttnExtras ex;
  if (int rc = fo::make_attn_extras(&ex, bias, bias_strides, bias_dtype, dtype, dropout_p, rng_seed, rng_offset))
    return rc;
  return attn_fwd_impl(q, k, v, o, lse, B, H, Sq, Sk, D, q_strides, k_strides, v_strides, o_strides, dtype, causal,
                       softmax_scale, &ex, device, stream);
}

// out[b, h, i, j] = 1 if element (i, j) of head (b, h) is kept by the dropout of
// fo_flash_attn_fwd_ex called with the same p, seed and offset; dense (B, H, Sq, Sk) bytes.
__global__ void dropout_mask_kernel(uint8_t* __restrict__ out, int64_t total, uint32_t base, uint32_t seed,
                                    uint32_t threshold) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    out[i] = fo::dropout_hash(base + static_cast<uint32_t>(i), seed) > threshold ? 1 : 0;
}

extern "C" int fo_dropout_mask(uint8_t* out, int B, int H, int Sq, int Sk, float dropout_p, uint64_t rng_seed,
                               uint64_t rng_offset, int device, void* stream) {
  fo::clear_error();
  FO_REQUIRE(out != nullptr, "null output pointer");
  FO_REQUIRE(B > 0 && H > 0 && Sq > 0 && Sk > 0, "B, H, Sq, Sk must be positive");
  FO_REQUIRE(dropout_p > 0.f && dropout_p < 1.f, "dropout_p must be in (0, 1) (got %g)", (double)dropout_p);
  fo::AttnExtras ex;
  if (int rc = fo::make_attn_extras(&ex, nullptr, nullptr, FO_F32, FO_BF16, dropout_p, rng_seed, rng_offset)) return rc;
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  const int64_t total = static_cast<int64_t>(B) * H * Sq * Sk;
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  dropout_mask_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, total, ex.drop_base, ex.drop_seed,
                                                                            ex.drop_threshold);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

extern "C" int fo_debug_umma_tile(const void* a, const void* b, float* c, int N, int K, int dtype, int mode,
                                  int device, void* stream) {
  fo::clear_error();
  FO_REQUIRE(a && b && c, "null pointer");
  FO_REQUIRE(dtype == FO_F16 || dtype == FO_BF16, "dtype must be fp16 or bf16");
  FO_REQUIRE((N == 64 || N == 128) && (K == 64 || K == 128), "N and K must be 64 or 128");
  FO_REQUIRE(mode == 0 || mode == 1, "mode must be 0 or 1");
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  int* status = fo::device_status_ptr(device);
  if (!status) return fo::fail(FO_ERR_CUDA, "cannot resolve the status word of device %d", device);
  CUtensorMap ta, tb;
  // A is (128 x K); B is (N x K) in mode 0 and (K x N) in mode 1, both row-major and dense.
  const int64_t sa[3] = {128LL * K, 128LL * K, K};
  if (int rc = make_tensor_map(&ta, a, dtype, 1, 1, 128, K, sa, "a")) return rc;
  const int b_rows = mode == 0 ? N : K, b_cols = mode == 0 ? K : N;
  const int64_t sb[3] = {static_cast<int64_t>(b_rows) * b_cols, static_cast<int64_t>(b_rows) * b_cols, b_cols};
  if (int rc = make_tensor_map(&tb, b, dtype, 1, 1, b_rows, b_cols, sb, "b")) return rc;
  const int smem = 4 * fo::kBoxBytes + 1024 + 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FO_BF16) {
    FO_CUDA_CHECK((fo::ensure_dynamic_smem<umma_tile_kernel<true>>(smem, device)));
    umma_tile_kernel<true><<<1, 128, smem, s>>>(ta, tb, static_cast<const uint16_t*>(a), c, N, K, mode, status);
  } else {
    FO_CUDA_CHECK((fo::ensure_dynamic_smem<umma_tile_kernel<false>>(smem, device)));
    umma_tile_kernel<false><<<1, 128, smem, s>>>(ta, tb, static_cast<const uint16_t*>(a), c, N, K, mode, status);
  }
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

// One warp waits, through the kernels' bounded wait, on a barrier that nobody arrives on.
__global__ void wait_timeout_kernel(int* device_status, unsigned long long budget_ns, int* returned) {
  using namespace fo;
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* cta_abort = &abort_word;
  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_budget(&bar, 0, cta_abort, device_status, FO_STATUS_TIMEOUT_SELFTEST, budget_ns);
  __syncthreads();
  if (threadIdx.x == 0 && returned != nullptr) *returned = ok ? 1 : 2;  // 2: gave up and came back
}

extern "C" int fo_debug_wait_timeout(int budget_us, int* returned, int device, void* stream) {
  fo::clear_error();
  FO_REQUIRE(budget_us >= 1 && budget_us <= 100000, "budget_us must be in [1, 100000] (got %d)", budget_us);
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  int* status = fo::device_status_ptr(device);
  if (!status) return fo::fail(FO_ERR_CUDA, "cannot resolve the status word of device %d", device);
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      status, static_cast<unsigned long long>(budget_us) * 1000ull, returned);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

extern "C" int fo_attn_configure(int impl, int ping_pong, int head_group) {
  fo::clear_error();
  FO_REQUIRE(impl >= -1 && impl <= 5,
             "impl must be -1 (keep), 0 (auto), 1 (simple), 2 (128-key), 3 (64-key), 4 (64-key, persistent grid) or 5 "
             "(64-key, one query tile per CTA)");
  FO_REQUIRE(ping_pong >= -1 && ping_pong <= 1, "ping_pong must be -1 (keep), 0 or 1");
  FO_REQUIRE(head_group >= -1, "head_group must be -1 (keep), 0 (automatic) or a positive head count");
  if (impl >= 0) fo::g_attn_options.impl.store(impl, std::memory_order_relaxed);
  if (ping_pong >= 0) fo::g_attn_options.ping_pong.store(ping_pong, std::memory_order_relaxed);
  if (head_group >= 0) fo::g_attn_options.head_group.store(head_group, std::memory_order_relaxed);
  return FO_OK;
}

extern "C" int fo_debug_set_attn_trace(void* device_buffer) {
  fo::clear_error();
#if FO_ATTN_TRACE
  g_attn_trace = static_cast<unsigned long long*>(device_buffer);
  return FO_OK;
#else
  if (device_buffer == nullptr) return FO_OK;
  return fo::fail(FO_ERR_UNSUPPORTED, "this build has no timeline hook: rebuild with -DFO_ATTN_TRACE=1");
#endif
}

extern "C" int fo_debug_attn_trace_shape(int* roles, int* iters, int* events) {
  *roles = fo::kTraceRoles;
  *iters = fo::kTraceIters;
  *events = fo::kTraceEvents;
  return FO_OK;
}
