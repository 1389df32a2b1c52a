// Host launcher of the attention backward (fo_flash_attn_bwd) and its two small helper kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>

#include "flash_attn_bwd.cuh"
#include "fo_host.h"
#include "fo_tma.h"

namespace {

template <bool kBf16>
__device__ __forceinline__ float to_f32(uint16_t raw) {
  if constexpr (kBf16) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  else return __half2float(*reinterpret_cast<const __half*>(&raw));
}

// delta[bh, row] = sum_d O[b,h,row,d] * dO[b,h,row,d]   (flash_attention_triton.py:273-315), and
// the fp32 dQ accumulation row is cleared.  One warp per query row.
template <bool kBf16>
__global__ void __launch_bounds__(256)
attn_bwd_prepare_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dout, float* __restrict__ delta,
                        float* __restrict__ dq_accum, int H, int Sq, int D, int64_t o_sb, int64_t o_sh, int64_t o_ss,
                        int64_t d_sb, int64_t d_sh, int64_t d_ss, int64_t rows) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t bh = r / Sq;
  const int row = static_cast<int>(r - bh * Sq);
  const int b = static_cast<int>(bh / H), h = static_cast<int>(bh - static_cast<int64_t>(b) * H);
  const uint16_t* orow = o + b * o_sb + h * o_sh + row * o_ss;
  const uint16_t* drow = dout + b * d_sb + h * d_sh + row * d_ss;
  float acc = 0.f;
  for (int d = lane; d < D; d += 32) {
    acc += to_f32<kBf16>(orow[d]) * to_f32<kBf16>(drow[d]);
    dq_accum[r * D + d] = 0.f;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[r] = acc;
}

// dQ = round(dq_accum) in the input type.  One thread per 8 elements.
template <bool kBf16>
__global__ void __launch_bounds__(256)
attn_bwd_finish_dq_kernel(const float* __restrict__ dq_accum, uint16_t* __restrict__ dq, int H, int Sq, int D,
                          int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t groups) {
  const int64_t g = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (g >= groups) return;
  const int per_row = D / 8;
  const int64_t r = g / per_row;
  const int d0 = static_cast<int>(g - r * per_row) * 8;
  const int64_t bh = r / Sq;
  const int row = static_cast<int>(r - bh * Sq);
  const int b = static_cast<int>(bh / H), h = static_cast<int>(bh - static_cast<int64_t>(b) * H);
  const float4 a0 = *reinterpret_cast<const float4*>(dq_accum + r * D + d0);
  const float4 a1 = *reinterpret_cast<const float4*>(dq_accum + r * D + d0 + 4);
  uint4 v;
  v.x = fo::pack2<kBf16>(a0.x, a0.y);
  v.y = fo::pack2<kBf16>(a0.z, a0.w);
  v.z = fo::pack2<kBf16>(a1.x, a1.y);
  v.w = fo::pack2<kBf16>(a1.z, a1.w);
  *reinterpret_cast<uint4*>(dq + b * q_sb + h * q_sh + row * q_ss + d0) = v;
}

template <int D, bool kBf16, int kExt>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               const CUtensorMap& tdq, const fo::AttnBwdParams& prm, cudaStream_t stream) {
  dim3 grid((prm.Sk + fo::kBlockN - 1) / fo::kBlockN, prm.B * prm.H);
  auto kernel = fo::attn_bwd_kernel<D, kBf16, kExt>;
  constexpr int smem = fo::BwdConfig<D>::kSmemBytes;
  FO_CUDA_CHECK((fo::ensure_dynamic_smem<fo::attn_bwd_kernel<D, kBf16, kExt>>(smem, prm.device)));
  kernel<<<grid, 512, smem, stream>>>(tq, tk, tv, tdo, tdq, prm);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

int check_out_strides(const int64_t s[3], const char* name) {
  for (int i = 0; i < 3; ++i)
    FO_REQUIRE(s[i] >= 0 && s[i] % 8 == 0, "%s: strides must be non-negative multiples of 8 elements", name);
  return FO_OK;
}

}  // namespace

namespace fo {
int make_attn_extras(AttnExtras* ex, const void* bias, const int64_t* bias_strides, int bias_dtype, int dtype,
                     float dropout_p, uint64_t rng_seed, uint64_t rng_offset);  // flash_attn_fwd.cu
}

static int attn_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* dout,
                         const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta,
                         int B, int H, int Sq, int Sk, int D,
                         const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                         const int64_t o_strides[3], const int64_t do_strides[3],
                         const int64_t dq_strides[3], const int64_t dk_strides[3],
                         const int64_t dv_strides[3],
                         int dtype, int causal, float softmax_scale, const fo::AttnExtras* ex, int device,
                         void* stream) {
  FO_REQUIRE(q && k && v && o && dout && lse && dq && dk && dv && dq_accum && delta, "null pointer");
  FO_REQUIRE(q_strides && k_strides && v_strides && o_strides && do_strides && dq_strides && dk_strides && dv_strides,
             "null stride array");
  FO_REQUIRE(dtype == FO_F16 || dtype == FO_BF16, "attention tensors must be fp16 or bf16 (got dtype %d)", dtype);
  FO_REQUIRE(B > 0 && H > 0 && Sq > 0 && Sk > 0, "B, H, Sq, Sk must be positive");
  FO_REQUIRE(static_cast<int64_t>(B) * H <= 65535, "B*H must be <= 65535");
  if (D <= 0 || D > 128 || D % 8 != 0)
    return fo::fail(FO_ERR_INVALID_ARGUMENT, "head_dim must be a multiple of 8 and <= 128 (got %d)", D);
  const int Dk = D <= 64 ? 64 : 128;  // head_dim the kernel is built for
  FO_REQUIRE(softmax_scale > 0.f && std::isfinite(softmax_scale), "softmax_scale must be positive and finite");
  for (const void* p : {static_cast<const void*>(o), static_cast<const void*>(dq), static_cast<const void*>(dk),
                        static_cast<const void*>(dv)})
    FO_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, "o, dq, dk, dv must be 16-byte aligned");
  FO_REQUIRE((reinterpret_cast<uintptr_t>(dq_accum) & 15) == 0, "dq_accum must be 16-byte aligned");
  if (int rc = check_out_strides(o_strides, "o")) return rc;
  if (int rc = check_out_strides(dq_strides, "dq")) return rc;
  if (int rc = check_out_strides(dk_strides, "dk")) return rc;
  if (int rc = check_out_strides(dv_strides, "dv")) return rc;

  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  int* status = fo::device_status_ptr(device);
  if (!status) return fo::fail(FO_ERR_CUDA, "cannot resolve the status word of device %d", device);

  CUtensorMap tq, tk, tv, tdo;
  if (int rc = fo::make_tensor_map(&tq, q, dtype, B, H, Sq, D, q_strides, "q")) return rc;
  if (int rc = fo::make_tensor_map(&tk, k, dtype, B, H, Sk, D, k_strides, "k")) return rc;
  if (int rc = fo::make_tensor_map(&tv, v, dtype, B, H, Sk, D, v_strides, "v")) return rc;
  if (int rc = fo::make_tensor_map(&tdo, dout, dtype, B, H, Sq, D, do_strides, "dout")) return rc;
  CUtensorMap tdq;
  if (int rc = fo::make_dq_accum_map(&tdq, dq_accum, static_cast<int64_t>(B) * H, Sq, D)) return rc;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == FO_BF16;
  const int64_t rows = static_cast<int64_t>(B) * H * Sq;
  {
    const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
    auto* op = static_cast<const uint16_t*>(o);
    auto* dp = static_cast<const uint16_t*>(dout);
    if (bf16)
      attn_bwd_prepare_kernel<true><<<blocks, 256, 0, s>>>(op, dp, delta, dq_accum, H, Sq, D, o_strides[0], o_strides[1],
                                                           o_strides[2], do_strides[0], do_strides[1], do_strides[2], rows);
    else
      attn_bwd_prepare_kernel<false><<<blocks, 256, 0, s>>>(op, dp, delta, dq_accum, H, Sq, D, o_strides[0], o_strides[1],
                                                            o_strides[2], do_strides[0], do_strides[1], do_strides[2], rows);
    fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
    FO_CUDA_CHECK(cudaGetLastError());
  }

  fo::AttnBwdParams prm;
  prm.lse = lse;
  prm.delta = delta;
  prm.dq_accum = dq_accum;
  prm.dk = dk;
  prm.dv = dv;
  prm.dk_stride_b = dk_strides[0];
  prm.dk_stride_h = dk_strides[1];
  prm.dk_stride_s = dk_strides[2];
  prm.dv_stride_b = dv_strides[0];
  prm.dv_stride_h = dv_strides[1];
  prm.dv_stride_s = dv_strides[2];
  prm.B = B;
  prm.H = H;
  prm.Sq = Sq;
  prm.Sk = Sk;
  prm.d_real = D;
  prm.causal = causal ? 1 : 0;
  prm.scale = softmax_scale;
  prm.scale_log2 = softmax_scale * 1.4426950408889634f;
  prm.device_status = status;
  prm.trace = fo::g_attn_trace;
  prm.device = device;
  std::memset(&prm.ex, 0, sizeof(prm.ex));
  prm.ex.drop_rescale = 1.f;
  const bool ext = ex != nullptr && (ex->bias != nullptr || ex->dropout);
  if (ext) prm.ex = *ex;
  int rc;
  const int mode = ext ? ((prm.ex.bias != nullptr ? 1 : 0) | (prm.ex.dropout ? 2 : 0)) : 0;
#define FO_BWD_MODE(M)                                                                                     \
  case M:                                                                                                  \
    if (Dk == 128) rc = bf16 ? launch_bwd<128, true, M>(tq, tk, tv, tdo, tdq, prm, s) : launch_bwd<128, false, M>(tq, tk, tv, tdo, tdq, prm, s); \
    else rc = bf16 ? launch_bwd<64, true, M>(tq, tk, tv, tdo, tdq, prm, s) : launch_bwd<64, false, M>(tq, tk, tv, tdo, tdq, prm, s);            \
    break;
  switch (mode) {
    FO_BWD_MODE(0)
    FO_BWD_MODE(1)
    FO_BWD_MODE(2)
    default:
    FO_BWD_MODE(3)
  }
#undef FO_BWD_MODE
  if (rc) return rc;

  {
    const int64_t groups = rows * (D / 8);
    const unsigned blocks = static_cast<unsigned>((groups + 255) / 256);
    auto* dqp = static_cast<uint16_t*>(dq);
    if (bf16)
      attn_bwd_finish_dq_kernel<true><<<blocks, 256, 0, s>>>(dq_accum, dqp, H, Sq, D, dq_strides[0], dq_strides[1],
                                                             dq_strides[2], groups);
    else
      attn_bwd_finish_dq_kernel<false><<<blocks, 256, 0, s>>>(dq_accum, dqp, H, Sq, D, dq_strides[0], dq_strides[1],
                                                              dq_strides[2], groups);
    fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
    FO_CUDA_CHECK(cudaGetLastError());
  }
  return FO_OK;
}

extern "C" int fo_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                 const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta,
                                 int B, int H, int Sq, int Sk, int D,
                                 const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                                 const int64_t o_strides[3], const int64_t do_strides[3],
                                 const int64_t dq_strides[3], const int64_t dk_strides[3],
                                 const int64_t dv_strides[3],
                                 int dtype, int causal, float softmax_scale, int device, void* stream) {
  fo::clear_error();
  return attn_bwd_impl(q, k, v, o, dout, lse, dq, dk, dv, dq_accum, delta, B, H, Sq, Sk, D, q_strides, k_strides,
                       v_strides, o_strides, do_strides, dq_strides, dk_strides, dv_strides, dtype, causal,
                       softmax_scale, nullptr, device, stream);
}

extern "C" int fo_flash_attn_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                    const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta,
                                    int B, int H, int Sq, int Sk, int D,
                                    const int64_t q_strides[3], const int64_t k_strides[3],
                                    const int64_t v_strides[3], const int64_t o_strides[3],
                                    const int64_t do_strides[3], const int64_t dq_strides[3],
                                    const int64_t dk_strides[3], const int64_t dv_strides[3],
                                    int dtype, int causal, float softmax_scale,
                                    const void* bias, const int64_t bias_strides[3], int bias_dtype,
                                    float dropout_p, uint64_t rng_seed, uint64_t rng_offset,
                                    int device, void* stream) {
  fo::clear_error();
  FO_REQUIRE(dtype == FO_F16 || dtype == FO_BF16, "attention tensors must be fp16 or bf16 (got dtype %d)", dtype);
  fo::AttnExtras ex;
  if (int rc = fo::make_attn_extras(&ex, bias, bias_strides, bias_dtype, dtype, dropout_p, rng_seed, rng_offset))
    return rc;
  return attn_bwd_impl(q, k, v, o, dout, lse, dq, dk, dv, dq_accum, delta, B, H, Sq, Sk, D, q_strides, k_strides,
                       v_strides, o_strides, do_strides, dq_strides, dk_strides, dv_strides, dtype, causal,
                       softmax_scale, &ex, device, stream);
}
