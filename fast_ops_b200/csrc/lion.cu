// Fused Lion step for sm_100a: one persistent multi-tensor kernel, one HBM pass.
//
// The arithmetic follows the reference torch implementation
// (fast_ops/lion/lion_optimizer_ref.py:51-67), where every product and sum is a
// separate tensor op whose result is rounded to the tensor's storage type:
//
//   p1 = R_p(p * c_wd)                      c_wd = float(1 - lr*wd)
//   t1 = R_m(m * c_b1)   t2 = R_g(g * c_1mb1)
//   u  = R_pm(t1 + t2)   s = sign(u) in {-1, 0, +1}        (pm = promote(m, g))
//   p2 = R_p(fma(c_nlr, s, p1))             c_nlr  = R_pm(-lr)
//   m1 = R_m(m * c_b2)   m2 = R_m(fma(c_1mb2, g, m1))       c_1mb2 = R_pm(1 - beta2)
//
// A scalar multiplier of `mul` stays fp32, while the `alpha` of `add_(x, alpha=...)` is
// first rounded to the promoted type of the two tensors and the sum is one fused
// multiply-add in fp32: that is what torch's vectorised CPU kernels compute, and it was
// checked bit for bit against the reference optimizer for every dtype combination below.
//
// The reference CUDA kernel (fast_ops/lion/lion_update.cu:15-107) computes in the
// storage type and uses sign(0) = -1; this kernel follows the torch semantics instead
// and computes in fp32 registers with explicit roundings.
//
// Memory: every element is read once (p, g, m) and written once (p, m) with 16-byte
// vector accesses; a chunk of kChunk elements is the unit handed to a CTA.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "fo_host.h"

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;     // elements per thread per group (16 B of a 16-bit type)
constexpr int kUnroll = 4;  // groups per thread per chunk
constexpr int kChunk = kThreads * kVec * kUnroll;  // 8192 elements

struct LionTensor {
  void* p;
  const void* g;
  void* m;
  int64_t numel;
};

struct LionConsts {
  float c_wd;    // 1 - lr*wd
  float c_b1;    // beta1
  float c_1mb1;  // 1 - beta1
  float c_nlr;   // -lr, rounded to promote(p, m)
  float c_b2;    // beta2
  float c_1mb2;  // 1 - beta2, rounded to promote(p, m)
};

// ---- storage-type helpers -------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(float x) { return x; }
  static __device__ __forceinline__ float round(float x) { return x; }
  static __device__ __forceinline__ float store(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ float round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
  }
  static __device__ __forceinline__ __nv_bfloat16 store(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float load(__half x) { return __half2float(x); }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ __half store(float x) { return __float2half_rn(x); }
};

// torch type promotion of the two operands of `exp_avg * beta1 + grad * (1 - beta1)`:
// equal types keep the type, anything else lands on fp32.
template <typename TM, typename TG> struct Promote { using type = float; };
template <typename T> struct Promote<T, T> { using type = T; };

// A group of kVec elements of T moved with 16-byte accesses.
template <typename T> struct alignas(16) Group {
  T v[kVec];
};

template <typename T>
__device__ __forceinline__ void load_group(Group<T>& dst, const T* src) {
  constexpr int n16 = sizeof(T) * kVec / 16;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst.v);
#pragma unroll
  for (int i = 0; i < n16; ++i) d[i] = __ldcs(s + i);  // streaming: every byte is touched once
}

template <typename T>
__device__ __forceinline__ void store_group(T* dst, const Group<T>& src) {
  constexpr int n16 = sizeof(T) * kVec / 16;
  uint4* d = reinterpret_cast<uint4*>(dst);
  const uint4* s = reinterpret_cast<const uint4*>(src.v);
#pragma unroll
  for (int i = 0; i < n16; ++i) __stcs(d + i, s[i]);
}

template <typename TP, typename TM>
__device__ __forceinline__ void lion_element(TP& p_io, TP g_in, TM& m_io, const LionConsts& c) {
  using TG = TP;
  using TU = typename Promote<TM, TG>::type;
  const float p = Elem<TP>::load(p_io);
  const float g = Elem<TG>::load(g_in);
  const float m = Elem<TM>::load(m_io);
  const float p1 = Elem<TP>::round(__fmul_rn(p, c.c_wd));
  const float t1 = Elem<TM>::round(__fmul_rn(m, c.c_b1));
  const float t2 = Elem<TG>::round(__fmul_rn(g, c.c_1mb1));
  const float u = Elem<TU>::round(__fadd_rn(t1, t2));
  const float s = (u > 0.f) ? 1.f : ((u < 0.f) ? -1.f : 0.f);
  p_io = Elem<TP>::store(__fmaf_rn(c.c_nlr, s, p1));
  const float m1 = Elem<TM>::round(__fmul_rn(m, c.c_b2));
  m_io = Elem<TM>::store(__fmaf_rn(c.c_1mb2, g, m1));
}

// One 16-byte-vector group of kVec elements.  (Packed fp32 pairs, mul/add.f32x2 through the
// __fmul2_rn / __fadd2_rn intrinsics, were tried here: no faster on all-16-bit tensors, and the
// compiler contracted the packed multiply and add into one fused multiply-add, which flips the
// sign of beta1*m + (1-beta1)*g where the two rounded terms cancel exactly.  The scalar _rn
// intrinsics below are never contracted.)
template <typename TP, typename TM>
__device__ __forceinline__ void lion_group(Group<TP>& pv, const Group<TP>& gv, Group<TM>& mv, const LionConsts& c) {
#pragma unroll
  for (int i = 0; i < kVec; ++i) lion_element<TP, TM>(pv.v[i], gv.v[i], mv.v[i], c);
}

// One chunk of kU * kThreads * kVec elements: `remaining` elements are left from p, g, m on (a full
// chunk of them are this chunk's unless the tensor ends earlier); `aligned` says that all three
// addresses allow 16-byte accesses.
template <typename TP, typename TM, int kU = kUnroll>
__device__ __forceinline__ void lion_chunk(TP* p, const TP* g, TM* m, int64_t remaining, bool aligned,
                                           const LionConsts& c) {
  constexpr int kElems = kThreads * kVec * kU;
  if (aligned && remaining >= kElems) {
    Group<TP> pv[kU], gv[kU];
    Group<TM> mv[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int off = (u * kThreads + threadIdx.x) * kVec;
      load_group(pv[u], p + off);
      load_group(gv[u], g + off);
      load_group(mv[u], m + off);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      lion_group<TP, TM>(pv[u], gv[u], mv[u], c);
      const int off = (u * kThreads + threadIdx.x) * kVec;
      store_group(p + off, pv[u]);
      store_group(m + off, mv[u]);
    }
  } else {
    // Ragged tail of a tensor, or a tensor whose storage is not 16-byte aligned.
    const int n = remaining < kElems ? static_cast<int>(remaining) : kElems;
    for (int i = threadIdx.x; i < n; i += kThreads) {
      TP pe = p[i];
      TM me = m[i];
      lion_element<TP, TM>(pe, g[i], me, c);
      p[i] = pe;
      m[i] = me;
    }
  }
}

__device__ __forceinline__ bool all_aligned16(const void* a, const void* b, const void* c) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

// One launch covers all tensors, described by a table of one entry per TENSOR (the form the
// allocation-free entry point can keep in a fixed device array).  `chunk_start[t]` is the index
// of tensor t's first chunk in the global chunk numbering (chunk_start[n_tensors] = total).  A
// resident wave of CTAs strides over the chunks; because a CTA's chunk index only grows, it finds
// the owning tensor by walking `t` forward from where the previous chunk left it.
template <typename TP, typename TM>
__global__ void __launch_bounds__(kThreads)
lion_table_walk_kernel(const LionTensor* __restrict__ tensors,
                         const int64_t* __restrict__ chunk_start, int n_tensors,
                         int64_t total_chunks, LionConsts c) {
  int t = 0;
  int64_t t_first = 0;            // chunk_start[t]
  int64_t t_end = __ldg(chunk_start + 1);  // chunk_start[t + 1]
  LionTensor cur = tensors[0];
  bool aligned = all_aligned16(cur.p, cur.g, cur.m);

  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    if (chunk >= t_end) {
      do {
        ++t;
        t_end = __ldg(chunk_start + t + 1);
      } while (chunk >= t_end && t + 1 < n_tensors);
      t_first = __ldg(chunk_start + t);
      cur = tensors[t];
      aligned = all_aligned16(cur.p, cur.g, cur.m);
    }
    const int64_t base = (chunk - t_first) * kChunk;
    lion_chunk<TP, TM>(static_cast<TP*>(cur.p) + base, static_cast<const TP*>(cur.g) + base,
                       static_cast<TM*>(cur.m) + base, cur.numel - base, aligned, c);
  }
}

// The same step on ONE tensor, described by the kernel's own arguments: no device table, so
// nothing is allocated, copied or cached for it (the per-tensor call of the reference's
// optimizer loop, and a ZeRO-1 shard, come through here).
// One 16-byte group per thread and array, and one CTA per 2048 elements instead of a resident
// wave that loops.  Measured on 6.7e9 bf16 elements (p, g, m all 16-bit), TB/s: a resident wave
// with 2 / 4 / 6 / 8 groups per thread 5.73 / 6.15 / 6.20 / 3.85; one CTA per chunk with
// 1 / 2 / 3 / 4 / 8 groups 7.01 / 7.03 / 6.59 / 6.80 / 4.40 (a torch elementwise add over three
// arrays of that size moves 7.08, a copy 6.59).  The multi-tensor kernel keeps its resident wave:
// with more CTAs each of them walks further through the tensor table (6.61 TB/s on the
// GPT-2-medium list with one wave, 6.56 with four, 6.05 with sixteen).
constexpr int kSingleUnroll = 1;

template <typename TP, typename TM>
__global__ void __launch_bounds__(kThreads)
lion_single_tensor_kernel(TP* __restrict__ p, const TP* __restrict__ g, TM* __restrict__ m, int64_t numel,
                          int64_t total_chunks, LionConsts c) {
  constexpr int kU = kSingleUnroll;
  constexpr int kElems = kThreads * kVec * kU;
  const bool aligned = all_aligned16(p, g, m);
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int64_t base = chunk * kElems;
    lion_chunk<TP, TM, kU>(p + base, g + base, m + base, numel - base, aligned, c);
  }
}

// One launch covers all tensors, described by one record per CHUNK of kChunk elements (pointers
// already advanced to the chunk, and how many elements are left of its tensor from there on): a
// CTA needs one 32-byte load to know its work, so the launch can use one CTA per quarter or half
// chunk like the single-tensor kernel instead of a resident wave that walks a tensor table.  The
// records cost 32 bytes of device memory and of traffic per kChunk elements (0.05 % of the
// step's traffic with 16-bit tensors).
struct ChunkRecord {
  void* p;
  const void* g;
  void* m;
  int64_t remaining;
};
static_assert(sizeof(ChunkRecord) == 32, "two 16-byte loads");

// Groups per thread.  Measured, one CTA per 2048 / 4096 / 8192 elements: GPT-2-medium list (fp32
// p, g) 6.94 / 6.83 / 6.89 TB/s, a list of 64 bf16 matrices of 4096 x 11008 6.39 / 6.65 / 6.50:
// with 16-bit parameters a CTA of one group moves 20 KB for its one dependent record load, with
// 32-bit ones 32 KB, so the former take two groups.
template <typename TP> struct MultiShape {
  static constexpr int kUnroll = sizeof(TP) == 2 ? 2 : 1;
  static constexpr int kSubElems = kThreads * kVec * kUnroll;  // elements of one CTA
  static constexpr int kSubsPerChunk = kChunk / kSubElems;
  static_assert(kChunk % kSubElems == 0 && kSubElems % 8 == 0,
                "a CTA's part starts 16-byte aligned whenever the tensor does");
};

template <typename TP, typename TM>
__global__ void __launch_bounds__(kThreads)
lion_multi_tensor_kernel(const ChunkRecord* __restrict__ records, int64_t total_subs, LionConsts c) {
  for (int64_t sub = blockIdx.x; sub < total_subs; sub += gridDim.x) {
    using Shape = MultiShape<TP>;
    const uint4* rp = reinterpret_cast<const uint4*>(records + sub / Shape::kSubsPerChunk);
    const uint4 lo = __ldg(rp), hi = __ldg(rp + 1);
    ChunkRecord r;
    memcpy(&r, &lo, 16);
    memcpy(reinterpret_cast<char*>(&r) + 16, &hi, 16);
    const int64_t off = (sub % Shape::kSubsPerChunk) * static_cast<int64_t>(Shape::kSubElems);
    if (off >= r.remaining) continue;  // the tensor ended in an earlier part of this chunk
    lion_chunk<TP, TM, Shape::kUnroll>(static_cast<TP*>(r.p) + off, static_cast<const TP*>(r.g) + off,
                                      static_cast<TM*>(r.m) + off, r.remaining - off, all_aligned16(r.p, r.g, r.m), c);
  }
}

// ---- host side --------------------------------------------------------------------------

struct Plan {
  int device = -1;
  int n_tensors = 0;
  int64_t total_chunks = 0;
  void* d_blob = nullptr;  // ChunkRecord x total_chunks (the allocation-free entry: [LionTensor x n][int64 x (n+1)])
  uint64_t last_use = 0;   // value of g_plan_clock at the latest call with this list
};

std::mutex g_plan_mutex;
std::map<std::string, Plan> g_plans;  // key: device + raw bytes of the tensor list
uint64_t g_plan_clock = 0;

constexpr size_t kMaxPlans = 32;

// cudaFree waits for the device's pending work, so a table still in use by a kernel
// in flight is not released under it.  A CUDA graph that captured a launch keeps the
// table's address: dropping the table invalidates that graph.
void free_plan_locked(Plan& plan) {
  if (!plan.d_blob) return;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(plan.device);
  cudaDeviceSynchronize();
  cudaFree(plan.d_blob);
  plan.d_blob = nullptr;
  if (prev >= 0) cudaSetDevice(prev);
}

void drop_all_plans_locked() {
  for (auto& kv : g_plans) free_plan_locked(kv.second);
  g_plans.clear();
}

// Makes room for one more list by dropping the one that has gone unused the longest.
void evict_oldest_plan_locked() {
  auto oldest = g_plans.begin();
  for (auto it = g_plans.begin(); it != g_plans.end(); ++it)
    if (it->second.last_use < oldest->second.last_use) oldest = it;
  if (oldest == g_plans.end()) return;
  free_plan_locked(oldest->second);
  g_plans.erase(oldest);
}

int sm_count(int device) {
  static std::mutex mu;
  static std::map<int, int> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
  cache[device] = n;
  return n;
}

// Rounds a double to `dtype` the way torch converts a Python scalar: through float.
float round_scalar(double x, int dtype) {
  const float f = static_cast<float>(x);
  if (dtype == FO_BF16) return __bfloat162float(__float2bfloat16_rn(f));
  if (dtype == FO_F16) return __half2float(__float2half_rn(f));
  return f;
}

int make_consts(double lr, double beta1, double beta2, double wd, int p_dtype, int m_dtype, LionConsts* c) {
  FO_REQUIRE(lr == lr && beta1 == beta1 && beta2 == beta2 && wd == wd, "Lion hyper-parameter is NaN");
  const int promoted = (p_dtype == m_dtype) ? p_dtype : FO_F32;
  c->c_wd = static_cast<float>(1.0 - lr * wd);
  c->c_b1 = static_cast<float>(beta1);
  c->c_1mb1 = static_cast<float>(1.0 - beta1);
  c->c_nlr = round_scalar(-lr, promoted);
  c->c_b2 = static_cast<float>(beta2);
  c->c_1mb2 = round_scalar(1.0 - beta2, promoted);
  return FO_OK;
}

// Size of the persistent grid: exactly one resident wave, as many CTAs per SM as the kernel's
// register use allows (a partial second wave costs up to 20 %), never more CTAs than chunks.
// The occupancy query is made once per kernel instantiation.
template <auto kKernel>
int64_t one_wave_grid(int device, int64_t total_chunks) {
  static std::atomic<int> cached_per_sm{0};  // one per kernel: the kernel is a template argument
  int per_sm = cached_per_sm.load(std::memory_order_relaxed);
  if (per_sm == 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kKernel, kThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 4;
    cached_per_sm.store(per_sm, std::memory_order_relaxed);
  }
  const int64_t grid = static_cast<int64_t>(sm_count(device)) * per_sm;
  return grid > total_chunks ? total_chunks : grid;
}

template <typename TP, typename TM>
int launch_records_typed(const Plan& plan, const LionConsts& c, cudaStream_t stream) {
  const int64_t total_subs = plan.total_chunks * MultiShape<TP>::kSubsPerChunk;
  // the kernel strides over its parts, so a grid cut at the launch limit still covers them all
  const int64_t grid = total_subs < 0x7fffffffll ? total_subs : 0x7fffffffll;
  lion_multi_tensor_kernel<TP, TM><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      static_cast<const ChunkRecord*>(plan.d_blob), total_subs, c);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

template <typename TP, typename TM>
int launch_walk_typed(const Plan& plan, const LionConsts& c, cudaStream_t stream) {
  const LionTensor* tensors = static_cast<const LionTensor*>(plan.d_blob);
  const int64_t* chunk_start = reinterpret_cast<const int64_t*>(tensors + plan.n_tensors);
  const int64_t grid = one_wave_grid<lion_table_walk_kernel<TP, TM>>(plan.device, plan.total_chunks);
  lion_table_walk_kernel<TP, TM><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      tensors, chunk_start, plan.n_tensors, plan.total_chunks, c);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

template <typename TP, typename TM>
int launch_single_typed(void* p, const void* g, void* m, int64_t numel, const LionConsts& c, int device,
                        cudaStream_t stream) {
  constexpr int kElems = kThreads * kVec * kSingleUnroll;
  const int64_t total_chunks = (numel + kElems - 1) / kElems;
  // the kernel strides over chunks, so a grid cut at the launch limit still covers them all
  const int64_t grid = total_chunks < 0x7fffffffll ? total_chunks : 0x7fffffffll;
  lion_single_tensor_kernel<TP, TM><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      static_cast<TP*>(p), static_cast<const TP*>(g), static_cast<TM*>(m), numel, total_chunks, c);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

#define FO_LION_DTYPE_CASES(CASE)                      \
  CASE(FO_BF16, FO_BF16, __nv_bfloat16, __nv_bfloat16) \
  CASE(FO_BF16, FO_F32, __nv_bfloat16, float)          \
  CASE(FO_BF16, FO_F16, __nv_bfloat16, __half)         \
  CASE(FO_F16, FO_F16, __half, __half)                 \
  CASE(FO_F16, FO_F32, __half, float)                  \
  CASE(FO_F16, FO_BF16, __half, __nv_bfloat16)         \
  CASE(FO_F32, FO_F32, float, float)                   \
  CASE(FO_F32, FO_BF16, float, __nv_bfloat16)          \
  CASE(FO_F32, FO_F16, float, __half)

// `plan.d_blob` holds chunk records.
int launch_records(const Plan& plan, int p_dtype, int m_dtype, const LionConsts& c, cudaStream_t stream) {
  if (plan.total_chunks == 0) return FO_OK;
#define FO_LION_CASE(PD, MD, TP, TM) \
  if (p_dtype == PD && m_dtype == MD) return launch_records_typed<TP, TM>(plan, c, stream);
  FO_LION_DTYPE_CASES(FO_LION_CASE)
#undef FO_LION_CASE
  return fo::fail(FO_ERR_INVALID_ARGUMENT, "unsupported Lion dtype combination p=%d m=%d", p_dtype, m_dtype);
}

// `plan.d_blob` holds the per-tensor table and its chunk prefix.
int launch_walk(const Plan& plan, int p_dtype, int m_dtype, const LionConsts& c, cudaStream_t stream) {
  if (plan.total_chunks == 0) return FO_OK;
#define FO_LION_CASE(PD, MD, TP, TM) \
  if (p_dtype == PD && m_dtype == MD) return launch_walk_typed<TP, TM>(plan, c, stream);
  FO_LION_DTYPE_CASES(FO_LION_CASE)
#undef FO_LION_CASE
  return fo::fail(FO_ERR_INVALID_ARGUMENT, "unsupported Lion dtype combination p=%d m=%d", p_dtype, m_dtype);
}

int launch_single(void* p, const void* g, void* m, int64_t numel, int p_dtype, int m_dtype, const LionConsts& c,
                  int device, cudaStream_t stream) {
#define FO_LION_CASE(PD, MD, TP, TM) \
  if (p_dtype == PD && m_dtype == MD) return launch_single_typed<TP, TM>(p, g, m, numel, c, device, stream);
  FO_LION_DTYPE_CASES(FO_LION_CASE)
#undef FO_LION_CASE
  return fo::fail(FO_ERR_INVALID_ARGUMENT, "unsupported Lion dtype combination p=%d m=%d", p_dtype, m_dtype);
}

int check_dtypes(int p_dtype, int g_dtype, int m_dtype) {
  FO_REQUIRE(p_dtype == FO_F16 || p_dtype == FO_BF16 || p_dtype == FO_F32, "bad param dtype %d", p_dtype);
  FO_REQUIRE(m_dtype == FO_F16 || m_dtype == FO_BF16 || m_dtype == FO_F32, "bad exp_avg dtype %d", m_dtype);
  FO_REQUIRE(p_dtype == g_dtype, "param and grad must have the same dtype (got %d and %d)", p_dtype, g_dtype);
  return FO_OK;
}

int dtype_size(int dtype) { return dtype == FO_F32 ? 4 : 2; }

// Builds the host image of the chunk records.
void build_records(void* const* params, const void* const* grads, void* const* exp_avgs, const int64_t* numels,
                   int n, int p_dtype, int m_dtype, std::vector<ChunkRecord>* records) {
  const int64_t ps = dtype_size(p_dtype), ms = dtype_size(m_dtype);
  int64_t total = 0;
  for (int i = 0; i < n; ++i) total += (numels[i] + kChunk - 1) / kChunk;
  records->clear();
  records->reserve(static_cast<size_t>(total));
  for (int i = 0; i < n; ++i) {
    for (int64_t off = 0; off < numels[i]; off += kChunk)
      records->push_back(ChunkRecord{static_cast<char*>(params[i]) + off * ps, static_cast<const char*>(grads[i]) + off * ps,
                                     static_cast<char*>(exp_avgs[i]) + off * ms, numels[i] - off});
  }
}

}  // namespace

extern "C" int fo_lion_multi_tensor_step(void* const* params, const void* const* grads,
                                         void* const* exp_avgs, const int64_t* numels, int n_tensors,
                                         int p_dtype, int g_dtype, int m_dtype,
                                         double lr, double beta1, double beta2, double weight_decay,
                                         int device, void* stream) {
  fo::clear_error();
  if (int rc = check_dtypes(p_dtype, g_dtype, m_dtype)) return rc;
  FO_REQUIRE(n_tensors >= 0, "n_tensors must be >= 0");
  if (n_tensors == 0) return FO_OK;
  FO_REQUIRE(params && grads && exp_avgs && numels, "null tensor list");
  LionConsts c;
  if (int rc = make_consts(lr, beta1, beta2, weight_decay, p_dtype, m_dtype, &c)) return rc;

  // Empty tensors carry no work and would break the forward walk; drop them here.
  std::vector<void*> ps;
  std::vector<const void*> gs;
  std::vector<void*> ms;
  std::vector<int64_t> ns;
  ps.reserve(n_tensors); gs.reserve(n_tensors); ms.reserve(n_tensors); ns.reserve(n_tensors);
  for (int i = 0; i < n_tensors; ++i) {
    FO_REQUIRE(numels[i] >= 0, "tensor %d has negative numel", i);
    if (numels[i] == 0) continue;
    FO_REQUIRE(params[i] && grads[i] && exp_avgs[i], "tensor %d has a null pointer", i);
    ps.push_back(params[i]); gs.push_back(grads[i]); ms.push_back(exp_avgs[i]); ns.push_back(numels[i]);
  }
  const int n = static_cast<int>(ps.size());
  if (n == 0) return FO_OK;

  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  if (n == 1)  // no table needed: the tensor travels in the kernel's arguments
    return launch_single(ps[0], gs[0], ms[0], ns[0], p_dtype, m_dtype, c, device, static_cast<cudaStream_t>(stream));

  // key: device, dtypes (the records hold byte addresses) and the raw list
  std::string key(reinterpret_cast<const char*>(&device), sizeof(device));
  key.append(reinterpret_cast<const char*>(&p_dtype), sizeof(p_dtype));
  key.append(reinterpret_cast<const char*>(&m_dtype), sizeof(m_dtype));
  key.append(reinterpret_cast<const char*>(ps.data()), sizeof(void*) * n);
  key.append(reinterpret_cast<const char*>(gs.data()), sizeof(void*) * n);
  key.append(reinterpret_cast<const char*>(ms.data()), sizeof(void*) * n);
  key.append(reinterpret_cast<const char*>(ns.data()), sizeof(int64_t) * n);

  // The lock is held across the launch: a table can then not be evicted (by another thread's
  // new list) between the lookup and the moment its kernel is in the stream, and cudaFree does
  // not release memory under a kernel that is already there.
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  auto it = g_plans.find(key);
  if (it == g_plans.end()) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    FO_CUDA_CHECK(cudaStreamIsCapturing(s, &capture));
    if (capture != cudaStreamCaptureStatusNone)
      return fo::fail(FO_ERR_UNSUPPORTED,
                      "first call with this tensor list on a capturing stream: call once outside the capture so "
                      "that the device table exists");
    // A caller whose pointers change every step would grow the cache without bound.
    if (g_plans.size() >= kMaxPlans) evict_oldest_plan_locked();
    std::vector<ChunkRecord> records;
    build_records(ps.data(), gs.data(), ms.data(), ns.data(), n, p_dtype, m_dtype, &records);
    Plan plan;
    plan.device = device;
    plan.n_tensors = n;
    plan.total_chunks = static_cast<int64_t>(records.size());
    const size_t bytes = records.size() * sizeof(ChunkRecord);
    FO_CUDA_CHECK(cudaMalloc(&plan.d_blob, bytes));
    // On the caller's stream, so that the copy and the kernel below are ordered whatever kind of
    // stream it is.  The source is pageable: the runtime has staged it when the call returns,
    // so the host image may die with this call.
    cudaError_t e = cudaMemcpyAsync(plan.d_blob, records.data(), bytes, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) {
      cudaFree(plan.d_blob);
      return fo::fail(FO_ERR_CUDA, "chunk record upload failed: %s", cudaGetErrorString(e));
    }
    it = g_plans.emplace(std::move(key), plan).first;
  }
  it->second.last_use = ++g_plan_clock;
  return launch_records(it->second, p_dtype, m_dtype, c, s);
}

extern "C" int fo_lion_clear_cache(void) {
  fo::clear_error();
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  drop_all_plans_locked();
  return FO_OK;
}

extern "C" int fo_lion_update(void* param, const void* grad, void* exp_avg, int64_t numel,
                              int p_dtype, int g_dtype, int m_dtype,
                              double lr, double beta1, double beta2, double weight_decay,
                              int device, void* stream) {
  fo::clear_error();
  if (int rc = check_dtypes(p_dtype, g_dtype, m_dtype)) return rc;
  FO_REQUIRE(numel >= 0, "negative numel");
  if (numel == 0) return FO_OK;
  FO_REQUIRE(param && grad && exp_avg, "null pointer");
  LionConsts c;
  if (int rc = make_consts(lr, beta1, beta2, weight_decay, p_dtype, m_dtype, &c)) return rc;
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  return launch_single(param, grad, exp_avg, numel, p_dtype, m_dtype, c, device, static_cast<cudaStream_t>(stream));
}

extern "C" int fo_lion_flat_step(void* param, const void* grad, void* exp_avg_shard,
                                 int64_t begin, int64_t end,
                                 int p_dtype, int g_dtype, int m_dtype,
                                 double lr, double beta1, double beta2, double weight_decay,
                                 int device, void* stream) {
  fo::clear_error();
  if (int rc = check_dtypes(p_dtype, g_dtype, m_dtype)) return rc;
  FO_REQUIRE(begin >= 0 && end >= begin, "bad shard range [%lld, %lld)", (long long)begin, (long long)end);
  if (end == begin) return FO_OK;
  FO_REQUIRE(param && grad && exp_avg_shard, "null pointer");
  const int64_t esz = (p_dtype == FO_F32) ? 4 : 2;
  void* p = static_cast<char*>(param) + begin * esz;
  const void* g = static_cast<const char*>(grad) + begin * esz;
  return fo_lion_update(p, g, exp_avg_shard, end - begin, p_dtype, g_dtype, m_dtype, lr, beta1, beta2,
                        weight_decay, device, stream);
}

// ---- allocation-free variant -----------------------------------------------------------------
//
// fo_lion_multi_tensor_step builds its device tensor table with cudaMalloc the first time it sees
// a pointer list.  Some callers cannot afford that: a trainer that has already handed every byte
// of device memory to its own pool (cudaMalloc then fails), or a step loop that must never hit
// the device-wide synchronisation an allocation or a free can imply.  For them the same kernel
// runs with its table in a fixed array that is part of the library image: nothing is allocated,
// on the device or through any allocating library routine.
//
// The array is a file-scope __device__ object, so every device that loads the library carries
// its kNoAllocTableBytes (about 40 KiB) until the process exits.  In host code the array's name is
// only a handle: the device address comes from cudaGetSymbolAddress, looked up once per device
// with that device current, and that address is what the kernel receives.

namespace {

constexpr int kNoAllocMaxTensors = 1024;
constexpr size_t kNoAllocTableBytes =
    ((sizeof(LionTensor) * kNoAllocMaxTensors + sizeof(int64_t) * (kNoAllocMaxTensors + 1)) + 255) / 256 * 256;

static __device__ __align__(256) unsigned char g_noalloc_table[kNoAllocTableBytes];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_dev_ptr[kNoAllocMaxDevices] = {};  // device address of g_noalloc_table, per device
// Host image of the table; guarded by g_noalloc_mutex.  Outside stream capture cudaMemcpyAsync
// from pageable memory has taken its copy of the source by the time it returns, so the image can
// be reused by the next call.  Inside a capture the copy would become a graph node that reads this
// shared image at every replay (by then it holds whatever list came last), so a capturing stream
// is refused.
alignas(16) unsigned char g_noalloc_host[kNoAllocTableBytes];

}  // namespace

extern "C" int fo_lion_multi_tensor_step_noalloc(void* const* params, const void* const* grads,
                                                 void* const* exp_avgs, const int64_t* numels, int n_tensors,
                                                 int p_dtype, int g_dtype, int m_dtype,
                                                 double lr, double beta1, double beta2, double weight_decay,
                                                 int device, void* stream) {
  fo::clear_error();
  if (int rc = check_dtypes(p_dtype, g_dtype, m_dtype)) return rc;
  FO_REQUIRE(n_tensors >= 0, "n_tensors must be >= 0");
  if (n_tensors == 0) return FO_OK;
  FO_REQUIRE(params && grads && exp_avgs && numels, "null tensor list");
  FO_REQUIRE(n_tensors <= kNoAllocMaxTensors,
             "the allocation-free Lion step takes at most %d tensors per call (got %d); split the list or use "
             "fo_lion_multi_tensor_step",
             kNoAllocMaxTensors, n_tensors);
  FO_REQUIRE(device >= 0 && device < kNoAllocMaxDevices, "device index %d outside [0, %d)", device,
             kNoAllocMaxDevices);
  LionConsts c;
  if (int rc = make_consts(lr, beta1, beta2, weight_decay, p_dtype, m_dtype, &c)) return rc;

  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    FO_CUDA_CHECK(cudaStreamIsCapturing(s, &capture));
    if (capture != cudaStreamCaptureStatusNone)
      return fo::fail(FO_ERR_UNSUPPORTED,
                      "the allocation-free Lion step cannot run on a capturing stream: its table upload would read "
                      "the shared host image at replay time");
  }

  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_dev_ptr[device] == nullptr) {
    // First call on this device: resolve the array's device address (the device is current).
    void* ptr = nullptr;
    FO_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_noalloc_table));
    FO_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address");
    g_noalloc_dev_ptr[device] = ptr;
  }
  void* d_table = g_noalloc_dev_ptr[device];

  // Compact the list (empty tensors carry no work) straight into the host image.
  int n = 0;
  for (int i = 0; i < n_tensors; ++i) {
    FO_REQUIRE(numels[i] >= 0, "tensor %d has negative numel", i);
    if (numels[i] > 0) {
      FO_REQUIRE(params[i] && grads[i] && exp_avgs[i], "tensor %d has a null pointer", i);
      ++n;
    }
  }
  if (n == 0) return FO_OK;
  LionTensor* tensors = reinterpret_cast<LionTensor*>(g_noalloc_host);
  int64_t* chunk_start = reinterpret_cast<int64_t*>(tensors + n);
  int64_t total = 0;
  int k = 0;
  for (int i = 0; i < n_tensors; ++i) {
    if (numels[i] == 0) continue;
    tensors[k] = LionTensor{params[i], grads[i], exp_avgs[i], numels[i]};
    chunk_start[k] = total;
    total += (numels[i] + kChunk - 1) / kChunk;
    ++k;
  }
  chunk_start[n] = total;
  const size_t bytes = sizeof(LionTensor) * n + sizeof(int64_t) * (n + 1);
  // Every entry the kernel reads is rewritten here, so nothing left by an earlier call is used.
  FO_CUDA_CHECK(cudaMemcpyAsync(d_table, g_noalloc_host, bytes, cudaMemcpyHostToDevice, s));

  Plan plan;
  plan.device = device;
  plan.n_tensors = n;
  plan.total_chunks = total;
  plan.d_blob = d_table;
  return launch_walk(plan, p_dtype, m_dtype, c, s);
}

// ---- ZeRO-1 step fused with the distribution of the updated weights ---------------------------
//
// The sharded step is followed by an all-gather of the updated parameters.  Here the kernel that
// computes a rank's slice also stores every updated 16-byte vector into the same position of
// each peer's flat parameter buffer (plain stores to peer memory over NVLink), so the transfer
// overlaps the HBM-bound update instead of following it.  The caller provides the peers' base
// pointers (the buffers must be mapped for peer access, e.g. a symmetric-memory allocation) and
// orders the ranks around the call: no peer may still read its buffer when the stores begin, and
// every rank must have finished before any of them reads the gathered weights.

namespace {

constexpr int kMaxPeers = 7;  // the other GPUs of one 8-GPU NVSwitch domain

struct PeerList {
  void* base[kMaxPeers];
  int n;
};

// One group per thread and one CTA per 2048 elements here too: on two GPUs the step with its
// peer stores takes 9.5 ms (709 GB/s leaving each GPU) against 10.5 ms (639) as a resident wave
// with four groups per thread; 1, 2 and 4 groups per thread measure the same with one CTA per chunk.
constexpr int kPushUnroll = 1;
constexpr int kPushElems = kThreads * kVec * kPushUnroll;

template <typename TP, typename TM>
__global__ void __launch_bounds__(kThreads)
lion_flat_push_kernel(TP* __restrict__ p_local, const TP* __restrict__ g, TM* __restrict__ m_shard,
                      int64_t begin, int64_t numel, PeerList peers, LionConsts c) {
  // p_local, g and the peers' bases address element 0 of the flat buffers; m_shard addresses the
  // momentum of element `begin`.
  const int64_t total_chunks = (numel + kPushElems - 1) / kPushElems;
  // 16-byte accesses need every address aligned, the peers' included (their buffers may start
  // anywhere an element may); one unaligned buffer sends the whole shard down the scalar path
  uintptr_t addr_bits = reinterpret_cast<uintptr_t>(p_local + begin) | reinterpret_cast<uintptr_t>(g + begin) |
                        reinterpret_cast<uintptr_t>(m_shard);
#pragma unroll
  for (int r = 0; r < kMaxPeers; ++r)
    if (r < peers.n) addr_bits |= reinterpret_cast<uintptr_t>(static_cast<TP*>(peers.base[r]) + begin);
  const bool aligned = (addr_bits & 15) == 0;
  for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int64_t base = chunk * kPushElems;
    const int64_t remaining = numel - base;
    TP* p = p_local + begin + base;
    const TP* gg = g + begin + base;
    TM* m = m_shard + base;
    if (aligned && remaining >= kPushElems) {
      Group<TP> pv[kPushUnroll], gv[kPushUnroll];
      Group<TM> mv[kPushUnroll];
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) {
        const int off = (u * kThreads + threadIdx.x) * kVec;
        load_group(pv[u], p + off);
        load_group(gv[u], gg + off);
        load_group(mv[u], m + off);
      }
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) {
        lion_group<TP, TM>(pv[u], gv[u], mv[u], c);
        const int off = (u * kThreads + threadIdx.x) * kVec;
        store_group(p + off, pv[u]);
        store_group(m + off, mv[u]);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
          if (r < peers.n) {
            TP* dst = static_cast<TP*>(peers.base[r]) + begin + base + off;
            constexpr int n16 = sizeof(TP) * kVec / 16;
#pragma unroll
            for (int q = 0; q < n16; ++q)
              reinterpret_cast<uint4*>(dst)[q] = reinterpret_cast<const uint4*>(pv[u].v)[q];
          }
        }
      }
    } else {
      const int n = remaining < kPushElems ? static_cast<int>(remaining) : kPushElems;
      for (int i = threadIdx.x; i < n; i += kThreads) {
        TP pe = p[i];
        TM me = m[i];
        lion_element<TP, TM>(pe, gg[i], me, c);
        p[i] = pe;
        m[i] = me;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
          if (r < peers.n) static_cast<TP*>(peers.base[r])[begin + base + i] = pe;
      }
    }
  }
}

template <typename TP, typename TM>
int launch_push(void* p, const void* g, void* m, int64_t begin, int64_t numel, const PeerList& peers,
                const LionConsts& c, int device, cudaStream_t stream) {
  const int64_t total_chunks = (numel + kPushElems - 1) / kPushElems;
  // the kernel strides over chunks, so a grid cut at the launch limit still covers them all
  const int64_t grid = total_chunks < 0x7fffffffll ? total_chunks : 0x7fffffffll;
  lion_flat_push_kernel<TP, TM><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      static_cast<TP*>(p), static_cast<const TP*>(g), static_cast<TM*>(m), begin, numel, peers, c);
  fo::g_launch_count.fetch_add(1, std::memory_order_relaxed);
  FO_CUDA_CHECK(cudaGetLastError());
  return FO_OK;
}

}  // namespace

extern "C" int fo_lion_flat_step_push(void* param, const void* grad, void* exp_avg_shard,
                                      int64_t begin, int64_t end,
                                      void* const* peer_params, int n_peers,
                                      int p_dtype, int g_dtype, int m_dtype,
                                      double lr, double beta1, double beta2, double weight_decay,
                                      int device, void* stream) {
  fo::clear_error();
  if (int rc = check_dtypes(p_dtype, g_dtype, m_dtype)) return rc;
  FO_REQUIRE(begin >= 0 && end >= begin, "bad shard range [%lld, %lld)", (long long)begin, (long long)end);
  FO_REQUIRE(n_peers >= 0 && n_peers <= kMaxPeers, "n_peers must be in [0, %d] (got %d)", kMaxPeers, n_peers);
  FO_REQUIRE(n_peers == 0 || peer_params != nullptr, "null peer list");
  if (end == begin) return FO_OK;
  FO_REQUIRE(param && grad && exp_avg_shard, "null pointer");
  PeerList peers;
  peers.n = n_peers;
  for (int i = 0; i < kMaxPeers; ++i) peers.base[i] = nullptr;
  for (int i = 0; i < n_peers; ++i) {
    FO_REQUIRE(peer_params[i] != nullptr, "peer %d has a null buffer", i);
    FO_REQUIRE(peer_params[i] != param, "peer %d is the local buffer", i);
    peers.base[i] = peer_params[i];
  }
  LionConsts c;
  if (int rc = make_consts(lr, beta1, beta2, weight_decay, p_dtype, m_dtype, &c)) return rc;
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n = end - begin;
#define FO_LION_PUSH_CASE(PD, MD, TP, TM) \
  if (p_dtype == PD && m_dtype == MD) return launch_push<TP, TM>(param, grad, exp_avg_shard, begin, n, peers, c, device, s);
  FO_LION_PUSH_CASE(FO_BF16, FO_BF16, __nv_bfloat16, __nv_bfloat16)
  FO_LION_PUSH_CASE(FO_BF16, FO_F32, __nv_bfloat16, float)
  FO_LION_PUSH_CASE(FO_F16, FO_F16, __half, __half)
  FO_LION_PUSH_CASE(FO_F16, FO_F32, __half, float)
  FO_LION_PUSH_CASE(FO_F32, FO_F32, float, float)
  FO_LION_PUSH_CASE(FO_F32, FO_BF16, float, __nv_bfloat16)
#undef FO_LION_PUSH_CASE
  return fo::fail(FO_ERR_UNSUPPORTED, "no fused-gather Lion kernel for dtypes p=%d m=%d", p_dtype, m_dtype);
}
