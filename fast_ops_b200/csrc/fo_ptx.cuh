// Hand-written PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, each CTA
// loading its own tiles), tcgen05 (tensor memory allocation, MMA, load/store, commit, fences) and
// the shared-memory / instruction descriptors the MMA consumes.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace fo {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ---------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes mbarrier initialisation visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking poll of a phase (try_wait may suspend the thread for a while when the phase is
// still open; test_wait returns at once).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Every wait in the attention kernels goes through here: it spins on
// try_wait, and once `kWaitBudgetNs` of wall time has passed it records `code` in the
// CTA's abort word (shared memory) and in the device status word and returns false.  From
// then on every wait of the CTA returns at once (the abort word is checked first), so the
// CTA still runs to its end, frees its tensor memory and exits; results are garbage and
// the host sees the status word.
constexpr uint64_t kWaitBudgetNs = 1000ull * 1000ull * 1000ull;  // 1 s

__device__ __forceinline__ bool mbar_wait_budget(uint64_t* bar, uint32_t parity, volatile int* cta_abort,
                                                 int* device_status, int code, uint64_t budget_ns) {
  // the common case first: a completed phase costs one try_wait and no shared-memory load
  if (mbar_try_wait(bar, parity)) return true;
  if (*cta_abort) return false;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*cta_abort) return false;
      if (global_timer_ns() - t0 > budget_ns) {
        *cta_abort = code;
        atomicOr(device_status, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* cta_abort,
                                          int* device_status, int code) {
  return mbar_wait_budget(bar, parity, cta_abort, device_status, code, kWaitBudgetNs);
}

// ---- TMA ------------------------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 4-D tiled load into this CTA's shared memory; completion is signalled on `bar` as
// transaction bytes.  c0 is the innermost coordinate and must keep c0 * elem_size a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src,
                                             int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// 3-D tiled reduction (element-wise add, type taken from the tensor map) of a shared-memory tile
// into global memory; out-of-range elements are dropped.  Coordinates must not be negative.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1,
                                                  int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Asks for the 128-byte line holding `p` to be brought into L2 (a hint: no fault on a bad address
// is specified, so callers pass addresses inside their tensors only).
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Register budget of the executing warpgroup (all four warps of an aligned group of four must
// execute it): raise after the other warpgroups have lowered theirs.
template <int kRegs> __device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs> __device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// bar.sync on a named barrier (id 1..15) among `count` threads of the CTA
__device__ __forceinline__ void named_barrier_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// bar.arrive: counts this thread in on a named barrier without waiting for it
__device__ __forceinline__ void named_barrier_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// The same two operations tied into the data flow, for use as scheduling fences around pure
// arithmetic (which the compiler otherwise moves freely across a barrier): the sync form
// "produces" `dep`, so nothing computed from it can start earlier; the arrive form "consumes"
// its operands, so it cannot be issued before they have been computed.
__device__ __forceinline__ void named_barrier_sync_dep(int id, int count, float& dep) {
  asm volatile("bar.sync %1, %2;" : "+f"(dep) : "r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive_dep(int id, int count, float a, float b) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count), "f"(a), "f"(b) : "memory");
}
// Arrive that is pinned on both sides: it consumes a and b and "produces" dep, so arithmetic that
// uses dep afterwards cannot be scheduled in front of it either.
__device__ __forceinline__ void named_barrier_arrive_mid(int id, int count, float& dep, float a, float b) {
  asm volatile("bar.arrive %1, %2;" : "+f"(dep) : "r"(id), "r"(count), "f"(a), "f"(b) : "memory");
}

// Turn-taking between two groups of warps that share an execution unit.  The operations above
// order the barrier against arithmetic only for the compiler's front end; the assembler schedules
// the machine code again and, since a barrier instruction has no register operands, may move pure
// arithmetic across it.  These two tie the barrier to memory operations, which are not moved
// across a barrier, and the arithmetic to the values those operations produce or consume:
//   turn_wait: bar.sync, then a volatile load of a shared-memory word that holds 0.0f; the caller
//              adds the loaded value into an operand of everything that must come after.
//   turn_pass: a volatile store of `v` (something computed from all the work that must come first)
//              into a private shared-memory slot, then bar.arrive.
__device__ __forceinline__ float turn_wait(int id, int count, const float* zero_word) {
  float v;
  asm volatile("bar.sync %1, %2;\n\tld.volatile.shared.f32 %0, [%3];"
               : "=f"(v)
               : "r"(id), "r"(count), "r"(smem_u32(zero_word))
               : "memory");
  return v;
}
__device__ __forceinline__ void turn_pass(int id, int count, float* slot, float v) {
  asm volatile("st.volatile.shared.f32 [%2], %3;\n\tbar.arrive %0, %1;"
               ::"r"(id), "r"(count), "r"(smem_u32(slot)), "f"(v)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the shared-memory source of all committed stores has been read.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tensor memory ---------------------------------------------------------------------------
// A tensor-memory address is (lane << 16) | column; 128 lanes x 512 columns of 32 bits per SM.

// One full warp allocates `ncols` (power of two >= 32) columns; the base address is written
// to *smem_result.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 bit, 32 consecutive columns: thread t of the warp gets lane (base_lane + t),
// columns [col, col+32).  The lane field of `taddr` must be the warp's own quarter
// (32 * (warp_id % 4)).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// tcgen05.wait::ld that also names the 32 destination registers of a preceding tmem_ld32 as
// read-write operands: the compiler then cannot schedule any use of those registers ahead of
// the wait (the load fills them asynchronously until the wait completes).
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---- descriptors -------------------------------------------------------------------------------
//
// Shared-memory matrix descriptor (64 bit) of tcgen05.mma:
//   [ 0,14) start address >> 4          [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4      [46,48) version = 1 on sm_100
//   [49,52) base offset = 0             [52,53) LBO mode = 0
//   [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
//
// Both operand layouts used here are what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B of a
// [rows x 64] 16-bit box produces: row r of the box sits at byte r*128, its eight 16-byte
// units XOR-permuted by (r % 8); the box base must be 1024-byte aligned.
//
//  * K-major operand (rows = M or N index, the 64 contiguous elements run along K):
//    SBO = 1024 (next group of 8 rows), LBO unused (1); one MMA consumes K = 16 elements =
//    32 bytes, so the k-th slice of the box starts 32*k bytes further.
//  * MN-major operand (rows = K index, the 64 contiguous elements run along N):
//    SBO = 1024 (next group of 8 k-rows), LBO = byte distance between consecutive
//    64-element column blocks (a separate box); the k-th slice (16 rows) starts 2048*k
//    bytes further.
constexpr uint64_t kDescFixed = (1ull << 46) | (2ull << 61);  // version 1, 128-byte swizzle

__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return kDescFixed | static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4) |
         (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32);
}

// Instruction descriptor (32 bit) of tcgen05.mma.kind::f16, fp32 accumulation:
//   [4,6) D format: 1 = f32     [7,10) A format: 0 = f16, 1 = bf16     [10,13) B format
//   [15] A major (0 = K)        [16] B major (0 = K, 1 = MN)
//   [17,23) N >> 3              [24,29) M >> 4
// A and B must have the same format: an fp16 A next to a bf16 B raises an illegal-instruction error.
__host__ __device__ constexpr uint32_t make_idesc(int is_bf16, int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(is_bf16) << 7) | (static_cast<uint32_t>(is_bf16) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A holds 16-bit values packed two per 32-bit column.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same two instructions with each descriptor given as two 32-bit halves.  The high half
// (stride offset 1024, version, 128-byte swizzle) is the same for every operand used here, and
// the k-th slice of an operand differs from the first only in the low half's address field,
// so an issue loop needs one 32-bit add per operand and instruction.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);

__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFF) >> 4) | ((lbo_bytes >> 4) << 16);
}

__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Warp-collective forms: every lane of a converged warp executes the call with the same
// (warp-uniform) operands, one elected lane issues the instruction.  Keeping the operand
// arithmetic outside any divergent branch lets it run on the uniform datapath.
__device__ __forceinline__ void umma_ss_lo_elect(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      ".reg .b64 da, db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_ts_lo_elect(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      ".reg .b64 db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tcgen05_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}"
      ::"r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// max of three floats in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace fo
