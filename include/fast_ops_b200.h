/*
 * fast_ops_b200 — C ABI of the two B200 (sm_100a) hot paths.
 *
 * Every entry point takes plain pointers and sizes; no torch type crosses this
 * boundary.  All device pointers must belong to `device`.  All launches are
 * asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 * default stream).  Functions return FO_OK (0) or a negative FO_ERR_* code; the
 * text of the most recent error on the calling thread is fo_last_error().
 *
 * Reference interfaces are cited by their path inside jfc4050/fast-ops.
 */
#ifndef FAST_OPS_B200_H
#define FAST_OPS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FO_OK 0
#define FO_ERR_INVALID_ARGUMENT (-1) /* shape / dtype / stride / alignment contract violated */
#define FO_ERR_CUDA (-2)             /* a CUDA runtime or driver call failed */
#define FO_ERR_UNSUPPORTED (-3)      /* valid request this build has no kernel for */
#define FO_ERR_DEVICE_STATUS (-4)    /* a kernel recorded a bounded-wait timeout */

/* Element types.  FO_F32 is accepted only by the Lion entry points. */
#define FO_F16 0
#define FO_BF16 1
#define FO_F32 2

/* Library version: major*10000 + minor*100 + patch. */
int fo_version(void);

/* Message of the last error returned on this host thread ("" if none). */
const char* fo_last_error(void);

/*
 * Device-side status word of `device`: 0 when every kernel launched by this
 * library so far finished its bounded waits, otherwise a code naming the wait
 * that gave up (the kernel still ran to its end and freed its tensor memory).
 * Synchronises the device.  If `reset` is non-zero the word is cleared.
 */
int fo_device_status(int device, int* status_out, int reset);

/*
 * FlashAttention forward:  O = softmax(scale * Q K^T + causal_mask) V,
 * LSE[b,h,i] = log(sum_j exp(scale * q_i . k_j))  (natural log, fp32).
 *
 * Replaces flash_attn_fwd_cuda(Q, K, V) (fast_ops/flash_attention/
 * flash_attention_fwd.cu:154-181), bound to Python as `forward`
 * (fast_ops/flash_attention/flash_attention.cpp:12-14).  The reference takes
 * (B,H,M,D)/(B,H,N,D) tensors and implies scale = 1/sqrt(D); the causal flag
 * and the LSE output follow the semantics of the reference's complete forward
 * (fast_ops/flash_attention/flash_attention_triton.py:149-150, :174-175, :255).
 *
 *   q, k, v, o : device pointers, fp16 or bf16 (`dtype`), 16-byte aligned.
 *   lse        : device pointer to B*H*Sq floats (contiguous), or NULL.
 *   *_strides  : element strides of the batch, head and sequence dimensions
 *                (in that order); the head_dim stride is 1.  Each stride must
 *                be a multiple of 8 elements (16 bytes).
 *   D          : a multiple of 8, at most 128 (the reference's contract,
 *                fast_ops/flash_attention/flash_attention.py:61-70).  The kernels are built for 64
 *                and 128; other values run zero-padded in the next larger one.
 *   causal     : non-zero masks column j > row i (top-left aligned).
 *   softmax_scale : multiplies Q K^T; pass 1/sqrt(D) for the reference default.
 */
int fo_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                      int B, int H, int Sq, int Sk, int D,
                      const int64_t q_strides[3], const int64_t k_strides[3],
                      const int64_t v_strides[3], const int64_t o_strides[3],
                      int dtype, int causal, float softmax_scale,
                      int device, void* stream);

/*
 * Process-wide options of the attention forward (tuning and tests; nothing in the reference
 * corresponds).  Each argument: -1 leaves the option as it is.
 *   impl       : 0 = chosen per call (default), 1 = the unoverlapped bring-up kernel, 2 = the
 *                warp-specialised kernel with 128-key softmax tiles, 3 = the one with 64-key steps,
 *                4 = the 64-key kernel as a persistent grid, 5 = the 64-key kernel with one query
 *                tile per CTA and two CTAs per SM (4 and 5: plain attention only).
 *   ping_pong  : 64-key kernel: 1 (default) = the two query tiles of a CTA take turns on the
 *                exponential units, 0 = they run free.
 *   head_group : heads scheduled together so that their K and V stay in L2; 0 (default) = derived
 *                from the K/V size.
 */
int fo_attn_configure(int impl, int ping_pong, int head_group);

/*
 * FlashAttention backward: dQ, dK, dV for the output gradient `dout`, given the forward's inputs,
 * its output O and its LSE.  The reference's CUDA path leaves backward unimplemented
 * (fast_ops/flash_attention/flash_attention.py:41-45); the semantics are those of its complete
 * implementation (fast_ops/flash_attention/flash_attention_triton.py:273-315, :322-638, :832-958).
 * Layouts, dtypes, D, causal and softmax_scale as in fo_flash_attn_fwd; every tensor has its own
 * batch/head/sequence strides.  `dq_accum` (B*H*Sq*D floats) and `delta` (B*H*Sq floats) are
 * scratch the caller provides; their contents on entry do not matter.  Three launches on `stream`:
 * delta = rowsum(O o dO), the main kernel (dK, dV per key tile; dQ added into dq_accum with
 * bulk reduce-adds, so dQ may differ in the last bit between runs), and the rounding of dq_accum into dq.
 */
int fo_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                      const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta,
                      int B, int H, int Sq, int Sk, int D,
                      const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                      const int64_t o_strides[3], const int64_t do_strides[3],
                      const int64_t dq_strides[3], const int64_t dk_strides[3], const int64_t dv_strides[3],
                      int dtype, int causal, float softmax_scale, int device, void* stream);

/*
 * FlashAttention forward and backward with the additive bias and the dropout of the reference's
 * complete implementation (forward: fast_ops/flash_attention/flash_attention_triton.py:176-199
 * bias, :215-219 dropout; backward: :496-510, :517-551, :580-603).  The arguments up to
 * softmax_scale are those of fo_flash_attn_fwd / fo_flash_attn_bwd.
 *
 *   bias         : NULL, or a device pointer to values added to softmax_scale * Q K^T before the
 *                  softmax: element (b, h, i, j) at bias + b*s[0] + h*s[1] + i*s[2] + j with
 *                  s = bias_strides in elements; a stride of 0 broadcasts that dimension (the
 *                  reference's "vector" bias is s[2] = 0, flash_attention_triton.py:760-769).
 *                  -inf entries mask; a row whose entries are all masked gets O = 0 and
 *                  LSE = -inf (the torch oracle gives NaN there).  No gradient is produced for
 *                  the bias, as in the reference (flash_attention_triton.py:854).
 *   bias_dtype   : FO_F32, or the dtype of q (flash_attention_triton.py:755).
 *   dropout_p    : in [0, 1).  Element (i, j) of head (b, h) is kept iff
 *                  hash((uint32)(rng_offset + ((b*H + h)*Sq + i)*Sk + j) ^ (uint32)rng_seed) >
 *                  (uint32)(dropout_p * 2^32) with the integer hash of
 *                  flash_attention_triton.py:38-50; kept probabilities are scaled by
 *                  1 / (1 - dropout_p) in P V, the row sums and LSE are those without dropout.
 *                  The backward must be given the forward's p, seed and offset.
 */
int fo_flash_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse,
                         int B, int H, int Sq, int Sk, int D,
                         const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t o_strides[3],
                         int dtype, int causal, float softmax_scale,
                         const void* bias, const int64_t bias_strides[3], int bias_dtype,
                         float dropout_p, uint64_t rng_seed, uint64_t rng_offset,
                         int device, void* stream);

int fo_flash_attn_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* dout,
                         const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta,
                         int B, int H, int Sq, int Sk, int D,
                         const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                         const int64_t o_strides[3], const int64_t do_strides[3],
                         const int64_t dq_strides[3], const int64_t dk_strides[3], const int64_t dv_strides[3],
                         int dtype, int causal, float softmax_scale,
                         const void* bias, const int64_t bias_strides[3], int bias_dtype,
                         float dropout_p, uint64_t rng_seed, uint64_t rng_offset,
                         int device, void* stream);

/*
 * Materialises the keep mask of the dropout above as B*H*Sq*Sk bytes (1 = kept), dense in
 * (b, h, i, j) order.  Replaces triton_dropout_mask / _dropout_mask_kernel
 * (fast_ops/flash_attention/flash_attention_triton.py:668-717), which the reference's tests use
 * to build the oracle's mask.
 */
int fo_dropout_mask(uint8_t* out, int B, int H, int Sq, int Sk, float dropout_p, uint64_t rng_seed,
                    uint64_t rng_offset, int device, void* stream);

/*
 * Fused Lion step on one dense tensor, in place:
 *   p <- p * (1 - lr*wd);  u = sign(beta1*m + (1-beta1)*g);  p <- p - lr*u;
 *   m <- beta2*m + (1-beta2)*g
 * with a rounding to the storage type after every product and sum, which is
 * what the reference torch implementation does
 * (fast_ops/lion/lion_optimizer_ref.py:51-67); sign(0) is 0.
 *
 * Replaces lion_update(param, grad, exp_avg, lr, beta1, beta2, weight_decay)
 * (fast_ops/lion/lion_update.cu:121-161, bound at fast_ops/lion/lion.cpp:13-15).
 * Hyper-parameters are doubles so that the derived constants (1 - lr*wd, ...)
 * are formed in double and rounded to float once, as torch does with Python
 * scalars.  p_dtype must equal g_dtype (lion_update.cu:132-133).
 */
int fo_lion_update(void* param, const void* grad, void* exp_avg, int64_t numel,
                   int p_dtype, int g_dtype, int m_dtype,
                   double lr, double beta1, double beta2, double weight_decay,
                   int device, void* stream);

/*
 * The same step over a list of tensors in ONE kernel launch.  Replaces the
 * per-tensor loop of Lion.step() (fast_ops/lion/lion_optimizer.py:57-76).
 * `params`, `grads`, `exp_avgs` and `numels` are HOST arrays of n_tensors
 * entries holding device pointers / element counts.  The device-side table
 * (one 32-byte record per 8192 elements of every tensor: 0.4 % of the bytes of
 * a 16-bit tensor) is built on the first call for a given list and dtypes
 * (cudaMalloc, and a copy on `stream`) and cached inside the library, keyed by
 * the list's contents, so later calls with the same list do no host-to-device
 * copy.  At most 32 lists are kept; the least recently used one is dropped for
 * a new one.  A list of one tensor needs no table.  CUDA graphs: a captured launch keeps its list's
 * table, so make the first call with a list outside the capture (on a capturing
 * stream it is refused with FO_ERR_UNSUPPORTED), and neither 32 other lists nor
 * fo_lion_clear_cache may come between the capture and a replay.
 */
int fo_lion_multi_tensor_step(void* const* params, const void* const* grads,
                              void* const* exp_avgs, const int64_t* numels, int n_tensors,
                              int p_dtype, int g_dtype, int m_dtype,
                              double lr, double beta1, double beta2, double weight_decay,
                              int device, void* stream);

/*
 * The same step on elements [begin, end) of flat buffers: the shard a rank owns
 * when parameters are partitioned ZeRO-1 style.  `exp_avg` points at the
 * momentum of element `begin` (a rank keeps momentum for its shard only);
 * `param` and `grad` point at element 0 of the flat buffers.  No counterpart in
 * the reference, whose step is per tensor (fast_ops/lion/lion_optimizer.py:64-76).
 */
int fo_lion_flat_step(void* param, const void* grad, void* exp_avg_shard,
                      int64_t begin, int64_t end,
                      int p_dtype, int g_dtype, int m_dtype,
                      double lr, double beta1, double beta2, double weight_decay,
                      int device, void* stream);

/*
 * fo_lion_flat_step fused with the distribution of the updated weights: every updated value of
 * [begin, end) is stored to the local flat buffer and, by plain stores over NVLink, to the same
 * position of each peer's flat buffer (`peer_params`: HOST array of n_peers <= 7 device pointers
 * to element 0 of the peers' buffers, mapped for peer access).  It replaces "step, then
 * all-gather" of a ZeRO-1 optimizer step; the reference has neither.  The caller orders the ranks:
 * no peer may still be reading its buffer when this kernel starts, and all ranks' kernels must
 * have finished before any rank reads the gathered weights.
 */
int fo_lion_flat_step_push(void* param, const void* grad, void* exp_avg_shard,
                           int64_t begin, int64_t end,
                           void* const* peer_params, int n_peers,
                           int p_dtype, int g_dtype, int m_dtype,
                           double lr, double beta1, double beta2, double weight_decay,
                           int device, void* stream);

/*
 * fo_lion_multi_tensor_step for callers that must not allocate: same arguments, same kernel,
 * same results, but the device-side tensor table lives in a fixed array inside the library
 * (about 40 KiB per device that loads the library, held until the process exits) instead of
 * memory obtained with cudaMalloc.  Meant for a step loop whose owner has given all device
 * memory to its own pool, or that cannot tolerate the device-wide synchronisation an
 * allocation may cause.  It has no counterpart in the reference.
 *
 *   - At most 1024 tensors per call; a longer list is rejected with FO_ERR_INVALID_ARGUMENT
 *     (split it, or use fo_lion_multi_tensor_step).
 *   - It calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a device
 *     looks up the array's device address.
 *   - A stream that is being captured is refused with FO_ERR_UNSUPPORTED: the table upload would
 *     turn into a graph node that reads the library's one host-side image at replay time, when it
 *     holds the list of whichever call came last.
 *   - The table is copied to the device on `stream` on every call, ahead of the kernel.  All
 *     calls on a device share the one array and every call rewrites the entries it uses:
 *     calls on the same stream are ordered, but two calls whose kernels can overlap on the GPU
 *     (different streams without an event between them) race on the table.
 */
int fo_lion_multi_tensor_step_noalloc(void* const* params, const void* const* grads,
                                      void* const* exp_avgs, const int64_t* numels, int n_tensors,
                                      int p_dtype, int g_dtype, int m_dtype,
                                      double lr, double beta1, double beta2, double weight_decay,
                                      int device, void* stream);

/* Drops the cached tensor tables of fo_lion_multi_tensor_step (all devices). */
int fo_lion_clear_cache(void);

/*
 * Number of kernels this library has launched since load (all entry points,
 * this process).  Lets a caller count launches inside a timed region.
 */
int64_t fo_launch_count(void);

/*
 * Self-test hooks for the tensor-core building blocks of the attention kernel
 * (one 128 x N x K tile through TMA + tcgen05.mma + tcgen05.ld).  mode 0:
 * C = A B^T with A (128 x K) and B (N x K) both K-major from shared memory;
 * mode 1: C = A B with A (128 x K) written to tensor memory by the threads and
 * B (K x N) N-major from shared memory.  a, b: device bf16/fp16; c: device
 * fp32 128 x N row-major.  K in {64,128}, N in {64,128}.  Test use only.
 */
int fo_debug_umma_tile(const void* a, const void* b, float* c, int N, int K,
                       int dtype, int mode, int device, void* stream);

/*
 * Self-test of the bounded device-side wait that every attention kernel uses: launches one warp
 * that waits, with a budget of `budget_us` microseconds (1 .. 100000), on a barrier nobody will
 * ever arrive on.  The wait must give up, OR FO_STATUS bit 0x10 into the device status word
 * (fo_device_status then reports it until reset) and the kernel must return normally; `returned`
 * (device int, may be NULL) receives 2 when that happened.  No fault is involved at any point.
 * Test use only; nothing in the reference corresponds.
 */
int fo_debug_wait_timeout(int budget_us, int* returned, int device, void* stream);

/*
 * Kernel-tuning aid, present only in a library built with -DFO_ATTN_TRACE=1 (the default build
 * returns FO_ERR_UNSUPPORTED for a non-NULL buffer): after fo_debug_set_attn_trace(buf) the
 * warp-specialised attention kernels record, for their first CTA, SM clock values of the
 * hand-offs between the softmax warps and the MMA issuer into `buf` (device memory of
 * roles*iters*events 64-bit words, see fo_debug_attn_trace_shape; zero it first).  NULL switches
 * the recording off.
 */
int fo_debug_set_attn_trace(void* device_buffer);
int fo_debug_attn_trace_shape(int* roles, int* iters, int* events);

#ifdef __cplusplus
}
#endif
#endif /* FAST_OPS_B200_H */
