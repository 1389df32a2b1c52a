/*
 * CPU oracle for the two hot paths.  TEST INFRASTRUCTURE ONLY: tests/, the smoke check and
 * the CPU-baseline leg of bench.py use it as the checker and as the timed CPU reference;
 * nothing in the product (fast_ops_b200/) may call it.
 *
 * It restates, in plain C, what the reference's torch implementations compute:
 *   - oracle_attention_fwd follows fast_ops/flash_attention/attention_ref.py:41-73
 *     (upcast to fp32, scores = (q/sqrt(d)) . k, causal triu(.,1) -> -inf, softmax, P V);
 *     the LSE it also returns is the quantity the reference's complete forward stores
 *     (fast_ops/flash_attention/flash_attention_triton.py:241-255).
 *   - oracle_lion_step follows fast_ops/lion/lion_optimizer_ref.py:51-67, including the
 *     rounding to the storage type after each tensor op and torch's handling of scalars
 *     (a `mul` scalar stays fp32; an `add_(..., alpha=a)` rounds a to the promoted tensor
 *     type and evaluates self + a*other as one fused multiply-add in fp32).
 *
 * Parity is pinned: tests/test_oracle_golden.py checks both functions against vectors
 * produced by importing the reference itself (tests/golden/make_golden.py).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#define ORACLE_F16 0
#define ORACLE_BF16 1
#define ORACLE_F32 2

/* ---- a small parallel-for on pthreads (this image's gcc ships no OpenMP runtime) -------- */

static int g_threads = 0; /* 0 = one per online core */

int oracle_num_threads(void) {
  if (g_threads > 0) return g_threads;
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

void oracle_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*range_fn)(int64_t begin, int64_t end, void* ctx);

typedef struct {
  range_fn fn;
  void* ctx;
  int64_t total, grain;
  int64_t next; /* next unclaimed index, advanced atomically */
} par_job;

static void* par_worker(void* arg) {
  par_job* job = (par_job*)arg;
  for (;;) {
    const int64_t b = __atomic_fetch_add(&job->next, job->grain, __ATOMIC_RELAXED);
    if (b >= job->total) break;
    const int64_t e = b + job->grain < job->total ? b + job->grain : job->total;
    job->fn(b, e, job->ctx);
  }
  return NULL;
}

/* Runs fn over [0, total) in pieces of `grain`, handed out dynamically to the threads. */
static void parallel_for(int64_t total, int64_t grain, range_fn fn, void* ctx) {
  if (total <= 0) return;
  int nt = oracle_num_threads();
  if ((int64_t)nt * grain > total) nt = (int)((total + grain - 1) / grain);
  par_job job = {fn, ctx, total, grain, 0};
  if (nt <= 1) {
    par_worker(&job);
    return;
  }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nt);
  int started = 0;
  for (int i = 0; i < nt - 1; ++i) {
    if (pthread_create(&th[started], NULL, par_worker, &job) == 0) ++started;
  }
  par_worker(&job);
  for (int i = 0; i < started; ++i) pthread_join(th[i], NULL);
  free(th);
}

/* ---- storage-type conversions (round to nearest even) ---------------------------------- */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}

static inline uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f; /* IEEE round-to-nearest-even */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}

static inline float round_to(float x, int dtype) {
  if (dtype == ORACLE_BF16) return bf16_to_f32(f32_to_bf16(x));
  if (dtype == ORACLE_F16) return f16_to_f32(f32_to_f16(x));
  return x;
}

static inline float load_elem(const void* base, int64_t i, int dtype) {
  if (dtype == ORACLE_F32) return ((const float*)base)[i];
  uint16_t h = ((const uint16_t*)base)[i];
  return dtype == ORACLE_BF16 ? bf16_to_f32(h) : f16_to_f32(h);
}

static inline void store_elem(void* base, int64_t i, int dtype, float x) {
  if (dtype == ORACLE_F32) ((float*)base)[i] = x;
  else if (dtype == ORACLE_BF16) ((uint16_t*)base)[i] = f32_to_bf16(x);
  else ((uint16_t*)base)[i] = f32_to_f16(x);
}

static inline int promote(int a, int b) { return a == b ? a : ORACLE_F32; }

/* ---- Lion -------------------------------------------------------------------------------
 * One step on one tensor, in place.  param/grad share p_dtype (the reference's fused kernel
 * requires it, fast_ops/lion/lion_update.cu:132-133); exp_avg has m_dtype.
 * Lines cited are of fast_ops/lion/lion_optimizer_ref.py. */
typedef struct {
  void* param;
  const void* grad;
  void* exp_avg;
  int p_dtype, m_dtype;
  double lr, beta1, beta2, weight_decay;
} lion_ctx;

static void lion_range(int64_t begin, int64_t end, void* vctx) {
  const lion_ctx* c = (const lion_ctx*)vctx;
  void* param = c->param;
  const void* grad = c->grad;
  void* exp_avg = c->exp_avg;
  const int p_dtype = c->p_dtype, m_dtype = c->m_dtype;
  const int u_dtype = promote(p_dtype, m_dtype);
  const float c_wd = (float)(1.0 - c->lr * c->weight_decay);
  const float c_b1 = (float)c->beta1;
  const float c_1mb1 = (float)(1.0 - c->beta1);
  const float c_b2 = (float)c->beta2;
  const float c_nlr = round_to((float)(-c->lr), u_dtype);
  const float c_1mb2 = round_to((float)(1.0 - c->beta2), u_dtype);
  for (int64_t i = begin; i < end; ++i) {
    const float p = load_elem(param, i, p_dtype);
    const float g = load_elem(grad, i, p_dtype);
    const float m = load_elem(exp_avg, i, m_dtype);
    /* :51  p.data.mul_(1 - lr * wd) */
    const float p1 = round_to(p * c_wd, p_dtype);
    /* :64  update = exp_avg * beta1 + grad * (1 - beta1)   (three ops, each rounded) */
    const float t1 = round_to(m * c_b1, m_dtype);
    const float t2 = round_to(g * c_1mb1, p_dtype);
    const float u = round_to(t1 + t2, u_dtype);
    const float s = (u > 0.f) ? 1.f : ((u < 0.f) ? -1.f : 0.f);
    /* :65  p.add_(torch.sign(update), alpha=-lr) */
    store_elem(param, i, p_dtype, fmaf(c_nlr, s, p1));
    /* :67  exp_avg.mul_(beta2).add_(grad, alpha=1 - beta2) */
    const float m1 = round_to(m * c_b2, m_dtype);
    store_elem(exp_avg, i, m_dtype, fmaf(c_1mb2, g, m1));
  }
}

void oracle_lion_step(void* param, const void* grad, void* exp_avg, int64_t numel, int p_dtype,
                      int m_dtype, double lr, double beta1, double beta2, double weight_decay) {
  lion_ctx ctx = {param, grad, exp_avg, p_dtype, m_dtype, lr, beta1, beta2, weight_decay};
  parallel_for(numel, 1 << 16, lion_range, &ctx);
}

/* ---- attention --------------------------------------------------------------------------
 * q: (B,H,Sq,D), k/v: (B,H,Sk,D), all fp32 and dense; out: (B,H,Sq,D) fp32; lse: (B,H,Sq)
 * fp32 or NULL.  `scale` multiplies q before the dot products (attention_ref.py:46 divides q
 * by sqrt(d); pass 1/sqrt(d)).  Causal masking is top-left aligned: column j > row i is
 * -inf (attention_ref.py:54-58).  `bh_begin/bh_end` restrict the work to a range of flattened
 * (batch, head) pairs, and `row_begin/row_end/row_stride` to query rows row_begin,
 * row_begin+row_stride, ... < row_end of each pair, so that a bounded sample of a large problem
 * can be checked or timed; rows outside the sample are left untouched. */
typedef struct {
  const float *q, *k, *v;
  float *out, *lse;
  int Sq, Sk, D, causal, bh_begin;
  int row_begin, row_stride, rows_per_bh;
  float scale;
} attn_ctx;

static void attn_range(int64_t begin, int64_t end, void* vctx) {
  const attn_ctx* c = (const attn_ctx*)vctx;
  const float *q = c->q, *k = c->k, *v = c->v;
  float *out = c->out, *lse = c->lse;
  const int Sq = c->Sq, Sk = c->Sk, D = c->D, causal = c->causal, bh_begin = c->bh_begin;
  const float scale = c->scale;
  {
    float* scores = (float*)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
    float* qs = (float*)malloc(sizeof(float) * (size_t)D);
    float* acc = (float*)malloc(sizeof(float) * (size_t)D);
    for (int64_t r = begin; r < end; ++r) {
      const int bh = bh_begin + (int)(r / c->rows_per_bh);
      const int i = c->row_begin + (int)(r % c->rows_per_bh) * c->row_stride;
      const float* qi = q + ((int64_t)bh * Sq + i) * D;
      const float* kb = k + (int64_t)bh * Sk * D;
      const float* vb = v + (int64_t)bh * Sk * D;
      float* oi = out + ((int64_t)bh * Sq + i) * D;
      int n = Sk;
      if (causal && i + 1 < n) n = i + 1;
      for (int d = 0; d < D; ++d) qs[d] = qi[d] * scale;
      float mx = -INFINITY;
      for (int j = 0; j < n; ++j) {
        const float* kj = kb + (int64_t)j * D;
        float s = 0.f;
#pragma omp simd reduction(+ : s)
        for (int d = 0; d < D; ++d) s += qs[d] * kj[d];
        scores[j] = s;
        if (s > mx) mx = s;
      }
      float sum = 0.f;
      for (int j = 0; j < n; ++j) {
        const float e = expf(scores[j] - mx);
        scores[j] = e;
        sum += e;
      }
      for (int d = 0; d < D; ++d) acc[d] = 0.f;
      for (int j = 0; j < n; ++j) {
        const float pj = scores[j];
        const float* vj = vb + (int64_t)j * D;
#pragma omp simd
        for (int d = 0; d < D; ++d) acc[d] += pj * vj[d];
      }
      const float inv = 1.f / sum;
      for (int d = 0; d < D; ++d) oi[d] = acc[d] * inv;
      if (lse) lse[(int64_t)bh * Sq + i] = mx + logf(sum);
    }
    free(scores);
    free(qs);
    free(acc);
  }
}

void oracle_attention_fwd(const float* q, const float* k, const float* v, float* out, float* lse,
                          int B, int H, int Sq, int Sk, int D, int causal, float scale,
                          int bh_begin, int bh_end, int row_begin, int row_end, int row_stride) {
  if (bh_begin < 0) bh_begin = 0;
  if (bh_end > B * H) bh_end = B * H;
  if (row_begin < 0) row_begin = 0;
  if (row_end > Sq) row_end = Sq;
  if (row_stride < 1) row_stride = 1;
  if (bh_end <= bh_begin || row_end <= row_begin || Sk <= 0) return;
  const int rows_per_bh = (row_end - row_begin + row_stride - 1) / row_stride;
  attn_ctx ctx = {q, k, v, out, lse, Sq, Sk, D, causal, bh_begin, row_begin, row_stride, rows_per_bh, scale};
  parallel_for((int64_t)(bh_end - bh_begin) * rows_per_bh, 16, attn_range, &ctx);
}

/* ---- attention backward ------------------------------------------------------------------
 * Gradients of out = softmax(scale * q k^T [+ causal mask]) v with respect to q, k, v for a
 * given d_out, all fp32 and dense (B,H,S,D): what torch autograd computes through
 * fast_ops/flash_attention/attention_ref.py:41-67 (the way the reference's own tests obtain
 * their expected gradients, tests/test_flash_attention_triton.py:118-131).
 *   P = softmax(S),  dV = P^T dO,  dP = dO V^T,  dS = P o (dP - rowsum(dP o P)) * scale,
 *   dQ = dS K,  dK = dS^T Q.
 * Pass 1 runs over query rows (row statistics and dQ), pass 2 over keys (dK, dV), so no two
 * threads ever add into the same output. */
typedef struct {
  const float *q, *k, *v, *dout;
  float *dq, *dk, *dv, *lse, *delta;
  int Sq, Sk, D, causal, bh_begin;
  float scale;
} attn_bwd_ctx;

static void attn_bwd_rows(int64_t begin, int64_t end, void* vctx) {
  const attn_bwd_ctx* c = (const attn_bwd_ctx*)vctx;
  const int Sq = c->Sq, Sk = c->Sk, D = c->D;
  float* p = (float*)malloc(sizeof(float) * (size_t)Sk);
  float* o = (float*)malloc(sizeof(float) * (size_t)D);
  float* acc = (float*)malloc(sizeof(float) * (size_t)D);
  for (int64_t r = begin; r < end; ++r) {
    const int bh = c->bh_begin + (int)(r / Sq);
    const int i = (int)(r % Sq);
    const float* qi = c->q + ((int64_t)bh * Sq + i) * D;
    const float* doi = c->dout + ((int64_t)bh * Sq + i) * D;
    const float* kb = c->k + (int64_t)bh * Sk * D;
    const float* vb = c->v + (int64_t)bh * Sk * D;
    int n = Sk;
    if (c->causal && i + 1 < n) n = i + 1;
    float mx = -INFINITY;
    for (int j = 0; j < n; ++j) {
      const float* kj = kb + (int64_t)j * D;
      float s = 0.f;
#pragma omp simd reduction(+ : s)
      for (int d = 0; d < D; ++d) s += qi[d] * kj[d];
      s *= c->scale;
      p[j] = s;
      if (s > mx) mx = s;
    }
    float sum = 0.f;
    for (int j = 0; j < n; ++j) {
      p[j] = expf(p[j] - mx);
      sum += p[j];
    }
    const float inv = 1.f / sum;
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    for (int j = 0; j < n; ++j) {
      p[j] *= inv;
      const float* vj = vb + (int64_t)j * D;
#pragma omp simd
      for (int d = 0; d < D; ++d) o[d] += p[j] * vj[d];
    }
    float delta = 0.f;
    for (int d = 0; d < D; ++d) delta += o[d] * doi[d];
    c->lse[(int64_t)bh * Sq + i] = mx + logf(sum);
    c->delta[(int64_t)bh * Sq + i] = delta;
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int j = 0; j < n; ++j) {
      const float* vj = vb + (int64_t)j * D;
      const float* kj = kb + (int64_t)j * D;
      float dp = 0.f;
#pragma omp simd reduction(+ : dp)
      for (int d = 0; d < D; ++d) dp += doi[d] * vj[d];
      const float ds = p[j] * (dp - delta) * c->scale;
#pragma omp simd
      for (int d = 0; d < D; ++d) acc[d] += ds * kj[d];
    }
    float* dqi = c->dq + ((int64_t)bh * Sq + i) * D;
    for (int d = 0; d < D; ++d) dqi[d] = acc[d];
  }
  free(p);
  free(o);
  free(acc);
}

static void attn_bwd_keys(int64_t begin, int64_t end, void* vctx) {
  const attn_bwd_ctx* c = (const attn_bwd_ctx*)vctx;
  const int Sq = c->Sq, Sk = c->Sk, D = c->D;
  float* ak = (float*)malloc(sizeof(float) * (size_t)D);
  float* av = (float*)malloc(sizeof(float) * (size_t)D);
  for (int64_t r = begin; r < end; ++r) {
    const int bh = c->bh_begin + (int)(r / Sk);
    const int j = (int)(r % Sk);
    const float* kj = c->k + ((int64_t)bh * Sk + j) * D;
    const float* vj = c->v + ((int64_t)bh * Sk + j) * D;
    for (int d = 0; d < D; ++d) ak[d] = av[d] = 0.f;
    for (int i = c->causal ? j : 0; i < Sq; ++i) {
      const float* qi = c->q + ((int64_t)bh * Sq + i) * D;
      const float* doi = c->dout + ((int64_t)bh * Sq + i) * D;
      float s = 0.f, dp = 0.f;
#pragma omp simd reduction(+ : s, dp)
      for (int d = 0; d < D; ++d) {
        s += qi[d] * kj[d];
        dp += doi[d] * vj[d];
      }
      const float p = expf(s * c->scale - c->lse[(int64_t)bh * Sq + i]);
      const float ds = p * (dp - c->delta[(int64_t)bh * Sq + i]) * c->scale;
#pragma omp simd
      for (int d = 0; d < D; ++d) {
        av[d] += p * doi[d];
        ak[d] += ds * qi[d];
      }
    }
    float* dkj = c->dk + ((int64_t)bh * Sk + j) * D;
    float* dvj = c->dv + ((int64_t)bh * Sk + j) * D;
    for (int d = 0; d < D; ++d) {
      dkj[d] = ak[d];
      dvj[d] = av[d];
    }
  }
  free(ak);
  free(av);
}

/* lse and delta are scratch of B*H*Sq floats supplied by the caller. */
void oracle_attention_bwd(const float* q, const float* k, const float* v, const float* dout, float* dq,
                          float* dk, float* dv, float* lse, float* delta, int B, int H, int Sq, int Sk,
                          int D, int causal, float scale, int bh_begin, int bh_end) {
  if (bh_begin < 0) bh_begin = 0;
  if (bh_end > B * H) bh_end = B * H;
  if (bh_end <= bh_begin || Sq <= 0 || Sk <= 0) return;
  attn_bwd_ctx ctx = {q, k, v, dout, dq, dk, dv, lse, delta, Sq, Sk, D, causal, bh_begin, scale};
  parallel_for((int64_t)(bh_end - bh_begin) * Sq, 8, attn_bwd_rows, &ctx);
  parallel_for((int64_t)(bh_end - bh_begin) * Sk, 8, attn_bwd_keys, &ctx);
}

/* ---- attention with bias and dropout -------------------------------------------------------
 * fast_ops/flash_attention/attention_ref.py:41-67 with its optional arguments:
 *   scores = (q / sqrt(d)) k^T;  scores += bias (:50-51);  causal triu(.,1) -> -inf (:54-58);
 *   attention = softmax(scores) (:59);  dropped entries -> 0 (:63-64);
 *   out = attention_drop (v / (1 - p)) (:67).
 * bias: fp32, element (b,h,i,j) at bias[b*sb + h*sh + i*sq + j] (0 strides broadcast), or NULL.
 * keep: dense (B,H,Sq,Sk) bytes, 1 = kept, or NULL.  A row whose scores are all -inf gives NaN,
 * as torch's softmax does.
 * The backward is what autograd computes through the same lines:
 *   Z = keep / (1 - p);  dV = (P o Z)^T dO;  dP = (dO V^T) o Z;
 *   dS = P o (dP - rowsum(dP o P)) * scale;  dQ = dS K;  dK = dS^T Q.
 *
 * oracle_dropout_mask restates the keep decision of
 * fast_ops/flash_attention/flash_attention_triton.py:38-50 with the element index of :125, :217
 * (all arithmetic modulo 2^32; the threshold is the fp32 product p * 2^32 truncated). */
static uint32_t dropout_hash(uint32_t idx, uint32_t seed) {
  uint32_t a = idx ^ seed;
  a ^= a >> 4;
  a = (a ^ 0xDEADBEEFu) + (a << 5);
  a ^= a >> 11;
  return a;
}

void oracle_dropout_mask(uint8_t* keep, int64_t total, float dropout_p, uint64_t seed, uint64_t offset) {
  const float prod = dropout_p * 4294967296.0f;
  const uint32_t thr = prod >= 4294967296.0f ? 0xffffffffu : (uint32_t)prod;
  for (int64_t i = 0; i < total; ++i)
    keep[i] = dropout_hash((uint32_t)offset + (uint32_t)i, (uint32_t)seed) > thr ? 1 : 0;
}

typedef struct {
  const float *q, *k, *v, *dout, *bias;
  const uint8_t* keep;
  float *out, *dq, *dk, *dv, *lse, *delta;
  int64_t bias_sb, bias_sh, bias_sq;
  int H, Sq, Sk, D, causal;
  float scale, rescale;
} attn_ex_ctx;

/* scaled, biased and masked score of (row i, key j) */
static float ex_score(const attn_ex_ctx* c, int bh, int i, int j) {
  if (c->causal && j > i) return -INFINITY;
  const float* qi = c->q + ((int64_t)bh * c->Sq + i) * c->D;
  const float* kj = c->k + ((int64_t)bh * c->Sk + j) * c->D;
  float s = 0.f;
#pragma omp simd reduction(+ : s)
  for (int d = 0; d < c->D; ++d) s += (qi[d] * c->scale) * kj[d];
  if (c->bias) {
    const int b = bh / c->H, h = bh % c->H;
    s += c->bias[b * c->bias_sb + h * c->bias_sh + (int64_t)i * c->bias_sq + j];
  }
  return s;
}

static void attn_ex_rows(int64_t begin, int64_t end, void* vctx) {
  const attn_ex_ctx* c = (const attn_ex_ctx*)vctx;
  const int Sq = c->Sq, Sk = c->Sk, D = c->D;
  float* p = (float*)malloc(sizeof(float) * (size_t)Sk);
  float* acc = (float*)malloc(sizeof(float) * (size_t)D);
  for (int64_t r = begin; r < end; ++r) {
    const int bh = (int)(r / Sq), i = (int)(r % Sq);
    const uint8_t* keep = c->keep ? c->keep + ((int64_t)bh * Sq + i) * Sk : NULL;
    const float* vb = c->v + (int64_t)bh * Sk * D;
    const float* kb = c->k + (int64_t)bh * Sk * D;
    float mx = -INFINITY;
    for (int j = 0; j < Sk; ++j) {
      p[j] = ex_score(c, bh, i, j);
      if (p[j] > mx) mx = p[j];
    }
    float sum = 0.f;
    for (int j = 0; j < Sk; ++j) {
      p[j] = expf(p[j] - mx);
      sum += p[j];
    }
    const float inv = 1.f / sum;
    for (int j = 0; j < Sk; ++j) p[j] *= inv;
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int j = 0; j < Sk; ++j) {
      if (keep && !keep[j]) continue;
      const float* vj = vb + (int64_t)j * D;
      for (int d = 0; d < D; ++d) acc[d] += p[j] * (vj[d] * c->rescale);
    }
    if (c->out) {
      float* oi = c->out + ((int64_t)bh * Sq + i) * D;
      for (int d = 0; d < D; ++d) oi[d] = acc[d];
    }
    if (c->lse) c->lse[(int64_t)bh * Sq + i] = mx + logf(sum);
    if (c->dout) {
      const float* doi = c->dout + ((int64_t)bh * Sq + i) * D;
      float delta = 0.f;
      for (int d = 0; d < D; ++d) delta += acc[d] * doi[d];
      c->delta[(int64_t)bh * Sq + i] = delta;
      for (int d = 0; d < D; ++d) acc[d] = 0.f;
      for (int j = 0; j < Sk; ++j) {
        float dp = 0.f;
        if (!keep || keep[j]) {
          const float* vj = vb + (int64_t)j * D;
          for (int d = 0; d < D; ++d) dp += doi[d] * vj[d];
          dp *= c->rescale;
        }
        const float ds = p[j] * (dp - delta) * c->scale;
        const float* kj = kb + (int64_t)j * D;
        for (int d = 0; d < D; ++d) acc[d] += ds * kj[d];
      }
      float* dqi = c->dq + ((int64_t)bh * Sq + i) * D;
      for (int d = 0; d < D; ++d) dqi[d] = acc[d];
    }
  }
  free(p);
  free(acc);
}

static void attn_ex_keys(int64_t begin, int64_t end, void* vctx) {
  const attn_ex_ctx* c = (const attn_ex_ctx*)vctx;
  const int Sq = c->Sq, Sk = c->Sk, D = c->D;
  float* ak = (float*)malloc(sizeof(float) * (size_t)D);
  float* av = (float*)malloc(sizeof(float) * (size_t)D);
  for (int64_t r = begin; r < end; ++r) {
    const int bh = (int)(r / Sk), j = (int)(r % Sk);
    const float* vj = c->v + ((int64_t)bh * Sk + j) * D;
    for (int d = 0; d < D; ++d) ak[d] = av[d] = 0.f;
    for (int i = 0; i < Sq; ++i) {
      const float lse = c->lse[(int64_t)bh * Sq + i];
      const float s = ex_score(c, bh, i, j);
      if (s == -INFINITY) continue;
      const float p = expf(s - lse);
      const int kept = !c->keep || c->keep[((int64_t)bh * Sq + i) * Sk + j];
      const float* qi = c->q + ((int64_t)bh * Sq + i) * D;
      const float* doi = c->dout + ((int64_t)bh * Sq + i) * D;
      float dp = 0.f;
      if (kept) {
        for (int d = 0; d < D; ++d) dp += doi[d] * vj[d];
        dp *= c->rescale;
      }
      const float ds = p * (dp - c->delta[(int64_t)bh * Sq + i]) * c->scale;
      for (int d = 0; d < D; ++d) {
        if (kept) av[d] += (p * c->rescale) * doi[d];
        ak[d] += ds * qi[d];
      }
    }
    float* dkj = c->dk + ((int64_t)bh * Sk + j) * D;
    float* dvj = c->dv + ((int64_t)bh * Sk + j) * D;
    for (int d = 0; d < D; ++d) {
      dkj[d] = ak[d];
      dvj[d] = av[d];
    }
  }
  free(ak);
  free(av);
}

/* Forward only when dout is NULL (dq, dk, dv, delta then unused); lse is required for the
 * backward (scratch of B*H*Sq floats) and optional otherwise. */
void oracle_attention_ex(const float* q, const float* k, const float* v, const float* bias,
                         const int64_t* bias_strides, const uint8_t* keep, float dropout_p,
                         float* out, float* lse, const float* dout, float* dq, float* dk, float* dv,
                         float* delta, int B, int H, int Sq, int Sk, int D, int causal, float scale) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return;
  attn_ex_ctx c;
  memset(&c, 0, sizeof(c));
  c.q = q; c.k = k; c.v = v; c.dout = dout; c.bias = bias; c.keep = keep;
  c.out = out; c.dq = dq; c.dk = dk; c.dv = dv; c.lse = lse; c.delta = delta;
  if (bias) { c.bias_sb = bias_strides[0]; c.bias_sh = bias_strides[1]; c.bias_sq = bias_strides[2]; }
  c.H = H; c.Sq = Sq; c.Sk = Sk; c.D = D; c.causal = causal;
  c.scale = scale;
  c.rescale = keep ? 1.0f / (1.0f - dropout_p) : 1.0f;
  parallel_for((int64_t)B * H * Sq, 8, attn_ex_rows, &c);
  if (dout) parallel_for((int64_t)B * H * Sk, 8, attn_ex_keys, &c);
}

