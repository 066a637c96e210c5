/*
 * CPU oracle for the fused AllReduce optimizer step.  TEST INFRASTRUCTURE
 * ONLY: see coconet_oracle.h.  Plain scalar C; build with
 *   gcc -O2 -ffp-contract=off -fPIC -shared coconet_oracle.c -lm
 * (-ffp-contract=off keeps every fp32 operation individually rounded, as the
 * reference's host loops are when built for baseline x86-64).
 *
 * Citations are paths inside parasailteam/coconet.
 */
#include "coconet_oracle.h"

#include <math.h>
#include <pthread.h>
#include <unistd.h>
#include <stdlib.h>
#include <string.h>

/* ---- binary16 <-> binary32 (round-to-nearest-even), via the compiler's
 * _Float16, which gcc implements in software on baseline x86-64. ---- */
uint16_t oracle_f32_to_f16(float f) {
  _Float16 h = (_Float16)f;
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

float oracle_f16_to_f32(uint16_t b) {
  _Float16 h;
  memcpy(&h, &b, 2);
  return (float)h;
}

/* ---- reductions --------------------------------------------------------- */

/* Rank-order fp32 sum; the reference leaves the order to MPI_Allreduce
 * (examples/test-sgd.cu:11, multi-process-adam-scattered.cpp:105); the new
 * kernels fix it to 0,1,...,R-1 so results are reproducible per world size. */
void oracle_reduce_f32(const float *const *g, int world, size_t n, float *out) {
  for (size_t i = 0; i < n; i++) {
    float s = g[0][i];
    for (int r = 1; r < world; r++) s = s + g[r][i];
    out[i] = s;
  }
}

void oracle_reduce_f16(const uint16_t *const *g, int world, size_t n,
                       float inv_scale, float *out) {
  for (size_t i = 0; i < n; i++) {
    float s = oracle_f16_to_f32(g[0][i]);
    for (int r = 1; r < world; r++) s = s + oracle_f16_to_f32(g[r][i]);
    out[i] = s * inv_scale;
  }
}

/* Ring reduce-scatter in fp16: the chunk that ends at `owner` starts at rank
 * owner+1 (send, all_reduce_computation.h:90), is accumulated by each
 * following rank (recvReduceSend, :96-102) and finally by the owner
 * (recvReduceCopySend, :110).  Each hop is one __hadd2
 * (FuncSumHalf, common_kernel.h:795-807) = one fp16 rounding. */
void oracle_reduce_f16_ring(const uint16_t *const *g, int world, int owner,
                            size_t n, uint16_t *out) {
  for (size_t i = 0; i < n; i++) {
    int r = (owner + 1) % world;
    _Float16 s = (_Float16)oracle_f16_to_f32(g[r][i]);
    for (int hop = 1; hop < world; hop++) {
      r = (r + 1) % world;
      _Float16 x = (_Float16)oracle_f16_to_f32(g[r][i]);
      s = (_Float16)((float)s + (float)x); /* exact in fp32, one fp16 rounding */
    }
    uint16_t b;
    memcpy(&b, &s, 2);
    out[i] = b;
  }
}

/* ---- SGD ---------------------------------------------------------------- */

/* examples/test-sgd.cu:17-23 (and the DSL program examples/sgd/sgd.cpp:45-47):
 * __S1 = __w - (__lr * __S0). */
void oracle_sgd(float *w, const float *gsum, size_t n, float lr) {
  for (size_t i = 0; i < n; i++) w[i] = w[i] - (lr * gsum[i]);
}

/* ---- Adam --------------------------------------------------------------- */

int oracle_adam(float *w, float *m, float *v, uint16_t *w_lp,
                const float *gsum, const uint16_t *gsum_h, size_t n,
                float lr, float beta1, float beta2, float eps, int step,
                int variant) {
  if (variant == ORACLE_VARIANT_OVERLAP) {
    /* multi-process-adam-scattered.cpp:112-123 with T = float.  pow(float,int)
     * is evaluated in double there, so 1 - pow() and the quotient are double
     * and then narrowed to T; sqrt(T) is the float overload.  stepsize there
     * carries the sign (w + x with stepsize = -lr), which is bit-identical to
     * w - lr*... because negation is exact. */
    const double bc1 = 1.0 - pow((double)beta1, (double)(step + 1));
    const double bc2 = 1.0 - pow((double)beta2, (double)(step + 1));
    for (size_t i = 0; i < n; i++) {
      const float g = gsum[i];
      const float mn = beta1 * m[i] + (1 - beta1) * g;
      const float vn = beta2 * v[i] + (1 - beta2) * g * g;
      const float m_ = (float)((double)mn / bc1);
      const float v_ = (float)((double)vn / bc2);
      const float x = lr * m_ / (sqrtf(v_) + eps);
      w[i] = w[i] - x;
      m[i] = mn;
      v[i] = vn;
      if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
    }
    return 0;
  }
  if (variant == ORACLE_VARIANT_DSL) {
    /* examples/test-adam.cu:14-38 (the frozen output of the DSL program
     * examples/adam/adam.cpp:65-71, which has lr == 1 implicitly):
     *   S2 = b2*v + (1-b2)*(g*g);  S4 = S2/b2;
     *   S1 = b1*m + (1-b1)*g;      S3 = S1/b1;
     *   S5 = w - (lr*S3)/S4. */
    for (size_t i = 0; i < n; i++) {
      const float g = gsum[i];
      const float s2 = (beta2 * v[i]) + ((1 - beta2) * (g * g));
      const float s4 = s2 / beta2;
      const float s1 = (beta1 * m[i]) + ((1 - beta1) * g);
      const float s3 = s1 / beta1;
      w[i] = w[i] - ((lr * s3) / s4);
      m[i] = s1;
      v[i] = s2;
      if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
    }
    return 0;
  }
  if (variant == ORACLE_VARIANT_NCCL) {
    /* nccl/src/collectives/device/reduce_kernel.h:27-62 as called from
     * common_kernel.h:875-887:
     *   v  = v*b2 + float(g*g in half)*(1-b2)         mixedbinOp1
     *   v_ = v/b2                                     binOp2
     *   m  = m*b2 + float(g)*(1-b2)   (beta2: the call site at :878 passes
     *                                  beta2 to the m functor)
     *   m_ = m/b1                                     binOp4
     *   w  = w - (m_*lr)/sqrtf(v_)                    delta + weightUpdate
     *   halfw = half(w)                               float4ToHalf4 :910 */
    if (!gsum_h) return -1;
    for (size_t i = 0; i < n; i++) {
      const float gf = oracle_f16_to_f32(gsum_h[i]);
      const float gg = oracle_f16_to_f32(oracle_f32_to_f16(gf * gf));
      const float vn = (v[i] * beta2) + (gg * (1 - beta2));
      const float v_ = vn / beta2;
      const float mn = (m[i] * beta2) + (gf * (1 - beta2));
      const float m_ = mn / beta1;
      const float d = (m_ * lr) / sqrtf(v_);
      w[i] = w[i] - d;
      m[i] = mn;
      v[i] = vn;
      if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
    }
    return 0;
  }
  return -1;
}

/* ---- LAMB --------------------------------------------------------------- */

int oracle_lamb(float *w, float *m, float *v, uint16_t *w_lp,
                const float *gsum, size_t n, float lr, float beta1,
                float beta2, float eps, float weight_decay, int step,
                int variant, unsigned flags, double *norms_out) {
  float *rbuf = (float *)malloc((n ? n : 1) * sizeof(float));
  if (!rbuf) return -1;
  double r2 = 0.0, w2 = 0.0;
  const int quirk = (flags & ORACLE_LAMB_REF_QUIRK) != 0;

  if (variant == ORACLE_VARIANT_OVERLAP) {
    /* multi-process-adam-scattered.cpp:402-435 (host checker of
     * nccl-overlap/src/collectives/device/all_reduce_scattered.h:106-282):
     * pass 1 updates m, v and accumulates the norms in double; pass 2
     * recomputes r from the stored m, v and applies the step.  The reference
     * hard-codes the decay factor 1.0f (line 416, reduce_kernel.h:57); here it
     * is the weight_decay argument. */
    const double bc1 = 1.0 - pow((double)beta1, (double)(step + 1));
    const double bc2 = 1.0 - pow((double)beta2, (double)(step + 1));
    for (size_t i = 0; i < n; i++) {
      const float g = gsum[i];
      const float mn = beta1 * m[i] + (1 - beta1) * g;
      const float vn = beta2 * v[i] + (1 - beta2) * g * g;
      const float m_ = (float)((double)mn / bc1);
      const float v_ = (float)((double)vn / bc2);
      const float r = m_ / (sqrtf(v_) + eps) + weight_decay * w[i];
      rbuf[i] = r;
      if (quirk) {
        r2 += (double)((r * r) / (float)n); /* line 418: float quotient */
      } else {
        r2 += (double)r * (double)r;
      }
      if (quirk) {
        w2 += (double)(w[i] * w[i]); /* line 419: float product */
      } else {
        w2 += (double)w[i] * (double)w[i];
      }
      m[i] = mn;
      v[i] = vn;
    }
  } else if (variant == ORACLE_VARIANT_DSL) {
    /* examples/lamb/lamb.cpp:79-88: m_ = m/(1-b1), v_ = v/(1-b2) (no power
     * of t), r = m_/Sqrt(v_) + lambda*w; epsilon is declared and unused. */
    for (size_t i = 0; i < n; i++) {
      const float g = gsum[i];
      const float mn = beta1 * m[i] + (1.0f - beta1) * g;
      const float vn = beta2 * v[i] + (1.0f - beta2) * g * g;
      const float m_ = mn / (1.0f - beta1);
      const float v_ = vn / (1.0f - beta2);
      const float r = m_ / sqrtf(v_) + weight_decay * w[i];
      rbuf[i] = r;
      r2 += (double)r * (double)r;
      w2 += (double)w[i] * (double)w[i];
      m[i] = mn;
      v[i] = vn;
    }
  } else if (variant == ORACLE_VARIANT_NCCL) {
    /* The forked-NCCL LAMB functors (AllReduce_pipe TYPE 1):
     * nccl/src/collectives/device/reduce_kernel.h:391-452 as called from
     * common_kernel.h:2472-2535 (first pass) and 2687-2726 (second pass);
     * norms: all_reduce_computation.h:929-977.
     *   v  = v*b2 + float(S0*S0 in half)*(1-b2)        mixedbinOp1
     *   v_ = v/b2                                      binOp2
     *   m  = m*b1 + float(S0)*(1-b1)                   mixedbinOp3 (beta1: the
     *        Simple-protocol copy passes the right coefficient, :2509)
     *   m_ = m/b1                                      binOp4
     *   r  = m_/sqrtf(v_) + 1.0f*w                     rOp: the decay factor is
     *        the constant 1.0f, whatever the caller wanted (reduce_kernel.h:427)
     *   wNorm = sqrtf(sum w*w), rNorm = sqrtf(sum r*r), sums in fp32
     *   scale = ((wNorm > 0) ? (rNorm > 0 ? wNorm/rNorm : 1) : 1) / rNorm   (:2699)
     *   w  = w - (lr*scale)*r;  halfw = half(w)        delta, weightUpdate, :2715
     * gsum holds S0, the fp16 ring sum, widened to float (exactly).  The
     * reference accumulates the two sums with atomics in no fixed order; this
     * restatement adds them in element order, in fp32 like the reference. */
    float w2f = 0.0f, r2f = 0.0f;
    for (size_t i = 0; i < n; i++) {
      const float gf = gsum[i];
      const float gg = oracle_f16_to_f32(oracle_f32_to_f16(gf * gf));
      const float vn = (v[i] * beta2) + (gg * (1 - beta2));
      const float v_ = vn / beta2;
      const float mn = (m[i] * beta1) + (gf * (1 - beta1));
      const float m_ = mn / beta1;
      const float r = m_ / sqrtf(v_) + 1.0f * w[i];
      rbuf[i] = r;
      w2f += w[i] * w[i];
      r2f += r * r;
      m[i] = mn;
      v[i] = vn;
    }
    const float wn = sqrtf(w2f), rn = sqrtf(r2f);
    if (norms_out) {
      norms_out[0] = wn;
      norms_out[1] = rn;
    }
    const float scale = ((wn > 0) ? (rn > 0 ? wn / rn : 1.0f) : 1.0f) / rn;
    for (size_t i = 0; i < n; i++) {
      const float d = (lr * scale) * rbuf[i];
      w[i] = w[i] - d;
      if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
    }
    free(rbuf);
    return 0;
  } else {
    free(rbuf);
    return -1;
  }

  double rnorm, wnorm;
  if (quirk) {
    rnorm = sqrt(r2);             /* line 424 */
    wnorm = sqrt(w2 / (double)n); /* line 425 */
  } else {
    rnorm = sqrt(r2);
    wnorm = sqrt(w2);
  }
  if (norms_out) {
    norms_out[0] = wnorm;
    norms_out[1] = rnorm;
  }
  /* Guards of line 433; the DSL meaning is the plain ratio wNorm/rNorm
   * (lamb.cpp:86).  The reference divides by rNorm once more (line 433,
   * nccl common_kernel.h:2699): kept only under ORACLE_LAMB_REF_QUIRK. */
  double sc = (wnorm > 0) ? (rnorm > 0 ? wnorm / rnorm : 1.0) : 1.0;
  if (quirk) sc = sc / rnorm;
  const float scale = (float)sc;
  for (size_t i = 0; i < n; i++) {
    const float x = lr * scale * rbuf[i];
    w[i] = w[i] - x;
    if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
  }
  free(rbuf);
  return 0;
}

/* ---- the reference's CPU path, as timed -------------------------------- */

int oracle_cpu_step_adam(const void *const *g, int world, int g_is_f16,
                         float inv_scale, float *w, float *m, float *v,
                         uint16_t *w_lp, size_t n, float lr, float beta1,
                         float beta2, float eps, int step) {
  /* Shape of examples/test-adam.cu:8-43: one reduction into a fresh array,
   * then one pass per intermediate (S2=v', S4=v^, S1=m', S3=m^, S5=w'), each
   * into its own temporary. */
  float *s0 = (float *)malloc(n * sizeof(float));
  float *s2 = (float *)malloc(n * sizeof(float));
  float *s4 = (float *)malloc(n * sizeof(float));
  float *s1 = (float *)malloc(n * sizeof(float));
  float *s3 = (float *)malloc(n * sizeof(float));
  if (!s0 || !s2 || !s4 || !s1 || !s3) {
    free(s0); free(s2); free(s4); free(s1); free(s3);
    return -1;
  }
  if (g_is_f16)
    oracle_reduce_f16((const uint16_t *const *)g, world, n, inv_scale, s0);
  else
    oracle_reduce_f32((const float *const *)g, world, n, s0);
  const double bc1 = 1.0 - pow((double)beta1, (double)(step + 1));
  const double bc2 = 1.0 - pow((double)beta2, (double)(step + 1));
  for (size_t i = 0; i < n; i++) s2[i] = beta2 * v[i] + (1 - beta2) * s0[i] * s0[i];
  for (size_t i = 0; i < n; i++) s4[i] = (float)((double)s2[i] / bc2);
  for (size_t i = 0; i < n; i++) s1[i] = beta1 * m[i] + (1 - beta1) * s0[i];
  for (size_t i = 0; i < n; i++) s3[i] = (float)((double)s1[i] / bc1);
  for (size_t i = 0; i < n; i++) {
    w[i] = w[i] - lr * s3[i] / (sqrtf(s4[i]) + eps);
    if (w_lp) w_lp[i] = oracle_f32_to_f16(w[i]);
  }
  memcpy(m, s1, n * sizeof(float));
  memcpy(v, s2, n * sizeof(float));
  free(s0); free(s2); free(s4); free(s1); free(s3);
  return 0;
}

struct cpu_step_job {
  const void *g[64];
  int world, g_is_f16, step, rc;
  float inv_scale, lr, beta1, beta2, eps;
  float *w, *m, *v;
  uint16_t *w_lp;
  size_t n;
};

static void *cpu_step_thread(void *arg) {
  struct cpu_step_job *j = (struct cpu_step_job *)arg;
  j->rc = oracle_cpu_step_adam(j->g, j->world, j->g_is_f16, j->inv_scale, j->w, j->m, j->v,
                               j->w_lp, j->n, j->lr, j->beta1, j->beta2, j->eps, j->step);
  return 0;
}

int oracle_cpu_step_adam_mt(const void *const *g, int world, int g_is_f16,
                            float inv_scale, float *w, float *m, float *v,
                            uint16_t *w_lp, size_t n, float lr, float beta1,
                            float beta2, float eps, int step, int threads) {
  /* The same passes on `threads` contiguous ranges of the elements, one host
   * thread each (the elements are independent, so the results are those of
   * the single-threaded call bit for bit). */
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if (world < 1 || world > 64) return -1;
  struct cpu_step_job *jobs = (struct cpu_step_job *)calloc((size_t)threads, sizeof(*jobs));
  pthread_t *tid = (pthread_t *)calloc((size_t)threads, sizeof(*tid));
  if (!jobs || !tid) {
    free(jobs); free(tid);
    return -1;
  }
  const size_t gs = g_is_f16 ? sizeof(uint16_t) : sizeof(float);
  int failed = 0;
  for (int t = 0; t < threads; t++) {
    const size_t a = n * (size_t)t / (size_t)threads, b = n * (size_t)(t + 1) / (size_t)threads;
    struct cpu_step_job *j = &jobs[t];
    for (int r = 0; r < world; r++) j->g[r] = (const char *)g[r] + a * gs;
    j->world = world, j->g_is_f16 = g_is_f16, j->step = step, j->rc = 0;
    j->inv_scale = inv_scale, j->lr = lr, j->beta1 = beta1, j->beta2 = beta2, j->eps = eps;
    j->w = w + a, j->m = m + a, j->v = v + a, j->w_lp = w_lp ? w_lp + a : 0;
    j->n = b - a;
    if (pthread_create(&tid[t], 0, cpu_step_thread, j) != 0) {  // run it here instead
      cpu_step_thread(j);
      tid[t] = 0;
      jobs[t].world = -1;  // marks "not joined"
    }
  }
  for (int t = 0; t < threads; t++) {
    if (jobs[t].world != -1) pthread_join(tid[t], 0);
    failed |= jobs[t].rc != 0;
  }
  free(jobs); free(tid);
  return failed ? -1 : 0;
}

int oracle_threads_available(void) {
  const long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}
