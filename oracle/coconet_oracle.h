/*
 * CPU oracle for the fused AllReduce optimizer step (reduce-scatter of Local
 * gradients -> sliced SGD / Adam / LAMB update -> all-gather of weights).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this code; it exists so that the CUDA path can be checked against a
 * scalar restatement of the reference's own host-side checks, and so that a
 * benchmark can time the reference's CPU loops beside the GPU numbers.
 *
 * Every function cites the reference file:line whose arithmetic it follows
 * (paths are relative to the root of parasailteam/coconet).
 *
 * Parity pins: the closed-form known-answer inputs of the reference's frozen
 * tests (examples/test-sgd.cu, examples/test-adam.cu:73-88) and the
 * reference's own host checkers compiled from where they lie (see
 * oracle/Makefile, target _ref) -- tests/test_oracle*.py run both.
 */
#ifndef COCONET_ORACLE_H_
#define COCONET_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Which of the reference's formulations of the update is evaluated. */
enum {
  /* nccl-overlap host checker and kernels: bias-corrected, eps inside the
   * denominator (nccl-overlap/samples/multi-process-adam-scattered.cpp:112-123,
   * nccl-overlap/src/collectives/device/reduce_kernel.h:143-246). */
  ORACLE_VARIANT_OVERLAP = 0,
  /* The DSL programs taken literally: examples/adam/adam.cpp:65-71
   * (m/beta1, v/beta2, w - m_/v_), examples/lamb/lamb.cpp:79-88. */
  ORACLE_VARIANT_DSL = 1,
  /* The forked-NCCL device functors.  Adam (AllReduce_pipe TYPE 0), including
   * the beta2-for-m slip: nccl/src/collectives/device/reduce_kernel.h:36-68,
   * common_kernel.h:862-923.  LAMB (TYPE 1): reduce_kernel.h:391-452,
   * common_kernel.h:2472-2535, 2687-2726 (decay factor 1.0, fp32 norms, the
   * trust ratio divided by ||r|| once more). */
  ORACLE_VARIANT_NCCL = 2,
};

/* LAMB flag: reproduce the reference checker's scale = trust / ||r|| with
 * norms of the MEAN square (multi-process-adam-scattered.cpp:415-433). */
#define ORACLE_LAMB_REF_QUIRK 1u

/* out[i] = g[0][i] + g[1][i] + ... in rank order, fp32 (stands in for the
 * MPI_Allreduce at examples/test-sgd.cu:11). */
void oracle_reduce_f32(const float *const *g, int world, size_t n, float *out);

/* fp16 gradients widened to fp32, summed in rank order in fp32, then
 * multiplied by inv_scale (loss-scale removal). */
void oracle_reduce_f16(const uint16_t *const *g, int world, size_t n,
                       float inv_scale, float *out);

/* fp16 gradients summed in fp16 (round-to-nearest after every add) in ring
 * order for the chunk owned by `owner`: ((g[o+1] + g[o+2]) + ...) + g[o],
 * as the ring reduce-scatter of all_reduce_computation.h:90-110 does with
 * __hadd2 (common_kernel.h:795-807).  Result is the fp16 sum as bits. */
void oracle_reduce_f16_ring(const uint16_t *const *g, int world, int owner,
                            size_t n, uint16_t *out);

/* examples/test-sgd.cu:17-23: w[i] = w[i] - lr * gsum[i]. */
void oracle_sgd(float *w, const float *gsum, size_t n, float lr);

/* One Adam step on n elements.  `step` counts from 0 (the reference's
 * `epoch`; t = step + 1).  w_lp may be NULL; otherwise receives
 * half_rn(w') as bits (common_kernel.h:655-670, 910).
 * For ORACLE_VARIANT_NCCL, gsum_h (fp16 bits of the reduced gradient) must be
 * given and gsum is ignored; for the others gsum_h is ignored. */
int oracle_adam(float *w, float *m, float *v, uint16_t *w_lp,
                const float *gsum, const uint16_t *gsum_h, size_t n,
                float lr, float beta1, float beta2, float eps, int step,
                int variant);

/* One LAMB step on one tensor of n elements (all slices together: the norms
 * are global).  Returns ||w|| and ||r|| as used through norms_out[2] when
 * non-NULL.  For ORACLE_VARIANT_NCCL gsum holds the fp16 ring sum widened to
 * float, and eps, weight_decay, step and flags are ignored (the functors have
 * no epsilon, no bias correction, and a decay factor of 1.0). */
int oracle_lamb(float *w, float *m, float *v, uint16_t *w_lp,
                const float *gsum, size_t n, float lr, float beta1,
                float beta2, float eps, float weight_decay, int step,
                int variant, unsigned flags, double *norms_out);

/* Conversions used by tests (IEEE binary16, round-to-nearest-even). */
uint16_t oracle_f32_to_f16(float f);
float oracle_f16_to_f32(uint16_t h);

/* The reference's CPU path as it would be timed: host sum of `world`
 * gradient arrays followed by the per-element passes with temporaries, in
 * the shape of examples/test-adam.cu:14-43 (bias-corrected math as in
 * ORACLE_VARIANT_OVERLAP).  g_is_f16 selects fp16 gradient inputs with
 * loss-scale removal and an fp16 weight copy.  Single-threaded, like the
 * reference loops.  Returns 0 on success, -1 if out of memory. */
int oracle_cpu_step_adam(const void *const *g, int world, int g_is_f16,
                         float inv_scale, float *w, float *m, float *v,
                         uint16_t *w_lp, size_t n, float lr, float beta1,
                         float beta2, float eps, int step);

/* The same step on `threads` host threads (pthreads, contiguous ranges of the
 * elements; results identical to the single-threaded call).  The reference's
 * loops carry no OpenMP pragma although -fopenmp is on its link line
 * (examples/sgd/Makefile:18); this is what they would do with one.  Used by
 * the benchmark's reference arm, which may use every host thread. */
int oracle_cpu_step_adam_mt(const void *const *g, int world, int g_is_f16,
                            float inv_scale, float *w, float *m, float *v,
                            uint16_t *w_lp, size_t n, float lr, float beta1,
                            float beta2, float eps, int step, int threads);
int oracle_threads_available(void);

#ifdef __cplusplus
}
#endif
#endif
