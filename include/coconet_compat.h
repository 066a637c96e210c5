/* Source compatibility for frozen programs that call the forked NCCL's fused
 * entry point `AllReduce_pipe` directly (C++ only, header only).  The fork
 * declares ONE signature per build, selected by a macro that the emitter
 * patches into the NCCL sources (nccl/src/nccl.h.in:211-216;
 * src/codegen.cpp:1921-1938); its frozen test programs use four arities
 * (examples/test-sgd.cu:3, examples/test-adam.cu:3, examples/test-adamf16.cu:3,
 * and the two of nccl.h.in).  Here they are overloads that forward to the C
 * ABI, so such a program keeps its call sites and changes only how it makes
 * its communicator (cocoCommInitRank instead of MPI + ncclCommInitRank).
 *
 * Differences that the overloads absorb:
 *  - the fork indexes m and v (full-size arrays) by GLOBAL element
 *    (nccl/src/collectives/device/all_reduce_computation.h:110); the runtime's
 *    m, v are slice-local, so the overloads pass m + slice_begin, v + slice_begin;
 *  - datatype / reduction-op arguments are accepted and ignored (the gradient
 *    type comes from the pointer type, the reduction is a sum);
 *  - the LAMB form's `r` scratch is ignored (r is recomputed).
 * Return value: 0 on success like ncclSuccess, so NCCLCHECK-style macros work. */
#ifndef COCONET_COMPAT_H_
#define COCONET_COMPAT_H_

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "coconet_rt.h"

namespace coco_compat {

template <typename T> struct GradType;
template <> struct GradType<float> { static constexpr cocoDataType_t value = cocoFloat32; };
template <> struct GradType<__half> { static constexpr cocoDataType_t value = cocoFloat16; };
template <> struct GradType<__nv_bfloat16> { static constexpr cocoDataType_t value = cocoBfloat16; };

/* First element of this rank's slice of `count` elements. */
inline int slice_begin(cocoComm_t comm, size_t count, size_t *begin) {
  int world = 0, rank = 0;
  size_t end = 0;
  int rc = cocoCommCount(comm, &world);
  if (rc == cocoSuccess) rc = cocoCommUserRank(comm, &rank);
  if (rc == cocoSuccess) rc = cocoSliceBounds(count, world, rank, begin, &end);
  return rc;
}

}  // namespace coco_compat

/* SGD: w -= lr * sum(g)   (examples/test-sgd.cu:3, check :17-23) */
template <typename T, typename DT, typename Op>
inline int AllReduce_pipe(float lr, T *g, float *w, size_t count, DT, cocoComm_t comm, Op,
                          cudaStream_t stream) {
  return cocoFusedSGD(comm, g, coco_compat::GradType<T>::value, w, nullptr, cocoFloat16, count, lr,
                      1.0f, stream);
}

/* Adam as the DSL program writes it, fp32 weights gathered
 * (examples/test-adam.cu:3 and test-adamf16.cu:3, check test-adam.cu:14-43) */
template <typename T, typename DT, typename Op>
inline int AllReduce_pipe(float lr, float beta1, float beta2, T *g, float *w, float *m, float *v,
                          size_t count, DT, cocoComm_t comm, Op, cudaStream_t stream) {
  size_t lo = 0;
  const int rc = coco_compat::slice_begin(comm, count, &lo);
  if (rc != cocoSuccess) return rc;
  return cocoFusedAdam(comm, g, coco_compat::GradType<T>::value, w, nullptr, cocoFloat16, m + lo,
                       v + lo, count, lr, beta1, beta2, 0.0f, 0, 1.0f, cocoVariantDsl, stream);
}

/* Mixed-precision Adam of the first fork, functor for functor: fp16 ring sum,
 * fp32 master weights, fp16 copy gathered (nccl/src/nccl.h.in:212;
 * reduce_kernel.h:36-68, common_kernel.h:862-923) */
template <typename DT, typename Op>
inline int AllReduce_pipe(float lr, float beta1, float beta2, __half *g, float *w, __half *halfw,
                          float *m, float *v, size_t count, DT, cocoComm_t comm, Op,
                          cudaStream_t stream) {
  size_t lo = 0;
  const int rc = coco_compat::slice_begin(comm, count, &lo);
  if (rc != cocoSuccess) return rc;
  return cocoFusedAdam(comm, g, cocoFloat16, w, halfw, cocoFloat16, m + lo, v + lo, count, lr,
                       beta1, beta2, 0.0f, 0, 1.0f, cocoVariantNccl, stream);
}

/* LAMB form of the first fork, functor for functor (nccl/src/nccl.h.in:215;
 * reduce_kernel.h:391-452, common_kernel.h:2472-2535, 2687-2726): fp16 ring
 * sum, decay factor 1.0, the trust ratio divided by ||r|| once more. */
template <typename DT, typename Op>
inline int AllReduce_pipe(float lr, float beta1, float beta2, __half *g, float *w, __half *halfw,
                          float *m, float *v, float *r, size_t count, DT, cocoComm_t comm, Op,
                          cudaStream_t stream) {
  (void)r;
  size_t lo = 0;
  const int rc = coco_compat::slice_begin(comm, count, &lo);
  if (rc != cocoSuccess) return rc;
  return cocoFusedLAMB(comm, g, cocoFloat16, w, halfw, cocoFloat16, m + lo, v + lo, count, lr,
                       beta1, beta2, 0.0f, 1.0f, 0, 1.0f, cocoVariantNccl, 0, stream);
}

#endif  /* COCONET_COMPAT_H_ */
