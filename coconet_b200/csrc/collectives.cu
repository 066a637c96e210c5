// Stand-alone collectives on the runtime's own peer memory, so that the
// unfused schedules of a generated program (AR_C, RS_C_AG) need no NCCL:
// cocoAllReduce, cocoReduceScatter, cocoAllGather.  Each is the generic fused
// kernel (include/coconet_fused_generic.cuh) with a trivial functor and, for
// the last two, one half of the exchange switched off.  fp32, sum, one-shot
// over peer loads/stores in fixed rank order -- the shape of the stock calls
// the reference emits (src/codegen.cpp:4146-4189), not a tuned replacement for
// NCCL: the fused step is the product, these keep the baseline self-contained.
#include <cuda_runtime.h>

#include "coconet_fused_generic.cuh"
#include "coconet_rt.h"

namespace {

struct SumOnly {  // all-reduce in place: every rank's buffer receives the sum
  __device__ __forceinline__ float operator()(size_t, size_t, float gsum, float) const { return gsum; }
};
struct SumToSlice {  // reduce-scatter: the sum of the rank's slice goes to recv[0..S)
  float *recv;
  __device__ __forceinline__ float operator()(size_t i, size_t, float gsum, float) const {
    recv[i] = gsum;
    return gsum;
  }
};
struct SendSlice {  // all-gather: the rank's send[0..S) goes to element lo + i of every recv
  const float *send;
  __device__ __forceinline__ float operator()(size_t i, size_t, float, float) const { return send[i]; }
};

}  // namespace

extern "C" {

int cocoAllReduce(cocoComm_t comm, float *buf, size_t count, cocoStream_t stream) {
  if (!comm || !buf) return cocoInvalidArgument;
  cocoGenericPlan plan;
  int rc = cocoFusedGenericPlan(comm, buf, cocoFloat32, buf, count, 1.0f, stream, &plan);
  if (rc != cocoSuccess) return rc;
  return cocoLaunchGenericFused<float>(plan, SumOnly{}, (cudaStream_t)stream);
}

int cocoReduceScatter(cocoComm_t comm, const float *send, float *recv, size_t count,
                      cocoStream_t stream) {
  if (!comm || !send || !recv) return cocoInvalidArgument;
  cocoGenericPlan plan;
  // `send` doubles as the weight argument: it is only read, and only locally
  int rc = cocoFusedGenericPlan(comm, send, cocoFloat32, (float *)send, count, 1.0f, stream, &plan);
  if (rc != cocoSuccess) return rc;
  plan.sa.flags |= coco::kFlagNoGather;
  return cocoLaunchGenericFused<float>(plan, SumToSlice{recv}, (cudaStream_t)stream);
}

int cocoAllGather(cocoComm_t comm, const float *send, float *recv, size_t count,
                  cocoStream_t stream) {
  if (!comm || !send || !recv) return cocoInvalidArgument;
  cocoGenericPlan plan;
  int rc = cocoFusedGenericPlan(comm, recv, cocoFloat32, recv, count, 1.0f, stream, &plan);
  if (rc != cocoSuccess) return rc;
  plan.sa.flags |= coco::kFlagNoReduce;
  return cocoLaunchGenericFused<float>(plan, SendSlice{send}, (cudaStream_t)stream);
}

}  // extern "C"
