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
#include "fused_step.cuh"

namespace {

struct SumOnly {  // all-reduce in place: every rank's buffer receives the sum
  __device__ __forceinline__ float operator()(size_t, size_t, float gsum, float) const { return gsum; }
};
struct SumToSlice {  // reduce-scatter: the sum of the rank's slice goes to recv[0..S)
  float *recv = nullptr;
  __device__ __forceinline__ float operator()(size_t i, size_t, float gsum, float) const {
    recv[i] = gsum;
    return gsum;
  }
};
struct SendSlice {  // all-gather: the rank's send[0..S) goes to element lo + i of every recv
  const float *send = nullptr;
  __device__ __forceinline__ float operator()(size_t i, size_t, float, float) const { return send[i]; }
};

}  // namespace

// ---- single-process groups ---------------------------------------------------------
// Ranks that share a GPU (virtual ranks) run as one cooperative launch, like
// the fused step's; a rank with a GPU of its own gets the ordinary kernel.
namespace coco {

namespace {

template <class F>
cudaError_t launch_group(const StepArgs &sa, const RankArgs *ranks, const F *fs, int nvirt,
                         RankArgs *table_dev, void *aux_dev, size_t slice, int sm_count,
                         cudaStream_t stream) {
  const int threads = 512;
  const long need = (long)((slice + 4 * (size_t)threads - 1) / (4 * (size_t)threads));
  if (nvirt == 1) {
    long ctas = 2L * sm_count;
    if (ctas > need) ctas = need;
    if (ctas < 1) ctas = 1;
    cocoGenericFusedKernel<float, F><<<(unsigned)ctas, threads, 0, stream>>>(sa, ranks[0], fs[0]);
    return cudaGetLastError();
  }
  int occ = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
      &occ, (const void *)cocoGenericFusedKernelMulti<float, F>, threads, 0);
  if (e != cudaSuccess) return e;
  if (occ < 1) return cudaErrorLaunchOutOfResources;
  long ctas = ((long)(occ > 2 ? 2 : occ) * sm_count) / nvirt;  // all ranks' CTAs are co-resident
  if (ctas > need) ctas = need;
  if (ctas < 1) ctas = 1;
  // pageable sources: staged before these calls return
  e = cudaMemcpyAsync(table_dev, ranks, sizeof(RankArgs) * nvirt, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(aux_dev, fs, sizeof(F) * nvirt, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  const RankArgs *tbl = table_dev;
  const F *ftbl = (const F *)aux_dev;
  void *params[] = {(void *)&sa, (void *)&tbl, (void *)&ftbl};
  return cudaLaunchCooperativeKernel((const void *)cocoGenericFusedKernelMulti<float, F>,
                                     dim3((unsigned)ctas, (unsigned)nvirt, 1), dim3(threads, 1, 1), params,
                                     0, stream);
}

}  // namespace

cudaError_t launch_collective_group(int kind, const StepArgs &sa_in, const RankArgs *ranks,
                                    void *const *aux, int nvirt, RankArgs *table_dev, void *aux_dev,
                                    int sm_count, cudaStream_t stream) {
  if (nvirt < 1 || nvirt > kMaxRanks) return cudaErrorInvalidValue;
  StepArgs sa = sa_in;
  const size_t slice = (sa.count + sa.world - 1) / sa.world;
  if (kind == kCollAllReduce) {
    SumOnly fs[kMaxRanks];
    return launch_group(sa, ranks, fs, nvirt, table_dev, aux_dev, slice, sm_count, stream);
  }
  if (kind == kCollReduceScatter) {
    sa.flags |= kFlagNoGather;
    SumToSlice fs[kMaxRanks];
    for (int k = 0; k < nvirt; ++k) fs[k].recv = (float *)aux[k];
    return launch_group(sa, ranks, fs, nvirt, table_dev, aux_dev, slice, sm_count, stream);
  }
  if (kind == kCollAllGather) {
    sa.flags |= kFlagNoReduce;
    SendSlice fs[kMaxRanks];
    for (int k = 0; k < nvirt; ++k) fs[k].send = (const float *)aux[k];
    return launch_group(sa, ranks, fs, nvirt, table_dev, aux_dev, slice, sm_count, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace coco

extern "C" {

int cocoAllReduce(cocoComm_t comm, float *buf, size_t count, cocoStream_t stream) {
  if (!comm || !buf) return cocoInvalidArgument;
  if (coco::comm_is_group(comm))
    return coco::comm_enqueue_collective(comm, coco::kCollAllReduce, buf, buf, nullptr, count, stream);
  cocoGenericPlan plan;
  int rc = cocoFusedGenericPlan(comm, buf, cocoFloat32, buf, count, 1.0f, stream, &plan);
  if (rc != cocoSuccess) return rc;
  return cocoLaunchGenericFused<float>(plan, SumOnly{}, (cudaStream_t)stream);
}

int cocoReduceScatter(cocoComm_t comm, const float *send, float *recv, size_t count,
                      cocoStream_t stream) {
  if (!comm || !send || !recv) return cocoInvalidArgument;
  if (coco::comm_is_group(comm))
    return coco::comm_enqueue_collective(comm, coco::kCollReduceScatter, send, (float *)send, recv,
                                         count, stream);
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
  if (coco::comm_is_group(comm))
    return coco::comm_enqueue_collective(comm, coco::kCollAllGather, recv, recv, (void *)send, count,
                                         stream);
  cocoGenericPlan plan;
  int rc = cocoFusedGenericPlan(comm, recv, cocoFloat32, recv, count, 1.0f, stream, &plan);
  if (rc != cocoSuccess) return rc;
  plan.sa.flags |= coco::kFlagNoReduce;
  return cocoLaunchGenericFused<float>(plan, SendSlice{send}, (cudaStream_t)stream);
}

}  // extern "C"
