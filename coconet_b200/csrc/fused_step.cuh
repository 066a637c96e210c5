// Shared between the runtime (host) and the fused-step kernels (device):
// argument blocks and the peer-visible flag page.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "coconet_rt.h"
#include "coconet_device.h"

namespace coco {

struct LaunchConfig {
  int ctas;        // CTAs per rank
  int threads;     // threads per CTA
  int nvirt;       // virtual ranks in this launch (grid.y)
  bool cooperative;
  size_t smem_bytes;  // dynamic shared memory of the tile pipeline
};

// Host entry: enqueue the fused kernel.  `table` (device memory, nvirt
// entries) is used when nvirt > 1, else `one` is passed by value.
cudaError_t launch_fused_step(int opt, cocoDataType_t g_type, bool has_lp, cocoDataType_t lp_type,
                              const StepArgs &sa, const RankArgs &one, const RankArgs *table,
                              const LaunchConfig &cfg, cudaStream_t stream);

// Largest number of co-resident CTAs per SM for the given kernel/threads.
cudaError_t fused_step_occupancy(int opt, cocoDataType_t g_type, bool has_lp,
                                 cocoDataType_t lp_type, int threads, size_t smem_bytes,
                                 int *ctas_per_sm);

}  // namespace coco
