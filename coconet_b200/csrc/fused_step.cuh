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
  size_t smem_bytes;  // dynamic shared memory of the warp rings
};

// Ring geometry shared by the host's sizing and the kernel: a stage of one
// warp holds 512 bytes (32 lanes x 16) per rank.
constexpr int kRingStagesMax = 4;
constexpr size_t kRingTileBytesPerRank = 512;

// Host entry: enqueue the fused kernel.  `table` (device memory, nvirt
// entries) is used when nvirt > 1, else `one` is passed by value.
cudaError_t launch_fused_step(int opt, cocoDataType_t g_type, bool has_lp, cocoDataType_t lp_type,
                              const StepArgs &sa, const RankArgs &one, const RankArgs *table,
                              const LaunchConfig &cfg, cudaStream_t stream);

// Data path (kernel instantiation) a call with these scalars takes.
int fused_step_path(const StepArgs &sa);
// Largest block size the kernel of that path is compiled for.
int fused_step_block_threads(int path, cocoDataType_t g_type);

// Largest number of co-resident CTAs per SM of the kernel that `path` selects,
// for this block size and dynamic shared memory (remembered per kernel).
cudaError_t fused_step_occupancy(int opt, cocoDataType_t g_type, bool has_lp,
                                 cocoDataType_t lp_type, int path, int threads,
                                 size_t smem_bytes, int *ctas_per_sm);

// Stand-alone collectives of single-process groups (collectives.cu).  The
// ranks that share the current device -- argument blocks `ranks`, per-rank
// buffer `aux` (reduce-scatter: recv, all-gather: send) -- become one launch;
// table_dev / aux_dev: device scratch for kMaxRanks argument blocks / pointers.
enum : int { kCollAllReduce = 1, kCollReduceScatter = 2, kCollAllGather = 3 };
cudaError_t launch_collective_group(int kind, const StepArgs &sa, const RankArgs *ranks,
                                    void *const *aux, int nvirt, RankArgs *table_dev, void *aux_dev,
                                    int sm_count, cudaStream_t stream);
// What collectives.cu needs from a communicator (runtime.cu).
bool comm_is_group(cocoComm_t c);
int comm_enqueue_collective(cocoComm_t c, int kind, const void *g, float *w, void *aux,
                            size_t count, cocoStream_t stream);

// Link probe (link_probe.cu): mode 0 pull, 1 push, 2 both over peer pointers;
// 4 multimem.ld_reduce, 5 multimem.st, 6 both through ra.mc_g / ra.mc_out;
// unroll 1, 2 or 4 16-byte units per thread and pass; sa.count in 16-byte units.
cudaError_t launch_link_probe(int mode, int unroll, const StepArgs &sa, const RankArgs &ra,
                              int sm_count, int threads, cudaStream_t stream);

}  // namespace coco
