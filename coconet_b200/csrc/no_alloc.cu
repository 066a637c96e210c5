// cocoLambStepNoAlloc: a single-GPU LAMB step that allocates nothing.
//
// Some callers of this library may not allocate device memory at the moment
// they step the optimizer: a training loop whose memory pool has been frozen or
// handed over entirely to a framework's caching allocator, a process close to
// the device's memory limit, or a latency-sensitive loop that must not take
// the driver's allocation locks.  Creating a communicator (cocoCommInitAll /
// cocoCommInitRank) calls cudaMalloc for the page that holds the kernel's
// counters and per-CTA partial norms, so those callers cannot use
// cocoFusedLAMB.  This entry point runs the same kernel with that page placed
// in a fixed array that is part of the library image instead.
//
// There is no counterpart of this entry point in the reference.
#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <mutex>

#include "coconet_rt.h"
#include "fused_step.cuh"

using namespace coco;

namespace {

// The scratch page.  Every GPU that loads this library holds one copy of it
// (sizeof(FlagPage), about 33 KB) until the process exits.  Its size bounds
// the launch at kMaxCtasPerRank CTAs (one row of partial norms per CTA).
static __device__ __align__(256) FlagPage g_no_alloc_page[1];

constexpr int kMaxDevices = 64;

struct PerDevice {
  FlagPage *page = nullptr;  // device address of g_no_alloc_page on this device
  unsigned long long seq = 0;
  int sm_count = 0;
  int coop = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

}  // namespace

extern "C" int cocoLambStepNoAlloc(const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                                   cocoDataType_t lp_type, float *m, float *v, size_t count,
                                   float lr, float beta1, float beta2, float eps,
                                   float weight_decay, int step, float grad_scale,
                                   cocoStream_t stream) {
  if (!g || !w || !m || !v || step < 0) return cocoInvalidArgument;
  if (g_type != cocoFloat32 && g_type != cocoFloat16 && g_type != cocoBfloat16)
    return cocoInvalidArgument;
  if (w_lp && lp_type != cocoFloat16 && lp_type != cocoBfloat16) return cocoInvalidArgument;
  if (count > (size_t)COCO_NO_ALLOC_MAX_COUNT) return cocoInvalidArgument;  // beyond the stated maximum
  if (count == 0) return cocoSuccess;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cocoCudaError;

  std::lock_guard<std::mutex> lock(g_mu);
  PerDevice &pd = g_dev[dev];
  if (!pd.page) {
    // Set-up, once per device, with that device current.  In host code the
    // array's name is only a handle: the kernel needs the address that
    // cudaGetSymbolAddress returns for THIS device.
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_no_alloc_page) != cudaSuccess || !ptr) {
      (void)cudaGetLastError();
      return cocoCudaError;
    }
    if (cudaDeviceGetAttribute(&pd.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&pd.coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return cocoCudaError;
    }
    pd.page = (FlagPage *)ptr;
  }
  if (!pd.coop) return cocoInvalidUsage;
  cudaStream_t st = (cudaStream_t)stream;

  // The page keeps what the previous call left.  Everything a call reads
  // before it has written it must start at zero even if an earlier kernel was
  // cut short: the norm flags and partials, the two CTA counters and the
  // status word.  They are one contiguous run of the page (checked below), so
  // one stream-ordered memset clears them; the per-CTA partial sums and the
  // last norms behind them are always written before they are read.
  static_assert(offsetof(FlagPage, norm_part) == offsetof(FlagPage, norm_flag) + sizeof(FlagPage::norm_flag) &&
                    offsetof(FlagPage, done_count) == offsetof(FlagPage, norm_part) + sizeof(FlagPage::norm_part) &&
                    offsetof(FlagPage, norm_count) == offsetof(FlagPage, done_count) + sizeof(unsigned int) &&
                    offsetof(FlagPage, status) == offsetof(FlagPage, norm_count) + sizeof(unsigned int),
                "cocoLambStepNoAlloc clears norm_flag .. status with one memset");
  constexpr size_t kClearBytes =
      offsetof(FlagPage, status) + sizeof(FlagPage::status) - offsetof(FlagPage, norm_flag);
  if (cudaMemsetAsync(pd.page->norm_flag, 0, kClearBytes, st) != cudaSuccess) {
    (void)cudaGetLastError();
    return cocoCudaError;
  }

  StepArgs sa = {};
  sa.count = count;
  sa.seq = ++pd.seq;
  sa.timeout_ns = 10ull * 1000 * 1000 * 1000;
  sa.world = 1;
  sa.variant = cocoVariantOverlap;
  sa.flags = 0;
  sa.lr = lr, sa.beta1 = beta1, sa.beta2 = beta2, sa.eps = eps;
  sa.weight_decay = weight_decay;
  sa.grad_scale = grad_scale;
  sa.d1d = 1.0 - std::pow((double)beta1, (double)(step + 1));
  sa.d2d = 1.0 - std::pow((double)beta2, (double)(step + 1));
  sa.d1 = (float)sa.d1d, sa.d2 = (float)sa.d2d;
  sa.omb1 = 1.0f - beta1, sa.omb2 = 1.0f - beta2;
  sa.r1d = 1.0 / sa.d1d, sa.r2d = 1.0 / sa.d2d;
  sa.pipe_stages = 0;

  RankArgs ra = {};
  ra.g[0] = g;
  ra.out[0] = w_lp ? w_lp : (void *)w;
  ra.flags[0] = pd.page;
  ra.w = w, ra.m = m, ra.v = v;
  ra.rank = 0;
  auto al16 = [](const void *p) { return (((uintptr_t)p) & 15u) == 0; };
  ra.aligned16 = (al16(g) && al16(w) && al16(m) && al16(v) && al16(ra.out[0])) ? 1 : 0;

  LaunchConfig cfg = {};
  cfg.threads = fused_step_block_threads(fused_step_path(sa), g_type);
  int occ = 0;
  if (fused_step_occupancy(kLAMB, g_type, w_lp != nullptr, lp_type, fused_step_path(sa),
                           cfg.threads, 0, &occ) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    return cocoCudaError;
  }
  long ctas = (long)(occ < 2 ? occ : 2) * pd.sm_count;
  const long need = (long)((count + 4 * (size_t)cfg.threads - 1) / (4 * (size_t)cfg.threads));
  if (ctas > need) ctas = need;
  if (ctas > kMaxCtasPerRank) ctas = kMaxCtasPerRank;
  if (ctas < 1) ctas = 1;
  cfg.ctas = (int)ctas;
  cfg.nvirt = 1;
  cfg.cooperative = true;  // every CTA waits for the rank's combined norms
  cfg.smem_bytes = 0;
  if (launch_fused_step(kLAMB, g_type, w_lp != nullptr, lp_type, sa, ra, nullptr, cfg, st) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return cocoCudaError;
  }
  return cocoSuccess;
}
