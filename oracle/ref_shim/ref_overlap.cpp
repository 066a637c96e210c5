// Builds the reference's scattered Adam/LAMB sample
// (nccl-overlap/samples/multi-process-adam-scattered.cpp) as a library and
// exposes its host checkers check_epoch_results_adam (lines 82-153) and
// check_epoch_results_lamb (lines 372-462).  Test infrastructure only.
#include "mpi.h"
FakeMpiWorld g_fake_mpi_world = {1, nullptr};
#define main coconet_ref_unused_main
#include "nccl-overlap/samples/multi-process-adam-scattered.cpp"
#undef main
#include "ref_unused_stubs.inc"

// Each returns 1 when the reference checker accepts w_new; cpu_m / cpu_v are
// advanced in place by the reference code (its running moments).
extern "C" int ref_overlap_adam_check(const float *const *grads, int world, int epoch, size_t n,
                                      const float *w_old, const float *w_new, float *cpu_m,
                                      float *cpu_v, float beta1, float beta2, float stepsize,
                                      float epsilon) {
  g_fake_mpi_world.size = world;
  g_fake_mpi_world.grads = grads;
  return check_epoch_results_adam<float>(0, 0, 0, epoch, n, (float *)grads[0], (float *)w_old,
                                         (float *)w_new, cpu_m, cpu_v, beta1, beta2, stepsize,
                                         epsilon)
             ? 1
             : 0;
}

extern "C" int ref_overlap_lamb_check(const float *const *grads, int world, int epoch, size_t n,
                                      const float *w_old, const float *w_new, float *cpu_m,
                                      float *cpu_v, float beta1, float beta2, float stepsize,
                                      float epsilon) {
  g_fake_mpi_world.size = world;
  g_fake_mpi_world.grads = grads;
  return check_epoch_results_lamb<float>(0, 0, 0, epoch, n, (float *)grads[0], (float *)w_old,
                                         (float *)w_new, cpu_m, cpu_v, beta1, beta2, stepsize,
                                         epsilon)
             ? 1
             : 0;
}
