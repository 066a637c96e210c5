// Builds the reference's frozen Adam test program (examples/test-adam.cu) as a
// library and exposes its host checker mpiRef (lines 6-45): the DSL program's
// formulation (m/beta1, v/beta2, w - lr*m_/v_).  Test infrastructure only.
#include "mpi.h"
FakeMpiWorld g_fake_mpi_world = {1, nullptr};
#define main coconet_ref_unused_main
#include "examples/test-adam.cu"
#undef main
#include "ref_unused_stubs.inc"

extern "C" int ref_adam_dsl_check(const float *const *grads, int world, const float *w_old,
                                  const float *m_old, const float *v_old, float lr, float beta1,
                                  float beta2, const float *w_new, size_t n) {
  g_fake_mpi_world.size = world;
  g_fake_mpi_world.grads = grads;
  return mpiRef((float *)grads[0], (float *)w_old, (float *)m_old, (float *)v_old, lr, beta1,
                beta2, (float *)w_new, nullptr, nullptr, n)
             ? 1
             : 0;
}
