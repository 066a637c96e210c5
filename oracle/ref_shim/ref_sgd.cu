// Builds the reference's frozen SGD test program (examples/test-sgd.cu) as a
// library and exposes its host checker mpiRef (lines 7-25).  Test
// infrastructure only; the reference source is compiled from where it lies.
#include "mpi.h"
FakeMpiWorld g_fake_mpi_world = {1, nullptr};
#define main coconet_ref_unused_main
#include "examples/test-sgd.cu"
#undef main
#include "ref_unused_stubs.inc"

// Returns 1 when the reference checker accepts `w_new` as the result of the
// step on (grads[0..world-1], w_old, lr).
extern "C" int ref_sgd_check(const float *const *grads, int world, const float *w_old,
                             float lr, const float *w_new, size_t n) {
  g_fake_mpi_world.size = world;
  g_fake_mpi_world.grads = grads;
  return mpiRef((float *)grads[0], (float *)w_old, lr, (float *)w_new, n) ? 1 : 0;
}
