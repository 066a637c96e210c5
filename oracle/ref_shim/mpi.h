/*
 * Stand-in for <mpi.h>, used only to compile the reference's own host-side
 * checkers (test infrastructure; nothing shipped includes it).  One process
 * plays every rank: MPI_Allreduce sums the gradient arrays registered with
 * fake_mpi_set_world() in rank order, in fp32.
 */
#ifndef COCONET_FAKE_MPI_H_
#define COCONET_FAKE_MPI_H_
#include <stddef.h>
#include <string.h>

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
#define MPI_COMM_WORLD 0
#define MPI_FLOAT 1
#define MPI_BYTE 2
#define MPI_SUM 1
#define MPI_SUCCESS 0

struct FakeMpiWorld {
  int size;
  const float *const *grads; /* size arrays; NULL = identity all-reduce */
};
extern FakeMpiWorld g_fake_mpi_world;

static inline int MPI_Init(int *, char ***) { return MPI_SUCCESS; }
static inline int MPI_Finalize() { return MPI_SUCCESS; }
static inline int MPI_Barrier(MPI_Comm) { return MPI_SUCCESS; }
static inline int MPI_Comm_size(MPI_Comm, int *s) { *s = g_fake_mpi_world.size; return MPI_SUCCESS; }
static inline int MPI_Comm_rank(MPI_Comm, int *r) { *r = 0; return MPI_SUCCESS; }
static inline int MPI_Bcast(void *, int, MPI_Datatype, int, MPI_Comm) { return MPI_SUCCESS; }
static inline int MPI_Allreduce(const void *in, void *out, size_t n, MPI_Datatype, MPI_Op, MPI_Comm) {
  float *o = (float *)out;
  if (!g_fake_mpi_world.grads) {
    memcpy(out, in, n * sizeof(float));
    return MPI_SUCCESS;
  }
  for (size_t i = 0; i < n; i++) {
    float s = g_fake_mpi_world.grads[0][i];
    for (int r = 1; r < g_fake_mpi_world.size; r++) s = s + g_fake_mpi_world.grads[r][i];
    o[i] = s;
  }
  return MPI_SUCCESS;
}
#endif
