/*
 * Force-included before each reference source that oracle/Makefile compiles
 * into oracle/_ref/ (test infrastructure only).  It lets the reference's
 * host-side checkers build and run in one process without a GPU:
 *  - device<->host copies inside the checkers become memcpy (the "device"
 *    result handed to a checker is a host array);
 *  - the fused collectives the reference programs call, which exist only in
 *    the reference's NCCL forks, are declared as no-ops so the files parse.
 * The checkers' arithmetic is compiled exactly as it is written there.
 */
#ifndef COCONET_REF_PRELUDE_H_
#define COCONET_REF_PRELUDE_H_
#include <cuda_runtime.h>
#include <nccl.h>
#include <string.h>

static inline cudaError_t coconet_fake_memcpy(void *d, const void *s, size_t n) {
  memcpy(d, s, n);
  return cudaSuccess;
}
#define cudaMemcpy(dst, src, n, kind) coconet_fake_memcpy((dst), (src), (n))

template <class... A> static inline ncclResult_t AllReduce_pipe(A...) { return ncclSuccess; }
template <class... A> static inline ncclResult_t ncclAllReduceScatteredAdam(A...) { return ncclSuccess; }
template <class... A> static inline ncclResult_t ncclAllReduceScatteredLAMB(A...) { return ncclSuccess; }
#endif
