// Support header of the programs the coconet-b200 DSL emitter generates.
// Same helper names as the reference's examples/header.h (CUDACHECK,
// NCCLCHECK, DIVUP, cudaMemRandInt, memset_value, eqFloat), without MPI: ranks
// find their place from RANK / WORLD_SIZE / LOCAL_RANK and rendezvous through
// the runtime (include/coconet_rt.h).
#ifndef COCONET_GENERATED_HEADER_H_
#define COCONET_GENERATED_HEADER_H_

#include <assert.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <curand.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <string>
#include <vector>

#include "coconet_rt.h"

#ifdef COCONET_USE_NCCL
#include <nccl.h>
#endif

#define DIVUP(x, y) (((x) + (y)-1) / (y))

#define CUDACHECK(cmd)                                                                    \
  do {                                                                                    \
    cudaError_t e = cmd;                                                                  \
    if (e != cudaSuccess) {                                                               \
      printf("Failed: Cuda error %s:%d '%s'\n", __FILE__, __LINE__, cudaGetErrorString(e)); \
      exit(EXIT_FAILURE);                                                                 \
    }                                                                                     \
  } while (0)

#define COCOCHECK(cmd)                                                                       \
  do {                                                                                       \
    int r_ = cmd;                                                                            \
    if (r_ != cocoSuccess) {                                                                 \
      printf("Failed, coconet_rt error %s:%d '%s'\n", __FILE__, __LINE__, cocoErrorString(r_)); \
      exit(EXIT_FAILURE);                                                                    \
    }                                                                                        \
  } while (0)

#define CURANDCHECK(x)                                 \
  do {                                                 \
    if ((x) != CURAND_STATUS_SUCCESS) {                \
      printf("Error at %s:%d\n", __FILE__, __LINE__);  \
      exit(EXIT_FAILURE);                              \
    }                                                  \
  } while (0)

#ifdef COCONET_USE_NCCL
#define NCCLCHECK(cmd)                                                                      \
  do {                                                                                      \
    ncclResult_t r = cmd;                                                                   \
    if (r != ncclSuccess) {                                                                 \
      printf("Failed, NCCL error %s:%d '%s'\n", __FILE__, __LINE__, ncclGetErrorString(r)); \
      exit(EXIT_FAILURE);                                                                   \
    }                                                                                       \
  } while (0)

// Stock NCCL communicator for the unfused schedules: rank 0's unique id is
// spread through the runtime's host all-gather instead of MPI_Bcast.
static inline ncclComm_t coconetNcclInit(cocoComm_t comm, int comm_size, int rank) {
  ncclUniqueId id;
  if (rank == 0) NCCLCHECK(ncclGetUniqueId(&id));
  std::vector<ncclUniqueId> all(comm_size);
  COCOCHECK(cocoAllGatherHost(comm, &id, all.data(), sizeof(id)));
  ncclComm_t nccl;
  NCCLCHECK(ncclCommInitRank(&nccl, comm_size, all[0], rank));
  return nccl;
}
#endif

static inline bool eqFloat(float u, float v) {
  if (u == 0.0f || v == 0.0f) return u == v;
  return fabsf((u - v) / u) <= 1e-3;
}

// Uniform [0,1) values, the same on every rank (seed 1234), as the reference's
// generated programs initialise their tensors.
template <class T> static inline void cudaMemRandInt(T *dst, size_t nelems) {
  curandGenerator_t gen;
  CURANDCHECK(curandCreateGenerator(&gen, CURAND_RNG_PSEUDO_DEFAULT));
  CURANDCHECK(curandSetPseudoRandomGeneratorSeed(gen, 1234ULL));
  if (sizeof(T) == sizeof(float))
    CURANDCHECK(curandGenerateUniform(gen, (float *)dst, nelems));
  else
    CURANDCHECK(curandGenerateUniformDouble(gen, (double *)dst, nelems));
  CURANDCHECK(curandDestroyGenerator(gen));
}

static __global__ void coconetFloatToHalf(half *h, const float *f, size_t n) {
  size_t i = threadIdx.x + (size_t)blockDim.x * blockIdx.x;
  if (i < n) h[i] = __float2half(f[i]);
}
template <> inline void cudaMemRandInt<half>(half *dst, size_t nelems) {
  float *tmp;
  CUDACHECK(cudaMalloc(&tmp, sizeof(float) * nelems));
  cudaMemRandInt(tmp, nelems);
  coconetFloatToHalf<<<(unsigned)DIVUP(nelems, (size_t)256), 256>>>(dst, tmp, nelems);
  CUDACHECK(cudaDeviceSynchronize());
  CUDACHECK(cudaFree(tmp));
}

template <class T> static __global__ void coconetMemsetKernel(T *f, T v, size_t n) {
  size_t i = threadIdx.x + (size_t)blockDim.x * blockIdx.x;
  if (i < n) f[i] = v;
}
template <class T> static inline void memset_value(T *f, T v, size_t nelems) {
  coconetMemsetKernel<<<(unsigned)DIVUP(nelems, (size_t)256), 256>>>(f, v, nelems);
  CUDACHECK(cudaDeviceSynchronize());
}

// Scalars of a generated program default to 1.0f like the reference's
// (src/codegen.cpp:4650-4660); COCONET_SCALAR_<name>=<value> overrides one.
static inline float coconetScalar(const char *name, float dflt) {
  const std::string key = std::string("COCONET_SCALAR_") + name;
  const char *e = getenv(key.c_str());
  return (e && e[0]) ? (float)atof(e) : dflt;
}
// Sum of `n` equal values in rank order (what the fused step computes when
// every rank holds the same gradient, as in the generated programs).
static inline float coconetRankSum(float x, int n) {
  float s = x;
  for (int r = 1; r < n; r++) s = s + x;
  return s;
}
static inline bool coconetClose(float ref, float got) {
  if (ref != ref && got != got) return true;  // both NaN
  const float d = fabsf(ref - got), m = fmaxf(fabsf(ref), fabsf(got));
  return d <= 1e-4f * m + 1e-6f;
}

// 16-bit results: one unit in the last place of a half is 2^-11 relative
static inline bool coconetCloseHalf(float ref, float got) {
  if (ref != ref && got != got) return true;
  const float d = fabsf(ref - got), m = fmaxf(fabsf(ref), fabsf(got));
  return d <= 1.5e-3f * m + 1e-6f;
}
static inline float coconetRoundHalf(float x) { return __half2float(__float2half(x)); }
// Device tensor -> host vector of float (the host check computes in float).
static inline void coconetToHost(std::vector<float> &h, const float *d, size_t n) {
  CUDACHECK(cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost));
}
static inline void coconetToHost(std::vector<float> &h, const half *d, size_t n) {
  std::vector<half> tmp(n);
  CUDACHECK(cudaMemcpy(tmp.data(), d, n * sizeof(half), cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < n; i++) h[i] = __half2float(tmp[i]);
}

// ---- pieces of the unfused schedules ------------------------------------------
static inline size_t coconetSliceLen(size_t n, int comm_size, int rank) {
  size_t b = 0, e = 0;
  cocoSliceBounds(n, comm_size, rank, &b, &e);
  return e - b;
}
static inline unsigned coconetBlocks(size_t n) {
  size_t b = DIVUP(n, (size_t)256);
  return (unsigned)(b < 1 ? 1 : (b > 4096 ? 4096 : b));
}
// acc += sum of x[i]^2 (grid-stride; one atomic per block)
template <class T> static __global__ void coconetSumSquares(const T *x, size_t n, double *acc) {
  __shared__ double part[256];
  double s = 0.0;
  for (size_t i = threadIdx.x + (size_t)blockDim.x * blockIdx.x; i < n;
       i += (size_t)blockDim.x * gridDim.x) {
    const double v = (double)(float)x[i];
    s += v * v;
  }
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) atomicAdd(acc, part[0]);
}
template <class T> static __global__ void coconetFinishNorm(const double *acc, T *out) {
  *out = (T)(float)sqrt(*acc);
}

// *acc (a device double) becomes the sum of the ranks' values: 8 bytes per rank
// through the runtime's host all-gather.  Used by Norm over a Sliced operand in
// the unfused schedules.
static inline void coconetSumOverRanks(cocoComm_t comm, double *acc, cudaStream_t stream) {
  int world = 1;
  COCOCHECK(cocoCommCount(comm, &world));
  if (world == 1) return;
  double mine = 0.0;
  CUDACHECK(cudaMemcpyAsync(&mine, acc, sizeof(double), cudaMemcpyDeviceToHost, stream));
  CUDACHECK(cudaStreamSynchronize(stream));
  std::vector<double> all(world);
  COCOCHECK(cocoAllGatherHost(comm, &mine, all.data(), sizeof(double)));
  double sum = 0.0;
  for (int r = 0; r < world; r++) sum += all[r];
  CUDACHECK(cudaMemcpyAsync(acc, &sum, sizeof(double), cudaMemcpyHostToDevice, stream));
  CUDACHECK(cudaStreamSynchronize(stream));
}

// Device-side failures (a bounded wait that expired) surface here.
static inline void coconetCheckStatus(cocoComm_t comm, int rank) {
  cocoStatus_t st;
  COCOCHECK(cocoGetStatus(comm, &st));
  if (st.code != 0) {
    printf("rank %d: fused step failed on the device: %s (phase %d, peer %d, call %llu)\n", rank,
           cocoErrorString(st.code), st.phase, st.peer, (unsigned long long)st.seq);
    exit(EXIT_FAILURE);
  }
}

#endif  // COCONET_GENERATED_HEADER_H_
