// A program in the style of the reference's frozen tests (examples/test-sgd.cu,
// test-adam.cu, test-adamf16.cu): it calls AllReduce_pipe in the four arities
// the fork and its tests use, through include/coconet_compat.h, and checks every
// result on the host the way those tests' mpiRef does (every rank holds the same
// inputs, as there, so the sum over ranks is a sum of `world` equal terms).
// Ranks come from RANK / WORLD_SIZE / LOCAL_RANK (one process per GPU).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "coconet_compat.h"

#define CUDACHECK(cmd) do { cudaError_t e = (cmd); if (e != cudaSuccess) { \
  printf("CUDA error %s:%d '%s'\n", __FILE__, __LINE__, cudaGetErrorString(e)); exit(1); } } while (0)
#define NCCLCHECK(cmd) do { int rc_ = (cmd); if (rc_ != 0) { \
  printf("runtime error %s:%d '%s'\n", __FILE__, __LINE__, cocoErrorString(rc_)); exit(1); } } while (0)

static bool eqFloat(float a, float b) {  // examples/header.h:55-62 (rel 1e-5), plus a floor
  const float d = fabsf(a - b), s = fmaxf(fabsf(a), fabsf(b));
  return d <= 1e-5f * s + 1e-8f;
}
static float frand(unsigned &s) {  // deterministic, the same on every rank
  s = s * 1664525u + 1013904223u;
  return (float)(s >> 8) / (float)(1u << 24);
}
template <typename T> static T *toDevice(const std::vector<T> &h) {
  T *d = nullptr;
  CUDACHECK(cudaMalloc(&d, h.size() * sizeof(T)));
  CUDACHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}
template <typename T> static std::vector<T> toHost(const T *d, size_t n) {
  std::vector<T> h(n);
  CUDACHECK(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
  return h;
}
static bool report(const char *what, size_t bad, int rank) {
  if (rank == 0) printf("%s %s\n", bad == 0 ? "PASSED" : "FAILED", what);
  return bad == 0;
}

int main(int argc, char **argv) {
  const size_t SZ = argc > 1 ? (size_t)atol(argv[1]) : 10007;
  int rank, world, local_rank, ndev;
  NCCLCHECK(cocoEnvRank(&rank, &world, &local_rank));
  CUDACHECK(cudaGetDeviceCount(&ndev));
  CUDACHECK(cudaSetDevice(local_rank % ndev));
  cocoComm_t comm;
  NCCLCHECK(cocoCommInitRank(&comm, world, rank, NULL));
  cudaStream_t stream;
  CUDACHECK(cudaStreamCreate(&stream));
  const float lr = 0.01f, beta1 = 0.9f, beta2 = 0.999f;
  size_t lo, hi;
  NCCLCHECK(cocoSliceBounds(SZ, world, rank, &lo, &hi));
  bool ok = true;

  unsigned seed = 1234;
  std::vector<float> hg(SZ), hw(SZ), hm(SZ), hv(SZ);
  std::vector<__half> hgh(SZ);
  for (size_t i = 0; i < SZ; i++) {
    hg[i] = 2.f * frand(seed) - 1.f;
    hw[i] = 0.04f * frand(seed) - 0.02f;
    hm[i] = 0.2f * frand(seed) - 0.1f;
    hv[i] = 0.5f + frand(seed);
    hgh[i] = __float2half(hg[i]);
  }
  std::vector<float> gsum(SZ), gsum16(SZ);  // sums of `world` equal terms, in rank order
  std::vector<__half> gring(SZ);            // the same accumulated in fp16, as the fork's ring does
  for (size_t i = 0; i < SZ; i++) {
    float a = hg[i], b = __half2float(hgh[i]);
    __half c = hgh[i];
    for (int r = 1; r < world; r++) {
      a = a + hg[i];
      b = b + __half2float(hgh[i]);
      c = __float2half(__half2float(c) + __half2float(hgh[i]));
    }
    gsum[i] = a, gsum16[i] = b, gring[i] = c;
  }

  {  // ---- SGD (test-sgd.cu) ----
    float *g = toDevice(hg), *w = toDevice(hw);
    NCCLCHECK(AllReduce_pipe(lr, g, w, SZ, 0, comm, 0, stream));
    CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<float> got = toHost(w, SZ);
    size_t bad = 0;
    for (size_t i = 0; i < SZ; i++) bad += !eqFloat(got[i], hw[i] - lr * gsum[i]);
    ok &= report("sgd", bad, rank);
    cudaFree(g), cudaFree(w);
  }
  {  // ---- Adam as the DSL writes it, full-size m and v indexed by global element (test-adam.cu) ----
    float *g = toDevice(hg), *w = toDevice(hw), *m = toDevice(hm), *v = toDevice(hv);
    NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g, w, m, v, SZ, 0, comm, 0, stream));
    CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<float> gw = toHost(w, SZ), gm = toHost(m, SZ), gv = toHost(v, SZ);
    size_t bad = 0;
    for (size_t i = 0; i < SZ; i++) {
      const float s = gsum[i];
      const float m1 = beta1 * hm[i] + (1.f - beta1) * s;
      const float v1 = beta2 * hv[i] + (1.f - beta2) * (s * s);
      const float w1 = hw[i] - (lr * (m1 / beta1)) / (v1 / beta2);
      bad += !eqFloat(gw[i], w1);
      if (i >= lo && i < hi) bad += !eqFloat(gm[i], m1) || !eqFloat(gv[i], v1);  // this rank's slice
      else bad += gm[i] != hm[i] || gv[i] != hv[i];                              // untouched elsewhere
    }
    ok &= report("adam", bad, rank);
    cudaFree(g), cudaFree(w), cudaFree(m), cudaFree(v);
  }
  {  // ---- the fork's mixed-precision Adam (nccl.h.in:212), functor for functor ----
    __half *g = toDevice(hgh), *halfw = nullptr;
    CUDACHECK(cudaMalloc(&halfw, SZ * sizeof(__half)));
    CUDACHECK(cudaMemset(halfw, 0, SZ * sizeof(__half)));
    float *w = toDevice(hw), *m = toDevice(hm), *v = toDevice(hv);
    NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g, w, halfw, m, v, SZ, 0, comm, 0, stream));
    CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<float> gw = toHost(w, SZ);
    std::vector<__half> gh = toHost(halfw, SZ);
    size_t bad = 0;
    for (size_t i = 0; i < SZ; i++) {
      const float s = __half2float(gring[i]);
      const float ss = __half2float(__float2half(s * s));          // the square is taken in fp16
      const float v1 = hv[i] * beta2 + ss * (1.f - beta2);
      const float m1 = hm[i] * beta2 + s * (1.f - beta2);          // beta2 for m: the fork's slip
      const float w1 = hw[i] - lr * (m1 / beta1) / sqrtf(v1 / beta2);
      if (i >= lo && i < hi) bad += !eqFloat(gw[i], w1);           // the fp32 master is slice-local
      bad += fabsf(__half2float(gh[i]) - w1) > 1e-3f * fabsf(w1) + 1e-6f;  // fp16 copy everywhere
    }
    ok &= report("adam-mixed", bad, rank);
    cudaFree(g), cudaFree(halfw), cudaFree(w), cudaFree(m), cudaFree(v);
  }
  {  // ---- LAMB form (nccl.h.in:215): the fork's LAMB functors (reduce_kernel.h:391-452) ----
    __half *g = toDevice(hgh), *halfw = nullptr;
    CUDACHECK(cudaMalloc(&halfw, SZ * sizeof(__half)));
    float *w = toDevice(hw), *m = toDevice(hm), *v = toDevice(hv), *r = nullptr;
    NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g, w, halfw, m, v, r, SZ, 0, comm, 0, stream));
    CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<float> gw = toHost(w, SZ);
    std::vector<__half> gh = toHost(halfw, SZ);
    std::vector<float> rr(SZ);
    float w2 = 0, r2 = 0;  // fp32 sums like the fork's (its order is not fixed: tolerance below)
    for (size_t i = 0; i < SZ; i++) {
      const float s = __half2float(gring[i]);                      // fp16 ring sum
      const float ss = __half2float(__float2half(s * s));          // the square is taken in fp16
      const float v1 = hv[i] * beta2 + ss * (1.f - beta2);
      const float m1 = hm[i] * beta1 + s * (1.f - beta1);          // beta1: the LAMB copy is right
      rr[i] = (m1 / beta1) / sqrtf(v1 / beta2) + 1.0f * hw[i];     // decay factor 1.0, no epsilon
      w2 += hw[i] * hw[i], r2 += rr[i] * rr[i];
    }
    const float wn = sqrtf(w2), rn = sqrtf(r2);
    const float scale = lr * (((wn > 0) ? (rn > 0 ? wn / rn : 1.0f) : 1.0f) / rn);  // the extra /||r||
    size_t bad = 0;
    for (size_t i = 0; i < SZ; i++) {
      const float w1 = hw[i] - scale * rr[i];
      if (i >= lo && i < hi) bad += fabsf(gw[i] - w1) > 1e-4f * fabsf(w1) + 1e-7f;
      bad += fabsf(__half2float(gh[i]) - w1) > 1e-3f * fabsf(w1) + 1e-6f;
    }
    ok &= report("lamb", bad, rank);
    cudaFree(g), cudaFree(halfw), cudaFree(w), cudaFree(m), cudaFree(v);
  }
  cocoStatus_t st;
  NCCLCHECK(cocoGetStatus(comm, &st));
  if (st.code != 0) { printf("device status %d\n", st.code); ok = false; }
  NCCLCHECK(cocoCommDestroy(comm));
  return ok ? 0 : 1;
}
