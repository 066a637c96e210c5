// A program in the style of the reference's frozen tests (examples/test-sgd.cu,
// test-adam.cu, test-adamf16.cu): it calls AllReduce_pipe in the four arities
// the fork and its tests use, through include/coconet_compat.h, and checks every
// result on the host the way those tests' mpiRef does (every rank holds the same
// inputs, as there, so the sum over ranks is a sum of `world` equal terms).
// Ranks come from RANK / WORLD_SIZE / LOCAL_RANK (one process per GPU), or, with
// COMPAT_VIRTUAL_RANKS=R, all R ranks live in this process on one GPU.
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

// The ranks this process drives: one (its own, from the environment), or, with
// COMPAT_VIRTUAL_RANKS=R, all R ranks of a single-process communicator on
// device 0 (virtual ranks: their calls are grouped into one launch).
struct Rank {
  cocoComm_t comm;
  int rank;
  size_t lo, hi;
};

int main(int argc, char **argv) {
  const size_t SZ = argc > 1 ? (size_t)atol(argv[1]) : 10007;
  int rank, world, local_rank, ndev;
  NCCLCHECK(cocoEnvRank(&rank, &world, &local_rank));
  CUDACHECK(cudaGetDeviceCount(&ndev));
  std::vector<Rank> ranks;
  const char *virt = getenv("COMPAT_VIRTUAL_RANKS");
  if (virt && atoi(virt) > 1) {
    world = atoi(virt);
    rank = 0;
    CUDACHECK(cudaSetDevice(0));
    std::vector<cocoComm_t> comms(world);
    std::vector<int> devs(world, 0);
    NCCLCHECK(cocoCommInitAll(comms.data(), world, devs.data()));
    for (int r = 0; r < world; r++) ranks.push_back({comms[r], r, 0, 0});
  } else {
    CUDACHECK(cudaSetDevice(local_rank % ndev));
    cocoComm_t comm;
    NCCLCHECK(cocoCommInitRank(&comm, world, rank, NULL));
    ranks.push_back({comm, rank, 0, 0});
  }
  for (Rank &r : ranks) NCCLCHECK(cocoSliceBounds(SZ, world, r.rank, &r.lo, &r.hi));
  const size_t V = ranks.size();
  cudaStream_t stream;
  CUDACHECK(cudaStreamCreate(&stream));
  const float lr = 0.01f, beta1 = 0.9f, beta2 = 0.999f;
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
    std::vector<float *> g(V), w(V);
    for (size_t k = 0; k < V; k++) g[k] = toDevice(hg), w[k] = toDevice(hw);
    NCCLCHECK(cocoGroupStart());
    for (size_t k = 0; k < V; k++) NCCLCHECK(AllReduce_pipe(lr, g[k], w[k], SZ, 0, ranks[k].comm, 0, stream));
    NCCLCHECK(cocoGroupEnd());
    CUDACHECK(cudaStreamSynchronize(stream));
    size_t bad = 0;
    for (size_t k = 0; k < V; k++) {
      std::vector<float> got = toHost(w[k], SZ);
      for (size_t i = 0; i < SZ; i++) bad += !eqFloat(got[i], hw[i] - lr * gsum[i]);
      cudaFree(g[k]), cudaFree(w[k]);
    }
    ok &= report("sgd", bad, rank);
  }
  {  // ---- Adam as the DSL writes it, full-size m and v indexed by global element (test-adam.cu) ----
    std::vector<float *> g(V), w(V), m(V), v(V);
    for (size_t k = 0; k < V; k++) g[k] = toDevice(hg), w[k] = toDevice(hw), m[k] = toDevice(hm), v[k] = toDevice(hv);
    NCCLCHECK(cocoGroupStart());
    for (size_t k = 0; k < V; k++)
      NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g[k], w[k], m[k], v[k], SZ, 0, ranks[k].comm, 0, stream));
    NCCLCHECK(cocoGroupEnd());
    CUDACHECK(cudaStreamSynchronize(stream));
    size_t bad = 0;
    for (size_t k = 0; k < V; k++) {
      const size_t lo = ranks[k].lo, hi = ranks[k].hi;
      std::vector<float> gw = toHost(w[k], SZ), gm = toHost(m[k], SZ), gv = toHost(v[k], SZ);
      for (size_t i = 0; i < SZ; i++) {
        const float s = gsum[i];
        const float m1 = beta1 * hm[i] + (1.f - beta1) * s;
        const float v1 = beta2 * hv[i] + (1.f - beta2) * (s * s);
        const float w1 = hw[i] - (lr * (m1 / beta1)) / (v1 / beta2);
        bad += !eqFloat(gw[i], w1);
        if (i >= lo && i < hi) bad += !eqFloat(gm[i], m1) || !eqFloat(gv[i], v1);  // this rank's slice
        else bad += gm[i] != hm[i] || gv[i] != hv[i];                              // untouched elsewhere
      }
      cudaFree(g[k]), cudaFree(w[k]), cudaFree(m[k]), cudaFree(v[k]);
    }
    ok &= report("adam", bad, rank);
  }
  // the fp16 ring sum of the slice owned by rank o starts behind the owner; with
  // equal terms on every rank the order does not change the result
  {  // ---- the fork's mixed-precision Adam (nccl.h.in:212), functor for functor ----
    std::vector<__half *> g(V), halfw(V);
    std::vector<float *> w(V), m(V), v(V);
    for (size_t k = 0; k < V; k++) {
      g[k] = toDevice(hgh), w[k] = toDevice(hw), m[k] = toDevice(hm), v[k] = toDevice(hv);
      CUDACHECK(cudaMalloc(&halfw[k], SZ * sizeof(__half)));
      CUDACHECK(cudaMemset(halfw[k], 0, SZ * sizeof(__half)));
    }
    NCCLCHECK(cocoGroupStart());
    for (size_t k = 0; k < V; k++)
      NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g[k], w[k], halfw[k], m[k], v[k], SZ, 0, ranks[k].comm, 0, stream));
    NCCLCHECK(cocoGroupEnd());
    CUDACHECK(cudaStreamSynchronize(stream));
    size_t bad = 0;
    for (size_t k = 0; k < V; k++) {
      const size_t lo = ranks[k].lo, hi = ranks[k].hi;
      std::vector<float> gw = toHost(w[k], SZ);
      std::vector<__half> gh = toHost(halfw[k], SZ);
      for (size_t i = 0; i < SZ; i++) {
        const float s = __half2float(gring[i]);
        const float ss = __half2float(__float2half(s * s));          // the square is taken in fp16
        const float v1 = hv[i] * beta2 + ss * (1.f - beta2);
        const float m1 = hm[i] * beta2 + s * (1.f - beta2);          // beta2 for m: the fork's slip
        const float w1 = hw[i] - lr * (m1 / beta1) / sqrtf(v1 / beta2);
        if (i >= lo && i < hi) bad += !eqFloat(gw[i], w1);           // the fp32 master is slice-local
        bad += fabsf(__half2float(gh[i]) - w1) > 1e-3f * fabsf(w1) + 1e-6f;  // fp16 copy everywhere
      }
      cudaFree(g[k]), cudaFree(halfw[k]), cudaFree(w[k]), cudaFree(m[k]), cudaFree(v[k]);
    }
    ok &= report("adam-mixed", bad, rank);
  }
  {  // ---- LAMB form (nccl.h.in:215): the fork's LAMB functors (reduce_kernel.h:391-452) ----
    std::vector<__half *> g(V), halfw(V);
    std::vector<float *> w(V), m(V), v(V);
    for (size_t k = 0; k < V; k++) {
      g[k] = toDevice(hgh), w[k] = toDevice(hw), m[k] = toDevice(hm), v[k] = toDevice(hv);
      CUDACHECK(cudaMalloc(&halfw[k], SZ * sizeof(__half)));
    }
    float *r = nullptr;
    NCCLCHECK(cocoGroupStart());
    for (size_t k = 0; k < V; k++)
      NCCLCHECK(AllReduce_pipe(lr, beta1, beta2, g[k], w[k], halfw[k], m[k], v[k], r, SZ, 0, ranks[k].comm, 0, stream));
    NCCLCHECK(cocoGroupEnd());
    CUDACHECK(cudaStreamSynchronize(stream));
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
    for (size_t k = 0; k < V; k++) {
      const size_t lo = ranks[k].lo, hi = ranks[k].hi;
      std::vector<float> gw = toHost(w[k], SZ);
      std::vector<__half> gh = toHost(halfw[k], SZ);
      for (size_t i = 0; i < SZ; i++) {
        const float w1 = hw[i] - scale * rr[i];
        if (i >= lo && i < hi) bad += fabsf(gw[i] - w1) > 1e-4f * fabsf(w1) + 1e-7f;
        bad += fabsf(__half2float(gh[i]) - w1) > 1e-3f * fabsf(w1) + 1e-6f;
      }
      cudaFree(g[k]), cudaFree(halfw[k]), cudaFree(w[k]), cudaFree(m[k]), cudaFree(v[k]);
    }
    ok &= report("lamb", bad, rank);
  }
  for (Rank &rk : ranks) {
    cocoStatus_t st;
    NCCLCHECK(cocoGetStatus(rk.comm, &st));
    if (st.code != 0) { printf("device status %d on rank %d\n", st.code, rk.rank); ok = false; }
  }
  for (Rank &rk : ranks) NCCLCHECK(cocoCommDestroy(rk.comm));
  return ok ? 0 : 1;
}
