// Header-only fused ReduceScatter -> <any pointwise update> -> AllGather
// kernel: the program supplies the update as a device functor, the runtime
// supplies the peer mappings, flags and launch shape.
//
// This is what lets ANY fused pointwise CoCoNet program run as one kernel, not
// only the three update rules the library ships optimised kernels for.  The
// reference planned the same with source templates that its code generator
// would fill in (the unreachable part of src/codegen.cpp:1948-3929, whose
// `.h.in` inputs are not in its tree); here it is a C++ template.
//
//   struct MyUpdate {                      // emitted by the DSL or written by hand
//     float *state; float lr;              // Sliced tensors and scalars it needs
//     __device__ float operator()(size_t i, size_t gi, float gsum, float w) const {
//       state[i] = ...;                    // i: index in the slice, gi: global index
//       return w - lr * gsum;              // the new weight, gathered to all ranks
//     }
//   };
//   cocoGenericPlan plan;
//   cocoFusedGenericPlan(comm, g, cocoFloat32, w, N, stream, &plan);   // host, per step
//   cocoLaunchGenericFused<float>(plan, MyUpdate{state, lr}, stream);
//
// Protocol and memory ordering are those of the library's own kernel
// (coconet_b200/csrc/fused_step.cu): start barrier, pull the slice from all R
// gradient buffers and sum in rank order in fp32, apply the functor, store the
// result into all R weight buffers, end barrier; every wait is bounded and
// records a status instead of hanging.  The flag helpers are restated here so
// that this header stands alone; they must stay in step with that file.
#ifndef COCONET_FUSED_GENERIC_CUH_
#define COCONET_FUSED_GENERIC_CUH_

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "coconet_device.h"
#include "coconet_rt.h"

struct cocoGenericPlan {
  coco::StepArgs sa;
  coco::RankArgs ra;
  int ctas;
  int threads;
};

namespace coco_generic {

__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float4 ld_sys_f4(const float *p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_sys_f(const float *p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_sys_h4(const __half *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned short ld_sys_h(const __half *p) {
  unsigned short v;
  asm volatile("ld.volatile.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_sys_f4(float *p, float4 v) {
  asm volatile("st.volatile.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_sys_f(float *p, float v) {
  asm volatile("st.volatile.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// false if the flag did not reach seq within the time limit (or 2^28 probes)
static __device__ __noinline__ bool wait_flag(const unsigned long long *flag, unsigned long long seq,
                                       unsigned long long timeout_ns) {
  if (ld_acquire(flag) >= seq) return true;
  const unsigned long long t0 = timer_ns();
  for (unsigned spins = 1; spins <= (1u << 28); ++spins) {
    if (ld_acquire(flag) >= seq) return true;
    if ((spins & 63u) == 0u) {
      if (timer_ns() - t0 > timeout_ns) return false;
      __nanosleep(32);
    }
  }
  return false;
}

static __device__ __noinline__ void record(coco::FlagPage *me, int code, int rank, int phase, int peer,
                                    unsigned long long seq) {
  if (atomicCAS(&me->status[0], 0, code) == 0) {
    me->status[1] = rank;
    me->status[2] = phase;
    me->status[3] = peer;
    me->status[4] = (int)(seq & 0xffffffffull);
    me->status[5] = (int)(seq >> 32);
  }
}

template <typename GT> struct Grad;
template <> struct Grad<float> {
  static __device__ __forceinline__ void load4(const void *base, size_t i, float (&x)[4]) {
    const float4 q = ld_sys_f4((const float *)base + i);
    x[0] = q.x, x[1] = q.y, x[2] = q.z, x[3] = q.w;
  }
  static __device__ __forceinline__ float load1(const void *base, size_t i) {
    return ld_sys_f((const float *)base + i);
  }
};
template <> struct Grad<__half> {
  static __device__ __forceinline__ void load4(const void *base, size_t i, float (&x)[4]) {
    const uint2 q = ld_sys_h4((const __half *)base + i);
    x[0] = __half2float(__ushort_as_half((unsigned short)(q.x & 0xffffu)));
    x[1] = __half2float(__ushort_as_half((unsigned short)(q.x >> 16)));
    x[2] = __half2float(__ushort_as_half((unsigned short)(q.y & 0xffffu)));
    x[3] = __half2float(__ushort_as_half((unsigned short)(q.y >> 16)));
  }
  static __device__ __forceinline__ float load1(const void *base, size_t i) {
    return __half2float(__ushort_as_half(ld_sys_h((const __half *)base + i)));
  }
};

}  // namespace coco_generic

// The vector loop of the data phase for a world size of at most RB (1, 2, 4 or
// 8): RB gradient slots per unit instead of always eight, of which all are
// loaded before the first is used.
template <typename GT, class F, int RB>
__device__ __forceinline__ void cocoGenericVectorLoop(const coco::StepArgs &sa, const coco::RankArgs &ra,
                                                      const F &f, size_t lo, size_t nvec, size_t tid,
                                                      size_t nth, int Rr, int Rw) {
  using namespace coco_generic;
  for (size_t u = tid; u < nvec; u += nth) {
    const size_t j = u * 4, gi = lo + j;
    float g[4] = {0.f, 0.f, 0.f, 0.f}, x[RB][4];
#pragma unroll
    for (int p = 0; p < RB; ++p)
      if (p < Rr) Grad<GT>::load4(ra.g[p], gi, x[p]);
#pragma unroll
    for (int p = 0; p < RB; ++p)
      if (p < Rr) {
#pragma unroll
        for (int e = 0; e < 4; ++e) g[e] = p == 0 ? x[0][e] : __fadd_rn(g[e], x[p][e]);
      }
    const float4 w4 = *reinterpret_cast<const float4 *>(ra.w + gi);
    float4 o;
    o.x = f(j + 0, gi + 0, __fmul_rn(g[0], sa.grad_scale), w4.x);
    o.y = f(j + 1, gi + 1, __fmul_rn(g[1], sa.grad_scale), w4.y);
    o.z = f(j + 2, gi + 2, __fmul_rn(g[2], sa.grad_scale), w4.z);
    o.w = f(j + 3, gi + 3, __fmul_rn(g[3], sa.grad_scale), w4.w);
#pragma unroll
    for (int p = 0; p < RB; ++p)
      if (p < Rw) st_sys_f4((float *)ra.out[p] + gi, o);
  }
}

// One rank's fused step with a caller-supplied update.  GT: gradient element
// type (float or __half); weights and the gathered output are fp32.  `src` is
// the rank's argument block (kernel parameter or device memory); the CTAs of
// one rank are blockIdx.x = 0 .. gridDim.x - 1.
template <typename GT, class F>
__device__ __forceinline__ void cocoGenericFusedBody(const coco::StepArgs &sa, const coco::RankArgs *src,
                                                     const F &f) {
  using namespace coco_generic;
  __shared__ coco::RankArgs ra;
  __shared__ int s_ok;
  {
    const int *s = reinterpret_cast<const int *>(src);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(coco::RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
  }
  __syncthreads();
  const int R = sa.world, rank = ra.rank;
  coco::FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;

  // ---- start barrier: lane p of warp 0 talks to rank p ----------------------
  if (R > 1) {
    if (threadIdx.x < 32) {
      const int p = threadIdx.x;
      const bool peer = p < R && p != rank;
      if (blockIdx.x == 0 && peer) st_release(&ra.flags[p]->arrive[rank], seq);
      bool late = false;
      if (peer) late = !wait_flag(&me->arrive[p], seq, sa.timeout_ns);
      const unsigned bad = __ballot_sync(0xffffffffu, late);
      if (bad && threadIdx.x == 0) {
        record(me, cocoTimeout, rank, coco::kPhaseStart, __ffs(bad) - 1, seq);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  const bool ok = s_ok != 0;

  // ---- data phase ------------------------------------------------------------------
  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const size_t nvec = ra.aligned16 ? L / 4 : 0;
  // The stand-alone collectives of the library are this kernel with one half
  // switched off: a reduce-scatter does not store to the ranks, an all-gather
  // does not read from them.
  const bool reduce = (sa.flags & coco::kFlagNoReduce) == 0;
  const bool gather = (sa.flags & coco::kFlagNoGather) == 0;
  const int Rr = reduce ? R : 0, Rw = gather ? R : 0;
  if (ok) {
    if (R == 1)
      cocoGenericVectorLoop<GT, F, 1>(sa, ra, f, lo, nvec, tid, nth, Rr, Rw);
    else if (R == 2)
      cocoGenericVectorLoop<GT, F, 2>(sa, ra, f, lo, nvec, tid, nth, Rr, Rw);
    else if (R <= 4)
      cocoGenericVectorLoop<GT, F, 4>(sa, ra, f, lo, nvec, tid, nth, Rr, Rw);
    else
      cocoGenericVectorLoop<GT, F, coco::kMaxRanks>(sa, ra, f, lo, nvec, tid, nth, Rr, Rw);
    for (size_t j = nvec * 4 + tid; j < L; j += nth) {
      const size_t gi = lo + j;
      float g = 0.f;
      for (int p = 0; p < Rr; ++p) {
        const float x = Grad<GT>::load1(ra.g[p], gi);
        g = p == 0 ? x : __fadd_rn(g, x);
      }
      const float o = f(j, gi, __fmul_rn(g, sa.grad_scale), ra.w[gi]);
      for (int p = 0; p < Rw; ++p) st_sys_f((float *)ra.out[p] + gi, o);
    }
  }

  // ---- end barrier -------------------------------------------------------------------
  if (R > 1) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < 32) {
      unsigned prev = 0;
      if (threadIdx.x == 0) {
        __threadfence_system();
        prev = atomicAdd(&me->done_count, 1u);
        if (prev == gridDim.x - 1) me->done_count = 0;
        __threadfence_system();
      }
      __syncwarp();
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == gridDim.x - 1) {
        __threadfence_system();
        const int p = threadIdx.x;
        const bool peer = p < R && p != rank;
        if (peer) st_release(&ra.flags[p]->done[rank], seq);
        if (ok) {
          bool late = false;
          if (peer) late = !wait_flag(&me->done[p], seq, sa.timeout_ns);
          const unsigned bad = __ballot_sync(0xffffffffu, late);
          if (bad && threadIdx.x == 0)
            record(me, cocoTimeout, rank, coco::kPhaseEnd, __ffs(bad) - 1, seq);
        }
      }
    }
  }
}

template <typename GT, class F>
__global__ void __launch_bounds__(512, 2)
    cocoGenericFusedKernel(const __grid_constant__ coco::StepArgs sa,
                           const __grid_constant__ coco::RankArgs ra_in, const F f) {
  cocoGenericFusedBody<GT, F>(sa, &ra_in, f);
}

// Several ranks that share one GPU (virtual ranks of a single-process
// communicator) as ONE cooperative launch: blockIdx.y is the rank, whose
// argument block and functor come from tables in device memory.  Kernels that
// wait for one another must never be separate launches on one GPU.
template <typename GT, class F>
__global__ void __launch_bounds__(512, 2)
    cocoGenericFusedKernelMulti(const __grid_constant__ coco::StepArgs sa,
                                const coco::RankArgs *__restrict__ table, const F *__restrict__ ftable) {
  const F f = ftable[blockIdx.y];
  cocoGenericFusedBody<GT, F>(sa, table + blockIdx.y, f);
}

// Host: enqueue one fused step with the update `f` on `stream`.
template <typename GT, class F>
inline int cocoLaunchGenericFused(const cocoGenericPlan &plan, const F &f, cudaStream_t stream) {
  if (plan.sa.count == 0) return cocoSuccess;
  cocoGenericFusedKernel<GT, F><<<plan.ctas, plan.threads, 0, stream>>>(plan.sa, plan.ra, f);
  return cudaGetLastError() == cudaSuccess ? cocoSuccess : cocoCudaError;
}

#endif  // COCONET_FUSED_GENERIC_CUH_
