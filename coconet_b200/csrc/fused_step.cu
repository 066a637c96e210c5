// Fused ReduceScatter -> sliced optimizer update -> AllGather, one kernel per
// step per GPU, for sm_100a.
//
// Replaces ncclAllReduceComputationRingKernel and its primitives
// (nccl/src/collectives/device/all_reduce_computation.h:35-150, 807-1054;
// primitives_computation.h:58-572; common_kernel.h:830-1172 in
// parasailteam/coconet).  The reference walks a ring: 2(R-1) serialised hops,
// each staged through a FIFO on the receiver.  On an NVSwitch node every peer
// is one hop away at full bandwidth, so this kernel is one-shot:
//
//   start barrier   every rank tells every peer "my kernel of call `seq` has
//                   started" (so its gradients are final and its weights may
//                   be overwritten) and waits for the same from all peers
//   reduce-scatter  each thread pulls 16-byte units of the rank's own slice
//                   from all R gradient buffers (R-1 of them over NVLink),
//                   sums them in fp32 in rank order 0..R-1
//   update          SGD / Adam / LAMB in registers on fp32 w, m, v
//   all-gather      the updated unit is stored straight into all R weight
//                   buffers (R-1 over NVLink)
//   end barrier     the last CTA of the rank announces "done" to the peers
//                   and waits for theirs, so the kernel only completes when
//                   nobody reads this rank's gradients or writes its weights
//
// The path is bandwidth-bound (NVLink for R > 1, HBM for R == 1); there is no
// contraction and no tensor-core work.  Every wait is bounded: on expiry the
// kernel records a status and runs to completion without touching peers.
#include "fused_step.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

namespace coco {
namespace {

// ---------------------------------------------------------------------------
// memory-model helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Loads/stores of data that another GPU writes or reads: system-coherent
// (never served from a stale L1 line), 16 bytes wide where possible.
__device__ __forceinline__ uint4 ld_sys_16(const void *p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned ld_sys_4(const void *p) {
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned short ld_sys_2(const void *p) {
  unsigned short v;
  asm volatile("ld.volatile.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_sys_16(void *p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_sys_8(void *p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_sys_4(void *p, unsigned v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_sys_2(void *p, unsigned short v) {
  asm volatile("st.volatile.global.u16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
}
__device__ __forceinline__ double ld_volatile_f64(const double *p) {
  double v;
  asm volatile("ld.volatile.global.f64 %0, [%1];" : "=d"(v) : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------
// bounded waits and the status word
// ---------------------------------------------------------------------------
constexpr unsigned kSpinHardCap = 1u << 28;  // backstop if the timer misbehaves

__device__ void record_status(FlagPage *me, int code, int rank, int phase, int peer,
                              unsigned long long seq) {
  if (atomicCAS(&me->status[0], 0, code) == 0) {
    me->status[1] = rank;
    me->status[2] = phase;
    me->status[3] = peer;
    me->status[4] = (int)(seq & 0xffffffffull);
    me->status[5] = (int)(seq >> 32);
  }
}

// Waits until flags[p] >= seq for every p in [0, world) except `skip`.
// Returns -1 on success, else the first peer that did not show up in time.
__device__ int wait_all(const unsigned long long *flags, int world, int skip,
                        unsigned long long seq, unsigned long long timeout_ns) {
  const unsigned long long t0 = globaltimer_ns();
  for (int p = 0; p < world; ++p) {
    if (p == skip) continue;
    unsigned spins = 0;
    while (ld_acquire_sys(flags + p) < seq) {
      ++spins;
      if ((spins & 63u) == 0u) {
        if (globaltimer_ns() - t0 > timeout_ns || spins > kSpinHardCap) return p;
        __nanosleep(64);
      }
    }
  }
  return -1;
}

// ---------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------
struct NoLp {};  // "no low-precision copy": the fp32 weights are what is gathered

template <typename T> struct Bits16;
template <> struct Bits16<__half> {
  static __device__ __forceinline__ float to_f32(unsigned short b) {
    return __half2float(__ushort_as_half(b));
  }
  static __device__ __forceinline__ unsigned short from_f32(float f) {
    return __half_as_ushort(__float2half_rn(f));
  }
};
template <> struct Bits16<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(unsigned short b) {
    return __uint_as_float(((unsigned)b) << 16);
  }
  static __device__ __forceinline__ unsigned short from_f32(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  }
};

template <typename GT> struct GradTraits {
  static constexpr int kVec = 8;  // 16 bytes of 16-bit elements
  static constexpr bool kIs16 = true;
};
template <> struct GradTraits<float> {
  static constexpr int kVec = 4;
  static constexpr bool kIs16 = false;
};

// Raw (unconverted) gradient unit of VEC elements.
template <typename GT, int VEC> struct RawUnit;
template <> struct RawUnit<float, 4> {
  uint4 q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_16((const float *)base + i);
  }
  __device__ __forceinline__ float get(int k) const {
    return __uint_as_float(k == 0 ? q.x : k == 1 ? q.y : k == 2 ? q.z : q.w);
  }
  __device__ __forceinline__ unsigned short bits(int) const { return 0; }
};
template <> struct RawUnit<float, 1> {
  unsigned q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_4((const float *)base + i);
  }
  __device__ __forceinline__ float get(int) const { return __uint_as_float(q); }
  __device__ __forceinline__ unsigned short bits(int) const { return 0; }
};
template <typename GT> struct RawUnit<GT, 8> {
  uint4 q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_16((const unsigned short *)base + i);
  }
  __device__ __forceinline__ unsigned short bits(int k) const {
    const unsigned wd = (k >> 1) == 0 ? q.x : (k >> 1) == 1 ? q.y : (k >> 1) == 2 ? q.z : q.w;
    return (unsigned short)((k & 1) ? (wd >> 16) : (wd & 0xffffu));
  }
  __device__ __forceinline__ float get(int k) const { return Bits16<GT>::to_f32(bits(k)); }
};
template <typename GT> struct RawUnit<GT, 1> {
  unsigned short q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_2((const unsigned short *)base + i);
  }
  __device__ __forceinline__ unsigned short bits(int) const { return q; }
  __device__ __forceinline__ float get(int) const { return Bits16<GT>::to_f32(q); }
};

// ---------------------------------------------------------------------------
// reduce-scatter of one unit: pull from every rank, sum in fp32 in rank order
// ---------------------------------------------------------------------------
template <typename GT, int VEC>
__device__ __forceinline__ void reduce_unit(const RankArgs &ra, const StepArgs &sa, size_t i,
                                            float (&g)[VEC], float (&gg)[VEC]) {
  RawUnit<GT, VEC> raw[kMaxRanks];
  const int R = sa.world;
  const bool ring = GradTraits<GT>::kIs16 && sa.variant == cocoVariantNccl;
  // The forked-NCCL variant reproduces the ring: the chunk owned by `rank`
  // starts at rank+1 and is accumulated hop by hop in fp16 (__hadd2,
  // common_kernel.h:795-807).  Everything else sums 0..R-1 in fp32.
  const int first = ring ? (ra.rank + 1) % R : 0;
#pragma unroll
  for (int k = 0; k < kMaxRanks; ++k) {
    if (k < R) {
      int p = first + k;
      if (p >= R) p -= R;
      raw[k].load(ra.g[p], i);
    }
  }
  if (ring) {
    if constexpr (std::is_same<GT, __half>::value) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        __half acc = __ushort_as_half(raw[0].bits(e));
#pragma unroll
        for (int k = 1; k < kMaxRanks; ++k)
          if (k < R) acc = __hadd(acc, __ushort_as_half(raw[k].bits(e)));
        g[e] = __half2float(acc);
        gg[e] = __half2float(__hmul(acc, acc));  // (float)(S0 * S0), reduce_kernel.h:29
      }
    }
    return;
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    float acc = raw[0].get(e);
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
      if (k < R) acc = __fadd_rn(acc, raw[k].get(e));
    g[e] = __fmul_rn(acc, sa.grad_scale);
    gg[e] = 0.f;
  }
}

// ---------------------------------------------------------------------------
// local fp32 state and the gathered output
// ---------------------------------------------------------------------------
template <int VEC> __device__ __forceinline__ void load_f32(const float *p, float (&x)[VEC]) {
  if constexpr (VEC == 1) {
    x[0] = *p;
  } else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      const float4 t = __ldcs(reinterpret_cast<const float4 *>(p) + q);
      x[4 * q] = t.x, x[4 * q + 1] = t.y, x[4 * q + 2] = t.z, x[4 * q + 3] = t.w;
    }
  }
}
template <int VEC> __device__ __forceinline__ void store_f32(float *p, const float (&x)[VEC]) {
  if constexpr (VEC == 1) {
    *p = x[0];
  } else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q)
      __stcs(reinterpret_cast<float4 *>(p) + q,
             make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]));
  }
}

// Store VEC updated weights at element i of every rank's gathered buffer.
template <typename LPT, int VEC>
__device__ __forceinline__ void gather_unit(const RankArgs &ra, int R, size_t i,
                                            const float (&x)[VEC]) {
  if constexpr (std::is_same<LPT, NoLp>::value) {
    if constexpr (VEC == 1) {
      const unsigned b = __float_as_uint(x[0]);
      for (int p = 0; p < R; ++p) st_sys_4((float *)ra.out[p] + i, b);
    } else {
      uint4 q[VEC / 4];
#pragma unroll
      for (int j = 0; j < VEC / 4; ++j)
        q[j] = make_uint4(__float_as_uint(x[4 * j]), __float_as_uint(x[4 * j + 1]),
                          __float_as_uint(x[4 * j + 2]), __float_as_uint(x[4 * j + 3]));
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < R) {
#pragma unroll
          for (int j = 0; j < VEC / 4; ++j) st_sys_16((float *)ra.out[p] + i + 4 * j, q[j]);
        }
    }
  } else {
    unsigned short h[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) h[e] = Bits16<LPT>::from_f32(x[e]);
    if constexpr (VEC == 1) {
      for (int p = 0; p < R; ++p) st_sys_2((unsigned short *)ra.out[p] + i, h[0]);
    } else if constexpr (VEC == 4) {
      const uint2 q = make_uint2(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16));
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < R) st_sys_8((unsigned short *)ra.out[p] + i, q);
    } else {
      const uint4 q = make_uint4(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16),
                                 h[4] | ((unsigned)h[5] << 16), h[6] | ((unsigned)h[7] << 16));
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < R) st_sys_16((unsigned short *)ra.out[p] + i, q);
    }
  }
}

// ---------------------------------------------------------------------------
// the update math.  Individually rounded fp32 operations in the order the
// reference's host checks evaluate them, so that m and v match a scalar CPU
// evaluation bit for bit.
// ---------------------------------------------------------------------------
struct Hyper {
  float lr, b1, b2, omb1, omb2, eps, wd, d1, d2;
  double d1d, d2d;
  int variant;
};

__device__ __forceinline__ Hyper make_hyper(const StepArgs &sa) {
  Hyper h;
  h.lr = sa.lr, h.b1 = sa.beta1, h.b2 = sa.beta2;
  h.omb1 = __fsub_rn(1.f, sa.beta1), h.omb2 = __fsub_rn(1.f, sa.beta2);
  h.eps = sa.eps, h.wd = sa.weight_decay, h.d1 = sa.d1, h.d2 = sa.d2;
  h.d1d = sa.d1d, h.d2d = sa.d2d;
  h.variant = sa.variant;
  return h;
}

// test-sgd.cu:18:  w - (lr * g)
__device__ __forceinline__ float sgd_elem(const Hyper &h, float w, float g) {
  return __fsub_rn(w, __fmul_rn(h.lr, g));
}

// New moments.  overlap: b*m + (1-b)*g, b*v + ((1-b)*g)*g
// (multi-process-adam-scattered.cpp:112-116); dsl: (1-b)*(g*g)
// (test-adam.cu:16); nccl: m*b2 + g*(1-b2) for BOTH moments, with the
// half-precision square (reduce_kernel.h:27-39, common_kernel.h:875-879).
__device__ __forceinline__ void moments_elem(const Hyper &h, float g, float gg, float &m,
                                             float &v) {
  if (h.variant == cocoVariantNccl) {
    v = __fadd_rn(__fmul_rn(v, h.b2), __fmul_rn(gg, h.omb2));
    m = __fadd_rn(__fmul_rn(m, h.b2), __fmul_rn(g, h.omb2));
  } else if (h.variant == cocoVariantDsl) {
    v = __fadd_rn(__fmul_rn(h.b2, v), __fmul_rn(h.omb2, __fmul_rn(g, g)));
    m = __fadd_rn(__fmul_rn(h.b1, m), __fmul_rn(h.omb1, g));
  } else {
    m = __fadd_rn(__fmul_rn(h.b1, m), __fmul_rn(h.omb1, g));
    v = __fadd_rn(__fmul_rn(h.b2, v), __fmul_rn(__fmul_rn(h.omb2, g), g));
  }
}

// m^ = m/d1, v^ = v/d2.  The bias-corrected form divides by the DOUBLE
// 1 - beta^t and narrows, exactly as the reference's host check does
// (multi-process-adam-scattered.cpp:118-119: pow() promotes to double), so the
// result can match a CPU evaluation bit for bit; the other forms divide by a
// float (test-adam.cu:21,29; reduce_kernel.h:33-47).
__device__ __forceinline__ void corrected_moments(const Hyper &h, float m, float v, float &m_,
                                                  float &v_) {
  if (h.variant == cocoVariantOverlap) {
    m_ = __double2float_rn(__ddiv_rn((double)m, h.d1d));
    v_ = __double2float_rn(__ddiv_rn((double)v, h.d2d));
  } else {
    m_ = __fdiv_rn(m, h.d1);
    v_ = __fdiv_rn(v, h.d2);
  }
}

__device__ __forceinline__ float adam_elem(const Hyper &h, float w, float m, float v) {
  float m_, v_;
  corrected_moments(h, m, v, m_, v_);
  if (h.variant == cocoVariantDsl)  // test-adam.cu:38:  w - (lr*m_)/v_
    return __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, m_), v_));
  // overlap (sample :121): lr*m_/(sqrt(v_)+eps); nccl (reduce_kernel.h:48-62) is
  // the same expression with eps == 0.
  return __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, m_), __fadd_rn(__fsqrt_rn(v_), h.eps)));
}

// r = m^/(sqrt(v^)+eps) + lambda*w  (sample :416; lamb.cpp:84 with eps == 0)
__device__ __forceinline__ float lamb_r_elem(const Hyper &h, float w, float m, float v) {
  float m_, v_;
  corrected_moments(h, m, v, m_, v_);
  return __fadd_rn(__fdiv_rn(m_, __fadd_rn(__fsqrt_rn(v_), h.eps)), __fmul_rn(h.wd, w));
}

// ---------------------------------------------------------------------------
// one unit of the data phase
// ---------------------------------------------------------------------------
// SGD and Adam: whole step.  LAMB phase 1: moments + norm partials only.
template <int OPT, typename GT, typename LPT, int VEC>
__device__ __forceinline__ void step_unit(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                          size_t lo, size_t i, double &sum_w2, double &sum_r2) {
  float g[VEC], gg[VEC], w[VEC];
  reduce_unit<GT, VEC>(ra, sa, i, g, gg);
  load_f32<VEC>(ra.w + i, w);
  if constexpr (OPT == kSGD) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) w[e] = sgd_elem(h, w[e], g[e]);
  } else {
    float m[VEC], v[VEC];
    load_f32<VEC>(ra.m + (i - lo), m);
    load_f32<VEC>(ra.v + (i - lo), v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      moments_elem(h, g[e], gg[e], m[e], v[e]);
      if constexpr (OPT == kAdam) {
        w[e] = adam_elem(h, w[e], m[e], v[e]);
      } else {
        const float r = lamb_r_elem(h, w[e], m[e], v[e]);
        if (sa.flags & COCO_LAMB_REF_QUIRK) {
          sum_r2 += (double)__fdiv_rn(__fmul_rn(r, r), (float)sa.count);
          sum_w2 += (double)__fmul_rn(w[e], w[e]);
        } else {
          sum_r2 += (double)r * (double)r;
          sum_w2 += (double)w[e] * (double)w[e];
        }
      }
    }
    store_f32<VEC>(ra.m + (i - lo), m);
    store_f32<VEC>(ra.v + (i - lo), v);
  }
  if constexpr (OPT != kLAMB) {
    if constexpr (!std::is_same<LPT, NoLp>::value) store_f32<VEC>(ra.w + i, w);
    gather_unit<LPT, VEC>(ra, sa.world, i, w);
  }
}

// LAMB phase 2: recompute r from the stored moments, apply the scaled step.
template <typename LPT, int VEC>
__device__ __forceinline__ void lamb_apply_unit(const RankArgs &ra, const StepArgs &sa,
                                                const Hyper &h, size_t lo, size_t i,
                                                float lr_scale) {
  float w[VEC], m[VEC], v[VEC];
  load_f32<VEC>(ra.w + i, w);
  load_f32<VEC>(ra.m + (i - lo), m);
  load_f32<VEC>(ra.v + (i - lo), v);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float r = lamb_r_elem(h, w[e], m[e], v[e]);
    w[e] = __fsub_rn(w[e], __fmul_rn(lr_scale, r));  // sample :434-435
  }
  if constexpr (!std::is_same<LPT, NoLp>::value) store_f32<VEC>(ra.w + i, w);
  gather_unit<LPT, VEC>(ra, sa.world, i, w);
}

__device__ __forceinline__ double warp_sum(double x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
  return x;
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int OPT, typename GT, typename LPT>
__global__ void __launch_bounds__(512)
    fused_step_kernel(const __grid_constant__ StepArgs sa, const __grid_constant__ RankArgs one,
                      const RankArgs *__restrict__ table) {
  __shared__ RankArgs ra;
  __shared__ int s_ok;
  __shared__ float s_lr_scale;
  __shared__ double s_red[2][16];

  {  // this (virtual) rank's pointers -> shared memory
    const RankArgs *src = table ? table + blockIdx.y : &one;
    const int *s = reinterpret_cast<const int *>(src);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
  }
  __syncthreads();

  const int R = sa.world;
  const int rank = ra.rank;
  FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;

  // ---- start barrier ------------------------------------------------------
  if (R > 1) {
    if (threadIdx.x == 0) {
      if (blockIdx.x == 0) {
        for (int p = 0; p < R; ++p)
          if (p != rank) st_release_sys(&ra.flags[p]->arrive[rank], seq);
      }
      const int late = wait_all(me->arrive, R, rank, seq, sa.timeout_ns);
      if (late >= 0) {
        record_status(me, cocoTimeout, rank, kPhaseStart, late, seq);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  bool ok = s_ok != 0;

  // ---- slice of this rank (same arithmetic as cocoSliceBounds) -------------
  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  constexpr int VEC = GradTraits<GT>::kVec;
  const size_t nvec = ra.pad ? L / VEC : 0;  // pad != 0: slice and pointers allow 16-byte units
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const Hyper h = make_hyper(sa);

  double sum_w2 = 0.0, sum_r2 = 0.0;
  if (ok) {
    for (size_t u = tid; u < nvec; u += nth)
      step_unit<OPT, GT, LPT, VEC>(ra, sa, h, lo, lo + u * VEC, sum_w2, sum_r2);
    for (size_t j = nvec * VEC + tid; j < L; j += nth)
      step_unit<OPT, GT, LPT, 1>(ra, sa, h, lo, lo + j, sum_w2, sum_r2);
  }

  if constexpr (OPT == kLAMB) {
    // ---- norms: thread -> warp -> CTA -> rank (fixed order) -> all ranks ---
    sum_w2 = warp_sum(sum_w2);
    sum_r2 = warp_sum(sum_r2);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) s_red[0][wid] = sum_w2, s_red[1][wid] = sum_r2;
    __syncthreads();
    if (threadIdx.x == 0) {
      double a = 0.0, b = 0.0;
      const int nw = (blockDim.x + 31) >> 5;
      for (int k = 0; k < nw; ++k) a += s_red[0][k], b += s_red[1][k];
      me->cta_part[blockIdx.x][0] = a;
      me->cta_part[blockIdx.x][1] = b;
      __threadfence();
      const unsigned prev = atomicAdd(&me->norm_count, 1u);
      if (prev == gridDim.x - 1) {  // last CTA of the rank: combine and publish
        __threadfence();
        a = 0.0, b = 0.0;
        for (unsigned c = 0; c < gridDim.x; ++c) {
          a += ld_volatile_f64(&me->cta_part[c][0]);
          b += ld_volatile_f64(&me->cta_part[c][1]);
        }
        me->norm_count = 0;
        for (int p = 0; p < R; ++p) {
          volatile double *dst = ra.flags[p]->norm_part[rank];
          dst[0] = a;
          dst[1] = b;
        }
        __threadfence_system();
        for (int p = 0; p < R; ++p) st_release_sys(&ra.flags[p]->norm_flag[rank], seq);
      }
      // every CTA: wait for all ranks' partials (bounded), sum in rank order
      float lr_scale = 0.f;
      if (ok) {
        const int late = wait_all(me->norm_flag, R, -1, seq, sa.timeout_ns);
        if (late >= 0) {
          record_status(me, cocoTimeout, rank, kPhaseNorm, late, seq);
          s_ok = 0;
        } else {
          double w2 = 0.0, r2 = 0.0;
          for (int p = 0; p < R; ++p) {
            w2 += ld_volatile_f64(&me->norm_part[p][0]);
            r2 += ld_volatile_f64(&me->norm_part[p][1]);
          }
          double wn, rn, sc;
          if (sa.flags & COCO_LAMB_REF_QUIRK) {  // sample :424-433
            rn = sqrt(r2);
            wn = sqrt(w2 / (double)N);
            sc = ((wn > 0) ? (rn > 0 ? wn / rn : 1.0) : 1.0) / rn;
          } else {  // lamb.cpp:86 with the sample's guards
            rn = sqrt(r2);
            wn = sqrt(w2);
            sc = (wn > 0) ? (rn > 0 ? wn / rn : 1.0) : 1.0;
          }
          lr_scale = __fmul_rn(sa.lr, (float)sc);
          if (blockIdx.x == 0) me->last_norms[0] = wn, me->last_norms[1] = rn;
        }
      }
      s_lr_scale = lr_scale;
    }
    __syncthreads();
    ok = s_ok != 0;
    if (ok) {
      const float lr_scale = s_lr_scale;
      for (size_t u = tid; u < nvec; u += nth)
        lamb_apply_unit<LPT, VEC>(ra, sa, h, lo, lo + u * VEC, lr_scale);
      for (size_t j = nvec * VEC + tid; j < L; j += nth)
        lamb_apply_unit<LPT, 1>(ra, sa, h, lo, lo + j, lr_scale);
    }
  }

  // ---- end barrier ----------------------------------------------------------
  if (R > 1) {
    __threadfence_system();  // this thread's peer stores before the "done" signal
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned prev = atomicAdd(&me->done_count, 1u);
      if (prev == gridDim.x - 1) {  // last CTA of the rank
        me->done_count = 0;
        __threadfence_system();
        for (int p = 0; p < R; ++p)
          if (p != rank) st_release_sys(&ra.flags[p]->done[rank], seq);
        if (ok) {
          const int late = wait_all(me->done, R, rank, seq, sa.timeout_ns);
          if (late >= 0) record_status(me, cocoTimeout, rank, kPhaseEnd, late, seq);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
typedef void (*KernelPtr)(const StepArgs, const RankArgs, const RankArgs *);

template <int OPT, typename GT> KernelPtr pick_lp(bool has_lp, cocoDataType_t lp) {
  if (!has_lp) return fused_step_kernel<OPT, GT, NoLp>;
  if (lp == cocoFloat16) return fused_step_kernel<OPT, GT, __half>;
  if (lp == cocoBfloat16) return fused_step_kernel<OPT, GT, __nv_bfloat16>;
  return nullptr;
}
template <int OPT> KernelPtr pick_g(cocoDataType_t g, bool has_lp, cocoDataType_t lp) {
  if (g == cocoFloat32) return pick_lp<OPT, float>(has_lp, lp);
  if (g == cocoFloat16) return pick_lp<OPT, __half>(has_lp, lp);
  if (g == cocoBfloat16) return pick_lp<OPT, __nv_bfloat16>(has_lp, lp);
  return nullptr;
}
KernelPtr pick(int opt, cocoDataType_t g, bool has_lp, cocoDataType_t lp) {
  switch (opt) {
    case kSGD: return pick_g<kSGD>(g, has_lp, lp);
    case kAdam: return pick_g<kAdam>(g, has_lp, lp);
    case kLAMB: return pick_g<kLAMB>(g, has_lp, lp);
  }
  return nullptr;
}

}  // namespace

cudaError_t launch_fused_step(int opt, cocoDataType_t g_type, bool has_lp, cocoDataType_t lp_type,
                              const StepArgs &sa, const RankArgs &one, const RankArgs *table,
                              const LaunchConfig &cfg, cudaStream_t stream) {
  KernelPtr k = pick(opt, g_type, has_lp, lp_type);
  if (!k) return cudaErrorInvalidValue;
  const dim3 grid(cfg.ctas, cfg.nvirt > 1 ? cfg.nvirt : 1, 1);
  const dim3 block(cfg.threads, 1, 1);
  const RankArgs *tbl = cfg.nvirt > 1 ? table : nullptr;
  void *params[] = {(void *)&sa, (void *)&one, (void *)&tbl};
  if (cfg.cooperative)
    return cudaLaunchCooperativeKernel((const void *)k, grid, block, params, 0, stream);
  return cudaLaunchKernel((const void *)k, grid, block, params, 0, stream);
}

cudaError_t fused_step_occupancy(int opt, cocoDataType_t g_type, bool has_lp,
                                 cocoDataType_t lp_type, int threads, int *ctas_per_sm) {
  KernelPtr k = pick(opt, g_type, has_lp, lp_type);
  if (!k) return cudaErrorInvalidValue;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(ctas_per_sm, (const void *)k, threads, 0);
}

}  // namespace coco
