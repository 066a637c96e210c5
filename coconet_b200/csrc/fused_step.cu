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

#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

// Build-time experiment switches of the single-rank 16-bit path (A/B runs).
#ifndef COCO_LOCAL16_SHUFFLE
#define COCO_LOCAL16_SHUFFLE 0   // 1: 16-byte gradient loads / copy stores, halves exchanged by shuffles
#endif
#ifndef COCO_CHECKED
#define COCO_CHECKED 0  // 1: bounds and alignment checks per unit that set the status word
#endif
// Block size the single-rank kernels are compiled for, two CTAs per SM: the
// register budget is 65536 / (2 x this).  The 16-bit-gradient kernels work on
// 8-element units and spill at 64 registers; at 384 threads they have 80 and
// measured 0.957 of the HBM copy peak against 0.910 at 512 (mixed-precision
// Adam, 334 M elements; 256 threads, 116 registers, no spills at all: 0.801 --
// too few warps).
#ifndef COCO_LOCAL16_THREADS
#define COCO_LOCAL16_THREADS 384
#endif
#ifndef COCO_LOCAL32_THREADS
#define COCO_LOCAL32_THREADS 512
#endif
// Threads per CTA the kernels for lists of tensors are compiled for.
#ifndef COCO_SEG_THREADS
#define COCO_SEG_THREADS 512
#endif
// The same for the multi-rank paths (register-staged, switch, warp rings) with
// 16-bit gradients.
#ifndef COCO_MULTI16_THREADS
#define COCO_MULTI16_THREADS 512
#endif
#ifndef COCO_MULTI32_THREADS
#define COCO_MULTI32_THREADS 512
#endif

namespace coco {

typedef void (*KernelPtr)(const StepArgs, const RankArgs, const RankArgs *);

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
__device__ __forceinline__ uint2 ld_sys_8(const void *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
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

__device__ __noinline__ void record_status(FlagPage *me, int code, int rank, int phase, int peer,
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
__device__ __noinline__ int wait_all(const unsigned long long *flags, int world, int skip,
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

// One flag.  Returns false if it did not reach seq in time.
__device__ __noinline__ bool wait_one(const unsigned long long *flag, unsigned long long seq,
                         unsigned long long timeout_ns) {
  if (ld_acquire_sys(flag) >= seq) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (unsigned spins = 1; spins <= kSpinHardCap; ++spins) {
    if (ld_acquire_sys(flag) >= seq) return true;
    if ((spins & 63u) == 0u) {
      if (globaltimer_ns() - t0 > timeout_ns) return false;
      __nanosleep(32);
    }
  }
  return false;
}

// Flags are exchanged by the first warp of a CTA, lane p talking to rank p, so
// that the R-1 remote stores (each a release: fence + store) and the R-1 polls
// proceed in parallel instead of one after the other.
// signal: store seq into slot `rank` of flags_of(p) for every peer p.
// wait:   until own slot p >= seq for every peer p; returns the first late peer or -1.
// Must be called by all 32 lanes of warp 0.
template <typename SlotOf>
__device__ __forceinline__ void warp_signal_peers(const RankArgs &ra, int R, int rank,
                                                  unsigned long long seq, SlotOf slot_of) {
  const int p = threadIdx.x & 31;
  if (p < R && p != rank) st_release_sys(slot_of(ra.flags[p]) + rank, seq);
}
__device__ __forceinline__ int warp_wait_peers(const unsigned long long *slots, int R, int rank,
                                               unsigned long long seq,
                                               unsigned long long timeout_ns) {
  const int p = threadIdx.x & 31;
  bool late = false;
  if (p < R && p != rank) late = !wait_one(slots + p, seq, timeout_ns);
  const unsigned bad = __ballot_sync(0xffffffffu, late);
  return bad ? __ffs(bad) - 1 : -1;
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
  static constexpr int kVec = 4;  // direct path: 4 elements per thread and pass
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
template <> struct RawUnit<float, 8> {
  uint4 q[2];
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q[0] = ld_sys_16((const float *)base + i);
    q[1] = ld_sys_16((const float *)base + i + 4);
  }
  template <int HS> __device__ __forceinline__ void load_halves(const void *base, size_t i) {
    q[0] = ld_sys_16((const float *)base + i);
    q[1] = ld_sys_16((const float *)base + i + HS);
  }
  __device__ __forceinline__ float get(int k) const {
    const uint4 &h = q[k >> 2];
    const int j = k & 3;
    return __uint_as_float(j == 0 ? h.x : j == 1 ? h.y : j == 2 ? h.z : h.w);
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
template <typename GT> struct RawUnit<GT, 4> {
  uint2 q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_8((const unsigned short *)base + i);
  }
  __device__ __forceinline__ unsigned short bits(int k) const {
    const unsigned wd = (k >> 1) == 0 ? q.x : q.y;
    return (unsigned short)((k & 1) ? (wd >> 16) : (wd & 0xffffu));
  }
  __device__ __forceinline__ float get(int k) const { return Bits16<GT>::to_f32(bits(k)); }
};
template <typename GT> struct RawUnit<GT, 8> {
  uint4 q;
  __device__ __forceinline__ void load(const void *base, size_t i) {
    q = ld_sys_16((const unsigned short *)base + i);
  }
  // elements i..i+3 and i+HS..i+HS+3
  template <int HS> __device__ __forceinline__ void load_halves(const void *base, size_t i) {
#if COCO_LOCAL16_SHUFFLE
    // The warp's 32 units are 256 consecutive elements (lane t: 4t.. and
    // 128+4t..).  Every lane loads 16 contiguous bytes of them (elements
    // 8t..8t+7) and the lanes exchange halves: element 4t+k sits in lane t/2,
    // words 2(t&1) and 2(t&1)+1; element 128+4t+k in lane 16 + t/2.  Must be
    // called by all 32 lanes.
    static_assert(HS == 128, "the exchange is written for the 128-element half stride");
    const int t = threadIdx.x & 31;
    const uint4 c = ld_sys_16((const unsigned short *)base + i + 4 * t);
    const int s0 = t >> 1, s1 = 16 + (t >> 1);
    const unsigned a0 = __shfl_sync(0xffffffffu, c.x, s0), a1 = __shfl_sync(0xffffffffu, c.y, s0);
    const unsigned a2 = __shfl_sync(0xffffffffu, c.z, s0), a3 = __shfl_sync(0xffffffffu, c.w, s0);
    const unsigned b0 = __shfl_sync(0xffffffffu, c.x, s1), b1 = __shfl_sync(0xffffffffu, c.y, s1);
    const unsigned b2 = __shfl_sync(0xffffffffu, c.z, s1), b3 = __shfl_sync(0xffffffffu, c.w, s1);
    q = (t & 1) ? make_uint4(a2, a3, b2, b3) : make_uint4(a0, a1, b0, b1);
#else
    const uint2 a = ld_sys_8((const unsigned short *)base + i);
    const uint2 b = ld_sys_8((const unsigned short *)base + i + HS);
    q = make_uint4(a.x, a.y, b.x, b.y);
#endif
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
// reduce-scatter of one unit: pull from every rank, sum in fp32 in rank order.
//
// RB is a compile-time bound on the world size (the kernel dispatches once on
// it): RB = 1 or 2 means R == RB exactly, RB = 4 / 8 covers R <= RB with a
// predicate per slot.  All RB loads are issued before the first use, so a
// thread has up to RB remote requests in flight.  RB = 0 is a plain loop over
// the R ranks (cold scalar path).
// ---------------------------------------------------------------------------
template <typename GT, int VEC, int RB, int HS = 4>
__device__ __forceinline__ void reduce_unit(const RankArgs &ra, const StepArgs &sa, size_t i,
                                            float (&g)[VEC]) {
  const int R = sa.world;
  const bool ring = GradTraits<GT>::kIs16 && sa.variant == cocoVariantNccl;
  // The forked-NCCL variant reproduces the ring: the chunk owned by `rank`
  // starts at rank+1 and is accumulated hop by hop in fp16 (__hadd2,
  // common_kernel.h:795-807).  Everything else sums 0..R-1 in fp32.
  const int first = ring ? (ra.rank + 1) % R : 0;
  if constexpr (RB == 0) {
    RawUnit<GT, VEC> raw;
    __half hacc[VEC];
    for (int k = 0; k < R; ++k) {
      int p = first + k;
      if (p >= R) p -= R;
      raw.load(ra.g[p], i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        if (ring) {
          if constexpr (std::is_same<GT, __half>::value)
            hacc[e] = k == 0 ? __ushort_as_half(raw.bits(e))
                             : __hadd(hacc[e], __ushort_as_half(raw.bits(e)));
        } else {
          g[e] = k == 0 ? raw.get(e) : __fadd_rn(g[e], raw.get(e));
        }
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      if (ring) {
        if constexpr (std::is_same<GT, __half>::value) g[e] = __half2float(hacc[e]);
      } else {
        g[e] = __fmul_rn(g[e], sa.grad_scale);
      }
    }
  } else {
    constexpr bool kExact = RB <= 2;  // R == RB: no per-slot predicate
    RawUnit<GT, VEC> raw[RB];
#pragma unroll
    for (int k = 0; k < RB; ++k) {
      if (kExact || k < R) {
        int p = first + k;
        if (p >= R) p -= R;
        if constexpr (VEC == 8 && HS != 4)
          raw[k].template load_halves<HS>(ra.g[p], i);
        else
          raw[k].load(ra.g[p], i);
      }
    }
    if (ring) {
      if constexpr (std::is_same<GT, __half>::value) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          __half acc = __ushort_as_half(raw[0].bits(e));
#pragma unroll
          for (int k = 1; k < RB; ++k)
            if (kExact || k < R) acc = __hadd(acc, __ushort_as_half(raw[k].bits(e)));
          g[e] = __half2float(acc);  // the update squares it in half precision
        }
      }
      return;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float acc = raw[0].get(e);
#pragma unroll
      for (int k = 1; k < RB; ++k)
        if (kExact || k < R) acc = __fadd_rn(acc, raw[k].get(e));
      g[e] = __fmul_rn(acc, sa.grad_scale);
    }
  }
}

// ---------------------------------------------------------------------------
// local fp32 state and the gathered output
// ---------------------------------------------------------------------------
// Plain (write-back, normally cached) accesses: the streaming hints ld.cs /
// st.cs measured 5 % slower for fp32 Adam on one GPU (0.908 -> 0.954 of the
// copy peak without them) and no faster anywhere else.
// HS: distance in elements between the first and the second four of an
// 8-element unit (4 = contiguous).
template <int VEC, int HS = 4>
__device__ __forceinline__ void load_f32(const float *p, float (&x)[VEC]) {
  if constexpr (VEC == 1) {
    x[0] = *p;
  } else if constexpr (VEC == 2) {
    const float2 t = *reinterpret_cast<const float2 *>(p);
    x[0] = t.x, x[1] = t.y;
  } else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      const float4 t = *reinterpret_cast<const float4 *>(p + q * HS);
      x[4 * q] = t.x, x[4 * q + 1] = t.y, x[4 * q + 2] = t.z, x[4 * q + 3] = t.w;
    }
  }
}
template <int VEC, int HS = 4>
__device__ __forceinline__ void store_f32(float *p, const float (&x)[VEC]) {
  if constexpr (VEC == 1) {
    *p = x[0];
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2 *>(p) = make_float2(x[0], x[1]);
  } else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q)
      *reinterpret_cast<float4 *>(p + q * HS) =
          make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
  }
}

// Store VEC updated weights at element i of every rank's gathered buffer.
// RB as in reduce_unit.
template <int VEC> struct Packed;  // VEC output elements as one store
template <typename LPT, int VEC, int RB, int HS = 4>
__device__ __forceinline__ void gather_unit(const RankArgs &ra, int R, size_t i,
                                            const float (&x)[VEC]) {
  constexpr bool kExact = RB == 1 || RB == 2;
  constexpr int kSlots = RB == 0 ? 1 : RB;
  if constexpr (std::is_same<LPT, NoLp>::value) {
    auto put = [&](int p) {
      float *dst = (float *)ra.out[p] + i;
      if constexpr (VEC == 1) {
        st_sys_4(dst, __float_as_uint(x[0]));
      } else if constexpr (VEC == 2) {
        st_sys_8(dst, make_uint2(__float_as_uint(x[0]), __float_as_uint(x[1])));
      } else {
#pragma unroll
        for (int j = 0; j < VEC / 4; ++j)
          st_sys_16(dst + HS * j,
                    make_uint4(__float_as_uint(x[4 * j]), __float_as_uint(x[4 * j + 1]),
                               __float_as_uint(x[4 * j + 2]), __float_as_uint(x[4 * j + 3])));
      }
    };
    if constexpr (RB == 0) {
      for (int p = 0; p < R; ++p) put(p);
    } else {
#pragma unroll
      for (int p = 0; p < kSlots; ++p)
        if (kExact || p < R) put(p);
    }
  } else {
    unsigned short h[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) h[e] = Bits16<LPT>::from_f32(x[e]);
    auto put = [&](int p) {
      unsigned short *dst = (unsigned short *)ra.out[p] + i;
      if constexpr (VEC == 1) {
        st_sys_2(dst, h[0]);
      } else if constexpr (VEC == 2) {
        st_sys_4(dst, h[0] | ((unsigned)h[1] << 16));
      } else if constexpr (VEC == 4) {
        st_sys_8(dst, make_uint2(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16)));
      } else if constexpr (HS == 4) {
        st_sys_16(dst, make_uint4(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16),
                                  h[4] | ((unsigned)h[5] << 16), h[6] | ((unsigned)h[7] << 16)));
      } else {
#if COCO_LOCAL16_SHUFFLE
        // the reverse exchange: lane s assembles elements 8s..8s+7 of the warp's
        // 256 from lanes 2(s&15) and 2(s&15)+1 (their first fours for s < 16,
        // their second fours otherwise) and stores 16 contiguous bytes
        static_assert(HS == 128, "the exchange is written for the 128-element half stride");
        const int t = threadIdx.x & 31;
        const unsigned A0 = h[0] | ((unsigned)h[1] << 16), A1 = h[2] | ((unsigned)h[3] << 16);
        const unsigned B0 = h[4] | ((unsigned)h[5] << 16), B1 = h[6] | ((unsigned)h[7] << 16);
        const int s0 = 2 * (t & 15), s1 = s0 + 1;
        const unsigned x0 = __shfl_sync(0xffffffffu, A0, s0), x1 = __shfl_sync(0xffffffffu, A1, s0);
        const unsigned x2 = __shfl_sync(0xffffffffu, A0, s1), x3 = __shfl_sync(0xffffffffu, A1, s1);
        const unsigned y0 = __shfl_sync(0xffffffffu, B0, s0), y1 = __shfl_sync(0xffffffffu, B1, s0);
        const unsigned y2 = __shfl_sync(0xffffffffu, B0, s1), y3 = __shfl_sync(0xffffffffu, B1, s1);
        st_sys_16(dst + 4 * t, t < 16 ? make_uint4(x0, x1, x2, x3) : make_uint4(y0, y1, y2, y3));
#else
        st_sys_8(dst, make_uint2(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16)));
        st_sys_8(dst + HS, make_uint2(h[4] | ((unsigned)h[5] << 16), h[6] | ((unsigned)h[7] << 16)));
#endif
      }
    };
    if constexpr (RB == 0) {
      for (int p = 0; p < R; ++p) put(p);
    } else {
#pragma unroll
      for (int p = 0; p < kSlots; ++p)
        if (kExact || p < R) put(p);
    }
  }
}

// ---------------------------------------------------------------------------
// the update math.  Individually rounded fp32 operations in the order the
// reference's host checks evaluate them, so that m and v match a scalar CPU
// evaluation bit for bit.
// ---------------------------------------------------------------------------
// The scalars of the update as the kernel uses them.  All but quirk_n are
// copies of kernel parameters, which live in the constant bank: arithmetic
// can take them as operands directly, so they need no registers of their own.
struct Hyper {
  float lr, b1, b2, omb1, omb2, eps, wd, d1, d2;
  double d1d, d2d, r1d, r2d;
  int variant;
  bool square_first;  // (1-b2)*(g*g) instead of ((1-b2)*g)*g
  bool nccl_m_beta2;  // forked-NCCL Adam: the first moment is updated with beta2
  float quirk_n;      // COCO_LAMB_REF_QUIRK: the element count r^2 is divided by
};

template <int OPT> __device__ __forceinline__ Hyper make_hyper(const StepArgs &sa) {
  Hyper h;
  h.lr = sa.lr, h.b1 = sa.beta1, h.b2 = sa.beta2;
  h.omb1 = sa.omb1, h.omb2 = sa.omb2;
  h.eps = sa.eps, h.wd = sa.weight_decay, h.d1 = sa.d1, h.d2 = sa.d2;
  h.d1d = sa.d1d, h.d2d = sa.d2d;
  h.r1d = sa.r1d, h.r2d = sa.r2d;
  h.variant = sa.variant;
  // test-adam.cu:16 squares first; lamb.cpp:81 multiplies left to right
  h.square_first = OPT == kAdam && sa.variant == cocoVariantDsl;
  // common_kernel.h:878 passes beta2 to the m functor (Adam); the LAMB copy at
  // :2509 passes beta1
  h.nccl_m_beta2 = OPT == kAdam;
  h.quirk_n = (float)sa.count;
  return h;
}

// test-sgd.cu:18:  w - (lr * g)
__device__ __forceinline__ float sgd_elem(const Hyper &h, float w, float g) {
  return __fsub_rn(w, __fmul_rn(h.lr, g));
}

// New moments.  overlap: b*m + (1-b)*g, b*v + ((1-b)*g)*g
// (multi-process-adam-scattered.cpp:112-116); dsl: (1-b)*(g*g)
// (test-adam.cu:16); nccl: v*b2 + gg*(1-b2) with the half-precision square
// and, for Adam, m*b2 + g*(1-b2) -- beta2 for BOTH moments
// (reduce_kernel.h:27-39, common_kernel.h:875-879); its LAMB copy uses beta1
// for m (reduce_kernel.h:391-400, common_kernel.h:2505-2511).
__device__ __forceinline__ void moments_elem(const Hyper &h, float g, float &m, float &v) {
  if (h.variant == cocoVariantNccl) {
    // g is the fp16 ring sum S0 widened to float (exactly), so S0 is recovered
    // exactly; the square is taken in half precision: (float)(S0 * S0),
    // reduce_kernel.h:29
    const __half s0 = __float2half_rn(g);
    const float gg = __half2float(__hmul(s0, s0));
    v = __fadd_rn(__fmul_rn(v, h.b2), __fmul_rn(gg, h.omb2));
    m = h.nccl_m_beta2 ? __fadd_rn(__fmul_rn(m, h.b2), __fmul_rn(g, h.omb2))
                       : __fadd_rn(__fmul_rn(m, h.b1), __fmul_rn(g, h.omb1));
  } else if (h.square_first) {
    v = __fadd_rn(__fmul_rn(h.b2, v), __fmul_rn(h.omb2, __fmul_rn(g, g)));
    m = __fadd_rn(__fmul_rn(h.b1, m), __fmul_rn(h.omb1, g));
  } else {
    m = __fadd_rn(__fmul_rn(h.b1, m), __fmul_rn(h.omb1, g));
    v = __fadd_rn(__fmul_rn(h.b2, v), __fmul_rn(__fmul_rn(h.omb2, g), g));
  }
}

// float(double(x) / d), exactly, at the price of one double multiply in the
// common case.  q = x * (1/d) is within a few units in the last place of the
// true quotient; narrowing q to float gives the same result as narrowing the
// true quotient unless a rounding boundary of the float format (the midpoint
// between two floats: dropped 29 bits == 0x10000000) lies within that error,
// or the result leaves the normal float range.  `risky` collects those rare
// cases so that ONE branch per batch of elements redoes them with the IEEE
// division (a branch per element would serialise the elements' dependency
// chains, and this kernel is latency-bound on them).
__device__ __forceinline__ float div_narrow_fast(float x, double rcp_d, bool &risky) {
  const double q = __dmul_rn((double)x, rcp_d);
  const unsigned lo = (unsigned)__double2loint(q);
  const unsigned ex = ((unsigned)__double2hiint(q) >> 20) & 0x7ffu;
  risky = risky || ((lo & 0x1fffffffu) - 0x0ffffff0u) <= 0x20u || ex <= 1023u - 126u ||
          ex >= 1023u + 127u;
  return __double2float_rn(q);
}

// m^ = m/d1, v^ = v/d2 for a batch of elements.  The bias-corrected form
// divides by the DOUBLE 1 - beta^t and narrows, exactly as the reference's
// host check does (multi-process-adam-scattered.cpp:118-119: pow() promotes to
// double), so the result matches a CPU evaluation bit for bit; the other
// forms divide by a float (test-adam.cu:21,29; reduce_kernel.h:33-47).
template <int V>
__device__ __forceinline__ void corrected_moments(const Hyper &h, const float (&m)[V],
                                                  const float (&v)[V], float (&m_)[V],
                                                  float (&v_)[V]) {
  if (h.variant == cocoVariantOverlap) {
    bool risky = false;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      m_[e] = div_narrow_fast(m[e], h.r1d, risky);
      v_[e] = div_narrow_fast(v[e], h.r2d, risky);
    }
    if (risky) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        m_[e] = __double2float_rn(__ddiv_rn((double)m[e], h.d1d));
        v_[e] = __double2float_rn(__ddiv_rn((double)v[e], h.d2d));
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      m_[e] = __fdiv_rn(m[e], h.d1);
      v_[e] = __fdiv_rn(v[e], h.d2);
    }
  }
}

__device__ __forceinline__ float adam_elem(const Hyper &h, float w, float m_, float v_) {
  if (h.variant == cocoVariantDsl)  // test-adam.cu:38:  w - (lr*m_)/v_
    return __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, m_), v_));
  // overlap (sample :121): lr*m_/(sqrt(v_)+eps); nccl (reduce_kernel.h:48-62) is
  // the same expression with eps == 0.
  return __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, m_), __fadd_rn(__fsqrt_rn(v_), h.eps)));
}

// r = m^/(sqrt(v^)+eps) + lambda*w  (sample :416; lamb.cpp:84 with eps == 0)
__device__ __forceinline__ float lamb_r_elem(const Hyper &h, float w, float m_, float v_) {
  return __fadd_rn(__fdiv_rn(m_, __fadd_rn(__fsqrt_rn(v_), h.eps)), __fmul_rn(h.wd, w));
}

// ---------------------------------------------------------------------------
// one unit of the data phase
// ---------------------------------------------------------------------------
// Everything after the reduction: SGD and Adam: the whole update and the
// all-gather of the unit.  LAMB phase 1: moments + norm partials only.
// g: reduced, scaled gradient.  NVLS: gather through the NVSwitch multicast
// address.  All loads of the unit are issued first; the arithmetic then runs
// in batches of four elements so that only four corrected moment pairs are
// live at a time (an 8-element unit otherwise spills).
template <typename LPT, int V>
__device__ __forceinline__ void nvls_gather(const RankArgs &ra, int R, size_t i,
                                            const float (&x)[V]);

template <int OPT, typename LPT, int VEC, int RB, int HS = 4, bool NVLS = false>
__device__ __forceinline__ void apply_unit(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                           size_t lo, size_t i, const float (&g)[VEC],
                                           double &sum_w2, double &sum_r2) {
#if COCO_CHECKED
  // Checked build (python -m coconet_b200.build --checked): every unit proves
  // that it lies inside the rank's slice and, for vector units, that its
  // addresses are 16-byte aligned; a unit that does not is skipped and the
  // status word says so (cocoInternalError), instead of a stray access.
  {
    const size_t S_ = (sa.count + sa.world - 1) / sa.world;
    const size_t lo_ = (size_t)ra.rank * S_ < sa.count ? (size_t)ra.rank * S_ : sa.count;
    const size_t hi_ = lo_ + S_ < sa.count ? lo_ + S_ : sa.count;
    const size_t last = i + (VEC > 4 ? HS + 4 : VEC);  // one past the unit's last element
    const bool in_slice = (sa.flags & kFlagScattered) || (i >= lo_ && last <= hi_);
    const bool aligned = VEC < 4 || ((((uintptr_t)(ra.w + i)) & 15u) == 0 &&
                                     (OPT == kSGD || ((((uintptr_t)(ra.m + (i - lo))) & 15u) == 0 &&
                                                      (((uintptr_t)(ra.v + (i - lo))) & 15u) == 0)));
    if (!in_slice || !aligned) {
      record_status(ra.flags[ra.rank], cocoInternalError, ra.rank, kPhaseCheck, -1, sa.seq);
      return;
    }
  }
#endif
  float w[VEC];
  load_f32<VEC, HS>(ra.w + i, w);
  if constexpr (OPT == kSGD) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) w[e] = sgd_elem(h, w[e], g[e]);
  } else {
    float m[VEC], v[VEC];
    load_f32<VEC, HS>(ra.m + (i - lo), m);
    load_f32<VEC, HS>(ra.v + (i - lo), v);
    constexpr int B = VEC < 4 ? VEC : 4;
#pragma unroll
    for (int q = 0; q < VEC; q += B) {
      float mb[B], vb[B], m_[B], v_[B];
#pragma unroll
      for (int e = 0; e < B; ++e) {
        mb[e] = m[q + e], vb[e] = v[q + e];
        moments_elem(h, g[q + e], mb[e], vb[e]);
        m[q + e] = mb[e], v[q + e] = vb[e];
      }
      corrected_moments<B>(h, mb, vb, m_, v_);
#pragma unroll
      for (int e = 0; e < B; ++e) {
        if constexpr (OPT == kAdam) {
          w[q + e] = adam_elem(h, w[q + e], m_[e], v_[e]);
        } else {
          const float r = lamb_r_elem(h, w[q + e], m_[e], v_[e]);
          if (sa.flags & COCO_LAMB_REF_QUIRK) {
            sum_r2 += (double)__fdiv_rn(__fmul_rn(r, r), h.quirk_n);
            sum_w2 += (double)__fmul_rn(w[q + e], w[q + e]);
          } else {
            sum_r2 += (double)r * (double)r;
            sum_w2 += (double)w[q + e] * (double)w[q + e];
          }
        }
      }
    }
    store_f32<VEC, HS>(ra.m + (i - lo), m);
    store_f32<VEC, HS>(ra.v + (i - lo), v);
  }
  if constexpr (OPT != kLAMB) {
    if constexpr (!std::is_same<LPT, NoLp>::value) store_f32<VEC, HS>(ra.w + i, w);
    if constexpr (NVLS)
      nvls_gather<LPT, VEC>(ra, sa.world, i, w);
    else
      gather_unit<LPT, VEC, RB, HS>(ra, sa.world, i, w);
  }
}

// One unit of the register-staged data phase: reduce, then apply.
template <int OPT, typename GT, typename LPT, int VEC, int RB, int HS = 4>
__device__ __forceinline__ void step_unit(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                          size_t lo, size_t i, double &sum_w2, double &sum_r2) {
  float g[VEC];
  reduce_unit<GT, VEC, RB, HS>(ra, sa, i, g);
  apply_unit<OPT, LPT, VEC, RB, HS>(ra, sa, h, lo, i, g, sum_w2, sum_r2);
}

// LAMB phase 2: recompute r from the stored moments, apply the scaled step.
template <typename LPT, int VEC, int RB, int HS = 4>
__device__ __forceinline__ void lamb_apply_unit(const RankArgs &ra, const StepArgs &sa,
                                                const Hyper &h, size_t lo, size_t i,
                                                float lr_scale) {
  float w[VEC], m[VEC], v[VEC];
  load_f32<VEC, HS>(ra.w + i, w);
  load_f32<VEC, HS>(ra.m + (i - lo), m);
  load_f32<VEC, HS>(ra.v + (i - lo), v);
  float m_[VEC], v_[VEC];
  corrected_moments<VEC>(h, m, v, m_, v_);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    const float r = lamb_r_elem(h, w[e], m_[e], v_[e]);
    w[e] = __fsub_rn(w[e], __fmul_rn(lr_scale, r));  // sample :434-435
  }
  if constexpr (!std::is_same<LPT, NoLp>::value) store_f32<VEC, HS>(ra.w + i, w);
  gather_unit<LPT, VEC, RB, HS>(ra, sa.world, i, w);
}

// ---------------------------------------------------------------------------
// NVLS path: the reduce-scatter is ONE multimem.ld_reduce per 16 bytes (the
// NVSwitch fetches the unit from all R gradient buffers and adds them on the
// way), the all-gather ONE multimem.st (the switch replicates it to all R
// output buffers).  Per GPU and direction this moves (1 + 1/R) * N * s bytes
// instead of 2 * (R-1)/R * N * s.  The order of the in-switch sum is not the
// rank order of the P2P path, and 16-bit sums are accumulated in fp32 but
// delivered rounded to 16 bits, so results agree with the P2P path only to
// within the stated tolerances, not bit for bit.
// ---------------------------------------------------------------------------
// ld_reduce returns the 16 raw bytes of the reduced unit (so that several can
// be kept in flight cheaply, 4 registers each); unpack converts them.
template <typename GT> struct Multimem;
template <> struct Multimem<float> {
  static constexpr int kN = 4;
  static __device__ __forceinline__ uint4 ld_reduce(const void *p) {
    float x[4];
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3])
                 : "l"(p));
    return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]),
                      __float_as_uint(x[3]));
  }
  static __device__ __forceinline__ void unpack(const uint4 &q, float (&x)[4]) {
    x[0] = __uint_as_float(q.x), x[1] = __uint_as_float(q.y);
    x[2] = __uint_as_float(q.z), x[3] = __uint_as_float(q.w);
  }
};
template <typename T16> struct Multimem16 {
  static constexpr int kN = 8;
  static __device__ __forceinline__ void unpack(const uint4 &q, float (&x)[8]) {
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      x[2 * k] = Bits16<T16>::to_f32((unsigned short)(w[k] & 0xffffu));
      x[2 * k + 1] = Bits16<T16>::to_f32((unsigned short)(w[k] >> 16));
    }
  }
};
template <> struct Multimem<__half> : Multimem16<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void *p) {
    uint4 q;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
        : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
        : "l"(p));
    return q;
  }
};
template <> struct Multimem<__nv_bfloat16> : Multimem16<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void *p) {
    uint4 q;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
        : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
        : "l"(p));
    return q;
  }
};
// 16 bytes to every rank's copy (typed .f32 only to name the register class;
// a store performs no arithmetic on the bits).
__device__ __forceinline__ void multimem_st_16(void *p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

template <typename LPT, int V>
__device__ __forceinline__ void nvls_gather(const RankArgs &ra, int R, size_t i,
                                            const float (&x)[V]) {
  if constexpr (std::is_same<LPT, NoLp>::value) {
#pragma unroll
    for (int j = 0; j < V / 4; ++j)
      multimem_st_16((float *)ra.mc_out + i + 4 * j,
                     make_uint4(__float_as_uint(x[4 * j]), __float_as_uint(x[4 * j + 1]),
                                __float_as_uint(x[4 * j + 2]), __float_as_uint(x[4 * j + 3])));
  } else {
    unsigned short h[V];
#pragma unroll
    for (int e = 0; e < V; ++e) h[e] = Bits16<LPT>::from_f32(x[e]);
    if constexpr (V == 8) {
      multimem_st_16((unsigned short *)ra.mc_out + i,
                     make_uint4(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16),
                                h[4] | ((unsigned)h[5] << 16), h[6] | ((unsigned)h[7] << 16)));
    } else {
      // 4 low-precision elements are only 8 bytes: plain peer stores
      gather_unit<LPT, V, 0>(ra, R, i, x);
    }
  }
}

// The in-switch reduction has a long round trip (the switch collects the unit
// from all R GPUs before it answers), so each thread keeps kNvlsDepth reduced
// units in flight: the loads of the next passes are issued before the current
// unit is worked on.  One ld_reduce per thread and pass reached 0.55 of the
// link rate at eight ranks.
#ifndef COCO_NVLS_DEPTH
#define COCO_NVLS_DEPTH 3
#endif
constexpr int kNvlsDepth = COCO_NVLS_DEPTH;

// Measured (mixed-precision Adam, 334 M elements; 0 = equal shares by grid stride): at two
// GPUs 1.166 -> 1.141 ms peer to peer and 1.758 -> 1.692 ms through the switch, fp32 Adam on
// 2^26 elements 0.452 -> 0.440 ms, the CTAs' finishing times 6-9 % apart before and 2-3 %
// after; at four GPUs, where the links are the bound whoever uses them, 1.632 -> 1.613 ms.
#ifndef COCO_MULTI_DYNAMIC
#define COCO_MULTI_DYNAMIC 1
#endif
#ifndef COCO_DYNAMIC_PASSES
#define COCO_DYNAMIC_PASSES 8
#endif
// Hands the units [0, nunits) out warp by warp from a counter in chunks of up to
// COCO_DYNAMIC_PASSES passes of a warp (32 units each), instead of by grid stride: the
// CTAs of a rank do not move their shares over the links at the same rate, and under
// equal shares the step ends with the slowest.  A chunk is at most a quarter of a warp's
// even share, down to one pass, so that a small message still spreads over all warps
// (with 8-pass chunks a 1 Mi-element step at two GPUs kept 512 warps busy for 8 passes
// each: 65 us against 43).  Lane 0 asks for the chunk after next when the warp enters a
// chunk, so the atomic's round trip is over long before its result is needed.  next()
// gives the warp's next unit (this lane's), or nunits when there is none.
struct WarpWork {
  unsigned *counter;
  size_t nunits, nchunks;
  size_t base;        // first unit of the current chunk
  unsigned pending;   // lane 0: number of the chunk after the current one
  int pass, passes, lane;
  bool done;          // no chunk is left (the same in every lane)
  __device__ __forceinline__ void start(unsigned *c, size_t n) {
    counter = c, nunits = n;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    const size_t quarter_share = n / (warps * 32 * 4);  // in passes
    passes = quarter_share >= COCO_DYNAMIC_PASSES ? COCO_DYNAMIC_PASSES
             : quarter_share >= 1 ? (int)quarter_share : 1;
    nchunks = (n + (size_t)(32 * passes) - 1) / (size_t)(32 * passes);
    lane = threadIdx.x & 31;
    pending = 0;
    if (lane == 0) pending = atomicAdd(counter, 1u);
    pass = passes;  // the first next() enters the first chunk
    base = 0;
    done = false;
  }
  __device__ __forceinline__ size_t next() {
    if (pass == passes) {
      const size_t c = __shfl_sync(0xffffffffu, pending, 0);
      if (c >= nchunks) {
        done = true;  // and stays so: pass is not reset
        return nunits;
      }
      if (lane == 0) pending = atomicAdd(counter, 1u);
      base = c * (size_t)(32 * passes);
      pass = 0;
    }
    const size_t u = base + (size_t)pass * 32 + lane;
    ++pass;
    return u < nunits ? u : nunits;
  }
};

// PHASE 0: SGD / Adam step or LAMB moments; PHASE 1: LAMB apply.
template <int OPT, typename GT, typename LPT, int PHASE>
__device__ __forceinline__ void nvls_phase(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                           size_t lo, size_t nunits, size_t tid, size_t nth,
                                           double &sum_w2, double &sum_r2, float lr_scale) {
  constexpr int V = Multimem<GT>::kN;
#if COCO_MULTI_DYNAMIC
  if constexpr (PHASE == 0 && OPT != kLAMB) {  // LAMB's norms are summed in the order of a fixed assignment
    const GT *src = (const GT *)ra.mc_g + lo;
    WarpWork ww;
    ww.start(&ra.flags[ra.rank]->work_next, nunits);
    uint4 raw[kNvlsDepth];
    size_t ids[kNvlsDepth];
#pragma unroll
    for (int k = 0; k < kNvlsDepth; ++k) {
      ids[k] = ww.next();
      if (ids[k] < nunits) raw[k] = Multimem<GT>::ld_reduce(src + ids[k] * V);
    }
    for (;;) {
      const uint4 cur = raw[0];
      const size_t u = ids[0];
#pragma unroll
      for (int k = 0; k + 1 < kNvlsDepth; ++k) raw[k] = raw[k + 1], ids[k] = ids[k + 1];
      const size_t un = ww.next();
      ids[kNvlsDepth - 1] = un;
      if (un < nunits) raw[kNvlsDepth - 1] = Multimem<GT>::ld_reduce(src + un * V);
      if (u < nunits) {
        float g[V];
        Multimem<GT>::unpack(cur, g);
#pragma unroll
        for (int e = 0; e < V; ++e) g[e] = __fmul_rn(g[e], sa.grad_scale);
        apply_unit<OPT, LPT, V, 0, 4, true>(ra, sa, h, lo, lo + u * V, g, sum_w2, sum_r2);
      }
      // units come in rising order, so nothing valid follows once the queue is empty
      // and this warp's current units are past the end
      if (ww.done && __all_sync(0xffffffffu, u >= nunits)) break;
    }
    return;
  }
#endif
  if constexpr (PHASE == 0) {
    const GT *src = (const GT *)ra.mc_g + lo;
    uint4 raw[kNvlsDepth];
#pragma unroll
    for (int k = 0; k < kNvlsDepth; ++k) {
      const size_t un = tid + (size_t)k * nth;
      if (un < nunits) raw[k] = Multimem<GT>::ld_reduce(src + un * V);
    }
    for (size_t u = tid; u < nunits; u += nth) {
      const uint4 cur = raw[0];
#pragma unroll
      for (int k = 0; k + 1 < kNvlsDepth; ++k) raw[k] = raw[k + 1];
      const size_t un = u + (size_t)kNvlsDepth * nth;
      if (un < nunits) raw[kNvlsDepth - 1] = Multimem<GT>::ld_reduce(src + un * V);
      float g[V];
      Multimem<GT>::unpack(cur, g);
#pragma unroll
      for (int e = 0; e < V; ++e) g[e] = __fmul_rn(g[e], sa.grad_scale);
      apply_unit<OPT, LPT, V, 0, 4, true>(ra, sa, h, lo, lo + u * V, g, sum_w2, sum_r2);
    }
  } else {
    for (size_t u = tid; u < nunits; u += nth) {
      const size_t i = lo + u * V;
      float w[V], m[V], v[V], m_[V], v_[V];
      load_f32<V>(ra.w + i, w);
      load_f32<V>(ra.m + (i - lo), m);
      load_f32<V>(ra.v + (i - lo), v);
      corrected_moments<V>(h, m, v, m_, v_);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float r = lamb_r_elem(h, w[e], m_[e], v_[e]);
        w[e] = __fsub_rn(w[e], __fmul_rn(lr_scale, r));
      }
      if constexpr (!std::is_same<LPT, NoLp>::value) store_f32<V>(ra.w + i, w);
      nvls_gather<LPT, V>(ra, sa.world, i, w);
    }
  }
}

// Grid-stride loops of the direct (register-staged) path over the elements
// [first, first + nelems), nelems a multiple of 4.
//
// Unit size: 4 elements per thread and pass, except on a single rank for
// 16-bit gradients and for SGD, which take 8 (with peers in flight the
// registers only allow 4: 8 measured 10 % slower at two ranks; fp32 Adam on
// one rank is 5 % faster with 4).  The 8 elements of a thread are NOT
// consecutive: a warp's 32 units are 256 consecutive elements, of which lane
// t takes 4t..4t+3 and 128+4t..128+4t+3, so that every load and store of the
// warp covers one contiguous run of whole 32-byte sectors (consecutive
// elements per lane made every fp32 access touch half sectors: 1.3 % slower).
constexpr int kHalfStride = 128;
// COCO_DIRECT_VEC8 (build-time experiment switch): 8-element units for 16-bit
// gradients at every world size, 1 = halves 128 elements apart (8-byte peer
// accesses, whole sectors of the fp32 state), 2 = 8 consecutive elements per
// lane (16-byte peer accesses).
#ifndef COCO_DIRECT_VEC8
#define COCO_DIRECT_VEC8 0
#endif
template <int OPT, typename GT, int RB> struct DirectVec {
  static constexpr int kVec =
      ((RB == 1 && (GradTraits<GT>::kIs16 || OPT == kSGD)) ||
       (COCO_DIRECT_VEC8 != 0 && RB >= 2 && GradTraits<GT>::kIs16)) ? 8 : 4;
  // distance between the two fours of an 8-element unit
  static constexpr int kStride = (RB == 1 || COCO_DIRECT_VEC8 == 1) ? kHalfStride : 4;
};

template <int OPT, typename GT, typename LPT, int RB>
__device__ __forceinline__ void direct_step(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                            size_t lo, size_t first, size_t nelems, size_t tid,
                                            size_t nth, double &sum_w2, double &sum_r2) {
  constexpr int VEC = DirectVec<OPT, GT, RB>::kVec;
  const size_t nunits = nelems / VEC;
  if constexpr (VEC == 8) {
    if constexpr (DirectVec<OPT, GT, RB>::kStride == kHalfStride) {
      // tid and nth are multiples of the warp size apart from the lane, so
      // u & 31 is the lane and u - lane the warp's first unit
      const size_t nfull = nunits / 32 * 32;
      for (size_t u = tid; u < nfull; u += nth)
        step_unit<OPT, GT, LPT, 8, RB, kHalfStride>(ra, sa, h, lo, first + u * 8 - (u & 31) * 4,
                                                    sum_w2, sum_r2);
      for (size_t u = nfull + tid; u < nunits; u += nth)  // last, partial warp: consecutive
        step_unit<OPT, GT, LPT, 8, RB>(ra, sa, h, lo, first + u * 8, sum_w2, sum_r2);
    } else {
      for (size_t u = tid; u < nunits; u += nth)
        step_unit<OPT, GT, LPT, 8, RB>(ra, sa, h, lo, first + u * 8, sum_w2, sum_r2);
    }
    // up to one 4-element unit may remain
    if ((nelems & 4) && tid == 0)
      step_unit<OPT, GT, LPT, 4, RB>(ra, sa, h, lo, first + nunits * 8, sum_w2, sum_r2);
  } else {
    for (size_t u = tid; u < nunits; u += nth)
      step_unit<OPT, GT, LPT, VEC, RB>(ra, sa, h, lo, first + u * VEC, sum_w2, sum_r2);
  }
}
#if COCO_MULTI_DYNAMIC
// The flat slice of a multi-rank SGD / Adam step with the units handed out warp by warp.
template <int OPT, typename GT, typename LPT, int RB>
__device__ __forceinline__ void direct_step_dynamic(const RankArgs &ra, const StepArgs &sa,
                                                    const Hyper &h, size_t lo, size_t first,
                                                    size_t nelems, size_t tid, size_t nth,
                                                    double &sum_w2, double &sum_r2) {
  constexpr int VEC = DirectVec<OPT, GT, RB>::kVec;
  if constexpr (VEC == 4 && OPT != kLAMB) {
    const size_t nunits = nelems / VEC;
    WarpWork ww;
    ww.start(&ra.flags[ra.rank]->work_next, nunits);
    for (;;) {
      const size_t u = ww.next();
      if (ww.done) break;
      if (u < nunits) step_unit<OPT, GT, LPT, VEC, RB>(ra, sa, h, lo, first + u * VEC, sum_w2, sum_r2);
    }
  } else {
    direct_step<OPT, GT, LPT, RB>(ra, sa, h, lo, first, nelems, tid, nth, sum_w2, sum_r2);
  }
}
#define COCO_DIRECT_STEP direct_step_dynamic
#else
#define COCO_DIRECT_STEP direct_step
#endif

template <typename GT, typename LPT, int RB>
__device__ __forceinline__ void direct_apply(const RankArgs &ra, const StepArgs &sa,
                                             const Hyper &h, size_t lo, size_t first,
                                             size_t nelems, size_t tid, size_t nth,
                                             float lr_scale) {
  constexpr int VEC = DirectVec<kLAMB, GT, RB>::kVec;
  const size_t nunits = nelems / VEC;
  if constexpr (VEC == 8) {
    const size_t nfull = nunits / 32 * 32;
    for (size_t u = tid; u < nfull; u += nth)
      lamb_apply_unit<LPT, 8, RB, kHalfStride>(ra, sa, h, lo, first + u * 8 - (u & 31) * 4, lr_scale);
    for (size_t u = nfull + tid; u < nunits; u += nth)
      lamb_apply_unit<LPT, 8, RB>(ra, sa, h, lo, first + u * 8, lr_scale);
    if ((nelems & 4) && tid == 0)
      lamb_apply_unit<LPT, 4, RB>(ra, sa, h, lo, first + nunits * 8, lr_scale);
  } else {
    for (size_t u = tid; u < nunits; u += nth)
      lamb_apply_unit<LPT, VEC, RB>(ra, sa, h, lo, first + u * VEC, lr_scale);
  }
}

__device__ __forceinline__ double warp_sum(double x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
  return x;
}

// ---------------------------------------------------------------------------
// warp rings: every warp stages the gradient tiles it is going to reduce in
// shared memory with bulk asynchronous copies (the TMA engine, 1-D form), a
// few tiles ahead of the math.  Latency of the peers' memory (2-3 us over
// NVLink) is then covered by bytes in flight in shared memory, of which there
// is plenty, instead of by registers, of which there are not.
//
//   tile   = 32 lanes x 16 bytes of gradient per rank (256 16-bit or 128 fp32
//            elements); stage = the R ranks' tiles, R x 512 bytes
//   ring   = D stages per warp, one mbarrier each; lane 0 issues the R copies
//            of a stage, all lanes wait for its barrier, read their 16 bytes of
//            every rank's tile, and lane 0 refills the stage for tile j + D
//            right away -- before the update math and the stores of tile j
//
// Warps never wait for one another (no CTA-wide barrier in the loop).  No
// cluster, no multicast: each warp fetches its own tiles, local or remote.
// Every wait is bounded; a warp that gives up still waits (bounded) for the
// copies it has in flight before the CTA may retire.
// ---------------------------------------------------------------------------
constexpr int kRingMaxStages = 4;
constexpr int kRingMaxWarps = 16;
constexpr unsigned kRingTileBytes = 512;  // 32 lanes x 16 bytes

__device__ __forceinline__ unsigned smem_u32(const void *p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded: gives up after timeout_ns (checked every 256 probes) or 2^26 probes.
__device__ __noinline__ bool mbar_wait_slow(unsigned long long *bar, unsigned parity,
                                            unsigned long long timeout_ns) {
  const unsigned long long t0 = globaltimer_ns();
  for (unsigned spin = 1; spin < (1u << 26); ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u && globaltimer_ns() - t0 > timeout_ns) return false;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity,
                                          unsigned long long timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, timeout_ns);
}
// global -> shared bulk copy; src, dst and bytes are multiples of 16.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, unsigned bytes,
                                          unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint4 ld_shared_16(const void *p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(smem_u32(p)));
  return v;
}

// Sum of the R ranks' 16 bytes of this lane, from one stage of the ring.
template <typename GT, int VEC>
__device__ __forceinline__ void ring_reduce(const unsigned char *stage, int lane,
                                            const RankArgs &ra, const StepArgs &sa,
                                            float (&g)[VEC]) {
  const int R = sa.world;
  const unsigned char *mine = stage + lane * 16;
  if constexpr (std::is_same<GT, __half>::value) {
    if (sa.variant == cocoVariantNccl) {
      // the forked-NCCL variant: fp16 sum in ring order, starting behind the owner
      __half acc[VEC];
      for (int k = 0; k < R; ++k) {
        int p = ra.rank + 1 + k;
        if (p >= R) p -= R;
        const uint4 q = ld_shared_16(mine + p * kRingTileBytes);
        const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const __half x = __ushort_as_half((unsigned short)((e & 1) ? (w[e >> 1] >> 16)
                                                                      : (w[e >> 1] & 0xffffu)));
          acc[e] = k == 0 ? x : __hadd(acc[e], x);
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) g[e] = __half2float(acc[e]);
      return;
    }
  }
  for (int p = 0; p < R; ++p) {  // rank order 0..R-1, fp32
    const uint4 q = ld_shared_16(mine + p * kRingTileBytes);
    float x[VEC];
    if constexpr (GradTraits<GT>::kIs16) {
      const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        x[e] = Bits16<GT>::to_f32((unsigned short)((e & 1) ? (w[e >> 1] >> 16)
                                                           : (w[e >> 1] & 0xffffu)));
    } else {
      x[0] = __uint_as_float(q.x), x[1] = __uint_as_float(q.y);
      x[2] = __uint_as_float(q.z), x[3] = __uint_as_float(q.w);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = p == 0 ? x[e] : __fadd_rn(g[e], x[e]);
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) g[e] = __fmul_rn(g[e], sa.grad_scale);
}

// This warp's share of the slice's full tiles: whole SGD / Adam step, or LAMB
// moments + norm partials.  `ring` is the warp's D stages, `bars` its D
// barriers (initialised, phase 0).  Returns false if a copy did not land in
// time (warp-uniform).
template <int OPT, typename GT, typename LPT>
__device__ __forceinline__ bool ring_step(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                          size_t lo, size_t ntiles, unsigned char *ring,
                                          unsigned long long *bars, double &sum_w2,
                                          double &sum_r2) {
  constexpr int VEC = 16 / (int)sizeof(GT);
  constexpr int TE = 32 * VEC;
  const int R = sa.world;
  const unsigned D = (unsigned)sa.pipe_stages;
  const int lane = threadIdx.x & 31;
  const size_t nwarp = blockDim.x >> 5;
  const size_t gw = (size_t)blockIdx.x * nwarp + (threadIdx.x >> 5);
  const size_t GW = (size_t)gridDim.x * nwarp;
  const size_t mine = ntiles > gw ? (ntiles - gw + GW - 1) / GW : 0;
  const unsigned stage_bytes = (unsigned)R * kRingTileBytes;

  auto issue = [&](size_t j) {  // lane 0 only
    const unsigned s = (unsigned)(j % D);
    const size_t e0 = lo + (gw + j * GW) * (size_t)TE;
    unsigned char *st = ring + (size_t)s * stage_bytes;
    mbar_expect_tx(&bars[s], stage_bytes);
    for (int p = 0; p < R; ++p)
      bulk_load(st + p * kRingTileBytes, (const GT *)ra.g[p] + e0, kRingTileBytes, &bars[s]);
  };

  if (lane == 0)
    for (size_t j = 0; j < mine && j < D; ++j) issue(j);

  bool ok = true;
  size_t j = 0;
  for (; j < mine; ++j) {
    const unsigned s = (unsigned)(j % D);
    const bool landed = mbar_wait(&bars[s], (unsigned)((j / D) & 1u), sa.timeout_ns);
    if (!__all_sync(0xffffffffu, landed)) {
      ok = false;
      break;
    }
    float g[VEC];
    ring_reduce<GT, VEC>(ring + (size_t)s * stage_bytes, lane, ra, sa, g);
    __syncwarp();  // every lane has read stage s: refill it for tile j + D
    if (lane == 0 && j + D < mine) issue(j + D);
    const size_t i = lo + (gw + j * GW) * (size_t)TE + (size_t)lane * VEC;
    apply_unit<OPT, LPT, VEC, 0, 4>(ra, sa, h, lo, i, g, sum_w2, sum_r2);
  }
  if (!ok && lane == 0) {
    // Copies may still be in flight into this warp's ring: give every issued
    // tile one more bounded wait before the CTA is allowed to retire.
    const size_t issued = mine < j + D ? mine : j + D;
    for (size_t k = j; k < issued; ++k)
      mbar_wait(&bars[k % D], (unsigned)((k / D) & 1u), sa.timeout_ns);
  }
  __syncwarp();
  return ok;
}

// LAMB's second phase over the elements the rings covered: 16 bytes of
// gathered output per lane and store.
template <typename GT, typename LPT>
__device__ __forceinline__ void ring_apply(const RankArgs &ra, const StepArgs &sa, const Hyper &h,
                                           size_t lo, size_t nelems, size_t tid, size_t nth,
                                           float lr_scale) {
  constexpr int VEC = std::is_same<LPT, NoLp>::value ? 4 : 8;
  const size_t nunits = nelems / VEC;  // nelems is a multiple of 128
  for (size_t u = tid; u < nunits; u += nth)
    lamb_apply_unit<LPT, VEC, 0>(ra, sa, h, lo, lo + u * VEC, lr_scale);
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
// PATH selects the data path at compile time so that each gets a register
// allocation of its own (with all three in one kernel the peer-to-peer loop
// spilled 376 bytes and lost 6 %): kPathDirect = register-staged peer loads
// and stores for world sizes 2..8, kPathLocal = the same for world size 1
// (wider units), kPathNvls = NVSwitch multimem, kPathRing = gradients staged
// in per-warp shared-memory rings by bulk copies (any world size),
// kPathSegments .. kPathSegments + 3 = peer-to-peer over a list of tensors
// (scattered calls), one kernel per world-size bucket.
// Every path ends with the same scalar loop for what it does not cover.
enum : int { kPathDirect = 0, kPathNvls = 1, kPathRing = 2, kPathLocal = 3, kPathSegments = 4 };

// Threads per CTA a path's kernel is compiled for (two CTAs per SM).
template <int PATH, typename GT> struct BlockThreads {
  static constexpr int value =
      PATH == kPathLocal ? (GradTraits<GT>::kIs16 ? COCO_LOCAL16_THREADS : COCO_LOCAL32_THREADS)
      : PATH >= kPathSegments ? COCO_SEG_THREADS
      : GradTraits<GT>::kIs16 ? COCO_MULTI16_THREADS : COCO_MULTI32_THREADS;
};

template <int OPT, typename GT, typename LPT, int PATH>
__global__ void __launch_bounds__((BlockThreads<PATH, GT>::value), 2)
    fused_step_kernel(const __grid_constant__ StepArgs sa, const __grid_constant__ RankArgs one,
                      const RankArgs *__restrict__ table) {
  extern __shared__ __align__(128) unsigned char ring_smem[];
  __shared__ RankArgs ra;
  __shared__ int s_ok;
  __shared__ int s_last_cta;
  __shared__ float s_lr_scale;
  __shared__ double s_red[2][16];
  __shared__ __align__(8) unsigned long long s_ring_bar[kRingMaxWarps][kRingMaxStages];

  {  // this (virtual) rank's pointers -> shared memory
    const RankArgs *src = table ? table + blockIdx.y : &one;
    const int *s = reinterpret_cast<const int *>(src);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
    if constexpr (PATH == kPathRing) {
      if ((threadIdx.x & 31) == 0) {  // every warp's own barriers, one arrival each
        for (int k = 0; k < sa.pipe_stages; ++k) mbar_init(&s_ring_bar[threadIdx.x >> 5][k], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      }
    }
  }
  __syncthreads();

  const int R = sa.world;
  const int rank = ra.rank;
  FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;

  // ---- start barrier ------------------------------------------------------
  if (R > 1) {
    if (threadIdx.x < 32) {
      if (blockIdx.x == 0)
        warp_signal_peers(ra, R, rank, seq, [](FlagPage *f) { return f->arrive; });
      const int late = warp_wait_peers(me->arrive, R, rank, seq, sa.timeout_ns);
      if (late >= 0 && threadIdx.x == 0) {
        record_status(me, cocoTimeout, rank, kPhaseStart, late, seq);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  bool ok = s_ok != 0;
  const bool started_ok = ok;
  // CTA 0 leaves its timer readings in the flag page (cocoLastPhaseTimes)
  const bool stamps = blockIdx.x == 0 && threadIdx.x == 0;
  if (stamps) {
    const unsigned long long t = globaltimer_ns();
    me->phase_ns[0] = me->phase_ns[1] = me->phase_ns[2] = t;
  }

  // ---- slice of this rank (same arithmetic as cocoSliceBounds) -------------
  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  constexpr int VEC = GradTraits<GT>::kVec;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const Hyper h = make_hyper<OPT>(sa);

  bool seg_norm_ok = true;  // scattered LAMB: the norm exchange completed
  if constexpr (PATH >= kPathSegments) {
    // Scattered call: the slice is a sequence of pieces of different tensors.
    // The pieces are cut into chunks of 2^chunk_shift elements, numbered
    // through all pieces (Segment::chunk0 = a piece's first chunk).  Every CTA
    // takes chunks q = its number, + number of CTAs, ..., and runs the
    // ordinary peer-to-peer loop on a chunk with all its threads (adjacent
    // warps on adjacent memory, like the flat call).  The bookkeeping is per
    // warp, so the walk has no CTA barrier: every warp finds a chunk's piece
    // by bisection over a shared-memory copy of the first-chunk numbers and
    // keeps the piece's pointers in its own RankArgs in shared memory.  The
    // NEXT chunk's piece is looked up before the current chunk's data loop and,
    // when it is another piece, its descriptor is fetched then (one 8-byte word
    // per lane, held in a register across the loop), so that the dependent
    // loads of the lookup overlap the data loop instead of standing between
    // two chunks.  The work is balanced to within one chunk per CTA whatever
    // the tensors' sizes.  (Walking the pieces one after the other with the
    // whole grid made every piece end in a partly filled pass and a grid-wide
    // drain: +17 % over the flat call for Adam, +43 % for LAMB, on a
    // BERT-large-shaped list of 398 tensors; a walk with the lookup between the
    // chunks: +17 to +26 % and +32 %.)
    // SGD and Adam: one walk.  LAMB: a walk for the moments that leaves every
    // chunk's partial norms (one pair per warp) in a table, the per-tensor sums
    // and their exchange between the ranks, and a walk that applies each
    // tensor's own trust ratio.
    //
    // SRB: the world-size bucket this kernel was built for (1, 2, <= 4, <= 8).
    // A kernel per bucket, because one kernel holding the loops of all four
    // spilled 400-550 bytes per thread against 16 and ran 8 % slower.
    constexpr int SRB = PATH == kPathSegments ? 1 : PATH == kPathSegments + 1 ? 2
                        : PATH == kPathSegments + 2 ? 4 : 8;
    // a piece as a warp holds it: the pointers inside a RankArgs (what the unit
    // functions take), the rest of the Segment's words behind it
    struct WarpPiece {
      RankArgs ra;
      unsigned long long meta[kSegWords - kSegPointerWords];
    };
    enum { kMBegin = 0, kMLen, kMAlignedTensor, kMTensorLen, kMRanks, kMChunk0 };
    static_assert(offsetof(Segment, len) == (kSegPointerWords + kMLen) * 8 &&
                      offsetof(Segment, aligned16) == (kSegPointerWords + kMAlignedTensor) * 8 &&
                      offsetof(Segment, tensor_len) == (kSegPointerWords + kMTensorLen) * 8 &&
                      offsetof(Segment, first_rank) == (kSegPointerWords + kMRanks) * 8 &&
                      offsetof(Segment, chunk0) == (kSegPointerWords + kMChunk0) * 8,
                  "WarpPiece::meta follows the Segment's words");
    __shared__ int s_last;
    __shared__ WarpPiece s_wp[kSegPartPerChunk][2];  // per warp, two so that the next piece can be installed early
    constexpr int kChunk0InSmem = 1536;
    __shared__ unsigned long long s_chunk0[kChunk0InSmem];
    __shared__ float s_scale[OPT == kLAMB ? kChunk0InSmem : 1];  // lr x trust ratio per piece
    const Segment *segs = ra.segs;
    const int nseg = ra.nseg;
    for (int k = threadIdx.x; k < nseg && k < kChunk0InSmem; k += blockDim.x) s_chunk0[k] = segs[k].chunk0;
    const bool chunk0_in_smem = nseg <= kChunk0InSmem;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    const size_t nchunk = (size_t)ra.nchunk;
    const int chunk_shift = ra.chunk_shift;
    const size_t chunk_elems = (size_t)1 << chunk_shift;
    // scattered LAMB: seg_part holds a pair of partial sums per chunk, and behind them a pair
    // per chunk and warp
    double *const warp_part = ra.seg_part + 2 * nchunk;
    for (int k = lane; k < (int)(sizeof(RankArgs) / sizeof(int)); k += 32) {
      const int x = reinterpret_cast<const int *>(&ra)[k];
      reinterpret_cast<int *>(&s_wp[wid][0].ra)[k] = x;
      reinterpret_cast<int *>(&s_wp[wid][1].ra)[k] = x;
    }
    __syncthreads();

    // the last piece whose first chunk is <= q
    auto find_piece = [&](size_t q) -> int {
      int a = 0, b = nseg - 1;
      while (a < b) {
        const int mid = (a + b + 1) >> 1;
        if ((chunk0_in_smem ? s_chunk0[mid] : segs[mid].chunk0) <= q) a = mid;
        else b = mid - 1;
      }
      return a;
    };
    // this lane's word of piece a's descriptor (the descriptors do not change during the kernel)
    auto fetch_word = [&](int a) -> unsigned long long {
      unsigned long long x = 0;
      if (lane < kSegWords) {
        const unsigned long long *src = reinterpret_cast<const unsigned long long *>(segs + a) + lane;
        asm volatile("ld.global.nc.u64 %0, [%1];" : "=l"(x) : "l"(src));
      }
      return x;
    };
    auto install = [&](WarpPiece &wp, unsigned long long word) {
      if (lane < kSegPointerWords) {
        reinterpret_cast<unsigned long long *>(&wp.ra)[lane] = word;
      } else if (lane < kSegWords) {
        wp.meta[lane - kSegPointerWords] = word;
        if (lane == kSegPointerWords + kMAlignedTensor) wp.ra.aligned16 = (int)(unsigned)word;
      }
      __syncwarp();
    };
    // body(piece as this warp holds it, chunk, piece number) for every chunk of this CTA
    auto walk = [&](auto &&body) {
      size_t q = blockIdx.x;
      if (q >= nchunk) return;
      int slot = 0;
      int a = find_piece(q);
      install(s_wp[wid][0], fetch_word(a));
#pragma unroll 1
      for (; q < nchunk; q += gridDim.x) {
        const size_t qn = q + gridDim.x;
        int an = a;
        unsigned long long next_word = 0;
        if (qn < nchunk) {
          an = find_piece(qn);
          if (an != a) next_word = fetch_word(an);
        }
        body(s_wp[wid][slot], q, a);
        if (an != a) {
          __syncwarp();  // every lane is done with what the other slot held
          slot ^= 1;
          install(s_wp[wid][slot], next_word);
          a = an;
        }
      }
    };
    // a chunk's place in its piece
    auto chunk_span = [&](const WarpPiece &wp, size_t q, size_t &seg_lo, size_t &c_lo, size_t &c_len) {
      seg_lo = (size_t)wp.meta[kMBegin];
      c_lo = (q - (size_t)wp.meta[kMChunk0]) << chunk_shift;
      const size_t rest = (size_t)wp.meta[kMLen] - c_lo;
      c_len = rest < chunk_elems ? rest : chunk_elems;
    };

    // ---- first walk: SGD / Adam step, or LAMB moments + the chunk's partial norms ----
    if (ok) {
      walk([&](WarpPiece &wp, size_t q, int) {
        size_t seg_lo, c_lo, c_len;
        chunk_span(wp, q, seg_lo, c_lo, c_len);
        const size_t nv = wp.ra.aligned16 ? c_len / VEC : 0;
        Hyper hs = h;
        if constexpr (OPT == kLAMB) hs.quirk_n = (float)wp.meta[kMTensorLen];
        double p_w2 = 0.0, p_r2 = 0.0;
        direct_step<OPT, GT, LPT, SRB>(wp.ra, sa, hs, seg_lo, seg_lo + c_lo, nv * VEC,
                                       (size_t)threadIdx.x, (size_t)blockDim.x, p_w2, p_r2);
        for (size_t j = nv * VEC + threadIdx.x; j < c_len; j += blockDim.x)
          step_unit<OPT, GT, LPT, 1, 0>(wp.ra, sa, hs, seg_lo, seg_lo + c_lo + j, p_w2, p_r2);
        if constexpr (OPT == kLAMB) {  // lane order, then a fixed shuffle tree: reproducible
          p_w2 = warp_sum(p_w2);
          p_r2 = warp_sum(p_r2);
          if (lane == 0) {
            double *dst = warp_part + 2 * (q * (size_t)nwarp + wid);
            dst[0] = p_w2, dst[1] = p_r2;
          }
        }
      });
    }

    if constexpr (OPT == kLAMB) {
      // ---- per-tensor norms: warp partials -> chunk (the CTA that walked it) -> rank
      // (last CTA) -> peers, every sum in a fixed order
      __syncthreads();
      if (started_ok) {
        for (size_t q = blockIdx.x + (size_t)threadIdx.x * gridDim.x; q < nchunk;
             q += (size_t)blockDim.x * gridDim.x) {
          const double2 *src = reinterpret_cast<const double2 *>(warp_part) + q * (size_t)nwarp;
          double x = 0.0, y = 0.0;
          for (int k = 0; k < nwarp; ++k) {
            const double2 pr = __ldcg(src + k);
            x += pr.x, y += pr.y;
          }
          reinterpret_cast<double2 *>(ra.seg_part)[q] = make_double2(x, y);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();  // this CTA's partial sums before the count
        const unsigned prev = atomicAdd(&me->norm_count, 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) me->norm_count = 0;
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        // A piece's chunks are summed in chunk order by one thread when they are few
        // (most tensors of a model are biases and norms of a chunk or two), by a warp
        // otherwise: in both cases an order that depends on the piece alone.  The stores
        // to the peers are ordered before the flag by the barrier and the one system
        // fence of the releasing threads below (a fence per piece cost ~10 us each).
        constexpr size_t kFewChunks = 32;
        auto first_chunk = [&](int k) -> size_t {
          if (k >= nseg) return nchunk;
          return (size_t)(chunk0_in_smem ? s_chunk0[k] : segs[k].chunk0);
        };
        auto publish = [&](int sidx, double x, double y) {
          const int t = segs[sidx].tensor;
          for (int p = 0; p < R; ++p) {
            volatile double *dst = tensor_norms_of(ra.flags[p])->part[rank][t];
            dst[0] = x;
            dst[1] = y;
          }
        };
        const double2 *part = reinterpret_cast<const double2 *>(ra.seg_part);
        for (int sidx = threadIdx.x; sidx < nseg; sidx += blockDim.x) {  // a thread per small piece
          const size_t c0 = first_chunk(sidx), nc = first_chunk(sidx + 1) - c0;
          if (nc > kFewChunks) continue;
          double x = 0.0, y = 0.0;
          if (started_ok) {  // a rank that never started publishes zeros
            for (size_t c = 0; c < nc; ++c) {
              const double2 pr = __ldcg(part + c0 + c);
              x += pr.x, y += pr.y;
            }
          }
          publish(sidx, x, y);
        }
        for (int sidx = wid; sidx < nseg; sidx += nwarp) {  // a warp per large piece
          const size_t c0 = first_chunk(sidx), nc = first_chunk(sidx + 1) - c0;
          if (nc <= kFewChunks) continue;
          double x = 0.0, y = 0.0;
          if (started_ok) {
            const double2 *src = part + c0;
            size_t c = lane;
            for (; c + 96 < nc; c += 128) {  // four loads in flight per lane
              const double2 p0 = __ldcg(src + c), p1 = __ldcg(src + c + 32), p2 = __ldcg(src + c + 64),
                            p3 = __ldcg(src + c + 96);
              x += p0.x, y += p0.y;
              x += p1.x, y += p1.y;
              x += p2.x, y += p2.y;
              x += p3.x, y += p3.y;
            }
            for (; c < nc; c += 32) {
              const double2 pr = __ldcg(src + c);
              x += pr.x, y += pr.y;
            }
          }
          x = warp_sum(x);
          y = warp_sum(y);
          if (lane == 0) publish(sidx, x, y);
        }
        __syncthreads();
        if ((int)threadIdx.x < R) {
          __threadfence_system();
          st_release_sys(&ra.flags[threadIdx.x]->norm_flag[rank], seq);
        }
      }
      // every CTA: wait (bounded) until all ranks' partials are in
      if (threadIdx.x == 0 && ok) {
        const int late = wait_all(me->norm_flag, R, -1, seq, sa.timeout_ns);
        if (late >= 0) {
          record_status(me, cocoTimeout, rank, kPhaseNorm, late, seq);
          s_ok = 0;
        }
      }
      __syncthreads();
      ok = ok && s_ok != 0;

      // ---- second walk: every tensor's own trust ratio ------------------------------
      if (ok) {
        // lr x trust ratio of piece a's tensor: the partials of the ranks that hold a
        // part of it, in rank order, so that every replica computes the same ratio
        auto piece_scale = [&](int a) -> float {
          TensorNorms *tn = tensor_norms_of(me);
          const int t = segs[a].tensor;
          double w2 = 0.0, r2 = 0.0;
          for (int p = segs[a].first_rank; p <= segs[a].last_rank; ++p) {
            w2 += ld_volatile_f64(&tn->part[p][t][0]);
            r2 += ld_volatile_f64(&tn->part[p][t][1]);
          }
          double wn, rn, sc;
          if (sa.flags & COCO_LAMB_REF_QUIRK) {  // sample :424-433, per buffer
            rn = sqrt(r2);
            wn = sqrt(w2 / (double)segs[a].tensor_len);
            sc = ((wn > 0) ? (rn > 0 ? wn / rn : 1.0) : 1.0) / rn;
          } else {
            rn = sqrt(r2);
            wn = sqrt(w2);
            sc = (wn > 0) ? (rn > 0 ? wn / rn : 1.0) : 1.0;
          }
          return __fmul_rn(sa.lr, (float)sc);
        };
        // all pieces' scales at once, a thread per piece (a stride of the walk is longer
        // than most tensors, so nearly every chunk enters another piece)
        for (int k = threadIdx.x; k < nseg && k < kChunk0InSmem; k += blockDim.x) s_scale[k] = piece_scale(k);
        __syncthreads();
        int scaled = -1;  // the piece lr_scale belongs to
        float lr_scale = 0.f;
        walk([&](WarpPiece &wp, size_t q, int a) {
          if (a != scaled) {
            if (a < kChunk0InSmem) {
              lr_scale = s_scale[a];
            } else {
              if (lane == 0) lr_scale = piece_scale(a);
              lr_scale = __shfl_sync(0xffffffffu, lr_scale, 0);
            }
            scaled = a;
          }
          size_t seg_lo, c_lo, c_len;
          chunk_span(wp, q, seg_lo, c_lo, c_len);
          const size_t nv = wp.ra.aligned16 ? c_len / VEC : 0;
          direct_apply<GT, LPT, SRB>(wp.ra, sa, h, seg_lo, seg_lo + c_lo, nv * VEC, (size_t)threadIdx.x,
                                     (size_t)blockDim.x, lr_scale);
          for (size_t j = nv * VEC + threadIdx.x; j < c_len; j += blockDim.x)
            lamb_apply_unit<LPT, 1, 0>(wp.ra, sa, h, seg_lo, seg_lo + c_lo + j, lr_scale);
        });
      }
    }
    seg_norm_ok = ok;
    ok = false;  // nothing is left for the flat-slice code below
    __syncthreads();
  }
  const bool seg_done = PATH >= kPathSegments;

  // Ring path: the slice's full warp tiles go through the rings; what is left
  // of the slice (and everything, when the slice or a pointer is not 16-byte
  // aligned) is done with direct loads.
  constexpr int kRingTileElems = 32 * (16 / (int)sizeof(GT));
  const size_t ring_tiles =
      (PATH == kPathRing && ra.aligned16 && sa.pipe_stages > 0) ? L / kRingTileElems : 0;
  const size_t piped = ring_tiles * kRingTileElems;  // elements covered by the rings
  const size_t nvec_rest = ra.aligned16 ? (L - piped) / VEC : 0;

  double sum_w2 = 0.0, sum_r2 = 0.0;
  if constexpr (PATH == kPathRing) {
    bool landed = true;
    if (ok && ring_tiles > 0) {
      const int wid = threadIdx.x >> 5;
      // ordering of the peers' gradient writes (made visible by the start
      // barrier's acquire) before this thread's copies through the async proxy
      asm volatile("fence.proxy.async;" ::: "memory");
      landed = ring_step<OPT, GT, LPT>(
          ra, sa, h, lo, ring_tiles,
          ring_smem + (size_t)wid * sa.pipe_stages * R * kRingTileBytes, s_ring_bar[wid], sum_w2,
          sum_r2);
      if (!landed && (threadIdx.x & 31) == 0)
        record_status(me, cocoTimeout, rank, kPhaseCopy, -1, seq);
    }
    // a warp whose copies did not land stops the whole CTA (uniformly)
    if (__syncthreads_or(!landed)) ok = false;
  }
  // NVLS: whole 16-byte units of the slice go through the switch; the rest
  // (and everything when unaligned) falls through to the peer-to-peer code.
  constexpr int NV = Multimem<GT>::kN;
  const bool nvls = PATH == kPathNvls && (sa.flags & kFlagNvls) && ra.aligned16 && ra.mc_g &&
                    ra.mc_out && sa.variant != cocoVariantNccl;
  const size_t nvls_units = nvls ? L / NV : 0;
  if constexpr (PATH == kPathNvls) {
    if (ok && nvls)
      nvls_phase<OPT, GT, LPT, 0>(ra, sa, h, lo, nvls_units, tid, nth, sum_w2, sum_r2, 0.f);
  }
  if (ok) {
    const size_t first = lo + piped;
    if constexpr (PATH == kPathLocal) {
      // Equal shares by grid stride.  The SMs do not stream from HBM at the same rate (their
      // active cycles differ by 8 % in a profile of this kernel), but handing the work out
      // warp by warp from a counter, 8 to 32 passes at a time with the next number asked for
      // ahead, measured no better: mixed-precision Adam on 334 M elements 1.53-1.56 ms
      // against 1.512, fp32 Adam on 2^26 0.304-0.324 ms against 0.312.
      direct_step<OPT, GT, LPT, 1>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, sum_w2, sum_r2);
    } else if constexpr (PATH != kPathDirect) {
      // vector loops of the direct path are not part of this kernel; the
      // scalar loop below takes what the path left over
      (void)first;
    } else if (R == 2)
      COCO_DIRECT_STEP<OPT, GT, LPT, 2>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, sum_w2, sum_r2);
    else if (R <= 4)
      COCO_DIRECT_STEP<OPT, GT, LPT, 4>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, sum_w2, sum_r2);
    else
      COCO_DIRECT_STEP<OPT, GT, LPT, 8>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, sum_w2, sum_r2);
    const size_t done_elems = PATH == kPathNvls ? nvls_units * NV
                              : PATH == kPathRing ? piped : piped + nvec_rest * VEC;
    for (size_t j = done_elems + tid; j < L; j += nth)
      step_unit<OPT, GT, LPT, 1, 0>(ra, sa, h, lo, lo + j, sum_w2, sum_r2);
  }

  if constexpr (OPT == kLAMB && PATH < kPathSegments) {
    // ---- norms: thread -> warp -> CTA -> rank (fixed order) -> all ranks ---
    sum_w2 = warp_sum(sum_w2);
    sum_r2 = warp_sum(sum_r2);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) s_red[0][wid] = sum_w2, s_red[1][wid] = sum_r2;
    __syncthreads();
    if (stamps) me->phase_ns[1] = me->phase_ns[2] = globaltimer_ns();
    if (threadIdx.x == 0) {
      double a = 0.0, b = 0.0;
      const int nw = (blockDim.x + 31) >> 5;
      for (int k = 0; k < nw; ++k) a += s_red[0][k], b += s_red[1][k];
      me->cta_part[blockIdx.x][0] = a;
      me->cta_part[blockIdx.x][1] = b;
      __threadfence();
      const unsigned prev = atomicAdd(&me->norm_count, 1u);
      s_last_cta = prev == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last_cta) {
      // Last CTA of the rank: combine and publish.  Thread c takes the CTAs c, c + block
      // size, ..., then the warps' shuffle tree, then the warps in order: a fixed order,
      // and the loads of all CTAs' pairs are in flight at once (one thread adding them
      // one after the other stood for ~100 us between the two phases of every step).
      __threadfence();
      double a = 0.0, b = 0.0;
      for (unsigned c = threadIdx.x; c < gridDim.x; c += blockDim.x) {
        a += ld_volatile_f64(&me->cta_part[c][0]);
        b += ld_volatile_f64(&me->cta_part[c][1]);
      }
      a = warp_sum(a);
      b = warp_sum(b);
      if (lane == 0) s_red[0][wid] = a, s_red[1][wid] = b;
      __syncthreads();
      if (threadIdx.x == 0) {
        a = 0.0, b = 0.0;
        const int nw = (blockDim.x + 31) >> 5;
        for (int k = 0; k < nw; ++k) a += s_red[0][k], b += s_red[1][k];
        me->norm_count = 0;
        for (int p = 0; p < R; ++p) {
          volatile double *dst = ra.flags[p]->norm_part[rank];
          dst[0] = a;
          dst[1] = b;
        }
        __threadfence_system();
        for (int p = 0; p < R; ++p) st_release_sys(&ra.flags[p]->norm_flag[rank], seq);
      }
    }
    if (threadIdx.x == 0) {
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
          if (sa.variant == cocoVariantNccl) {
            // forked-NCCL LAMB: float norms, the ratio divided by ||r|| once
            // more, all in float (common_kernel.h:2699)
            const float wf = (float)sqrt(w2), rf = (float)sqrt(r2);
            wn = wf, rn = rf;
            sc = (double)__fdiv_rn((wf > 0) ? (rf > 0 ? __fdiv_rn(wf, rf) : 1.0f) : 1.0f, rf);
          } else if (sa.flags & COCO_LAMB_REF_QUIRK) {  // sample :424-433
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
      if (stamps) me->phase_ns[2] = globaltimer_ns();
    }
    __syncthreads();
    ok = s_ok != 0;
    if (ok) {
      const float lr_scale = s_lr_scale;
      if constexpr (PATH == kPathRing) ring_apply<GT, LPT>(ra, sa, h, lo, piped, tid, nth, lr_scale);
      if constexpr (PATH == kPathNvls) {
        if (ok && nvls)
          nvls_phase<OPT, GT, LPT, 1>(ra, sa, h, lo, nvls_units, tid, nth, sum_w2, sum_r2,
                                      lr_scale);
      }
      if (ok) {
        const size_t first = lo + piped;
        if constexpr (PATH == kPathLocal) {
          direct_apply<GT, LPT, 1>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, lr_scale);
        } else if constexpr (PATH != kPathDirect) {
          (void)first;
        } else if (R == 2)
          direct_apply<GT, LPT, 2>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, lr_scale);
        else if (R <= 4)
          direct_apply<GT, LPT, 4>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, lr_scale);
        else
          direct_apply<GT, LPT, 8>(ra, sa, h, lo, first, nvec_rest * VEC, tid, nth, lr_scale);
        const size_t done_elems = PATH == kPathNvls ? nvls_units * NV
                                  : PATH == kPathRing ? piped : piped + nvec_rest * VEC;
        for (size_t j = done_elems + tid; j < L; j += nth)
          lamb_apply_unit<LPT, 1, 0>(ra, sa, h, lo, lo + j, lr_scale);
      }
    }
  }

  if (seg_done) ok = started_ok && seg_norm_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long t = globaltimer_ns();
    if (blockIdx.x < kMaxCtasPerRank) me->cta_end_ns[blockIdx.x] = t;  // cocoLastCtaSpread
    if (stamps) me->phase_ns[3] = t;
  }

  // ---- end barrier ----------------------------------------------------------
  if (R > 1) {
    __threadfence_system();  // this thread's peer stores before the "done" signal
    __syncthreads();
    if (threadIdx.x < 32) {
      unsigned prev = 0;
      if (threadIdx.x == 0) {
        __threadfence_system();
        prev = atomicAdd(&me->done_count, 1u);
        if (prev == gridDim.x - 1) {
          me->done_count = 0;
          me->work_next = 0;  // every CTA of the rank has stopped taking chunks
        }
        __threadfence_system();
      }
      __syncwarp();
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == gridDim.x - 1) {  // last CTA of the rank
        __threadfence_system();
        warp_signal_peers(ra, R, rank, seq, [](FlagPage *f) { return f->done; });
        if (ok) {
          const int late = warp_wait_peers(me->done, R, rank, seq, sa.timeout_ns);
          if (late >= 0 && threadIdx.x == 0)
            record_status(me, cocoTimeout, rank, kPhaseEnd, late, seq);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
template <int OPT, typename GT, typename LPT> KernelPtr pick_path(int path) {
  switch (path) {
    case kPathNvls: return fused_step_kernel<OPT, GT, LPT, kPathNvls>;
    case kPathRing: return fused_step_kernel<OPT, GT, LPT, kPathRing>;
    case kPathLocal: return fused_step_kernel<OPT, GT, LPT, kPathLocal>;
    case kPathSegments:
    case kPathSegments + 1:
    case kPathSegments + 2:
    case kPathSegments + 3:
      // lists of tensors gather fp32 weights only: no low-precision variants
      if constexpr (!std::is_same<LPT, NoLp>::value) return nullptr;
      else if (path == kPathSegments) return fused_step_kernel<OPT, GT, LPT, kPathSegments>;
      else if (path == kPathSegments + 1) return fused_step_kernel<OPT, GT, LPT, kPathSegments + 1>;
      else if (path == kPathSegments + 2) return fused_step_kernel<OPT, GT, LPT, kPathSegments + 2>;
      else return fused_step_kernel<OPT, GT, LPT, kPathSegments + 3>;
    default: return fused_step_kernel<OPT, GT, LPT, kPathDirect>;
  }
}
template <int OPT, typename GT> KernelPtr pick_lp(bool has_lp, cocoDataType_t lp, int path) {
  if (!has_lp) return pick_path<OPT, GT, NoLp>(path);
  if (lp == cocoFloat16) return pick_path<OPT, GT, __half>(path);
  if (lp == cocoBfloat16) return pick_path<OPT, GT, __nv_bfloat16>(path);
  return nullptr;
}
template <int OPT> KernelPtr pick_g(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path) {
  if (g == cocoFloat32) return pick_lp<OPT, float>(has_lp, lp, path);
  if (g == cocoFloat16) return pick_lp<OPT, __half>(has_lp, lp, path);
  if (g == cocoBfloat16) return pick_lp<OPT, __nv_bfloat16>(has_lp, lp, path);
  return nullptr;
}
}  // namespace

// The kernels are instantiated in three translation units (COCO_PART = 0, 1,
// 2: SGD, Adam, LAMB) so that they compile in parallel; COCO_PART = 3 holds
// the dispatch.  Without COCO_PART everything is in one unit.
#if !defined(COCO_PART) || COCO_PART == 0
KernelPtr pick_sgd(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path) {
  return pick_g<kSGD>(g, has_lp, lp, path);
}
#endif
#if !defined(COCO_PART) || COCO_PART == 1
KernelPtr pick_adam(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path) {
  return pick_g<kAdam>(g, has_lp, lp, path);
}
#endif
#if !defined(COCO_PART) || COCO_PART == 2
KernelPtr pick_lamb(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path) {
  return pick_g<kLAMB>(g, has_lp, lp, path);
}
#endif

#if !defined(COCO_PART) || COCO_PART == 3
KernelPtr pick_sgd(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path);
KernelPtr pick_adam(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path);
KernelPtr pick_lamb(cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path);

namespace {

KernelPtr pick(int opt, cocoDataType_t g, bool has_lp, cocoDataType_t lp, int path) {
  switch (opt) {
    case kSGD: return pick_sgd(g, has_lp, lp, path);
    case kAdam: return pick_adam(g, has_lp, lp, path);
    case kLAMB: return pick_lamb(g, has_lp, lp, path);
  }
  return nullptr;
}

}  // namespace

// The path a launch takes: the segment kernels for lists of tensors, NVLS when
// the call carries multicast addresses, the warp rings when it was given
// stages, else the register-staged path.
int fused_step_path(const StepArgs &sa) {
  if (sa.flags & kFlagScattered)  // one kernel per world-size bucket: 1, 2, <= 4, <= 8
    return kPathSegments + (sa.world == 1 ? 0 : sa.world == 2 ? 1 : sa.world <= 4 ? 2 : 3);
  if (sa.flags & kFlagNvls) return kPathNvls;
  if (sa.pipe_stages > 0) return kPathRing;
  return sa.world == 1 ? kPathLocal : kPathDirect;
}

int fused_step_block_threads(int path, cocoDataType_t g_type) {
  const bool is16 = g_type != cocoFloat32;
  if (path == kPathLocal) return is16 ? COCO_LOCAL16_THREADS : COCO_LOCAL32_THREADS;
  if (path >= kPathSegments) return COCO_SEG_THREADS;
  return is16 ? COCO_MULTI16_THREADS : COCO_MULTI32_THREADS;
}

namespace {

// Per (kernel, threads, dynamic shared memory): the attribute is set and the
// occupancy queried once, then remembered (both are host calls in the path of
// every small-message step otherwise).
struct KernelInfo {
  int occupancy;
};
std::mutex g_info_mu;
std::map<std::tuple<const void *, int, int, size_t>, KernelInfo> g_info;  // + device

cudaError_t kernel_info(KernelPtr k, int threads, size_t smem_bytes, KernelInfo *out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_info_mu);
  const auto key = std::make_tuple((const void *)k, dev, threads, smem_bytes);
  auto it = g_info.find(key);
  if (it != g_info.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  if (smem_bytes > 0) {  // static + dynamic may exceed the 48 KB default together
    e = cudaFuncSetAttribute((const void *)k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes);
    if (e != cudaSuccess) return e;
  }
  KernelInfo ki = {};
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ki.occupancy, (const void *)k, threads,
                                                    smem_bytes);
  if (e != cudaSuccess) return e;
  g_info[key] = ki;
  *out = ki;
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_fused_step(int opt, cocoDataType_t g_type, bool has_lp, cocoDataType_t lp_type,
                              const StepArgs &sa, const RankArgs &one, const RankArgs *table,
                              const LaunchConfig &cfg, cudaStream_t stream) {
  KernelPtr k = pick(opt, g_type, has_lp, lp_type, fused_step_path(sa));
  if (!k) return cudaErrorInvalidValue;
  const dim3 grid(cfg.ctas, cfg.nvirt > 1 ? cfg.nvirt : 1, 1);
  const dim3 block(cfg.threads, 1, 1);
  const RankArgs *tbl = cfg.nvirt > 1 ? table : nullptr;
  void *params[] = {(void *)&sa, (void *)&one, (void *)&tbl};
  if (cfg.smem_bytes > 0) {  // sets the shared-memory attribute on first use
    KernelInfo ki;
    cudaError_t e = kernel_info(k, cfg.threads, cfg.smem_bytes, &ki);
    if (e != cudaSuccess) return e;
  }
  if (cfg.cooperative)
    return cudaLaunchCooperativeKernel((const void *)k, grid, block, params, cfg.smem_bytes, stream);
  return cudaLaunchKernel((const void *)k, grid, block, params, cfg.smem_bytes, stream);
}

cudaError_t fused_step_occupancy(int opt, cocoDataType_t g_type, bool has_lp,
                                 cocoDataType_t lp_type, int path, int threads, size_t smem_bytes,
                                 int *ctas_per_sm) {
  KernelPtr k = pick(opt, g_type, has_lp, lp_type, path);  // the instantiation that is launched
  if (!k) return cudaErrorInvalidValue;
  KernelInfo ki;
  cudaError_t e = kernel_info(k, threads, smem_bytes, &ki);
  if (e != cudaSuccess) return e;
  *ctas_per_sm = ki.occupancy;
  return cudaSuccess;
}
#endif  // dispatch part

}  // namespace coco
