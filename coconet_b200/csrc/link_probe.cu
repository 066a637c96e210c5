// Link probe: what this node's NVLink gives a kernel that has the fused
// step's access shape and nothing else to do.  Every rank pulls its slice of a
// peer-mapped buffer from all peers (16-byte loads, U of them in flight per
// thread and peer), or pushes its slice to all peers (16-byte stores), or both
// at once -- the communication skeleton of the fused step without the update.
//
// It is a yardstick, not a product path: the benchmark prints its figures next
// to the fused step's so that a reader can tell how much of the gap to the
// nominal link rate is the kernel's and how much is the link's.  The reference
// has no counterpart (its ring kernels were measured end to end only,
// experiments/generate-pdf/dsl_vs_apex.py:93-96).
//
// Protocol and memory ordering are the fused kernel's: start barrier (every
// rank has launched), data loop, end barrier (nobody touches a peer's buffer
// any more); every wait is bounded and records a status instead of hanging.
#include <cuda_runtime.h>

#include "coconet_fused_generic.cuh"
#include "fused_step.cuh"

namespace coco {

namespace {

__device__ __forceinline__ uint4 ld_peer_16(const void *p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_peer_16(void *p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint4 mc_ld_reduce_16(const void *p) {
  float x[4];
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3])
               : "l"(p));
  return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]),
                    __float_as_uint(x[3]));
}
__device__ __forceinline__ void mc_st_16(void *p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// The same through the NVSwitch multicast address of the buffer: MODE 0 one
// multimem.ld_reduce (fp32 add) per unit of the rank's slice, 1 one
// multimem.st per unit, 2 both.  U reductions in flight per thread.
template <int MODE, int U>
__global__ void __launch_bounds__(512)
    switch_probe_kernel(const __grid_constant__ StepArgs sa, const __grid_constant__ RankArgs ra_in) {
  using namespace coco_generic;
  __shared__ RankArgs ra;
  __shared__ int s_ok;
  {
    const int *s = reinterpret_cast<const int *>(&ra_in);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
  }
  __syncthreads();
  const int R = sa.world, rank = ra.rank;
  FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;
  if (threadIdx.x < 32) {
    const int p = threadIdx.x;
    const bool peer = p < R && p != rank;
    if (blockIdx.x == 0 && peer) st_release(&ra.flags[p]->arrive[rank], seq);
    bool late = false;
    if (peer) late = !wait_flag(&me->arrive[p], seq, sa.timeout_ns);
    const unsigned bad = __ballot_sync(0xffffffffu, late);
    if (bad && threadIdx.x == 0) {
      record(me, cocoTimeout, rank, kPhaseStart, __ffs(bad) - 1, seq);
      s_ok = 0;
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  if (ok) {
    uint4 sink = make_uint4(0, 0, 0, 0);
    for (size_t u0 = tid; u0 < L; u0 += nth * U) {
      uint4 x[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t u = u0 + (size_t)k * nth;
        x[k] = make_uint4(rank, (unsigned)u, k, 0);
        if (MODE != 1 && u < L) x[k] = mc_ld_reduce_16((const uint4 *)ra.mc_g + lo + u);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t u = u0 + (size_t)k * nth;
        if (u >= L) continue;
        if (MODE == 0)
          sink.x ^= x[k].x, sink.y ^= x[k].y, sink.z ^= x[k].z, sink.w ^= x[k].w;
        else
          mc_st_16((uint4 *)ra.mc_out + lo + u, x[k]);
      }
    }
    // keep the reductions alive without a store per unit
    if (MODE == 0 && (sink.x ^ sink.y ^ sink.z ^ sink.w) == 0x9e3779b9u && tid == 0)
      st_peer_16((uint4 *)ra.out[rank] + lo, sink);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned prev = 0;
    if (threadIdx.x == 0) {
      prev = atomicAdd(&me->done_count, 1u);
      if (prev == gridDim.x - 1) me->done_count = 0;
      __threadfence_system();
    }
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev == gridDim.x - 1) {
      const int p = threadIdx.x;
      const bool peer = p < R && p != rank;
      if (peer) st_release(&ra.flags[p]->done[rank], seq);
      bool late = false;
      if (peer && ok) late = !wait_flag(&me->done[p], seq, sa.timeout_ns);
      const unsigned bad = __ballot_sync(0xffffffffu, late);
      if (bad && threadIdx.x == 0) record(me, cocoTimeout, rank, kPhaseEnd, __ffs(bad) - 1, seq);
    }
  }
}

// Hybrid: the even CTAs take the first `sa.pad` sixteenths of the rank's slice
// through the switch (multimem.ld_reduce + multimem.st), the odd CTAs the rest
// peer to peer (pull from all peers + push to all peers), at the same time.
// Tells whether the switch's reductions and plain peer traffic compete for
// the same resource or can overlap.
template <int RB>
__global__ void __launch_bounds__(512)
    hybrid_probe_kernel(const __grid_constant__ StepArgs sa, const __grid_constant__ RankArgs ra_in) {
  using namespace coco_generic;
  __shared__ RankArgs ra;
  __shared__ int s_ok;
  {
    const int *s = reinterpret_cast<const int *>(&ra_in);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
  }
  __syncthreads();
  const int R = sa.world, rank = ra.rank;
  FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;
  if (threadIdx.x < 32) {
    const int p = threadIdx.x;
    const bool peer = p < R && p != rank;
    if (blockIdx.x == 0 && peer) st_release(&ra.flags[p]->arrive[rank], seq);
    bool late = false;
    if (peer) late = !wait_flag(&me->arrive[p], seq, sa.timeout_ns);
    const unsigned bad = __ballot_sync(0xffffffffu, late);
    if (bad && threadIdx.x == 0) {
      record(me, cocoTimeout, rank, kPhaseStart, __ffs(bad) - 1, seq);
      s_ok = 0;
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  const size_t cut = L / 16 * (size_t)sa.pad;  // units [0, cut) through the switch
  const bool via_switch = (blockIdx.x & 1) == 0;
  const size_t half_ctas = via_switch ? (gridDim.x + 1) / 2 : gridDim.x / 2;
  const size_t tid = (size_t)(blockIdx.x >> 1) * blockDim.x + threadIdx.x;
  const size_t nth = half_ctas * blockDim.x;
  if (ok && via_switch) {
    for (size_t u = tid; u < cut; u += 2 * nth) {
      const size_t u2 = u + nth;
      uint4 a = mc_ld_reduce_16((const uint4 *)ra.mc_g + lo + u), b = a;
      if (u2 < cut) b = mc_ld_reduce_16((const uint4 *)ra.mc_g + lo + u2);
      mc_st_16((uint4 *)ra.mc_out + lo + u, a);
      if (u2 < cut) mc_st_16((uint4 *)ra.mc_out + lo + u2, b);
    }
  } else if (ok && nth > 0) {
    for (size_t u = cut + tid; u < L; u += nth) {
      uint4 acc = make_uint4(rank, (unsigned)u, 0, 0), x[RB - 1];
#pragma unroll
      for (int q = 0; q < RB - 1; ++q) {
        int p = rank + 1 + q;
        if (p >= R) p -= R;
        if (q < R - 1) x[q] = ld_peer_16((const uint4 *)ra.g[p] + lo + u);
      }
#pragma unroll
      for (int q = 0; q < RB - 1; ++q)
        if (q < R - 1) acc.x ^= x[q].x, acc.y ^= x[q].y, acc.z ^= x[q].z, acc.w ^= x[q].w;
#pragma unroll
      for (int q = 0; q < RB - 1; ++q) {
        int p = rank + 1 + q;
        if (p >= R) p -= R;
        if (q < R - 1) st_peer_16((uint4 *)ra.out[p] + lo + u, acc);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned prev = 0;
    if (threadIdx.x == 0) {
      prev = atomicAdd(&me->done_count, 1u);
      if (prev == gridDim.x - 1) me->done_count = 0;
      __threadfence_system();
    }
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev == gridDim.x - 1) {
      const int p = threadIdx.x;
      const bool peer = p < R && p != rank;
      if (peer) st_release(&ra.flags[p]->done[rank], seq);
      bool late = false;
      if (peer && ok) late = !wait_flag(&me->done[p], seq, sa.timeout_ns);
      const unsigned bad = __ballot_sync(0xffffffffu, late);
      if (bad && threadIdx.x == 0) record(me, cocoTimeout, rank, kPhaseEnd, __ffs(bad) - 1, seq);
    }
  }
}

// MODE 0 pull, 1 push, 2 both.  U: units of 16 bytes per thread and pass.
// RB: compile-time bound on the world size (RB - 1 peer slots per unit).
// sa.count = 16-byte units of the whole buffer; the rank's slice is sliced as
// the fused step slices elements.
template <int MODE, int U, int RB>
__global__ void __launch_bounds__(512)
    link_probe_kernel(const __grid_constant__ StepArgs sa, const __grid_constant__ RankArgs ra_in) {
  using namespace coco_generic;
  __shared__ RankArgs ra;
  __shared__ int s_ok;
  {
    const int *s = reinterpret_cast<const int *>(&ra_in);
    int *d = reinterpret_cast<int *>(&ra);
    for (int k = threadIdx.x; k < (int)(sizeof(RankArgs) / sizeof(int)); k += blockDim.x)
      d[k] = s[k];
    if (threadIdx.x == 0) s_ok = 1;
  }
  __syncthreads();
  const int R = sa.world, rank = ra.rank;
  FlagPage *me = ra.flags[rank];
  const unsigned long long seq = sa.seq;

  if (R > 1) {  // start barrier: lane p of warp 0 talks to rank p
    if (threadIdx.x < 32) {
      const int p = threadIdx.x;
      const bool peer = p < R && p != rank;
      if (blockIdx.x == 0 && peer) st_release(&ra.flags[p]->arrive[rank], seq);
      bool late = false;
      if (peer) late = !wait_flag(&me->arrive[p], seq, sa.timeout_ns);
      const unsigned bad = __ballot_sync(0xffffffffu, late);
      if (bad && threadIdx.x == 0) {
        record(me, cocoTimeout, rank, kPhaseStart, __ffs(bad) - 1, seq);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  const bool ok = s_ok != 0;

  const size_t N = sa.count;
  const size_t S = (N + R - 1) / R;
  const size_t lo = (size_t)rank * S < N ? (size_t)rank * S : N;
  const size_t hi = lo + S < N ? lo + S : N;
  const size_t L = hi - lo;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  if (ok) {
    for (size_t u0 = tid; u0 < L; u0 += nth * U) {
      uint4 acc[U];
#pragma unroll
      for (int k = 0; k < U; ++k) acc[k] = make_uint4(rank, (unsigned)u0, k, 0);
      if (MODE != 1) {
        // all loads of the pass are issued before the first use
        uint4 x[U][RB - 1];
#pragma unroll
        for (int k = 0; k < U; ++k) {
          const size_t u = u0 + (size_t)k * nth;
#pragma unroll
          for (int q = 0; q < RB - 1; ++q) {
            int p = rank + 1 + q;
            if (p >= R) p -= R;
            if (q < R - 1 && u < L) x[k][q] = ld_peer_16((const uint4 *)ra.g[p] + lo + u);
          }
        }
#pragma unroll
        for (int k = 0; k < U; ++k)
#pragma unroll
          for (int q = 0; q < RB - 1; ++q)
            if (q < R - 1 && u0 + (size_t)k * nth < L) {
              acc[k].x ^= x[k][q].x, acc[k].y ^= x[k][q].y;
              acc[k].z ^= x[k][q].z, acc[k].w ^= x[k][q].w;
            }
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const size_t u = u0 + (size_t)k * nth;
        if (u >= L) continue;
        if (MODE == 0) {
          // keep the loads alive: one local store per unit (a fraction of the traffic)
          st_peer_16((uint4 *)ra.out[rank] + lo + u, acc[k]);
        } else {
#pragma unroll
          for (int q = 0; q < RB - 1; ++q) {
            int p = rank + 1 + q;
            if (p >= R) p -= R;
            if (q < R - 1) st_peer_16((uint4 *)ra.out[p] + lo + u, acc[k]);
          }
        }
      }
    }
  }

  if (R > 1) {  // end barrier
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < 32) {
      unsigned prev = 0;
      if (threadIdx.x == 0) {
        prev = atomicAdd(&me->done_count, 1u);
        if (prev == gridDim.x - 1) me->done_count = 0;
        __threadfence_system();
      }
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == gridDim.x - 1) {
        const int p = threadIdx.x;
        const bool peer = p < R && p != rank;
        if (peer) st_release(&ra.flags[p]->done[rank], seq);
        bool late = false;
        if (peer && ok) late = !wait_flag(&me->done[p], seq, sa.timeout_ns);
        const unsigned bad = __ballot_sync(0xffffffffu, late);
        if (bad && threadIdx.x == 0) record(me, cocoTimeout, rank, kPhaseEnd, __ffs(bad) - 1, seq);
      }
    }
  }
}

typedef void (*ProbePtr)(const StepArgs, const RankArgs);

template <int MODE, int RB> ProbePtr pick_unroll(int unroll) {
  switch (unroll) {
    case 1: return link_probe_kernel<MODE, 1, RB>;
    case 2: return link_probe_kernel<MODE, 2, RB>;
    case 4: return link_probe_kernel<MODE, 4, RB>;
  }
  return nullptr;
}
template <int MODE> ProbePtr pick_world(int world, int unroll) {
  if (world <= 2) return pick_unroll<MODE, 2>(unroll);
  if (world <= 4) return pick_unroll<MODE, 4>(unroll);
  return pick_unroll<MODE, 8>(unroll);
}

template <int MODE> ProbePtr pick_switch(int unroll) {
  switch (unroll) {
    case 1: return switch_probe_kernel<MODE, 1>;
    case 2: return switch_probe_kernel<MODE, 2>;
    case 4: return switch_probe_kernel<MODE, 4>;
  }
  return nullptr;
}

}  // namespace

cudaError_t launch_link_probe(int mode, int unroll, const StepArgs &sa, const RankArgs &ra,
                              int sm_count, int threads, cudaStream_t stream) {
  ProbePtr k = mode == 0 ? pick_world<0>(sa.world, unroll)
               : mode == 1 ? pick_world<1>(sa.world, unroll)
               : mode == 2 ? pick_world<2>(sa.world, unroll)
               : mode == 4 ? pick_switch<0>(unroll)
               : mode == 5 ? pick_switch<1>(unroll)
               : mode == 6 ? pick_switch<2>(unroll)
               : mode == 7 ? (sa.world <= 2 ? (ProbePtr)hybrid_probe_kernel<2>
                              : sa.world <= 4 ? (ProbePtr)hybrid_probe_kernel<4>
                                              : (ProbePtr)hybrid_probe_kernel<8>)
                           : nullptr;
  if (!k) return cudaErrorInvalidValue;
  int occ = 0;  // the deeper unrolls hold more registers: fewer CTAs per SM
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void *)k, threads, 0);
  if (e != cudaSuccess) return e;
  if (occ < 1) return cudaErrorLaunchOutOfResources;
  const int ctas = (occ > 2 ? 2 : occ) * sm_count;
  void *params[] = {(void *)&sa, (void *)&ra};
  return cudaLaunchKernel((const void *)k, dim3(ctas), dim3(threads), params, 0, stream);
}

}  // namespace coco
