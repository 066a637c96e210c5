/*
 * coconet_rt — C ABI of the B200 runtime for CoCoNet's fused AllReduce
 * optimizer step:  ReduceScatter(sum) of Local gradients  ->  sliced
 * SGD / Adam / LAMB update  ->  AllGather of the Replicated weights, as ONE
 * kernel per step per GPU over NVLink peer memory.
 *
 * It replaces, for this one call, the reference's patched NCCL 2.6.4 fork.
 * Reference interfaces are cited as file:line inside parasailteam/coconet.
 *
 * Conventions
 *  - plain C: pointers and sizes only; every entry point returns an int
 *    (cocoSuccess == 0), never throws, never terminates the process.
 *  - one communicator per GPU per process (or several per process through
 *    cocoCommInitAll); all ranks call the collective entry points in the same
 *    order, like NCCL.  One fused operation in flight per communicator.
 *  - data layout: N elements, world size R, S = ceil(N/R); rank r owns the
 *    contiguous slice [r*S, min(N,(r+1)*S)) — the element count the reference
 *    gives a `Sliced` tensor (src/codegen.cpp:139-165).
 *      g      Local       N elements per rank (fp32 | fp16 | bf16), read-only
 *      w      Replicated  N fp32.  Without w_lp it is gathered to all ranks;
 *                         with w_lp only the own slice (the fp32 master) is
 *                         updated, indexed by global element like the
 *                         reference (all_reduce_computation.h:110)
 *      w_lp   Replicated  N fp16/bf16 copy of w, gathered to all ranks; or NULL
 *      m, v   Sliced      S fp32 per rank, indexed from the slice start
 *                         (examples/adam/adam.cpp:62-63)
 *  - buffers read or written by peers (g, and w or w_lp) are peer-mapped on
 *    first use (a collective host-side exchange) unless registered before
 *    with cocoRegister.
 *  - a fused call that fails on the host at world size > 1 (a buffer that
 *    cannot be mapped, a launch error) leaves this rank's call count ahead of
 *    its peers': the communicator then refuses every further call with
 *    cocoInvalidUsage.  Destroy it, as after a device-side timeout.  Argument
 *    errors (cocoInvalidArgument) are found before that and are harmless.
 *  - buffers that the runtime peer-mapped on first use stay mapped for the
 *    life of the communicator: keep them allocated until it is destroyed, or
 *    hand them to cocoDeregister first (an allocator that reuses the address
 *    for another tensor would otherwise meet the peers' old mappings).
 *  - every device-side wait is bounded (COCO_TIMEOUT_MS, default 10000); on
 *    expiry the kernel records {code, rank, phase, peer} in a host-visible
 *    status word and returns.  Read it with cocoGetStatus after synchronising
 *    the stream.
 */
#ifndef COCONET_RT_H_
#define COCONET_RT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COCO_VERSION 100
#define COCO_MAX_RANKS 8
#define COCO_MAX_LAMB_TENSORS 2048 /* tensors of one cocoFusedLAMBScattered call */

typedef struct cocoComm *cocoComm_t;

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer so that this
 * header needs no CUDA include. */
typedef void *cocoStream_t;

typedef enum {
  cocoSuccess = 0,
  cocoInvalidArgument = 1,
  cocoInvalidUsage = 2,
  cocoCudaError = 3,
  cocoSystemError = 4,   /* sockets / bootstrap */
  cocoTimeout = 5,       /* a bounded device- or host-side wait expired */
  cocoPeerError = 6,     /* no peer access between two ranks */
  cocoInternalError = 7,
  cocoNumResults = 8
} cocoResult_t;

/* Element types; values of the first three match ncclDataType_t's
 * ncclFloat32 = 7, ncclFloat16 = 6, ncclBfloat16 = 9 so that emitted
 * programs can pass either (nccl/src/nccl.h.in:104-118). */
typedef enum { cocoFloat16 = 6, cocoFloat32 = 7, cocoBfloat16 = 9 } cocoDataType_t;

/* Which of the reference's three formulations the update evaluates. */
typedef enum {
  /* bias-corrected, eps in the denominator:  nccl-overlap/src/collectives/
   * device/reduce_kernel.h:143-246; host check nccl-overlap/samples/
   * multi-process-adam-scattered.cpp:112-123 (Adam), 402-435 (LAMB). */
  cocoVariantOverlap = 0,
  /* the DSL programs as written: examples/adam/adam.cpp:65-71 and its frozen
   * check examples/test-adam.cu:14-38; examples/lamb/lamb.cpp:79-88. */
  cocoVariantDsl = 1,
  /* the forked-NCCL functors, fp16 gradient sum in ring order included.
   * Adam (AllReduce_pipe TYPE 0): nccl/src/collectives/device/
   * reduce_kernel.h:27-62, common_kernel.h:853-923.  LAMB (TYPE 1):
   * reduce_kernel.h:391-452, common_kernel.h:2472-2535, 2687-2726 -- decay
   * factor 1.0 whatever weight_decay says, no epsilon, m/beta1 and v/beta2,
   * scale = (||w||/||r||)/||r||.  Needs fp16 gradients and an fp16 w_lp. */
  cocoVariantNccl = 2
} cocoVariant_t;

/* flags */
#define COCO_LAMB_REF_QUIRK 0x1u /* scale = trust/||r||, norms of the mean
                                    square (multi-process-adam-scattered.cpp:
                                    415-433); for known-answer tests only */

typedef struct {
  int code;        /* cocoResult_t of the first device-side failure, 0 if none */
  int rank;        /* rank that recorded it */
  int phase;       /* 1 start barrier, 2 norm exchange, 3 end barrier, 4 bulk copy of a
                      gradient tile, 5 a bounds / alignment check of the checked build */
  int peer;        /* peer rank that was waited for, -1 if n/a */
  uint64_t seq;    /* sequence number of the fused call */
} cocoStatus_t;

int cocoGetVersion(int *version);
const char *cocoErrorString(int result);

/* ---- communicators ------------------------------------------------------
 * Replaces ncclGetUniqueId + MPI_Bcast + ncclCommInitRank in the emitted
 * main() (src/codegen.cpp:4587-4601).  `bootstrap` is "host:port" of a TCP
 * rendezvous that rank 0 listens on; NULL reads COCO_BOOTSTRAP, else
 * MASTER_ADDR:MASTER_PORT+1.  The calling thread's current CUDA device
 * becomes the communicator's device. */
int cocoCommInitRank(cocoComm_t *comm, int world, int rank, const char *bootstrap);

/* Single-process variant (counterpart of ncclCommInitAll, used by
 * nccl-overlap/samples/single-process-adam-scattered.cu:179-281).  devices[i]
 * is the CUDA device of rank i; NULL means 0..n-1.  The same device may be
 * listed several times: those ranks become virtual ranks whose fused calls,
 * issued between cocoGroupStart/cocoGroupEnd, run as ONE cooperative launch
 * (kernels that wait for one another must never be separate launches on one
 * GPU). */
int cocoCommInitAll(cocoComm_t *comms, int n, const int *devices);

/* Collective in process mode (all ranks call it; bounded by the bootstrap's
 * timeout): every rank synchronises its device, symmetric allocations that
 * were not freed with cocoMemFree are released, and only when all ranks have
 * arrived are the peers' mappings closed and the flag page freed -- a peer may
 * still be finishing its last kernel on this rank's memory before that. */
int cocoCommDestroy(cocoComm_t comm);
int cocoCommCount(cocoComm_t comm, int *world);
int cocoCommUserRank(cocoComm_t comm, int *rank);
int cocoCommCuDevice(cocoComm_t comm, int *device);

/* What cocoCommInitRank learned about the links between the ranks' GPUs: the
 * counterpart of the reference's peer-access check and topology search
 * (nccl/src/transport/p2p.cc:118-238, nccl/src/graph/*.cc), reduced to what a
 * one-hop NVSwitch node needs.  Every rank asks the driver, for each peer's
 * GPU (found by PCI bus id), whether it can map that GPU's memory and at
 * which relative performance (cudaDeviceGetP2PAttribute), and the rows are
 * gathered over the bootstrap.  A pair WITHOUT peer access fails the
 * communicator at creation with cocoPeerError (the fused step is built on
 * peer loads and stores; there is no staged fallback); unequal performance
 * ranks are reported (uniform = 0, a warning under COCO_DEBUG=WARN) because
 * the one-shot exchange assumes every peer is equally near.
 * [a][b] is rank a's view of rank b's GPU; -1 = the driver did not say (the
 * peer's GPU is not visible to this process); the diagonal is 1 / 0 / 1. */
typedef struct {
  int world;
  int access[COCO_MAX_RANKS][COCO_MAX_RANKS];
  int perf_rank[COCO_MAX_RANKS][COCO_MAX_RANKS];
  int native_atomics[COCO_MAX_RANKS][COCO_MAX_RANKS];
  int uniform; /* every pair reachable, all known performance ranks equal */
} cocoTopology_t;
int cocoCommTopology(cocoComm_t comm, cocoTopology_t *topology);
/* The rule above on a caller-supplied table (row-major world x world, needs
 * no GPU): cocoPeerError if some access[a][b] == 0 for a != b, else
 * cocoSuccess with *uniform set. */
int cocoTopologyCheck(int world, const int *access, const int *perf_rank, int *uniform);

/* Host-side barrier and all-gather of small blobs over the bootstrap (what
 * the emitted programs used MPI_Barrier / MPI_Bcast for). */
int cocoBarrier(cocoComm_t comm);
int cocoAllGatherHost(cocoComm_t comm, const void *send, void *recv, size_t bytes_per_rank);

/* ---- host rendezvous, usable without a GPU ---------------------------------
 * What the emitted main() did with MPI_Init / MPI_Comm_rank / MPI_Bcast /
 * MPI_Barrier (src/codegen.cpp:4587-4601, 4471-4487): a star of TCP
 * connections to rank 0.  `addr` as for cocoCommInitRank.  Every call is
 * collective and bounded by timeout_ms (a missing rank yields cocoTimeout). */
typedef struct cocoBootstrap *cocoBootstrap_t;
int cocoBootstrapInit(cocoBootstrap_t *bs, int world, int rank, const char *addr, int timeout_ms);
int cocoBootstrapAllGather(cocoBootstrap_t bs, const void *send, void *recv, size_t bytes_per_rank);
int cocoBootstrapBarrier(cocoBootstrap_t bs);
int cocoBootstrapDestroy(cocoBootstrap_t bs);
/* RANK / WORLD_SIZE / LOCAL_RANK as set by torchrun-style launchers (0, 1, 0
 * when unset): how an emitted program finds its place without MPI. */
int cocoEnvRank(int *rank, int *world, int *local_rank);

/* Like ncclGroupStart/End: fused calls issued in between are launched at
 * cocoGroupEnd.  Required when several ranks share one device. */
int cocoGroupStart(void);
int cocoGroupEnd(void);

/* Collective.  Peer-maps [ptr, ptr+bytes) for the other ranks (CUDA IPC
 * between processes; peer access inside one process), the counterpart of the
 * reference's P2P transport set-up (nccl/src/transport/p2p.cc:118-238). */
int cocoRegister(cocoComm_t comm, void *ptr, size_t bytes);
/* Collective (for buffers registered by cocoRegister or on first use): every
 * rank unmaps its peers' buffers and waits for the others, so that the buffer
 * may be freed afterwards.  `ptr` is the pointer that was registered. */
int cocoDeregister(cocoComm_t comm, void *ptr);

/* Local (not collective).  Registers a buffer whose peer mappings the caller
 * already holds -- symmetric memory made with cuMemCreate/cuMemMap or by
 * another library: peer_ptrs[r] is this process's address of rank r's buffer
 * (peer_ptrs[rank] == ptr).  multicast_ptr, when not NULL, is an NVLS
 * multicast address bound to the same R buffers (cuMulticastCreate /
 * cuMulticastBindMem); it enables the NVSwitch path selected by
 * cocoSetAlgo(comm, 1) or COCO_ALGO=nvls: one multimem.ld_reduce per 16 bytes
 * for the reduce-scatter and one multimem.st for the all-gather.  The
 * reference's nearest counterpart is CollNet (nccl/src/collectives/device/
 * all_reduce_computation.h:262-316, left as assert(false) there). */
int cocoRegisterMapped(cocoComm_t comm, void *ptr, size_t bytes, void *const *peer_ptrs,
                       void *multicast_ptr);
/* Collective.  Symmetric device memory made by the runtime (the counterpart of
 * ncclMemAlloc + registration): `bytes` on every rank, each rank's buffer
 * mapped into every other rank (cuMemCreate, POSIX-fd exchange, cuMemMap) and,
 * where all devices support it, an NVSwitch multicast mapping over the R
 * buffers (cuMulticastCreate / BindMem).  The buffer is registered with the
 * communicator; put the gradients and the gathered weights in such buffers to
 * get the NVLS path without any other library.  At world size 1 this is
 * cudaMalloc.  COCO_NO_MULTICAST=1 skips the multicast mapping.  Free with
 * cocoMemFree (collective); what is still allocated when the communicator is
 * destroyed is released then. */
int cocoMemAlloc(cocoComm_t comm, void **ptr, size_t bytes);
int cocoMemFree(cocoComm_t comm, void *ptr);
int cocoMemHasMulticast(cocoComm_t comm, const void *ptr, int *yes);

/* 0: peer-to-peer loads and stores, gradients summed in fixed rank order
 * (results reproducible bit for bit).  1: NVLS wherever both buffers have a
 * multicast address (in-switch summation order; 16-bit sums delivered rounded
 * to 16 bits; within the stated tolerances, not bit-exact).  2 (default, also
 * COCO_ALGO=auto): NVLS from world size 4 on, where it moves fewer bytes per
 * link, but only for 16-bit gradients (tolerance rel 2e-3); fp32 gradients
 * keep the fixed-order peer-to-peer path, whose results are reproducible per
 * world size to the last bit (the rel 1e-5 contract), unless the caller asks
 * for the switch with algo 1.  Buffers without a multicast address always
 * take the peer-to-peer path. */
int cocoSetAlgo(cocoComm_t comm, int algo);

/* ---- the fused step -----------------------------------------------------
 * All three enqueue one kernel on `stream` and return.  grad_scale multiplies
 * the reduced gradient (1/loss_scale for mixed precision; pass 1.0f else).
 * step counts from 0 (the reference's `epoch`; t = step + 1). */

/* w' = w - lr * sum_r g_r   (examples/sgd/sgd.cpp:45-47, test-sgd.cu:17-23) */
int cocoFusedSGD(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                 cocoDataType_t lp_type, size_t count, float lr, float grad_scale,
                 cocoStream_t stream);

/* Replaces AllReduce_pipe(lr,beta1,beta2,g,w,halfw,m,v,count,...)
 * (nccl/src/nccl.h.in:211-212, nccl/src/collectives/all_reduce.cc:41-48). */
int cocoFusedAdam(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                  cocoDataType_t lp_type, float *m, float *v, size_t count, float lr,
                  float beta1, float beta2, float eps, int step, float grad_scale,
                  cocoVariant_t variant, cocoStream_t stream);

/* Replaces the LAMB form AllReduce_pipe(...,m,v,r,count,...)
 * (nccl/src/nccl.h.in:214-215, all_reduce.cc:50-58).  No `r` buffer is
 * needed: r is recomputed from m, v, w in the second phase, as the
 * reference's host checker does (multi-process-adam-scattered.cpp:427-431). */
int cocoFusedLAMB(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                  cocoDataType_t lp_type, float *m, float *v, size_t count, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step,
                  float grad_scale, cocoVariant_t variant, unsigned flags, cocoStream_t stream);

/* One LAMB step on ONE GPU (world size 1, bias-corrected formulation, same
 * arguments and arithmetic as cocoFusedLAMB) for callers that may not
 * allocate device memory when they step the optimizer: with a frozen or fully
 * reserved memory pool, near the device's memory limit, or in a loop that
 * must stay clear of the driver's allocation locks.  It needs no communicator and calls no
 * cudaMalloc/cudaFree nor any allocating library routine: the kernel's scratch
 * (CTA counters, per-CTA partial norms, status; about 33 KB) lives in a fixed
 * __device__ array inside the library image, held by every GPU that loads the
 * library until the process exits.
 *  - Limit: count <= COCO_NO_ALLOC_MAX_COUNT, else cocoInvalidArgument.
 *  - The first call on a device looks up the array's device address (once per
 *    device, with that device current); make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the array: two calls whose kernels overlap
 *    on the GPU race.  Serialise them (one stream, or events).
 *  - The current device is used; m, v hold `count` elements.
 * This entry point has no counterpart in the reference. */
#define COCO_NO_ALLOC_MAX_COUNT (1ull << 31)
int cocoLambStepNoAlloc(const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                        cocoDataType_t lp_type, float *m, float *v, size_t count, float lr,
                        float beta1, float beta2, float eps, float weight_decay, int step,
                        float grad_scale, cocoStream_t stream);

/* ---- lists of tensors ("scattered" calls) -----------------------------------
 * Replace ncclAllReduceScatteredWeights / ...Adam of the reference's second
 * NCCL fork (nccl-overlap/src/collectives/all_reduce.cc:21-59; kernel
 * nccl-overlap/src/collectives/device/all_reduce_scattered.h:15-105): the
 * parameters are nbuff separate tensors (g[b], w[b] of counts[b] elements,
 * e.g. one per layer) instead of one flat buffer; ONE kernel per step still.
 * The tensors form a virtual flat buffer in which tensor b starts at the next
 * multiple of 8 elements; that buffer is sliced over the ranks like a single
 * tensor with slices of cocoScatteredSliceElems elements, and m, v are
 * slice-local arrays of that many fp32 elements.  Every rank passes the same
 * list in the same order; each tensor is peer-mapped on first use.  fp32
 * weights are gathered (no low-precision copy); peer-to-peer path.
 * cocoFusedLAMBScattered replaces ncclAllReduceScatteredLAMB (all_reduce.cc:
 * 61-75; all_reduce_scattered.h:106-282): the trust ratio is PER TENSOR, from
 * ||w_b|| and ||r_b|| of tensor b alone (double sums, fixed order: CTA, rank),
 * exchanged between the ranks whose slices hold parts of b; everything else is
 * cocoFusedLAMB's arithmetic, `flags` included.  At most COCO_MAX_LAMB_TENSORS
 * tensors per call. */
int cocoScatteredSliceElems(size_t nbuff, const size_t *counts, int world, size_t *slice_elems);
/* Where tensor `tensor` of such a list lives in the flat Sliced moments (host
 * only, no GPU needed; e.g. to save or reload the optimizer state of one layer):
 * element e of the tensor is element flat_offset + e of the virtual flat buffer,
 * i.e. element (flat_offset + e) % slice_elems of m / v on rank
 * (flat_offset + e) / slice_elems; first_rank..last_rank are the ranks that hold
 * a part of it (first_rank = last_rank = -1 for an empty tensor).  No reference
 * counterpart: the fork indexes full-size moment arrays by global element. */
int cocoScatteredTensorPlace(size_t nbuff, const size_t *counts, int world, size_t tensor,
                             size_t *flat_offset, int *first_rank, int *last_rank);
int cocoFusedSGDScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                          cocoDataType_t g_type, float *const *w, const size_t *counts, float lr,
                          float grad_scale, cocoStream_t stream);
int cocoFusedAdamScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                           cocoDataType_t g_type, float *const *w, const size_t *counts, float *m,
                           float *v, float lr, float beta1, float beta2, float eps, int step,
                           float grad_scale, cocoVariant_t variant, cocoStream_t stream);

int cocoFusedLAMBScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                           cocoDataType_t g_type, float *const *w, const size_t *counts, float *m,
                           float *v, float lr, float beta1, float beta2, float eps,
                           float weight_decay, int step, float grad_scale, cocoVariant_t variant,
                           unsigned flags, cocoStream_t stream);

/* ---- stand-alone collectives (fp32, sum) ------------------------------------
 * What the unfused schedules of a generated program call where the reference
 * emits ncclAllReduce / ncclReduceScatter / ncclAllGather
 * (src/codegen.cpp:4146-4189), on the runtime's own peer memory: `count` is the
 * TOTAL element count N; slices are those of cocoSliceBounds.
 *   cocoAllReduce      buf[0..N) on every rank becomes the sum over ranks
 *   cocoReduceScatter  recv[0..S_r) = sum over ranks of send[lo_r .. hi_r)
 *   cocoAllGather      recv[lo_r .. hi_r) on every rank = rank r's send[0..S_r)
 * Buffers that peers touch (buf; send of a reduce-scatter; recv of an
 * all-gather) are peer-mapped on first use like the fused calls' buffers. */
int cocoAllReduce(cocoComm_t comm, float *buf, size_t count, cocoStream_t stream);
int cocoReduceScatter(cocoComm_t comm, const float *send, float *recv, size_t count,
                      cocoStream_t stream);
int cocoAllGather(cocoComm_t comm, const float *send, float *recv, size_t count,
                  cocoStream_t stream);

/* Prepares one fused step whose update the CALLER supplies as a device
 * functor (include/coconet_fused_generic.cuh: cocoLaunchGenericFused): peer
 * views of g and w, flag pages, sequence number and launch shape.  Collective
 * like the fused calls; call it once per step, then launch.  The counterpart
 * of the template-filling generator the reference left unreachable
 * (src/codegen.cpp:1948-3929). */
struct cocoGenericPlan;
int cocoFusedGenericPlan(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w,
                         size_t count, float grad_scale, cocoStream_t stream,
                         struct cocoGenericPlan *plan);

/* Collective diagnostic: what the links between the ranks' GPUs give a kernel
 * with the fused step's access shape and nothing else to do.  `buf` holds
 * `bytes` on every rank (16-byte aligned; peer-mapped on first use like the
 * fused calls' buffers; its contents are overwritten).  mode 0: every rank
 * pulls its slice of `buf` from all peers with 16-byte loads, `unroll` (1, 2
 * or 4) units in flight per thread and peer; 1: pushes its slice to all peers
 * with 16-byte stores; 2: both at once (the fused step's traffic without the
 * update); 3: the copy engine moves half of the next rank's buffer
 * (cudaMemcpyAsync; `unroll` ignored); 4 / 5 / 6: the same three through the
 * NVSwitch -- one multimem.ld_reduce per 16 bytes of the rank's slice, one
 * multimem.st, or both (`buf` must come from cocoMemAlloc with a multicast
 * mapping, else cocoInvalidUsage; its bytes are read as fp32); 7: both ways
 * at once -- the even CTAs take the first `unroll` sixteenths of the slice
 * through the switch, the odd CTAs the rest peer to peer -- and the result is
 * the time of one iteration in MICROSECONDS instead of a rate (it tells
 * whether the two kinds of traffic overlap or compete).  One untimed iteration, then `iters`
 * timed with CUDA events on `stream`; the call synchronises the stream.
 * *gbs_per_direction = bytes that cross one GPU's links in one direction per
 * iteration / the slowest rank's time per iteration, in GB/s (0 at world size
 * 1), identical on all ranks.  The reference has no counterpart: its kernels
 * were only timed end to end (experiments/generate-pdf/dsl_vs_apex.py:93-96). */
int cocoLinkProbe(cocoComm_t comm, void *buf, size_t bytes, int mode, int unroll, int iters,
                  double *gbs_per_direction, cocoStream_t stream);

/* Norms of the last LAMB step on this communicator: out[0] = ||w||,
 * out[1] = ||r|| as used for the trust ratio.  Synchronise the stream first. */
int cocoLastLambNorms(cocoComm_t comm, double out[2]);

/* Where the last fused call on this communicator spent its time, as seen by
 * CTA 0 of this rank, in nanoseconds of the GPU's timer: out[0] = from the
 * start barrier to the end of the first data phase (LAMB: reduce + moments +
 * norms; otherwise 0), out[1] = the exchange of the norms (LAMB; otherwise
 * 0), out[2] = the last data phase (LAMB: scale + gather; otherwise the
 * whole reduce + update + gather).  Synchronise the stream first.  The
 * reference has no counterpart; its programs time whole stages with events
 * (src/codegen.cpp:4330-4380). */
int cocoLastPhaseTimes(cocoComm_t comm, unsigned long long out_ns[3]);

/* How evenly the last fused call's work was spread over this rank's CTAs:
 * the time from the start barrier to the end of a CTA's data, in nanoseconds
 * of the GPU's timer, for the CTA that finished first (out[0]), the median
 * CTA (out[1]) and the last (out[2]).  The step ends with the last.
 * Synchronise the stream first.  No reference counterpart. */
int cocoLastCtaSpread(cocoComm_t comm, unsigned long long out_ns[3]);

/* First device-side failure since the last call (then cleared); the
 * counterpart of ncclCommGetAsyncError (nccl/src/init.cc:996-1021). */
int cocoGetStatus(cocoComm_t comm, cocoStatus_t *status);

/* Slice bounds of `rank` for `count` elements over `world` ranks. */
int cocoSliceBounds(size_t count, int world, int rank, size_t *begin, size_t *end);

/* Per-launch tunables (also COCO_CTAS_PER_SM / COCO_THREADS / COCO_TIMEOUT_MS
 * in the environment, in the style of NCCL_PARAM, nccl/src/include/param.h:
 * 48-64).  Values <= 0 keep the current setting. */
int cocoSetTunables(cocoComm_t comm, int ctas_per_sm, int threads, int timeout_ms);

/* Number of kernels this communicator has launched (for accounting). */
int cocoLaunchCount(cocoComm_t comm, uint64_t *launches);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* COCONET_RT_H_ */
