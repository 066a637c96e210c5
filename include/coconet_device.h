// Device-side ABI of the fused step: the argument blocks a kernel receives and
// the peer-visible flag page.  Shared by the runtime library and by kernels
// that programs instantiate themselves (coconet_fused_generic.cuh).  CUDA C++.
#ifndef COCONET_DEVICE_H_
#define COCONET_DEVICE_H_

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "coconet_rt.h"

namespace coco {

constexpr int kMaxRanks = COCO_MAX_RANKS;
constexpr int kMaxCtasPerRank = 2048;  // rows of the per-CTA partial-norm table
constexpr int kMaxLambTensors = COCO_MAX_LAMB_TENSORS;  // tensors of one scattered LAMB call

enum Opt : int { kSGD = 0, kAdam = 1, kLAMB = 2 };

// Phases recorded in the status word when a bounded wait gives up.
enum Phase : int { kPhaseStart = 1, kPhaseNorm = 2, kPhaseEnd = 3, kPhaseCopy = 4, kPhaseCheck = 5 };

// One per rank, in device memory, mapped into every peer.  Zero at creation;
// every flag only ever grows (it holds the sequence number of a fused call),
// so nothing is reset between steps and a late reader can never miss a value.
struct FlagPage {
  // --- written by peers (slot = writer's rank), polled locally -------------
  unsigned long long arrive[kMaxRanks];     // "my kernel for call seq has started"
  unsigned long long done[kMaxRanks];       // "all my reads/writes of call seq are complete"
  unsigned long long norm_flag[kMaxRanks];  // "norm_part[slot] of call seq is valid"
  double norm_part[kMaxRanks][2];           // per-rank partial sums {sum w^2, sum r^2}
  // --- local only ---------------------------------------------------------
  unsigned int done_count;  // CTAs of this rank that finished their data phase
  unsigned int norm_count;  // CTAs of this rank that posted their partial norms
  int status[8];            // cocoStatus_t image: code, rank, phase, peer, seq lo/hi
  double last_norms[2];     // {||w||, ||r||} of the last LAMB step
  // GPU timer (ns) at which this rank's CTA 0 passed, in the last fused call: the start
  // barrier, the end of its first data phase (LAMB), the arrival of all ranks' norms (LAMB),
  // the end of its data; entries a call does not pass are set to the previous one
  unsigned long long phase_ns[4];
  double cta_part[kMaxCtasPerRank][2];
  // GPU timer (ns) at which every CTA of this rank finished its data in the last fused call
  unsigned long long cta_end_ns[kMaxCtasPerRank];
  // multi-rank kernels that hand their work out warp by warp: the next chunk to take (set
  // back to zero by the rank's last CTA at the end barrier)
  unsigned int work_next;
  unsigned int pad_;
};

// Per-tensor norm partials of a scattered LAMB call.  A communicator allocates
// its flag page and this table as ONE peer-mapped block, the table right
// behind the page (tensor_norms_of); pages made elsewhere have no table.
struct TensorNorms {
  // written by peers (first index = writer's rank): {sum w^2, sum r^2} of the
  // part of tensor b that lies in the writer's slice; valid for call seq once
  // the writer's norm_flag says so, and only for writers whose slice meets b
  double part[kMaxRanks][kMaxLambTensors][2];
};
__host__ __device__ inline TensorNorms *tensor_norms_of(FlagPage *page) {
  return reinterpret_cast<TensorNorms *>(page + 1);
}

// One piece of a rank's slice when the parameters are a LIST of tensors
// (scattered calls): the part of one tensor that falls into the slice.
struct Segment {
  const void *g[kMaxRanks];   // that tensor's gradient on every rank, element 0
  void *out[kMaxRanks];       // that tensor's weights on every rank, element 0
  float *w;                   // own weights of the tensor, element 0
  float *m;                   // own moments, positioned so that [i - begin] is element i's
  float *v;
  unsigned long long begin;   // first element of the tensor inside the slice
  unsigned long long len;     // number of elements
  int aligned16;
  int tensor;
  unsigned long long tensor_len;  // elements of the whole tensor
  int first_rank, last_rank;      // ranks whose slices hold a part of the tensor
  unsigned long long chunk0;      // number of chunks in the pieces before this one
};
// A list of tensors is walked in chunks of 2^RankArgs::chunk_shift elements, one CTA per
// chunk at a time.  The host picks the size per call: large enough that the lookup between
// two chunks is rare (64 Ki elements: 32 passes of a 512-thread CTA), small enough that
// every CTA gets at least kSegChunksPerCta of them, so that the last, partly filled round
// of the walk stays a few percent of the step.
constexpr int kSegChunkShiftMin = 13, kSegChunkShiftMax = 16;
constexpr int kSegChunksPerCta = 16;
constexpr int kSegWords = 25;         // a Segment is this many 8-byte words
constexpr int kSegPointerWords = 2 * kMaxRanks + 3;  // g, out, w, m, v: the words a RankArgs starts with too
constexpr int kSegPartPerChunk = 16;  // scattered LAMB: partial sums kept per chunk (one per warp of a CTA)

// Per-rank pointers of one fused call.  Indexed tables hold the view THIS
// rank has of every peer's buffer (entry [rank] is the rank's own buffer).
// The first kSegPointerWords words are laid out like a Segment's, so that a
// piece of a list of tensors is entered by copying those words.
struct RankArgs {
  const void *g[kMaxRanks];   // gradients of each peer, element 0
  void *out[kMaxRanks];       // gathered output of each peer (fp32 w, or w_lp), element 0
  float *w;                   // own fp32 weights, element 0 (N elements)
  float *m;                   // own first moment, slice-local (S elements)
  float *v;                   // own second moment, slice-local
  FlagPage *flags[kMaxRanks]; // flag page of each peer
  const void *mc_g;           // NVLS multicast address of the gradient buffers, or null
  void *mc_out;               // NVLS multicast address of the gathered output, or null
  int rank;
  int aligned16;              // non-zero: slice start and all pointers are 16-byte aligned
  const Segment *segs;        // scattered calls: this rank's segments (device memory)
  int nseg;
  int nchunk;                 // chunks of all segments together
  int chunk_shift;            // log2 of the elements per chunk
  int pad_;
  double *seg_part;           // scattered LAMB: [chunk][2] partial sums of this rank's pieces, then [chunk][warp][2]
};
static_assert(sizeof(Segment) == kSegWords * 8, "Segment is walked as 8-byte words");
static_assert(offsetof(Segment, g) == offsetof(RankArgs, g) && offsetof(Segment, out) == offsetof(RankArgs, out) &&
                  offsetof(Segment, w) == offsetof(RankArgs, w) && offsetof(Segment, m) == offsetof(RankArgs, m) &&
                  offsetof(Segment, v) == offsetof(RankArgs, v) &&
                  offsetof(Segment, begin) == kSegPointerWords * 8,
              "a Segment's pointers and a RankArgs' pointers share one layout");

// Internal StepArgs::flags bit (public flags use the low byte).
constexpr unsigned kFlagNvls = 0x100u;  // reduce / gather through NVSwitch multicast
constexpr unsigned kFlagScattered = 0x200u;  // the parameters are a list of tensors (RankArgs::segs)
constexpr unsigned kFlagNoGather = 0x400u;   // generic kernel: do not store the result to the ranks
constexpr unsigned kFlagNoReduce = 0x800u;   // generic kernel: do not read the ranks' gradients

// Scalars of one fused call, identical on every rank.
struct StepArgs {
  unsigned long long count;   // N
  unsigned long long seq;     // sequence number of this call on the communicator (>= 1)
  unsigned long long timeout_ns;
  int world;
  int variant;                // cocoVariant_t
  unsigned flags;
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  float d1, d2;               // denominators of m^ = m/d1, v^ = v/d2 ...
  double d1d, d2d;            // ... in double for the bias-corrected form
  int pipe_stages;            // stages of each warp's gradient ring (bulk copies), 0 = off
  int pad;
  // Derived on the host so that the kernel reads them as constants instead of
  // holding them in registers: 1 - beta (float subtraction), 1/d in double.
  float omb1, omb2;
  double r1d, r2d;
};

}  // namespace coco

#endif  // COCONET_DEVICE_H_
