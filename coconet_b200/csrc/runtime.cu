// Host side of the C ABI declared in coconet_rt.h: communicators, peer
// mapping of caller buffers, the flag page, launch configuration.
//
// Replaces, for the fused optimizer step only, what the reference gets from
// its NCCL 2.6.4 fork (parasailteam/coconet): communicator set-up
// (nccl/src/init.cc), the P2P transport's IPC mapping
// (nccl/src/transport/p2p.cc:118-238), argument marshalling and launch
// (nccl/src/enqueue.cc:200-343) and async error reporting
// (nccl/src/init.cc:972-1021).
#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "bootstrap.h"
#include "coconet_rt.h"
#include "coconet_fused_generic.cuh"
#include "fused_step.cuh"

using namespace coco;

namespace {

int env_int(const char *name, int dflt) {
  const char *e = getenv(name);
  if (!e || !e[0]) return dflt;
  return atoi(e);
}

int debug_level() {
  static int lvl = [] {
    const char *e = getenv("COCO_DEBUG");
    if (!e) return 0;
    if (!strcmp(e, "INFO")) return 2;
    if (!strcmp(e, "WARN")) return 1;
    return atoi(e);
  }();
  return lvl;
}

#define COCO_WARN(...)                      \
  do {                                      \
    if (debug_level() >= 1) {               \
      fprintf(stderr, "[coconet_rt] WARN ");\
      fprintf(stderr, __VA_ARGS__);         \
      fprintf(stderr, "\n");                \
    }                                       \
  } while (0)
#define COCO_INFO(...)                      \
  do {                                      \
    if (debug_level() >= 2) {               \
      fprintf(stderr, "[coconet_rt] INFO ");\
      fprintf(stderr, __VA_ARGS__);         \
      fprintf(stderr, "\n");                \
    }                                       \
  } while (0)

#define CUDA_TRY(expr)                                                            \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess) {                                                      \
      COCO_WARN("%s:%d %s -> %s", __FILE__, __LINE__, #expr, cudaGetErrorString(e_)); \
      (void)cudaGetLastError();                                                   \
      return cocoCudaError;                                                       \
    }                                                                             \
  } while (0)

#define COCO_TRY(expr)             \
  do {                             \
    int r_ = (expr);               \
    if (r_ != cocoSuccess) return r_; \
  } while (0)

size_t dtype_size(cocoDataType_t t) {
  switch (t) {
    case cocoFloat32: return 4;
    case cocoFloat16:
    case cocoBfloat16: return 2;
  }
  return 0;
}

// A caller buffer that peers can address.  peer[r] is this rank's view of
// rank r's buffer start (peer[rank] == base).
struct Region {
  char *base = nullptr;
  size_t bytes = 0;
  char *peer[kMaxRanks] = {};
  char *multicast = nullptr;  // NVLS address of the same buffers, when the caller mapped one
  std::vector<std::string> ipc_keys;  // mappings this region holds a reference on
  bool external = false;              // registered with cocoRegisterMapped: nothing to close
};

struct IpcMapping {
  void *base = nullptr;
  int refs = 0;
};

struct IpcBlob {
  cudaIpcMemHandle_t handle;
  unsigned long long offset;  // of the registered pointer inside its allocation
  unsigned long long bytes;
  int valid;
  int pad;
};

// One fused call waiting for its launch (single-process groups).
struct PendingCall {
  int opt = 0;
  cocoDataType_t g_type = cocoFloat32, lp_type = cocoFloat16;
  const void *g = nullptr;
  float *w = nullptr;
  void *w_lp = nullptr;
  float *m = nullptr, *v = nullptr;
  StepArgs sa = {};
  cudaStream_t stream = nullptr;
  // stand-alone collective of a single-process group (kCollAllReduce ...), 0 = a fused step
  int coll = 0;
  void *aux = nullptr;  // reduce-scatter: recv; all-gather: send
  // scattered calls: the parameters are lists of tensors
  std::vector<const void *> sg;
  std::vector<float *> sw;
  std::vector<size_t> scounts;
};

// Flat layout of a list of tensors: each tensor starts at a multiple of 8
// elements of a virtual flat buffer that is sliced over the ranks like a
// single tensor (slice length a multiple of 8 too), so that every piece keeps
// 16-byte alignment in the moments whatever the tensors' sizes.
struct FlatLayout {
  std::vector<size_t> off;
  size_t total = 0;
  size_t slice = 0;
};
FlatLayout flat_layout(const size_t *counts, size_t n, int world) {
  FlatLayout L;
  L.off.resize(n);
  size_t at = 0;
  for (size_t b = 0; b < n; ++b) {
    L.off[b] = at;
    at += (counts[b] + 7) / 8 * 8;
  }
  L.total = at;
  L.slice = ((at + world - 1) / world + 7) / 8 * 8;
  return L;
}

struct LocalGroup;  // ranks that live in one process

constexpr size_t kCommPageBytes = sizeof(FlagPage) + sizeof(TensorNorms);
// per device of a single-process group: the virtual ranks' argument blocks and,
// behind them, one pointer-sized functor per rank for the stand-alone collectives
constexpr size_t kGroupTableBytes = sizeof(RankArgs) * kMaxRanks + 16 * kMaxRanks;

}  // namespace

struct cocoComm {
  int world = 1, rank = 0, device = 0;
  int sm_count = 0;
  bool coop_supported = false;
  // process mode
  std::unique_ptr<Bootstrap> boot;
  std::vector<Region> regions;
  std::map<std::string, IpcMapping> ipc_open;  // "<peer>:<handle bytes>" -> mapped base
  // single-process mode
  std::shared_ptr<LocalGroup> group;
  bool has_pending = false;
  PendingCall pending;
  // both
  FlagPage *flags = nullptr;
  FlagPage *peer_flags[kMaxRanks] = {};
  unsigned long long seq = 0;
  unsigned long long launches = 0;
  unsigned long long session = 0;  // random id shared by the ranks (names of side channels)
  std::vector<Segment> seg_host;   // last segment table uploaded
  Segment *seg_dev = nullptr;
  size_t seg_cap = 0;
  double *seg_part = nullptr;      // scattered LAMB: per-segment, per-CTA partial sums
  size_t seg_part_cap = 0;         // in doubles
  int ctas_per_sm = 0;  // 0 = automatic
  int threads = 512;
  int timeout_ms = 10000;
  int smem_budget_kb = 200;  // shared memory the warp rings may use per SM
  int pipeline = -1;         // COCO_PIPELINE: 1 warp rings (bulk copies), 0 register-staged, unset: by world size
  int ring_stages = 0;       // COCO_RING_STAGES: cap on the stages of a ring, 0 = as many as fit
  int seg_chunk_shift = 0;   // COCO_SEG_CHUNK_SHIFT: log2 of the chunk of a list walk, 0 = by size
  int last_ctas = 0;         // CTAs of this rank in the last fused launch
  int algo = 2;              // 0 p2p, 1 nvls, 2 auto (COCO_ALGO=p2p|nvls|auto)
  cocoTopology_t topo = {};  // peer access / performance between the ranks' GPUs
};

namespace {

struct LocalGroup {
  std::vector<cocoComm *> comms;         // index = rank
  std::map<int, RankArgs *> table_dev;   // device -> table for virtual ranks (+ kMaxRanks pointers behind it)
  std::mutex mu;
};

thread_local int g_group_depth = 0;
thread_local std::vector<cocoComm *> g_group_touched;

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
    if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

int init_common(cocoComm *c) {
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, c->device));
  c->sm_count = prop.multiProcessorCount;
  c->coop_supported = prop.cooperativeLaunch != 0;
  c->ctas_per_sm = env_int("COCO_CTAS_PER_SM", 0);
  c->threads = env_int("COCO_THREADS", 512);
  if (c->threads < 32 || c->threads > 512 || (c->threads % 32) != 0) c->threads = 512;
  c->pipeline = env_int("COCO_PIPELINE", -1);
  c->ring_stages = env_int("COCO_RING_STAGES", 0);
  c->seg_chunk_shift = env_int("COCO_SEG_CHUNK_SHIFT", 0);
  {
    const char *algo = getenv("COCO_ALGO");
    c->algo = !algo ? 2 : !strcmp(algo, "nvls") ? 1 : !strcmp(algo, "p2p") ? 0 : 2;
  }
  c->smem_budget_kb = std::max(16, std::min(220, env_int("COCO_SMEM_KB", 200)));
  c->timeout_ms = env_int("COCO_TIMEOUT_MS", 10000);
  if (c->timeout_ms <= 0) c->timeout_ms = 10000;
  // one block: the flag page, and behind it the per-tensor norm table of
  // scattered LAMB calls (tensor_norms_of)
  CUDA_TRY(cudaMalloc((void **)&c->flags, kCommPageBytes));
  CUDA_TRY(cudaMemset(c->flags, 0, kCommPageBytes));
  CUDA_TRY(cudaDeviceSynchronize());
  c->peer_flags[c->rank] = c->flags;
  return cocoSuccess;
}

// ---- process mode: CUDA IPC ------------------------------------------------
int alloc_range(const void *ptr, char **base, size_t *size) {
  // The driver entry point is looked up at run time so that the library has
  // no link-time dependency on libcuda (it must load on machines without a
  // driver, e.g. to list its symbols).
  typedef CUresult (*GetRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
  static GetRangeFn fn = [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess)
      f = nullptr;
    return (GetRangeFn)f;
  }();
  if (!fn) return cocoCudaError;
  CUdeviceptr b = 0;
  size_t s = 0;
  CUresult r = fn(&b, &s, (CUdeviceptr)ptr);
  if (r != CUDA_SUCCESS) return cocoInvalidArgument;
  *base = (char *)b;
  *size = s;
  return cocoSuccess;
}

int map_region_ipc(cocoComm *c, void *ptr, size_t bytes, Region *out) {
  IpcBlob mine;
  memset(&mine, 0, sizeof(mine));
  char *abase = nullptr;
  size_t asize = 0;
  int rc = alloc_range(ptr, &abase, &asize);
  if (rc == cocoSuccess) {
    cudaError_t e = cudaIpcGetMemHandle(&mine.handle, abase);
    if (e == cudaSuccess) {
      mine.offset = (unsigned long long)((char *)ptr - abase);
      mine.bytes = bytes;
      mine.valid = 1;
    } else {
      COCO_WARN("cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
    }
  }
  // Always take part in the exchange so that a local failure cannot leave
  // the peers blocked in the collective.
  std::vector<IpcBlob> all(c->world);
  COCO_TRY(c->boot->all_gather(&mine, all.data(), sizeof(IpcBlob)));
  for (int r = 0; r < c->world; ++r)
    if (!all[r].valid) return cocoCudaError;

  out->base = (char *)ptr;
  out->bytes = bytes;
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) {
      out->peer[r] = (char *)ptr;
      continue;
    }
    if (all[r].bytes < bytes) return cocoInvalidUsage;  // ranks disagree on the size
    std::string key = std::to_string(r) + ":" +
                      std::string((const char *)&all[r].handle, sizeof(cudaIpcMemHandle_t));
    void *mapped = nullptr;
    auto it = c->ipc_open.find(key);
    if (it != c->ipc_open.end()) {
      mapped = it->second.base;
      it->second.refs++;
    } else {
      cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        COCO_WARN("cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        (void)cudaGetLastError();
        return cocoPeerError;
      }
      IpcMapping mp;
      mp.base = mapped;
      mp.refs = 1;
      c->ipc_open[key] = mp;
    }
    out->ipc_keys.push_back(key);
    out->peer[r] = (char *)mapped + all[r].offset;
  }
  return cocoSuccess;
}

const Region *find_region(const cocoComm *c, const void *ptr, size_t bytes) {
  const char *p = (const char *)ptr;
  for (const Region &r : c->regions)
    if (p >= r.base && p + bytes <= r.base + r.bytes) return &r;
  return nullptr;
}

// Peer views of [ptr, ptr+bytes); registers the buffer on first use.
int peer_views(cocoComm *c, const void *ptr, size_t bytes, char *views[kMaxRanks],
               char **multicast) {
  *multicast = nullptr;
  if (c->world == 1) {
    views[0] = (char *)ptr;
    return cocoSuccess;
  }
  const Region *r = find_region(c, ptr, bytes);
  if (!r) {
    Region fresh;
    COCO_TRY(map_region_ipc(c, (void *)ptr, bytes, &fresh));
    c->regions.push_back(fresh);
    r = &c->regions.back();
    COCO_INFO("rank %d registered %p (+%zu bytes)", c->rank, ptr, bytes);
  }
  const size_t off = (const char *)ptr - r->base;
  for (int p = 0; p < c->world; ++p) views[p] = r->peer[p] + off;
  if (r->multicast) *multicast = r->multicast + off;
  return cocoSuccess;
}

// ---- launch configuration ---------------------------------------------------
bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

// Which data path serves the peer-to-peer step when COCO_PIPELINE is unset:
// the warp rings from four ranks on for SGD and Adam (measured 6 % faster than
// the register-staged path at four and at eight GPUs, slower at two: 1.66
// against 1.77 ms, 1.97 against 2.09 ms and 1.30 against 1.17 ms for the
// 334 M-element mixed-precision step), the register-staged path below that,
// for LAMB (4.15 against 4.19 ms at eight GPUs: its second phase is the same
// in both) and for virtual ranks sharing a GPU.
bool ring_by_default(int opt, int world, int nvirt) { return world >= 4 && nvirt <= 1 && opt != kLAMB; }

int pick_launch(const cocoComm *c, int opt, cocoDataType_t g_type, bool has_lp,
                cocoDataType_t lp_type, size_t count, int world, int nvirt, StepArgs *sa,
                LaunchConfig *cfg) {
  const bool coop = (opt == kLAMB) || nvirt > 1;
  if (coop && !c->coop_supported) return cocoInvalidUsage;
  const size_t slice = (count + world - 1) / world;

  // Warp rings (gradients staged in shared memory by bulk copies): every warp
  // of a CTA holds D stages of `world` 512-byte tiles.  As many stages (up to
  // 4, or COCO_RING_STAGES) as fit the shared-memory budget of one CTA; off
  // when the slice has no full tile, for lists of tensors and on the NVLS path.
  int want_per_sm = c->ctas_per_sm > 0 ? c->ctas_per_sm : 2;
  // block size of the multi-rank paths (the ring's shared memory depends on it)
  const size_t warps = (size_t)std::min(c->threads, fused_step_block_threads(0, g_type)) / 32;
  const size_t stage_bytes = (size_t)world * kRingTileBytesPerRank * warps;
  const size_t tile_elems = 32 * (16 / dtype_size(g_type));
  int stages = 0;
  const bool ring_wanted = c->pipeline > 0 || (c->pipeline < 0 && ring_by_default(opt, world, nvirt));
  if (ring_wanted && slice >= tile_elems && !(sa->flags & (kFlagScattered | kFlagNvls))) {
    const size_t budget_sm = (size_t)c->smem_budget_kb * 1024;
    // at large world sizes one stage of two CTAs may not fit: one CTA per SM then
    if (budget_sm / want_per_sm < stage_bytes && c->ctas_per_sm <= 0) want_per_sm = 1;
    stages = (int)std::min<size_t>(kRingStagesMax, budget_sm / want_per_sm / stage_bytes);
    if (c->ring_stages > 0) stages = std::min(stages, c->ring_stages);
    if (stages < 1) stages = 0;
  }
  sa->pipe_stages = stages;
  cfg->smem_bytes = (size_t)stages * stage_bytes;
  const int path = fused_step_path(*sa);
  const int threads = std::min(c->threads, fused_step_block_threads(path, g_type));

  int occ = 0;
  CUDA_TRY(fused_step_occupancy(opt, g_type, has_lp, lp_type, path, threads, cfg->smem_bytes, &occ));
  if (occ < 1) return cocoInternalError;
  int per_sm = std::min(want_per_sm, occ);
  long ctas = (long)per_sm * c->sm_count;
  if (nvirt > 1) ctas = std::max(1L, ((long)occ * c->sm_count) / nvirt);
  // no more CTAs than there is work: one warp tile (or 16-byte unit) per thread pass
  const size_t vec = 4;
  const size_t per_cta = stages > 0 ? tile_elems * warps : vec * (size_t)threads;
  const long need = (long)std::max<size_t>(1, (slice + per_cta - 1) / per_cta);
  ctas = std::max(1L, std::min(ctas, need));
  ctas = std::min<long>(ctas, kMaxCtasPerRank);
  cfg->ctas = (int)ctas;
  cfg->threads = threads;
  cfg->nvirt = nvirt;
  cfg->cooperative = coop;
  return cocoSuccess;
}

int validate(const cocoComm *c, const PendingCall &pc) {
  if (!c) return cocoInvalidArgument;
  if (!pc.scounts.empty()) {
    if (pc.w_lp) return cocoInvalidArgument;  // low-precision copies of a list: not built
    if (pc.opt == kLAMB && pc.scounts.size() > (size_t)kMaxLambTensors) return cocoInvalidArgument;
    for (size_t b = 0; b < pc.scounts.size(); ++b)
      if (!pc.sg[b] || !pc.sw[b]) return cocoInvalidArgument;
  } else if (!pc.g || !pc.w) {
    return cocoInvalidArgument;
  }
  if (dtype_size(pc.g_type) == 0) return cocoInvalidArgument;
  if (pc.w_lp && pc.lp_type != cocoFloat16 && pc.lp_type != cocoBfloat16)
    return cocoInvalidArgument;
  if (pc.opt != kSGD && (!pc.m || !pc.v)) return cocoInvalidArgument;
  if (pc.sa.variant < cocoVariantOverlap || pc.sa.variant > cocoVariantNccl)
    return cocoInvalidArgument;
  if (pc.sa.variant == cocoVariantNccl) {
    // the forked-NCCL formulations (Adam, LAMB) are defined for fp16 gradients
    // + fp16 copy of one flat buffer only
    if (pc.opt == kSGD || pc.g_type != cocoFloat16 || !pc.w_lp || pc.lp_type != cocoFloat16 ||
        !pc.scounts.empty())
      return cocoInvalidArgument;
  }
  if (pc.sa.variant == cocoVariantDsl && pc.opt == kAdam && !(pc.sa.beta1 != 0.f && pc.sa.beta2 != 0.f))
    return cocoInvalidArgument;
  return cocoSuccess;
}

void fill_rank_args(RankArgs *ra, int rank, int world, char *const g_views[], char *const out_views[],
                    FlagPage *const flags[], const PendingCall &pc) {
  memset(ra, 0, sizeof(*ra));
  bool ok16 = aligned16(pc.w) && (pc.opt == kSGD || (aligned16(pc.m) && aligned16(pc.v)));
  for (int p = 0; p < world; ++p) {
    ra->g[p] = g_views[p];
    ra->out[p] = out_views[p];
    ra->flags[p] = flags[p];
    ok16 = ok16 && aligned16(g_views[p]) && aligned16(out_views[p]);
  }
  ra->w = pc.w;
  ra->m = pc.m;
  ra->v = pc.v;
  ra->rank = rank;
  const size_t S = (pc.sa.count + world - 1) / world;
  const size_t vec = 8;  // 16 bytes of the narrowest element type
  size_t lo = (size_t)rank * S;
  if (lo > pc.sa.count) lo = pc.sa.count;
  ra->aligned16 = (ok16 && (lo % vec) == 0) ? 1 : 0;
}

// log2 of the chunk size for a walk over `slice_elems` elements by `ctas` CTAs.
int seg_chunk_shift(const cocoComm *c, size_t slice_elems, long ctas) {
  if (c->seg_chunk_shift > 0)
    return std::min(kSegChunkShiftMax, std::max(kSegChunkShiftMin, c->seg_chunk_shift));
  int shift = kSegChunkShiftMax;
  while (shift > kSegChunkShiftMin &&
         (slice_elems >> shift) < (size_t)std::max(1L, ctas) * kSegChunksPerCta)
    --shift;
  return shift;
}

int seg_chunk_count(const std::vector<Segment> &segs, int chunk_shift) {
  if (segs.empty()) return 0;
  return (int)(segs.back().chunk0 + ((segs.back().len + ((1ull << chunk_shift) - 1)) >> chunk_shift));
}

// This rank's pieces of a list of tensors.  views_g[b][p] / views_w[b][p]: rank
// p's copy of tensor b as this rank addresses it.
std::vector<Segment> build_segments(int rank, int world, const FlatLayout &L,
                                    const std::vector<size_t> &counts,
                                    const std::vector<std::vector<char *>> &views_g,
                                    const std::vector<std::vector<char *>> &views_w, float *m,
                                    float *v, size_t gsize, int chunk_shift) {
  std::vector<Segment> out;
  const size_t lo = std::min(L.total, (size_t)rank * L.slice);
  const size_t hi = std::min(L.total, lo + L.slice);
  for (size_t b = 0; b < counts.size(); ++b) {
    const size_t t0 = L.off[b], t1 = L.off[b] + counts[b];
    const size_t s0 = std::max(t0, lo), s1 = std::min(t1, hi);
    if (s0 >= s1) continue;
    Segment sg;
    memset(&sg, 0, sizeof(sg));
    bool al = true;
    for (int p = 0; p < world; ++p) {
      sg.g[p] = views_g[b][p];
      sg.out[p] = views_w[b][p];
      al = al && aligned16(views_g[b][p]) && aligned16(views_w[b][p]);
    }
    sg.w = (float *)views_w[b][rank];
    sg.begin = s0 - t0;
    sg.len = s1 - s0;
    // element i of the tensor lives at flat index t0 + i, i.e. at m[(t0 + i) - lo];
    // the kernel indexes m[i - begin]
    sg.m = m ? m + (s0 - lo) : nullptr;
    sg.v = v ? v + (s0 - lo) : nullptr;
    al = al && (sg.begin % 8 == 0) && aligned16(sg.m) && aligned16(sg.v) && gsize != 0;
    sg.aligned16 = al ? 1 : 0;
    sg.tensor = (int)b;
    sg.tensor_len = counts[b];
    sg.first_rank = (int)(t0 / L.slice);          // counts[b] > 0 here: t1 - 1 >= t0
    sg.last_rank = (int)((t1 - 1) / L.slice);
    out.push_back(sg);
  }
  unsigned long long chunks = 0;  // chunk numbering through all pieces
  for (Segment &sg : out) {
    sg.chunk0 = chunks;
    chunks += (sg.len + ((1ull << chunk_shift) - 1)) >> chunk_shift;
  }
  return out;
}

// Puts `segs` into the communicator's device table (re-uploading only when it
// changed) and returns the device pointer.
int upload_segments(cocoComm *c, const std::vector<Segment> &segs, cudaStream_t stream,
                    const Segment **dev) {
  *dev = nullptr;
  if (segs.empty()) return cocoSuccess;
  if (segs.size() > c->seg_cap) {
    CUDA_TRY(cudaStreamSynchronize(stream));
    if (c->seg_dev) CUDA_TRY(cudaFree(c->seg_dev));
    c->seg_dev = nullptr;
    c->seg_cap = std::max<size_t>(64, segs.size() * 2);
    CUDA_TRY(cudaMalloc((void **)&c->seg_dev, c->seg_cap * sizeof(Segment)));
    c->seg_host.clear();
  }
  const bool same = c->seg_host.size() == segs.size() &&
                    memcmp(c->seg_host.data(), segs.data(), segs.size() * sizeof(Segment)) == 0;
  if (!same) {
    c->seg_host = segs;
    // pageable source: staged before the call returns; ordered on the stream
    // after the previous step's kernel, which may still be reading the table
    CUDA_TRY(cudaMemcpyAsync(c->seg_dev, c->seg_host.data(), segs.size() * sizeof(Segment),
                             cudaMemcpyHostToDevice, stream));
  }
  *dev = c->seg_dev;
  return cocoSuccess;
}

// Scattered LAMB: room for one partial-sum pair per chunk of this rank's pieces,
// and behind them one per chunk and warp of a CTA.  Nothing is cleared: a step reads only the entries it wrote.
int ensure_seg_part(cocoComm *c, size_t nchunk, cudaStream_t stream, double **dev) {
  const size_t need = std::max<size_t>(1, nchunk) * (1 + kSegPartPerChunk) * 2;
  if (need > c->seg_part_cap) {
    CUDA_TRY(cudaStreamSynchronize(stream));
    if (c->seg_part) CUDA_TRY(cudaFree(c->seg_part));
    c->seg_part = nullptr;
    c->seg_part_cap = 0;
    CUDA_TRY(cudaMalloc((void **)&c->seg_part, need * sizeof(double)));
    c->seg_part_cap = need;
  }
  *dev = c->seg_part;
  return cocoSuccess;
}

// Launch of one rank that owns its device alone (process mode, or a
// single-process rank with a device of its own).
int launch_single(cocoComm *c, const PendingCall &pc, char *const g_views[],
                  char *const out_views[], char *mc_g, char *mc_out) {
  RankArgs ra;
  fill_rank_args(&ra, c->rank, c->world, g_views, out_views, c->peer_flags, pc);
  LaunchConfig cfg;
  StepArgs sa = pc.sa;
  if (!pc.scounts.empty()) {  // scattered: peer views per tensor, pieces of this rank's slice
    const FlatLayout L = flat_layout(pc.scounts.data(), pc.scounts.size(), c->world);
    std::vector<std::vector<char *>> vg(pc.scounts.size()), vw(pc.scounts.size());
    for (size_t b = 0; b < pc.scounts.size(); ++b) {
      vg[b].resize(kMaxRanks);
      vw[b].resize(kMaxRanks);
      char *mc = nullptr;
      COCO_TRY(peer_views(c, pc.sg[b], pc.scounts[b] * dtype_size(pc.g_type), vg[b].data(), &mc));
      COCO_TRY(peer_views(c, pc.sw[b], pc.scounts[b] * sizeof(float), vw[b].data(), &mc));
    }
    ra.chunk_shift = seg_chunk_shift(c, L.slice, 2L * c->sm_count);
    const std::vector<Segment> segs = build_segments(c->rank, c->world, L, pc.scounts, vg, vw, pc.m,
                                                     pc.v, dtype_size(pc.g_type), ra.chunk_shift);
    COCO_TRY(upload_segments(c, segs, pc.stream, &ra.segs));
    ra.nseg = (int)segs.size();
    ra.nchunk = seg_chunk_count(segs, ra.chunk_shift);
    sa.flags |= kFlagScattered;
    mc_g = mc_out = nullptr;
  }
  // NVLS moves (1 + 1/R) N s bytes per direction, peer-to-peer 2 (R-1)/R N s:
  // the switch wins from R = 4 on.  "auto" takes it there for 16-bit gradients
  // only: the in-switch sum has no fixed order, which the 2e-3 tolerance of
  // 16-bit gradients absorbs but the 1e-5 contract of fp32 gradients (fixed
  // reduction order per world size) does not; fp32 gradients go through the
  // switch only when the caller asks with cocoSetAlgo(comm, 1).  It needs
  // multicast addresses for both buffers (cocoMemAlloc / cocoRegisterMapped).
  const bool want_nvls =
      c->algo == 1 || (c->algo == 2 && c->world >= 4 && dtype_size(pc.g_type) == 2);
  if (want_nvls && mc_g && mc_out && aligned16(mc_g) && aligned16(mc_out)) {
    ra.mc_g = mc_g;
    ra.mc_out = mc_out;
    sa.flags |= kFlagNvls;
  }
  COCO_TRY(pick_launch(c, pc.opt, pc.g_type, pc.w_lp != nullptr, pc.lp_type, pc.sa.count,
                       c->world, 1, &sa, &cfg));
  if (pc.opt == kLAMB && ra.nseg > 0)
    COCO_TRY(ensure_seg_part(c, (size_t)ra.nchunk, pc.stream, &ra.seg_part));
  CUDA_TRY(launch_fused_step(pc.opt, pc.g_type, pc.w_lp != nullptr, pc.lp_type, sa, ra, nullptr,
                             cfg, pc.stream));
  c->launches++;
  c->last_ctas = cfg.ctas;
  return cocoSuccess;
}

// Launch every queued call of a single-process group: one launch per device;
// ranks that share a device become virtual ranks of one cooperative launch.
int flush_group(LocalGroup *grp) {
  std::lock_guard<std::mutex> lock(grp->mu);
  const int R = (int)grp->comms.size();
  for (cocoComm *c : grp->comms)
    if (!c->has_pending) return cocoInvalidUsage;  // every rank must have called
  const PendingCall &first = grp->comms[0]->pending;
  char *g_views[kMaxRanks], *out_views[kMaxRanks];
  FlagPage *flags[kMaxRanks];
  for (int r = 0; r < R; ++r) {
    const PendingCall &pc = grp->comms[r]->pending;
    if (pc.opt != first.opt || pc.g_type != first.g_type || pc.sa.count != first.sa.count ||
        (pc.w_lp != nullptr) != (first.w_lp != nullptr) || pc.lp_type != first.lp_type ||
        pc.sa.seq != first.sa.seq || pc.coll != first.coll) {
      for (cocoComm *c : grp->comms) c->has_pending = false;
      return cocoInvalidUsage;  // ranks disagree on the operation
    }
    g_views[r] = (char *)pc.g;
    out_views[r] = pc.w_lp ? (char *)pc.w_lp : (char *)pc.w;
    flags[r] = grp->comms[r]->flags;
  }
  std::map<int, std::vector<int>> by_dev;
  for (int r = 0; r < R; ++r) by_dev[grp->comms[r]->device].push_back(r);
  int result = cocoSuccess;
  for (auto &kv : by_dev) {
    const std::vector<int> &ranks = kv.second;
    cocoComm *lead = grp->comms[ranks[0]];
    DeviceGuard guard(kv.first);
    if (!guard.ok) {
      result = cocoCudaError;
      break;
    }
    const PendingCall &pc0 = lead->pending;
    std::vector<RankArgs> host(ranks.size());
    for (size_t k = 0; k < ranks.size(); ++k)
      fill_rank_args(&host[k], ranks[k], R, g_views, out_views, flags,
                     grp->comms[ranks[k]]->pending);
    if (pc0.coll != 0) {  // stand-alone collective: the generic kernel, one launch per device
      RankArgs *&slot = grp->table_dev[kv.first];
      if (!slot && cudaMalloc((void **)&slot, kGroupTableBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        result = cocoCudaError;
        break;
      }
      void *aux[kMaxRanks] = {};
      for (size_t k = 0; k < ranks.size(); ++k) aux[k] = grp->comms[ranks[k]]->pending.aux;
      cudaError_t e = launch_collective_group(pc0.coll, pc0.sa, host.data(), aux, (int)ranks.size(), slot,
                                              (char *)slot + sizeof(RankArgs) * kMaxRanks,
                                              lead->sm_count, pc0.stream);
      if (e != cudaSuccess) {
        COCO_WARN("collective launch failed: %s", cudaGetErrorString(e));
        (void)cudaGetLastError();
        result = cocoCudaError;
        break;
      }
      lead->launches++;
      continue;
    }
    const bool scattered = !pc0.scounts.empty();
    if (scattered) {  // one address space: every rank's tensors are addressed directly
      const size_t nb = pc0.scounts.size();
      const FlatLayout L = flat_layout(pc0.scounts.data(), nb, R);
      std::vector<std::vector<char *>> vg(nb), vw(nb);
      bool same = true;
      for (size_t b = 0; b < nb; ++b) {
        vg[b].resize(kMaxRanks);
        vw[b].resize(kMaxRanks);
        for (int r = 0; r < R; ++r) {
          const PendingCall &pr = grp->comms[r]->pending;
          same = same && pr.scounts.size() == nb && pr.scounts[b] == pc0.scounts[b];
          if (!same) break;
          vg[b][r] = (char *)pr.sg[b];
          vw[b][r] = (char *)pr.sw[b];
        }
      }
      if (!same) {
        result = cocoInvalidUsage;
        break;
      }
      bool failed = false;
      for (size_t k = 0; k < ranks.size() && !failed; ++k) {
        cocoComm *ck = grp->comms[ranks[k]];
        // virtual ranks share the device's CTAs
        host[k].chunk_shift = seg_chunk_shift(ck, L.slice, 2L * ck->sm_count / (long)ranks.size());
        const std::vector<Segment> segs = build_segments(ranks[k], R, L, pc0.scounts, vg, vw,
                                                         ck->pending.m, ck->pending.v,
                                                         dtype_size(pc0.g_type), host[k].chunk_shift);
        int rc2 = upload_segments(ck, segs, pc0.stream, &host[k].segs);
        host[k].nseg = (int)segs.size();
        host[k].nchunk = seg_chunk_count(segs, host[k].chunk_shift);
        if (rc2 != cocoSuccess) {
          result = rc2;
          failed = true;
        }
      }
      if (failed) break;
    }
    LaunchConfig cfg;
    StepArgs sa = pc0.sa;
    if (scattered) sa.flags |= kFlagScattered;
    int rc = pick_launch(lead, pc0.opt, pc0.g_type, pc0.w_lp != nullptr, pc0.lp_type,
                         pc0.sa.count, R, (int)ranks.size(), &sa, &cfg);
    if (rc != cocoSuccess) {
      result = rc;
      break;
    }
    if (scattered && pc0.opt == kLAMB) {
      bool failed = false;
      for (size_t k = 0; k < ranks.size() && !failed; ++k)
        if (host[k].nseg > 0) {
          int rc2 = ensure_seg_part(grp->comms[ranks[k]], (size_t)host[k].nchunk, pc0.stream,
                                    &host[k].seg_part);
          if (rc2 != cocoSuccess) result = rc2, failed = true;
        }
      if (failed) break;
    }
    RankArgs *table = nullptr;
    if (ranks.size() > 1) {
      RankArgs *&slot = grp->table_dev[kv.first];
      if (!slot && cudaMalloc((void **)&slot, kGroupTableBytes) != cudaSuccess) {
        result = cocoCudaError;
        break;
      }
      table = slot;
      // pageable source: the copy is staged before this call returns
      if (cudaMemcpyAsync(table, host.data(), sizeof(RankArgs) * ranks.size(),
                          cudaMemcpyHostToDevice, pc0.stream) != cudaSuccess) {
        result = cocoCudaError;
        break;
      }
    }
    cudaError_t e = launch_fused_step(pc0.opt, pc0.g_type, pc0.w_lp != nullptr, pc0.lp_type,
                                      sa, host[0], table, cfg, pc0.stream);
    if (e != cudaSuccess) {
      COCO_WARN("launch failed: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
      result = cocoCudaError;
      break;
    }
    lead->launches++;
    for (int r : ranks) grp->comms[r]->last_ctas = cfg.ctas;
  }
  for (cocoComm *c : grp->comms) c->has_pending = false;
  return result;
}

// NVTX range around the host side of a fused call (the reference marks its
// kernels for the profiler the same way, nccl/src/include/nvtx.h, used from
// enqueue.cc): named after the update rule, visible to any attached tool,
// free when none is.  COCO_NVTX=0 switches it off.
struct NvtxRange {
  bool on;
  explicit NvtxRange(const PendingCall &pc) {
    static const bool enabled = env_int("COCO_NVTX", 1) != 0;
    on = enabled;
    if (on)
      nvtxRangePushA(pc.coll ? "coconet collective"
                     : pc.opt == kSGD ? "coconet fused SGD"
                     : pc.opt == kAdam ? "coconet fused Adam" : "coconet fused LAMB");
  }
  ~NvtxRange() {
    if (on) nvtxRangePop();
  }
};

int enqueue(cocoComm *c, PendingCall &pc) {
  NvtxRange range(pc);
  COCO_TRY(validate(c, pc));
  if (pc.sa.count == 0) return cocoSuccess;
  pc.sa.world = c->world;
  pc.sa.seq = ++c->seq;
  pc.sa.timeout_ns = (unsigned long long)c->timeout_ms * 1000000ull;

  if (c->group) {  // single-process: wait until every rank of the group has called
    if (c->has_pending) return cocoInvalidUsage;
    c->pending = pc;
    c->has_pending = true;
    if (g_group_depth > 0) {
      if (std::find(g_group_touched.begin(), g_group_touched.end(), c) == g_group_touched.end())
        g_group_touched.push_back(c);
      return cocoSuccess;
    }
    for (cocoComm *o : c->group->comms)
      if (!o->has_pending) return cocoSuccess;  // more ranks to come
    return flush_group(c->group.get());
  }

  DeviceGuard guard(c->device);
  if (!guard.ok) return cocoCudaError;
  char *g_views[kMaxRanks] = {}, *out_views[kMaxRanks] = {};
  char *mc_g = nullptr, *mc_out = nullptr;
  if (!pc.scounts.empty()) return launch_single(c, pc, g_views, out_views, nullptr, nullptr);
  COCO_TRY(peer_views(c, pc.g, pc.sa.count * dtype_size(pc.g_type), g_views, &mc_g));
  if (pc.w_lp)
    COCO_TRY(peer_views(c, pc.w_lp, pc.sa.count * dtype_size(pc.lp_type), out_views, &mc_out));
  else
    COCO_TRY(peer_views(c, pc.w, pc.sa.count * sizeof(float), out_views, &mc_out));
  return launch_single(c, pc, g_views, out_views, mc_g, mc_out);
}

// What the kernel would otherwise derive per thread: 1 - beta as a float
// subtraction, the reciprocals of the double denominators.
void finish_scalars(StepArgs *sa) {
  sa->omb1 = 1.0f - sa->beta1;
  sa->omb2 = 1.0f - sa->beta2;
  sa->r1d = 1.0 / sa->d1d;
  sa->r2d = 1.0 / sa->d2d;
}

void set_denominators(StepArgs *sa, int opt, int step) {
  // m^ = m/d1, v^ = v/d2.  overlap: 1 - beta^t evaluated in double as the
  // reference's host check does (multi-process-adam-scattered.cpp:118-119);
  // dsl Adam / nccl Adam and LAMB: beta (adam.cpp:68-69, reduce_kernel.h:33-47,
  // 403-410); dsl LAMB: 1 - beta (lamb.cpp:82-83).
  sa->d1d = sa->d2d = 1.0;
  if (sa->variant == cocoVariantOverlap) {
    sa->d1d = 1.0 - std::pow((double)sa->beta1, (double)(step + 1));
    sa->d2d = 1.0 - std::pow((double)sa->beta2, (double)(step + 1));
    sa->d1 = (float)sa->d1d;
    sa->d2 = (float)sa->d2d;
  } else if (opt == kLAMB && sa->variant == cocoVariantDsl) {
    sa->d1 = 1.0f - sa->beta1;
    sa->d2 = 1.0f - sa->beta2;
  } else {
    sa->d1 = sa->beta1;
    sa->d2 = sa->beta2;
  }
  finish_scalars(sa);
}

}  // namespace

// One rank's row of the topology table: what the driver says about reaching
// each peer's GPU from this rank's.
struct TopoRow {
  int access[kMaxRanks], perf[kMaxRanks], atomics[kMaxRanks];
};

int discover_topology(cocoComm *c) {
  const int R = c->world;
  char mine[32] = {};
  if (cudaDeviceGetPCIBusId(mine, sizeof(mine), c->device) != cudaSuccess) {
    (void)cudaGetLastError();
    mine[0] = 0;
  }
  std::vector<char> ids(32 * (size_t)R);
  COCO_TRY(c->boot->all_gather(mine, ids.data(), 32));
  TopoRow row;
  for (int p = 0; p < R; ++p) {
    row.access[p] = row.perf[p] = row.atomics[p] = -1;
    if (p == c->rank) {
      row.access[p] = 1, row.perf[p] = 0, row.atomics[p] = 1;
      continue;
    }
    int dev = -1;
    const char *id = ids.data() + 32 * (size_t)p;
    if (!id[0] || cudaDeviceGetByPCIBusId(&dev, id) != cudaSuccess) {
      (void)cudaGetLastError();
      continue;  // that GPU is not visible to this process: the driver cannot say
    }
    if (dev == c->device) {  // two ranks on one GPU
      row.access[p] = 1, row.perf[p] = 0, row.atomics[p] = 1;
      continue;
    }
    int v = 0;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrAccessSupported, c->device, dev) == cudaSuccess)
      row.access[p] = v;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrPerformanceRank, c->device, dev) == cudaSuccess)
      row.perf[p] = v;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrNativeAtomicSupported, c->device, dev) == cudaSuccess)
      row.atomics[p] = v;
    (void)cudaGetLastError();
  }
  std::vector<TopoRow> all(R);
  COCO_TRY(c->boot->all_gather(&row, all.data(), sizeof(TopoRow)));
  cocoTopology_t &t = c->topo;
  memset(&t, 0, sizeof(t));
  t.world = R;
  std::vector<int> acc(R * R), perf(R * R);
  for (int a = 0; a < R; ++a)
    for (int b = 0; b < R; ++b) {
      t.access[a][b] = acc[a * R + b] = all[a].access[b];
      t.perf_rank[a][b] = perf[a * R + b] = all[a].perf[b];
      t.native_atomics[a][b] = all[a].atomics[b];
    }
  const int rc = cocoTopologyCheck(R, acc.data(), perf.data(), &t.uniform);
  if (rc != cocoSuccess)
    COCO_WARN("rank %d: some pair of GPUs has no peer access; the fused step needs it", c->rank);
  else if (!t.uniform)
    COCO_WARN("rank %d: the GPUs are not equally near to one another (unequal P2P performance ranks)",
              c->rank);
  return rc;
}

// What symm_mem.cu needs from a communicator.
namespace coco {
int comm_world(cocoComm_t c) { return c->world; }
int comm_rank(cocoComm_t c) { return c->rank; }
int comm_device(cocoComm_t c) { return c->device; }
bool comm_is_group(cocoComm_t c) { return (bool)c->group; }
unsigned long long comm_session(cocoComm_t c) { return c->session; }
int comm_all_gather(cocoComm_t c, const void *send, void *recv, size_t bytes) {
  if (!c->boot) return cocoInvalidUsage;
  return c->boot->all_gather(send, recv, bytes);
}
int comm_enqueue_collective(cocoComm_t c, int kind, const void *g, float *w, void *aux,
                            size_t count, cocoStream_t stream) {
  if (!c->group) return cocoInvalidUsage;
  PendingCall pc;
  pc.opt = kSGD;  // no optimizer state: the collective's functor is chosen by `coll`
  pc.coll = kind;
  pc.aux = aux;
  pc.g = g, pc.g_type = cocoFloat32, pc.w = w;
  pc.sa.count = count;
  pc.sa.grad_scale = 1.0f;
  pc.sa.variant = cocoVariantOverlap;
  pc.sa.d1 = pc.sa.d2 = 1.f;
  pc.sa.d1d = pc.sa.d2d = 1.0;
  pc.stream = (cudaStream_t)stream;
  return enqueue(c, pc);
}
int comm_release_allocs(cocoComm_t c);  // symm_mem.cu
int comm_add_mapped_region(cocoComm_t c, void *ptr, size_t bytes, void *const *peers, void *mc) {
  return cocoRegisterMapped(c, ptr, bytes, peers, mc);
}
int comm_remove_region(cocoComm_t c, void *ptr) {
  auto &v = c->regions;
  for (size_t k = 0; k < v.size(); ++k)
    if (v[k].base == (char *)ptr) {
      v.erase(v.begin() + k);
      return cocoSuccess;
    }
  return cocoInvalidArgument;
}
}  // namespace coco

// ============================================================================
// C ABI
// ============================================================================
extern "C" {

int cocoGetVersion(int *version) {
  if (!version) return cocoInvalidArgument;
  *version = COCO_VERSION;
  return cocoSuccess;
}

const char *cocoErrorString(int result) {
  switch (result) {
    case cocoSuccess: return "success";
    case cocoInvalidArgument: return "invalid argument";
    case cocoInvalidUsage: return "invalid usage";
    case cocoCudaError: return "CUDA error";
    case cocoSystemError: return "system error (bootstrap)";
    case cocoTimeout: return "timed out waiting for a peer";
    case cocoPeerError: return "no peer access";
    case cocoInternalError: return "internal error";
  }
  return "unknown result code";
}

int cocoSliceBounds(size_t count, int world, int rank, size_t *begin, size_t *end) {
  if (world < 1 || rank < 0 || rank >= world || !begin || !end) return cocoInvalidArgument;
  const size_t S = (count + world - 1) / world;
  size_t lo = (size_t)rank * S;
  if (lo > count) lo = count;
  size_t hi = lo + S;
  if (hi > count) hi = count;
  *begin = lo;
  *end = hi;
  return cocoSuccess;
}

int cocoCommInitRank(cocoComm_t *comm, int world, int rank, const char *bootstrap) {
  if (!comm || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return cocoInvalidArgument;
  std::unique_ptr<cocoComm> c(new cocoComm);
  c->world = world;
  c->rank = rank;
  CUDA_TRY(cudaGetDevice(&c->device));
  CUDA_TRY(cudaFree(0));
  c->boot.reset(new Bootstrap);
  const int boot_timeout = env_int("COCO_BOOTSTRAP_TIMEOUT_MS", 120000);
  COCO_TRY(c->boot->init(world, rank, resolve_bootstrap_addr(bootstrap), boot_timeout));
  {  // a session id all ranks share: rank 0's random number
    unsigned long long mine = 0;
    FILE *f = fopen("/dev/urandom", "rb");
    if (f) {
      if (fread(&mine, sizeof(mine), 1, f) != 1) mine = 0;
      fclose(f);
    }
    if (!mine) mine = (unsigned long long)getpid() * 2654435761ull + (unsigned long long)time(nullptr);
    std::vector<unsigned long long> all(world);
    COCO_TRY(c->boot->all_gather(&mine, all.data(), sizeof(mine)));
    c->session = all[0];
  }
  int rc = init_common(c.get());
  // agree on success before anyone maps anything
  std::vector<int> rcs(world);
  COCO_TRY(c->boot->all_gather(&rc, rcs.data(), sizeof(int)));
  for (int r : rcs)
    if (r != cocoSuccess) return r;
  if (world > 1) {
    COCO_TRY(discover_topology(c.get()));  // same verdict on every rank: the table is shared
    Region reg;
    COCO_TRY(map_region_ipc(c.get(), c->flags, kCommPageBytes, &reg));
    for (int p = 0; p < world; ++p) c->peer_flags[p] = (FlagPage *)reg.peer[p];
    COCO_TRY(c->boot->barrier());
  }
  COCO_INFO("rank %d/%d on device %d (%d SMs) ready", rank, world, c->device, c->sm_count);
  *comm = c.release();
  return cocoSuccess;
}

int cocoCommInitAll(cocoComm_t *comms, int n, const int *devices) {
  if (!comms || n < 1 || n > kMaxRanks) return cocoInvalidArgument;
  int ndev = 0;
  CUDA_TRY(cudaGetDeviceCount(&ndev));
  std::vector<int> devs(n);
  for (int r = 0; r < n; ++r) {
    devs[r] = devices ? devices[r] : r;
    if (devs[r] < 0 || devs[r] >= ndev) return cocoInvalidArgument;
  }
  int prev = 0;
  CUDA_TRY(cudaGetDevice(&prev));
  auto grp = std::make_shared<LocalGroup>();
  std::vector<std::unique_ptr<cocoComm>> made;
  int rc = cocoSuccess;
  for (int r = 0; r < n && rc == cocoSuccess; ++r) {
    std::unique_ptr<cocoComm> c(new cocoComm);
    c->world = n;
    c->rank = r;
    c->device = devs[r];
    if (cudaSetDevice(devs[r]) != cudaSuccess) {
      rc = cocoCudaError;
      break;
    }
    rc = init_common(c.get());
    made.push_back(std::move(c));
  }
  // peer access between distinct devices
  for (int a = 0; a < n && rc == cocoSuccess; ++a)
    for (int b = 0; b < n && rc == cocoSuccess; ++b) {
      if (devs[a] == devs[b]) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, devs[a], devs[b]) != cudaSuccess || !can) {
        rc = cocoPeerError;
        break;
      }
      cudaSetDevice(devs[a]);
      cudaError_t e = cudaDeviceEnablePeerAccess(devs[b], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
      } else if (e != cudaSuccess) {
        (void)cudaGetLastError();
        rc = cocoPeerError;
      }
    }
  cudaSetDevice(prev);
  if (rc != cocoSuccess) {
    for (auto &c : made)
      if (c->flags) cudaFree(c->flags);
    return rc;
  }
  for (int r = 0; r < n; ++r) {
    made[r]->group = n > 1 ? grp : nullptr;
    for (int p = 0; p < n; ++p) made[r]->peer_flags[p] = made[p]->flags;
  }
  for (int r = 0; r < n; ++r) {
    grp->comms.push_back(made[r].get());
    comms[r] = made[r].release();
  }
  return cocoSuccess;
}

int cocoCommDestroy(cocoComm_t comm) {
  if (!comm) return cocoInvalidArgument;
  DeviceGuard guard(comm->device);
  cudaDeviceSynchronize();
  // symmetric allocations the caller did not free: released here (collective
  // in process mode), so that nothing stays bound to a multicast object
  int result = comm_release_allocs(comm);
  if (comm->boot && comm->world > 1) {
    // Peers have this rank's flag page (and buffers) mapped and may still be
    // in the end phase of their last kernel: nobody unmaps or frees before
    // every rank has synchronised its device and arrived here.  Bounded by the
    // bootstrap's timeout; a rank that is gone does not hold the others up
    // for ever.
    const int rc = comm->boot->barrier();
    if (rc != cocoSuccess && result == cocoSuccess) result = rc;
  }
  for (auto &kv : comm->ipc_open) cudaIpcCloseMemHandle(kv.second.base);
  if (comm->group) {
    std::lock_guard<std::mutex> lock(comm->group->mu);
    auto &v = comm->group->comms;
    // the last member frees what the group owns
    bool last = true;
    for (cocoComm *&o : v) {
      if (o == comm) o = nullptr;
      if (o) last = false;
    }
    if (last)
      for (auto &kv : comm->group->table_dev) {
        DeviceGuard g2(kv.first);
        cudaFree(kv.second);
      }
  }
  if (comm->seg_part) cudaFree(comm->seg_part);
  if (comm->flags) cudaFree(comm->flags);
  if (comm->seg_dev) cudaFree(comm->seg_dev);
  (void)cudaGetLastError();
  delete comm;
  return result;
}

int cocoTopologyCheck(int world, const int *access, const int *perf_rank, int *uniform) {
  if (world < 1 || world > kMaxRanks || !access || !perf_rank || !uniform) return cocoInvalidArgument;
  *uniform = 1;
  int seen = -1;
  for (int a = 0; a < world; ++a)
    for (int b = 0; b < world; ++b) {
      if (a == b) continue;
      if (access[a * world + b] == 0) return cocoPeerError;
      if (access[a * world + b] < 0) *uniform = 0;  // unknown is not "uniform"
      const int p = perf_rank[a * world + b];
      if (p < 0) continue;
      if (seen < 0) seen = p;
      else if (p != seen) *uniform = 0;
    }
  return cocoSuccess;
}

int cocoCommTopology(cocoComm_t comm, cocoTopology_t *topology) {
  if (!comm || !topology) return cocoInvalidArgument;
  if (comm->group || comm->world == 1) {  // one process: every pair was checked at creation
    memset(topology, 0, sizeof(*topology));
    topology->world = comm->world;
    for (int a = 0; a < comm->world; ++a)
      for (int b = 0; b < comm->world; ++b) {
        topology->access[a][b] = 1;
        topology->perf_rank[a][b] = a == b ? 0 : -1;
        topology->native_atomics[a][b] = a == b ? 1 : -1;
      }
    topology->uniform = comm->world == 1;
    return cocoSuccess;
  }
  *topology = comm->topo;
  return cocoSuccess;
}

int cocoCommCount(cocoComm_t comm, int *world) {
  if (!comm || !world) return cocoInvalidArgument;
  *world = comm->world;
  return cocoSuccess;
}
int cocoCommUserRank(cocoComm_t comm, int *rank) {
  if (!comm || !rank) return cocoInvalidArgument;
  *rank = comm->rank;
  return cocoSuccess;
}
int cocoCommCuDevice(cocoComm_t comm, int *device) {
  if (!comm || !device) return cocoInvalidArgument;
  *device = comm->device;
  return cocoSuccess;
}

int cocoBarrier(cocoComm_t comm) {
  if (!comm) return cocoInvalidArgument;
  if (comm->boot) return comm->boot->barrier();
  return cocoSuccess;  // single-process groups share one host thread of control
}

int cocoAllGatherHost(cocoComm_t comm, const void *send, void *recv, size_t bytes_per_rank) {
  if (!comm || !send || !recv) return cocoInvalidArgument;
  if (comm->boot) return comm->boot->all_gather(send, recv, bytes_per_rank);
  if (comm->world == 1) {
    if (send != recv) memcpy(recv, send, bytes_per_rank);
    return cocoSuccess;
  }
  return cocoInvalidUsage;
}

struct cocoBootstrap {
  Bootstrap impl;
};

int cocoBootstrapInit(cocoBootstrap_t *bs, int world, int rank, const char *addr, int timeout_ms) {
  if (!bs) return cocoInvalidArgument;
  std::unique_ptr<cocoBootstrap> b(new cocoBootstrap);
  COCO_TRY(b->impl.init(world, rank, resolve_bootstrap_addr(addr),
                        timeout_ms > 0 ? timeout_ms : 120000));
  *bs = b.release();
  return cocoSuccess;
}
int cocoBootstrapAllGather(cocoBootstrap_t bs, const void *send, void *recv,
                           size_t bytes_per_rank) {
  if (!bs || !send || !recv) return cocoInvalidArgument;
  return bs->impl.all_gather(send, recv, bytes_per_rank);
}
int cocoBootstrapBarrier(cocoBootstrap_t bs) {
  if (!bs) return cocoInvalidArgument;
  return bs->impl.barrier();
}
int cocoBootstrapDestroy(cocoBootstrap_t bs) {
  if (!bs) return cocoInvalidArgument;
  delete bs;
  return cocoSuccess;
}
int cocoEnvRank(int *rank, int *world, int *local_rank) {
  if (!rank || !world || !local_rank) return cocoInvalidArgument;
  *rank = env_int("RANK", 0);
  *world = env_int("WORLD_SIZE", 1);
  *local_rank = env_int("LOCAL_RANK", *rank);
  return cocoSuccess;
}

int cocoGroupStart(void) {
  ++g_group_depth;
  return cocoSuccess;
}

int cocoGroupEnd(void) {
  if (g_group_depth <= 0) return cocoInvalidUsage;
  if (--g_group_depth > 0) return cocoSuccess;
  std::vector<cocoComm *> touched;
  touched.swap(g_group_touched);
  int result = cocoSuccess;
  std::vector<LocalGroup *> done;
  for (cocoComm *c : touched) {
    if (!c->group) continue;
    LocalGroup *g = c->group.get();
    if (std::find(done.begin(), done.end(), g) != done.end()) continue;
    done.push_back(g);
    int rc = flush_group(g);
    if (rc != cocoSuccess && result == cocoSuccess) result = rc;
  }
  return result;
}

int cocoRegister(cocoComm_t comm, void *ptr, size_t bytes) {
  if (!comm || !ptr || bytes == 0) return cocoInvalidArgument;
  if (comm->world == 1 || comm->group) return cocoSuccess;  // one address space: nothing to map
  if (find_region(comm, ptr, bytes)) return cocoSuccess;
  DeviceGuard guard(comm->device);
  Region reg;
  COCO_TRY(map_region_ipc(comm, ptr, bytes, &reg));
  comm->regions.push_back(reg);
  return cocoSuccess;
}

int cocoRegisterMapped(cocoComm_t comm, void *ptr, size_t bytes, void *const *peer_ptrs,
                       void *multicast_ptr) {
  if (!comm || !ptr || bytes == 0 || !peer_ptrs) return cocoInvalidArgument;
  if (comm->group) return cocoInvalidUsage;
  if (peer_ptrs[comm->rank] != ptr) return cocoInvalidArgument;
  Region reg;
  reg.base = (char *)ptr;
  reg.bytes = bytes;
  for (int p = 0; p < comm->world; ++p) {
    if (!peer_ptrs[p]) return cocoInvalidArgument;
    reg.peer[p] = (char *)peer_ptrs[p];
  }
  reg.multicast = (char *)multicast_ptr;
  reg.external = true;
  // newest first, so that it wins over an older registration of the same range
  comm->regions.insert(comm->regions.begin(), reg);
  return cocoSuccess;
}

int cocoSetAlgo(cocoComm_t comm, int algo) {
  if (!comm || algo < 0 || algo > 2) return cocoInvalidArgument;
  comm->algo = algo;
  return cocoSuccess;
}

int cocoDeregister(cocoComm_t comm, void *ptr) {
  if (!comm || !ptr) return cocoInvalidArgument;
  if (comm->world == 1 || comm->group) return cocoSuccess;
  DeviceGuard guard(comm->device);
  // finish whatever still uses the mapping on this rank
  CUDA_TRY(cudaDeviceSynchronize());
  auto &v = comm->regions;
  bool found = false, external = false;
  for (size_t k = 0; k < v.size(); ++k)
    if (v[k].base == (char *)ptr) {
      external = v[k].external;
      for (const std::string &key : v[k].ipc_keys) {
        auto it = comm->ipc_open.find(key);
        if (it != comm->ipc_open.end() && --it->second.refs == 0) {
          cudaIpcCloseMemHandle(it->second.base);
          comm->ipc_open.erase(it);
        }
      }
      v.erase(v.begin() + k);
      found = true;
      break;
    }
  if (external) return cocoSuccess;  // local registration, local removal
  // collective: nobody may free its buffer before every peer has unmapped it
  int ok = found ? 1 : 0;
  std::vector<int> all(comm->world);
  COCO_TRY(comm->boot->all_gather(&ok, all.data(), sizeof(int)));
  return found ? cocoSuccess : cocoInvalidArgument;
}

int cocoFusedSGD(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                 cocoDataType_t lp_type, size_t count, float lr, float grad_scale,
                 cocoStream_t stream) {
  if (!comm) return cocoInvalidArgument;
  PendingCall pc;
  pc.opt = kSGD;
  pc.g = g, pc.g_type = g_type, pc.w = w, pc.w_lp = w_lp, pc.lp_type = lp_type;
  pc.sa.count = count;
  pc.sa.lr = lr;
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = cocoVariantOverlap;
  pc.sa.d1 = pc.sa.d2 = 1.f;
  pc.sa.d1d = pc.sa.d2d = 1.0;
  pc.stream = (cudaStream_t)stream;
  return enqueue(comm, pc);
}

int cocoFusedAdam(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                  cocoDataType_t lp_type, float *m, float *v, size_t count, float lr,
                  float beta1, float beta2, float eps, int step, float grad_scale,
                  cocoVariant_t variant, cocoStream_t stream) {
  if (!comm || step < 0) return cocoInvalidArgument;
  PendingCall pc;
  pc.opt = kAdam;
  pc.g = g, pc.g_type = g_type, pc.w = w, pc.w_lp = w_lp, pc.lp_type = lp_type;
  pc.m = m, pc.v = v;
  pc.sa.count = count;
  pc.sa.lr = lr, pc.sa.beta1 = beta1, pc.sa.beta2 = beta2;
  // only the bias-corrected form has an epsilon (reduce_kernel.h:243 of
  // nccl-overlap); the other two divide by v^ / sqrt(v^) directly
  pc.sa.eps = variant == cocoVariantOverlap ? eps : 0.f;
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = (int)variant;
  set_denominators(&pc.sa, kAdam, step);
  pc.stream = (cudaStream_t)stream;
  return enqueue(comm, pc);
}

int cocoFusedLAMB(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w, void *w_lp,
                  cocoDataType_t lp_type, float *m, float *v, size_t count, float lr,
                  float beta1, float beta2, float eps, float weight_decay, int step,
                  float grad_scale, cocoVariant_t variant, unsigned flags, cocoStream_t stream) {
  if (!comm || step < 0) return cocoInvalidArgument;
  PendingCall pc;
  pc.opt = kLAMB;
  pc.g = g, pc.g_type = g_type, pc.w = w, pc.w_lp = w_lp, pc.lp_type = lp_type;
  pc.m = m, pc.v = v;
  pc.sa.count = count;
  pc.sa.lr = lr, pc.sa.beta1 = beta1, pc.sa.beta2 = beta2;
  pc.sa.eps = variant == cocoVariantOverlap ? eps : 0.f;  // lamb.cpp:72,84: epsilon unused
  // the forked-NCCL functor hard-codes the decay factor (reduce_kernel.h:427)
  pc.sa.weight_decay = variant == cocoVariantNccl ? 1.0f : weight_decay;
  if (variant == cocoVariantNccl) flags &= ~COCO_LAMB_REF_QUIRK;  // it has its own norm rule
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = (int)variant;
  pc.sa.flags = flags;
  set_denominators(&pc.sa, kLAMB, step);
  pc.stream = (cudaStream_t)stream;
  return enqueue(comm, pc);
}

int cocoFusedGenericPlan(cocoComm_t comm, const void *g, cocoDataType_t g_type, float *w,
                         size_t count, float grad_scale, cocoStream_t stream,
                         cocoGenericPlan *plan) {
  (void)stream;
  if (!comm || !g || !w || !plan) return cocoInvalidArgument;
  if (g_type != cocoFloat32 && g_type != cocoFloat16) return cocoInvalidArgument;
  if (comm->group) return cocoInvalidUsage;  // one process per GPU (or world size 1)
  memset(plan, 0, sizeof(*plan));
  plan->sa.count = count;
  plan->sa.world = comm->world;
  plan->sa.grad_scale = grad_scale;
  plan->sa.timeout_ns = (unsigned long long)comm->timeout_ms * 1000000ull;
  if (count == 0) return cocoSuccess;
  plan->sa.seq = ++comm->seq;
  DeviceGuard guard(comm->device);
  if (!guard.ok) return cocoCudaError;
  char *g_views[kMaxRanks] = {}, *out_views[kMaxRanks] = {};
  char *mc_g = nullptr, *mc_out = nullptr;
  COCO_TRY(peer_views(comm, g, count * dtype_size(g_type), g_views, &mc_g));
  COCO_TRY(peer_views(comm, w, count * sizeof(float), out_views, &mc_out));
  PendingCall pc;
  pc.opt = kSGD;  // no m, v of the library's own: the functor owns its state
  pc.g = g, pc.g_type = g_type, pc.w = w;
  pc.sa = plan->sa;
  fill_rank_args(&plan->ra, comm->rank, comm->world, g_views, out_views, comm->peer_flags, pc);
  const size_t slice = (count + comm->world - 1) / comm->world;
  const int threads = 512;
  long ctas = 2L * comm->sm_count;
  const long need = (long)std::max<size_t>(1, (slice + 4 * (size_t)threads - 1) / (4 * (size_t)threads));
  plan->ctas = (int)std::max(1L, std::min(ctas, need));
  plan->threads = threads;
  comm->launches++;
  return cocoSuccess;
}

int cocoScatteredSliceElems(size_t nbuff, const size_t *counts, int world, size_t *slice_elems) {
  if (!counts || !slice_elems || world < 1 || world > kMaxRanks) return cocoInvalidArgument;
  *slice_elems = flat_layout(counts, nbuff, world).slice;
  return cocoSuccess;
}

int cocoScatteredTensorPlace(size_t nbuff, const size_t *counts, int world, size_t tensor,
                             size_t *flat_offset, int *first_rank, int *last_rank) {
  if (!counts || !flat_offset || !first_rank || !last_rank || world < 1 || world > kMaxRanks ||
      tensor >= nbuff)
    return cocoInvalidArgument;
  const FlatLayout L = flat_layout(counts, nbuff, world);
  *flat_offset = L.off[tensor];
  if (counts[tensor] == 0) {
    *first_rank = *last_rank = -1;
  } else {  // the same arithmetic as build_segments
    *first_rank = (int)(L.off[tensor] / L.slice);
    *last_rank = (int)((L.off[tensor] + counts[tensor] - 1) / L.slice);
  }
  return cocoSuccess;
}

static int enqueue_scattered(cocoComm_t comm, int opt, size_t nbuff, const void *const *g,
                             cocoDataType_t g_type, float *const *w, const size_t *counts,
                             float *m, float *v, PendingCall &pc, cocoStream_t stream) {
  if (!comm || !g || !w || !counts || nbuff == 0) return cocoInvalidArgument;
  pc.opt = opt;
  pc.g_type = g_type;
  pc.m = m, pc.v = v;
  pc.sg.assign(g, g + nbuff);
  pc.sw.assign(w, w + nbuff);
  pc.scounts.assign(counts, counts + nbuff);
  pc.g = g[0];
  pc.w = w[0];
  pc.sa.count = flat_layout(counts, nbuff, comm->world).total;
  pc.stream = (cudaStream_t)stream;
  return enqueue(comm, pc);
}

int cocoFusedSGDScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                          cocoDataType_t g_type, float *const *w, const size_t *counts, float lr,
                          float grad_scale, cocoStream_t stream) {
  PendingCall pc;
  pc.sa.lr = lr;
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = cocoVariantOverlap;
  pc.sa.d1 = pc.sa.d2 = 1.f;
  pc.sa.d1d = pc.sa.d2d = 1.0;
  return enqueue_scattered(comm, kSGD, nbuff, g, g_type, w, counts, nullptr, nullptr, pc, stream);
}

int cocoFusedAdamScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                           cocoDataType_t g_type, float *const *w, const size_t *counts, float *m,
                           float *v, float lr, float beta1, float beta2, float eps, int step,
                           float grad_scale, cocoVariant_t variant, cocoStream_t stream) {
  if (step < 0 || variant == cocoVariantNccl || !m || !v) return cocoInvalidArgument;
  PendingCall pc;
  pc.sa.lr = lr, pc.sa.beta1 = beta1, pc.sa.beta2 = beta2;
  pc.sa.eps = variant == cocoVariantOverlap ? eps : 0.f;
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = (int)variant;
  set_denominators(&pc.sa, kAdam, step);
  return enqueue_scattered(comm, kAdam, nbuff, g, g_type, w, counts, m, v, pc, stream);
}

int cocoFusedLAMBScattered(cocoComm_t comm, size_t nbuff, const void *const *g,
                           cocoDataType_t g_type, float *const *w, const size_t *counts, float *m,
                           float *v, float lr, float beta1, float beta2, float eps,
                           float weight_decay, int step, float grad_scale, cocoVariant_t variant,
                           unsigned flags, cocoStream_t stream) {
  if (step < 0 || variant == cocoVariantNccl || !m || !v) return cocoInvalidArgument;
  if (nbuff > (size_t)kMaxLambTensors) return cocoInvalidArgument;
  PendingCall pc;
  pc.sa.lr = lr, pc.sa.beta1 = beta1, pc.sa.beta2 = beta2;
  pc.sa.eps = variant == cocoVariantOverlap ? eps : 0.f;
  pc.sa.weight_decay = weight_decay;
  pc.sa.grad_scale = grad_scale;
  pc.sa.variant = (int)variant;
  pc.sa.flags = flags;
  set_denominators(&pc.sa, kLAMB, step);
  return enqueue_scattered(comm, kLAMB, nbuff, g, g_type, w, counts, m, v, pc, stream);
}

int cocoLinkProbe(cocoComm_t comm, void *buf, size_t bytes, int mode, int unroll, int iters,
                  double *gbs_per_direction, cocoStream_t stream) {
  if (!comm || !buf || !gbs_per_direction || iters < 1 || mode < 0 || mode > 7)
    return cocoInvalidArgument;
  // mode 7 (hybrid): `unroll` is the number of sixteenths of the slice that go through the switch
  if (mode == 7 && (unroll < 0 || unroll > 16)) return cocoInvalidArgument;
  if (mode != 3 && mode != 7 && unroll != 1 && unroll != 2 && unroll != 4) return cocoInvalidArgument;
  if ((((uintptr_t)buf) & 15u) != 0 || bytes < 32u * (size_t)comm->world) return cocoInvalidArgument;
  if (comm->group) return cocoInvalidUsage;  // one process per GPU
  *gbs_per_direction = 0.0;
  if (comm->world == 1) return cocoSuccess;  // no link to measure
  DeviceGuard guard(comm->device);
  if (!guard.ok) return cocoCudaError;
  const int R = comm->world;
  cudaStream_t st = (cudaStream_t)stream;
  char *views[kMaxRanks] = {};
  char *mc = nullptr;
  COCO_TRY(peer_views(comm, buf, bytes, views, &mc));

  PendingCall pc;
  pc.opt = kSGD;
  pc.g = buf, pc.w = (float *)buf;
  pc.sa.count = bytes / 16;  // 16-byte units
  pc.sa.world = R;
  pc.sa.timeout_ns = (unsigned long long)comm->timeout_ms * 1000000ull;
  RankArgs ra;
  fill_rank_args(&ra, comm->rank, R, views, views, comm->peer_flags, pc);
  if (mode >= 4) {  // through the switch: the buffer needs a multicast mapping
    if (!mc || !aligned16(mc)) return cocoInvalidUsage;
    ra.mc_g = mc;
    ra.mc_out = mc;
  }
  const size_t slice_units = (pc.sa.count + R - 1) / R;
  double dir_bytes = 0.0;  // bytes crossing this GPU's links in one direction per iteration
  const size_t half = bytes / 2 / 16 * 16;
  if (mode == 3) {
    dir_bytes = (double)half;
  } else {
    size_t lo = (size_t)comm->rank * slice_units;
    if (lo > pc.sa.count) lo = pc.sa.count;
    const size_t len = std::min<size_t>(pc.sa.count - lo, slice_units);
    if (mode == 7) {  // reported as the time of one iteration in microseconds instead of a rate
      pc.sa.pad = unroll;
      dir_bytes = 1e3;
    } else if (mode <= 2)  // peer to peer: R - 1 slices in (pull) and / or out (push)
      dir_bytes = (double)(R - 1) * (double)len * 16.0 * (mode == 2 ? 2.0 : 1.0);
    else  // switch: the whole buffer leaves (reduce) or arrives (store) once, the slice the other way
      dir_bytes = (double)pc.sa.count * 16.0 + (mode == 6 ? (double)len * 16.0 : 0.0);
  }

  cudaEvent_t e0 = nullptr, e1 = nullptr;
  CUDA_TRY(cudaEventCreate(&e0));
  CUDA_TRY(cudaEventCreate(&e1));
  int result = cocoSuccess;
  auto once = [&]() -> int {
    if (mode == 3) {  // copy engine: the next rank's first half into this rank's second half
      const int p = (comm->rank + 1) % R;
      if (cudaMemcpyAsync((char *)buf + half, views[p], half, cudaMemcpyDefault, st) != cudaSuccess)
        return cocoCudaError;
      return cocoSuccess;
    }
    pc.sa.seq = ++comm->seq;
    if (launch_link_probe(mode, unroll, pc.sa, ra, comm->sm_count, 512, st) != cudaSuccess) {
      (void)cudaGetLastError();
      return cocoCudaError;
    }
    comm->launches++;
    return cocoSuccess;
  };
  // every rank takes every step whatever happens locally, so that the ranks'
  // sequence numbers stay in step
  int rc = once();  // warm-up
  if (rc != cocoSuccess) result = rc;
  if (cudaStreamSynchronize(st) != cudaSuccess) result = cocoCudaError;
  rc = comm->boot->barrier();
  if (rc != cocoSuccess && result == cocoSuccess) result = rc;
  cudaEventRecord(e0, st);
  for (int i = 0; i < iters; ++i) {
    rc = once();
    if (rc != cocoSuccess && result == cocoSuccess) result = rc;
  }
  cudaEventRecord(e1, st);
  if (cudaStreamSynchronize(st) != cudaSuccess) result = cocoCudaError;
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) result = cocoCudaError;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  (void)cudaGetLastError();
  // the slowest rank's time and the smallest byte count give the figure all ranks report
  std::vector<double> all(2 * (size_t)R);
  const double mine[2] = {(double)ms / iters, dir_bytes};
  rc = comm->boot->all_gather(mine, all.data(), sizeof(mine));
  if (rc != cocoSuccess) return rc;
  if (result != cocoSuccess) return result;
  double worst_ms = 0.0, least_bytes = dir_bytes;
  for (int r = 0; r < R; ++r) {
    worst_ms = std::max(worst_ms, all[2 * r]);
    least_bytes = std::min(least_bytes, all[2 * r + 1]);
  }
  if (worst_ms > 0.0) *gbs_per_direction = least_bytes / (worst_ms * 1e-3) / 1e9;
  if (mode == 7) *gbs_per_direction = worst_ms * 1e3;  // microseconds per iteration
  return cocoSuccess;
}

int cocoLastLambNorms(cocoComm_t comm, double out[2]) {
  if (!comm || !out) return cocoInvalidArgument;
  DeviceGuard guard(comm->device);
  CUDA_TRY(cudaMemcpy(out, comm->flags->last_norms, 2 * sizeof(double), cudaMemcpyDeviceToHost));
  return cocoSuccess;
}

int cocoLastPhaseTimes(cocoComm_t comm, unsigned long long out_ns[3]) {
  if (!comm || !out_ns) return cocoInvalidArgument;
  DeviceGuard guard(comm->device);
  unsigned long long t[4];
  CUDA_TRY(cudaMemcpy(t, comm->flags->phase_ns, sizeof(t), cudaMemcpyDeviceToHost));
  for (int k = 0; k < 3; ++k) out_ns[k] = t[k + 1] >= t[k] ? t[k + 1] - t[k] : 0;
  return cocoSuccess;
}

int cocoLastCtaSpread(cocoComm_t comm, unsigned long long out_ns[3]) {
  if (!comm || !out_ns) return cocoInvalidArgument;
  DeviceGuard guard(comm->device);
  const int n = comm->last_ctas;
  out_ns[0] = out_ns[1] = out_ns[2] = 0;
  if (n <= 0) return cocoSuccess;
  unsigned long long t0 = 0;
  std::vector<unsigned long long> end((size_t)n);
  CUDA_TRY(cudaMemcpy(&t0, &comm->flags->phase_ns[0], sizeof(t0), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemcpy(end.data(), comm->flags->cta_end_ns, sizeof(unsigned long long) * n,
                      cudaMemcpyDeviceToHost));
  std::sort(end.begin(), end.end());
  out_ns[0] = end.front() >= t0 ? end.front() - t0 : 0;
  out_ns[1] = end[n / 2] >= t0 ? end[n / 2] - t0 : 0;
  out_ns[2] = end.back() >= t0 ? end.back() - t0 : 0;
  return cocoSuccess;
}

int cocoGetStatus(cocoComm_t comm, cocoStatus_t *status) {
  if (!comm || !status) return cocoInvalidArgument;
  DeviceGuard guard(comm->device);
  int raw[8];
  CUDA_TRY(cudaMemcpy(raw, comm->flags->status, sizeof(raw), cudaMemcpyDeviceToHost));
  status->code = raw[0];
  status->rank = raw[1];
  status->phase = raw[2];
  status->peer = raw[3];
  status->seq = ((uint64_t)(unsigned)raw[5] << 32) | (unsigned)raw[4];
  if (raw[0] != 0) CUDA_TRY(cudaMemset(comm->flags->status, 0, sizeof(raw)));
  return cocoSuccess;
}

int cocoSetTunables(cocoComm_t comm, int ctas_per_sm, int threads, int timeout_ms) {
  if (!comm) return cocoInvalidArgument;
  if (ctas_per_sm > 0) comm->ctas_per_sm = ctas_per_sm;
  if (threads > 0) {
    if (threads < 32 || threads > 512 || (threads % 32) != 0) return cocoInvalidArgument;
    comm->threads = threads;
  }
  if (timeout_ms > 0) comm->timeout_ms = timeout_ms;
  return cocoSuccess;
}

int cocoLaunchCount(cocoComm_t comm, uint64_t *launches) {
  if (!comm || !launches) return cocoInvalidArgument;
  *launches = comm->launches;
  return cocoSuccess;
}

}  // extern "C"
