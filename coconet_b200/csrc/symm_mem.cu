// cocoMemAlloc / cocoMemFree: symmetric device memory with an NVSwitch
// multicast mapping, made by the runtime itself.
//
// Every rank creates one physical allocation (cuMemCreate), exports it as a
// POSIX file descriptor, passes the descriptor to every other rank over UNIX
// datagram sockets (SCM_RIGHTS) and maps all R allocations into its address
// space.  Where the devices support it, rank 0 also creates a multicast object
// over the R allocations (cuMulticastCreate / AddDevice / BindMem) and every
// rank maps it: loads and stores through that address are reduced and
// replicated by the NVSwitch (multimem.ld_reduce / multimem.st in
// fused_step.cu).  The buffer is then registered with the communicator like a
// cocoRegisterMapped buffer.
//
// The reference's counterpart is NCCL's own buffer set-up
// (nccl/src/transport/p2p.cc:118-238 for peer mappings; it has no in-switch
// path: its CollNet kernel is `assert(false)`,
// nccl/src/collectives/device/all_reduce_computation.h:262-316).
//
// The driver API is reached through cudaGetDriverEntryPoint so that the
// library keeps no link-time dependency on libcuda.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "coconet_rt.h"
#include "fused_step.cuh"

using namespace coco;

// Implemented in runtime.cu: what this file needs from a communicator.
namespace coco {
int comm_world(cocoComm_t c);
int comm_rank(cocoComm_t c);
int comm_device(cocoComm_t c);
bool comm_is_group(cocoComm_t c);
int comm_all_gather(cocoComm_t c, const void *send, void *recv, size_t bytes);
int comm_add_mapped_region(cocoComm_t c, void *ptr, size_t bytes, void *const *peers, void *mc);
int comm_remove_region(cocoComm_t c, void *ptr);
unsigned long long comm_session(cocoComm_t c);
}  // namespace coco

namespace {

#define DRV_FN(name) decltype(&name) p_##name = nullptr

struct Driver {
  DRV_FN(cuMemGetAllocationGranularity);
  DRV_FN(cuMemCreate);
  DRV_FN(cuMemRelease);
  DRV_FN(cuMemExportToShareableHandle);
  DRV_FN(cuMemImportFromShareableHandle);
  DRV_FN(cuMemAddressReserve);
  DRV_FN(cuMemAddressFree);
  DRV_FN(cuMemMap);
  DRV_FN(cuMemUnmap);
  DRV_FN(cuMemSetAccess);
  DRV_FN(cuMulticastCreate);
  DRV_FN(cuMulticastAddDevice);
  DRV_FN(cuMulticastBindMem);
  DRV_FN(cuMulticastUnbind);
  DRV_FN(cuMulticastGetGranularity);
  DRV_FN(cuDeviceGetAttribute);
  DRV_FN(cuDeviceGet);
  bool ok = false;
};

template <typename F> bool resolve(const char *name, F *out) {
  void *f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || !f ||
      q != cudaDriverEntryPointSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  *out = (F)f;
  return true;
}

Driver &driver() {
  static Driver d = [] {
    Driver x;
#define GET(name) resolve(#name, &x.p_##name)
    x.ok = GET(cuMemGetAllocationGranularity) && GET(cuMemCreate) && GET(cuMemRelease) &&
           GET(cuMemExportToShareableHandle) && GET(cuMemImportFromShareableHandle) &&
           GET(cuMemAddressReserve) && GET(cuMemAddressFree) && GET(cuMemMap) && GET(cuMemUnmap) &&
           GET(cuMemSetAccess) && GET(cuDeviceGetAttribute) && GET(cuDeviceGet);
    // multicast entry points are optional (older drivers)
    if (!(GET(cuMulticastCreate) && GET(cuMulticastAddDevice) && GET(cuMulticastBindMem) &&
          GET(cuMulticastUnbind) && GET(cuMulticastGetGranularity)))
      x.p_cuMulticastCreate = nullptr;
#undef GET
    return x;
  }();
  return d;
}

struct SymmAlloc {
  size_t size = 0;
  CUmemGenericAllocationHandle local = 0;
  CUmemGenericAllocationHandle peer_handle[kMaxRanks] = {};
  CUdeviceptr va[kMaxRanks] = {};
  bool has_mc = false;
  bool bound = false;
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_va = 0;
  CUdevice dev = 0;
  bool plain = false;  // world size 1: plain cudaMalloc
};

std::mutex g_mu;
std::map<cocoComm_t, std::map<void *, SymmAlloc>> g_allocs;

// ---- file descriptors between processes ------------------------------------------
std::string sock_name(unsigned long long session, int rank) {
  char buf[96];
  snprintf(buf, sizeof(buf), "coco-fd-%llx-%d", session, rank);
  return buf;
}

int make_socket(unsigned long long session, int rank) {
  int fd = ::socket(AF_UNIX, SOCK_DGRAM, 0);
  if (fd < 0) return -1;
  struct sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  const std::string n = sock_name(session, rank);
  memcpy(a.sun_path + 1, n.data(), n.size());  // abstract namespace: leading NUL
  if (::bind(fd, (struct sockaddr *)&a, (socklen_t)(sizeof(sa_family_t) + 1 + n.size())) != 0) {
    ::close(fd);
    return -1;
  }
  struct timeval tv = {30, 0};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  return fd;
}

bool send_fd(int sock, unsigned long long session, int to_rank, int src_rank, int tag, int fd) {
  struct sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  const std::string n = sock_name(session, to_rank);
  memcpy(a.sun_path + 1, n.data(), n.size());
  int payload[2] = {src_rank, tag};
  struct iovec iov = {payload, sizeof(payload)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &a;
  msg.msg_namelen = (socklen_t)(sizeof(sa_family_t) + 1 + n.size());
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr *c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return ::sendmsg(sock, &msg, 0) == (ssize_t)sizeof(payload);
}

bool recv_fd(int sock, int *src_rank, int *tag, int *fd) {
  int payload[2] = {-1, -1};
  struct iovec iov = {payload, sizeof(payload)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t k;
  do {
    k = ::recvmsg(sock, &msg, 0);
  } while (k < 0 && errno == EINTR);
  if (k != (ssize_t)sizeof(payload)) return false;
  struct cmsghdr *c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return false;
  memcpy(fd, CMSG_DATA(c), sizeof(int));
  *src_rank = payload[0];
  *tag = payload[1];
  return true;
}

// every rank reports ok/failed; true only if all are ok
bool all_ok(cocoComm_t comm, bool mine) {
  const int R = comm_world(comm);
  int v = mine ? 1 : 0;
  std::vector<int> all(R, 0);
  if (comm_all_gather(comm, &v, all.data(), sizeof(int)) != cocoSuccess) return false;
  for (int x : all)
    if (!x) return false;
  return true;
}

bool map_rw(Driver &d, CUdeviceptr *va, size_t size, size_t gran, CUmemGenericAllocationHandle h,
            CUdevice dev) {
  if (d.p_cuMemAddressReserve(va, size, gran, 0, 0) != CUDA_SUCCESS) return false;
  if (d.p_cuMemMap(*va, size, 0, h, 0) != CUDA_SUCCESS) {
    d.p_cuMemAddressFree(*va, size);
    *va = 0;
    return false;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.p_cuMemSetAccess(*va, size, &acc, 1) != CUDA_SUCCESS) {
    d.p_cuMemUnmap(*va, size);
    d.p_cuMemAddressFree(*va, size);
    *va = 0;
    return false;
  }
  return true;
}

void unmap(Driver &d, CUdeviceptr va, size_t size) {
  if (!va) return;
  d.p_cuMemUnmap(va, size);
  d.p_cuMemAddressFree(va, size);
}

void release_all(Driver &d, SymmAlloc &a, int R, int rank) {
  if (a.mc_va) unmap(d, a.mc_va, a.size);
  if (a.bound) d.p_cuMulticastUnbind(a.mc, a.dev, 0, a.size);
  if (a.mc) d.p_cuMemRelease(a.mc);
  for (int p = 0; p < R; ++p) {
    if (p == rank) continue;
    if (a.va[p]) unmap(d, a.va[p], a.size);
    if (a.peer_handle[p]) d.p_cuMemRelease(a.peer_handle[p]);
  }
  if (a.va[rank]) unmap(d, a.va[rank], a.size);
  if (a.local) d.p_cuMemRelease(a.local);
}

}  // namespace

extern "C" int cocoMemAlloc(cocoComm_t comm, void **ptr, size_t bytes) {
  if (!comm || !ptr || bytes == 0) return cocoInvalidArgument;
  if (comm_is_group(comm)) return cocoInvalidUsage;  // one address space: use cudaMalloc
  const int R = comm_world(comm), rank = comm_rank(comm);
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(comm_device(comm)) != cudaSuccess) return cocoCudaError;
  struct Restore {
    int d;
    ~Restore() {
      if (d >= 0) cudaSetDevice(d);
    }
  } restore{prev};

  if (R == 1) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      return cocoCudaError;
    }
    SymmAlloc a;
    a.plain = true;
    a.size = bytes;
    std::lock_guard<std::mutex> lock(g_mu);
    g_allocs[comm][p] = a;
    *ptr = p;
    return cocoSuccess;
  }

  Driver &d = driver();
  SymmAlloc a;
  bool ok = d.ok;
  const unsigned long long session = comm_session(comm);
  int sock = -1;
  size_t gran = 0;

  if (ok) ok = d.p_cuDeviceGet(&a.dev, comm_device(comm)) == CUDA_SUCCESS;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = a.dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  if (ok)
    ok = d.p_cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) ==
         CUDA_SUCCESS;

  // multicast: supported by every device?
  int mc_supported = 0;
  if (ok && d.p_cuMulticastCreate && getenv("COCO_NO_MULTICAST") == nullptr)
    d.p_cuDeviceGetAttribute(&mc_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, a.dev);
  bool want_mc = all_ok(comm, ok && mc_supported != 0);
  CUmulticastObjectProp mcprop;
  memset(&mcprop, 0, sizeof(mcprop));
  if (want_mc) {
    mcprop.numDevices = (unsigned)R;
    mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcprop.size = gran;  // provisional, for the granularity query
    size_t mg = 0;
    if (d.p_cuMulticastGetGranularity(&mg, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
            CUDA_SUCCESS && mg > gran)
      gran = mg;
  }
  if (ok) {
    a.size = (bytes + gran - 1) / gran * gran;
    ok = d.p_cuMemCreate(&a.local, a.size, &prop, 0) == CUDA_SUCCESS;
    if (!ok) a.local = 0;
  }
  if (ok) ok = map_rw(d, &a.va[rank], a.size, gran, a.local, a.dev);
  if (ok) {
    sock = make_socket(session, rank);
    ok = sock >= 0;
  }
  // every rank has its socket bound (or has failed) before anyone sends
  ok = all_ok(comm, ok);

  // ---- exchange the allocations ---------------------------------------------------
  if (ok) {
    int myfd = -1;
    ok = d.p_cuMemExportToShareableHandle(&myfd, a.local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                          0) == CUDA_SUCCESS;
    if (ok) {
      for (int p = 0; p < R && ok; ++p)
        if (p != rank) ok = send_fd(sock, session, p, rank, /*tag*/ 1, myfd);
      ::close(myfd);
    }
    // receive whatever arrives (allocations now, the multicast object later)
    int got = 0;
    while (ok && got < R - 1) {
      int src = -1, tag = -1, fd = -1;
      if (!recv_fd(sock, &src, &tag, &fd)) {
        ok = false;
        break;
      }
      if (tag == 1 && src >= 0 && src < R && src != rank && !a.peer_handle[src]) {
        ok = d.p_cuMemImportFromShareableHandle(&a.peer_handle[src], (void *)(uintptr_t)fd,
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) ==
             CUDA_SUCCESS;
        if (!ok) a.peer_handle[src] = 0;
        if (ok) ok = map_rw(d, &a.va[src], a.size, gran, a.peer_handle[src], a.dev);
        ++got;
      }
      ::close(fd);
    }
  }
  ok = all_ok(comm, ok);

  // ---- multicast object ---------------------------------------------------------------
  if (ok && want_mc) {
    bool mok = true;
    if (rank == 0) {
      mcprop.size = a.size;
      mok = d.p_cuMulticastCreate(&a.mc, &mcprop) == CUDA_SUCCESS;
      if (!mok) a.mc = 0;
      int mfd = -1;
      if (mok)
        mok = d.p_cuMemExportToShareableHandle(&mfd, a.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                               0) == CUDA_SUCCESS;
    // tell everyone whether an object is coming before anyone waits for it
      const bool coming = all_ok(comm, mok);
      if (coming)
        for (int p = 1; p < R && mok; ++p) mok = send_fd(sock, session, p, 0, /*tag*/ 2, mfd);
      else
        mok = false;
      if (mfd >= 0) ::close(mfd);
    } else {
      const bool coming = all_ok(comm, true);
      if (coming) {
        int src = -1, tag = -1, fd = -1;
        mok = recv_fd(sock, &src, &tag, &fd) && tag == 2;
        if (mok) {
          mok = d.p_cuMemImportFromShareableHandle(&a.mc, (void *)(uintptr_t)fd,
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) ==
                CUDA_SUCCESS;
          if (!mok) a.mc = 0;
        }
        if (fd >= 0) ::close(fd);
      } else {
        mok = false;
      }
    }
    if (mok) mok = d.p_cuMulticastAddDevice(a.mc, a.dev) == CUDA_SUCCESS;
    mok = all_ok(comm, mok);  // all devices added before anyone binds
    if (mok) {
      mok = d.p_cuMulticastBindMem(a.mc, 0, a.local, 0, a.size, 0) == CUDA_SUCCESS;
      a.bound = mok;
    }
    mok = all_ok(comm, mok);
    if (mok) mok = map_rw(d, &a.mc_va, a.size, gran, a.mc, a.dev);
    mok = all_ok(comm, mok);
    if (!mok) {  // carry on without the switch path
      if (a.mc_va) unmap(d, a.mc_va, a.size);
      a.mc_va = 0;
      if (a.bound) d.p_cuMulticastUnbind(a.mc, a.dev, 0, a.size);
      a.bound = false;
      if (a.mc) d.p_cuMemRelease(a.mc);
      a.mc = 0;
    }
    a.has_mc = mok;
  }
  if (sock >= 0) ::close(sock);

  if (!ok) {
    release_all(d, a, R, rank);
    return cocoCudaError;
  }
  void *peers[kMaxRanks] = {};
  for (int p = 0; p < R; ++p) peers[p] = (void *)a.va[p];
  int rc = comm_add_mapped_region(comm, (void *)a.va[rank], a.size, peers,
                                  a.has_mc ? (void *)a.mc_va : nullptr);
  if (rc != cocoSuccess) {
    release_all(d, a, R, rank);
    return rc;
  }
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_allocs[comm][(void *)a.va[rank]] = a;
  }
  *ptr = (void *)a.va[rank];
  return cocoSuccess;
}

extern "C" int cocoMemFree(cocoComm_t comm, void *ptr) {
  if (!comm || !ptr) return cocoInvalidArgument;
  SymmAlloc a;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_allocs.find(comm);
    if (it == g_allocs.end() || !it->second.count(ptr)) return cocoInvalidArgument;
    a = it->second[ptr];
    it->second.erase(ptr);
  }
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(comm_device(comm));
  cudaDeviceSynchronize();
  int rc = cocoSuccess;
  if (a.plain) {
    if (cudaFree(ptr) != cudaSuccess) rc = cocoCudaError;
  } else {
    const int R = comm_world(comm), rank = comm_rank(comm);
    comm_remove_region(comm, ptr);
    // nobody unmaps while a peer's kernel may still use the memory
    all_ok(comm, true);
    release_all(driver(), a, R, rank);
    all_ok(comm, true);
  }
  if (prev >= 0) cudaSetDevice(prev);
  return rc;
}

// Called by cocoCommDestroy: whatever the communicator still holds is freed
// (collectively, like cocoMemFree: every rank must hold the same number of
// allocations) and its entry disappears, so that memory bound to a multicast
// object does not outlive the communicator and a later communicator at the same
// address inherits nothing.
namespace coco {
int comm_release_allocs(cocoComm_t comm) {
  int result = cocoSuccess;
  for (;;) {
    void *next = nullptr;
    {
      std::lock_guard<std::mutex> lock(g_mu);
      auto it = g_allocs.find(comm);
      if (it == g_allocs.end()) break;
      if (it->second.empty()) {
        g_allocs.erase(it);
        break;
      }
      next = it->second.begin()->first;
    }
    const int rc = cocoMemFree(comm, next);
    if (rc != cocoSuccess) {
      if (result == cocoSuccess) result = rc;
      std::lock_guard<std::mutex> lock(g_mu);
      auto it = g_allocs.find(comm);
      if (it != g_allocs.end()) it->second.erase(next);  // never loop on a failing entry
    }
  }
  return result;
}
}  // namespace coco

extern "C" int cocoMemHasMulticast(cocoComm_t comm, const void *ptr, int *yes) {
  if (!comm || !ptr || !yes) return cocoInvalidArgument;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_allocs.find(comm);
  if (it == g_allocs.end() || !it->second.count((void *)ptr)) return cocoInvalidArgument;
  *yes = it->second[(void *)ptr].has_mc ? 1 : 0;
  return cocoSuccess;
}
