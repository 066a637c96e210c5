// Out-of-band rendezvous between the ranks of a communicator: a star of TCP
// connections to rank 0.  Stands where the reference uses MPI_Bcast of the
// ncclUniqueId plus NCCL's own TCP bootstrap (src/codegen.cpp:4587-4601 and
// nccl/src/bootstrap.cc:227-359 in parasailteam/coconet).  Host code only.
#pragma once

#include <stddef.h>

#include <string>
#include <vector>

namespace coco {

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  Bootstrap(const Bootstrap &) = delete;
  Bootstrap &operator=(const Bootstrap &) = delete;

  // addr is "host:port"; rank 0 listens there, the others connect (retrying
  // until timeout_ms).  Returns 0, or a cocoResult_t.
  int init(int world, int rank, const std::string &addr, int timeout_ms);

  // recv must hold world * bytes; slot r receives rank r's `send`.  Ranks that
  // are not in the same collective (count, kind or size differ) get
  // cocoInvalidUsage, and so does every later call.
  int all_gather(const void *send, void *recv, size_t bytes);
  int barrier();

  int world() const { return world_; }
  int rank() const { return rank_; }

 private:
  int exchange(const void *send, void *recv, size_t bytes, unsigned kind);
  int world_ = 0, rank_ = -1;
  unsigned long long op_ = 0;   // collectives issued so far on this rank
  bool broken_ = false;         // the ranks fell out of step
  int listen_fd_ = -1;
  int root_fd_ = -1;            // non-root: connection to rank 0
  std::vector<int> peer_fd_;    // root: connection to each rank (index = rank)
};

// Resolves the rendezvous address: explicit argument, else COCO_BOOTSTRAP,
// else MASTER_ADDR:(MASTER_PORT+1), else 127.0.0.1:29533.
std::string resolve_bootstrap_addr(const char *explicit_addr);

}  // namespace coco
