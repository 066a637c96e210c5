#include "bootstrap.h"

#include <algorithm>

#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include "coconet_rt.h"

namespace coco {
namespace {

int send_all(int fd, const void *buf, size_t n) {
  const char *p = (const char *)buf;
  while (n > 0) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR) continue;
      return (errno == EAGAIN || errno == EWOULDBLOCK) ? cocoTimeout : cocoSystemError;
    }
    p += k;
    n -= (size_t)k;
  }
  return cocoSuccess;
}

int recv_all(int fd, void *buf, size_t n) {
  char *p = (char *)buf;
  while (n > 0) {
    ssize_t k = ::recv(fd, p, n, 0);
    if (k < 0) {
      if (errno == EINTR) continue;
      return (errno == EAGAIN || errno == EWOULDBLOCK) ? cocoTimeout : cocoSystemError;
    }
    if (k == 0) return cocoSystemError;  // peer closed
    p += k;
    n -= (size_t)k;
  }
  return cocoSuccess;
}

void set_timeouts(int fd, int timeout_ms) {
  struct timeval tv;
  tv.tv_sec = timeout_ms / 1000;
  tv.tv_usec = (timeout_ms % 1000) * 1000;
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

double now_ms() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

bool split_addr(const std::string &addr, std::string *host, int *port) {
  size_t c = addr.rfind(':');
  if (c == std::string::npos) return false;
  *host = addr.substr(0, c);
  *port = atoi(addr.c_str() + c + 1);
  return *port > 0 && *port < 65536 && !host->empty();
}

}  // namespace

std::string resolve_bootstrap_addr(const char *explicit_addr) {
  if (explicit_addr && explicit_addr[0]) return explicit_addr;
  if (const char *e = getenv("COCO_BOOTSTRAP"))
    if (e[0]) return e;
  const char *ma = getenv("MASTER_ADDR");
  const char *mp = getenv("MASTER_PORT");
  if (ma && mp && ma[0] && mp[0]) return std::string(ma) + ":" + std::to_string(atoi(mp) + 1);
  return "127.0.0.1:29533";
}

Bootstrap::~Bootstrap() {
  if (root_fd_ >= 0) ::close(root_fd_);
  for (int fd : peer_fd_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
}

int Bootstrap::init(int world, int rank, const std::string &addr, int timeout_ms) {
  if (world < 1 || rank < 0 || rank >= world) return cocoInvalidArgument;
  world_ = world;
  rank_ = rank;
  if (world == 1) return cocoSuccess;

  std::string host;
  int port = 0;
  if (!split_addr(addr, &host, &port)) return cocoInvalidArgument;

  struct addrinfo hints;
  memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo *res = nullptr;
  if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res)
    return cocoSystemError;
  struct sockaddr_in sa = *(struct sockaddr_in *)res->ai_addr;
  freeaddrinfo(res);

  const double deadline = now_ms() + timeout_ms;
  if (rank == 0) {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (listen_fd_ < 0) return cocoSystemError;
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (::bind(listen_fd_, (struct sockaddr *)&sa, sizeof(sa)) != 0) return cocoSystemError;
    if (::listen(listen_fd_, world) != 0) return cocoSystemError;
    struct timeval tv;
    tv.tv_sec = timeout_ms / 1000;
    tv.tv_usec = (timeout_ms % 1000) * 1000;
    setsockopt(listen_fd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));  // bounds accept()
    peer_fd_.assign(world, -1);
    for (int k = 1; k < world; ++k) {
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) return (errno == EAGAIN || errno == EWOULDBLOCK) ? cocoTimeout : cocoSystemError;
      set_timeouts(fd, timeout_ms);
      int32_t hello[2];
      int rc = recv_all(fd, hello, sizeof(hello));
      if (rc != cocoSuccess) {
        ::close(fd);
        return rc;
      }
      if (hello[0] != world || hello[1] <= 0 || hello[1] >= world || peer_fd_[hello[1]] >= 0) {
        ::close(fd);
        return cocoInvalidUsage;  // mismatched world size or duplicate rank
      }
      peer_fd_[hello[1]] = fd;
    }
    return cocoSuccess;
  }

  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return cocoSystemError;
    if (::connect(fd, (struct sockaddr *)&sa, sizeof(sa)) == 0) {
      set_timeouts(fd, timeout_ms);
      int32_t hello[2] = {world, rank};
      int rc = send_all(fd, hello, sizeof(hello));
      if (rc != cocoSuccess) {
        ::close(fd);
        return rc;
      }
      root_fd_ = fd;
      return cocoSuccess;
    }
    ::close(fd);
    if (now_ms() > deadline) return cocoTimeout;
    usleep(20 * 1000);
  }
}

// Every exchange starts with a small header -- which collective this is (a
// running count kept by every rank), of what kind, and how many bytes the rank
// contributes -- so that ranks that fell out of step (one of them skipped or
// added a collective, or disagrees on the size) get cocoInvalidUsage instead of
// one rank's handle blob being read as another's barrier byte.  After a
// mismatch the connection is out of step for good: every later call fails.
namespace {
constexpr uint32_t kMagic = 0xC0C0B007u;
struct Header {
  uint32_t magic;
  uint32_t kind;    // 0 all-gather, 1 barrier; in rank 0's reply: 0 ok, 1 mismatch
  uint64_t op;      // index of this collective on the communicator
  uint64_t bytes;   // per-rank payload
};
}  // namespace

int Bootstrap::exchange(const void *send, void *recv, size_t bytes, unsigned kind) {
  if (broken_) return cocoInvalidUsage;
  const uint64_t op = ++op_;
  if (world_ == 1) {
    if (recv != send) memcpy(recv, send, bytes);
    return cocoSuccess;
  }
  char *out = (char *)recv;
  if (rank_ == 0) {
    memmove(out, send, bytes);
    bool mismatch = false;
    for (int r = 1; r < world_; ++r) {
      Header h;
      int rc = recv_all(peer_fd_[r], &h, sizeof(h));
      if (rc != cocoSuccess) return rc;
      if (h.magic != kMagic || h.kind != kind || h.op != op || h.bytes != bytes) {
        mismatch = true;  // drain what the rank sends behind its header, within reason
        std::vector<char> sink(4096);
        uint64_t left = h.magic == kMagic ? std::min<uint64_t>(h.bytes, 1u << 24) : 0;
        while (left > 0) {
          const size_t n = (size_t)std::min<uint64_t>(left, sink.size());
          if (recv_all(peer_fd_[r], sink.data(), n) != cocoSuccess) break;
          left -= n;
        }
        continue;
      }
      rc = recv_all(peer_fd_[r], out + (size_t)r * bytes, bytes);
      if (rc != cocoSuccess) return rc;
    }
    Header reply = {kMagic, mismatch ? 1u : 0u, op, (uint64_t)bytes};
    int result = mismatch ? cocoInvalidUsage : cocoSuccess;
    for (int r = 1; r < world_; ++r) {
      int rc = send_all(peer_fd_[r], &reply, sizeof(reply));
      if (rc == cocoSuccess && !mismatch) rc = send_all(peer_fd_[r], out, bytes * world_);
      if (rc != cocoSuccess && result == cocoSuccess) result = rc;
    }
    if (mismatch) broken_ = true;
    return result;
  }
  const Header h = {kMagic, kind, op, (uint64_t)bytes};
  int rc = send_all(root_fd_, &h, sizeof(h));
  if (rc == cocoSuccess) rc = send_all(root_fd_, send, bytes);
  if (rc != cocoSuccess) return rc;
  Header reply;
  rc = recv_all(root_fd_, &reply, sizeof(reply));
  if (rc != cocoSuccess) return rc;
  if (reply.magic != kMagic || reply.kind != 0 || reply.op != op) {
    broken_ = true;
    return cocoInvalidUsage;
  }
  return recv_all(root_fd_, out, bytes * world_);
}

int Bootstrap::all_gather(const void *send, void *recv, size_t bytes) {
  return exchange(send, recv, bytes, 0);
}

int Bootstrap::barrier() {
  std::vector<char> tmp(world_ > 0 ? world_ : 1);
  char me = 1;
  return exchange(&me, tmp.data(), 1, 1);
}

}  // namespace coco
