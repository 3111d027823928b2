// TCP rendezvous and host-side messaging between the ranks of a communicator.
//
// Role in the library: (1) carry the 256-byte unique id semantics of
// flagcxGetUniqueId / flagcxCommInitRank (reference: flagcx/service/bootstrap.cc:124-332),
// (2) exchange set-up data (memory export handles, peer info, tuner timings),
// (3) serve as the transport of the CPU host-collective path.
//
// Differences from the reference's bootstrap: the root hands every rank the
// whole address table (no ring hand-off), pairwise connections are opened on
// first use, every blocking step has a deadline and polls an abort flag, and
// a host-side fault injector can be armed through FLAGCX_FAULT_INJECT.
#pragma once
#include "flagcx.h"
#include <atomic>
#include <cstdint>
#include <deque>
#include <mutex>
#include <sys/socket.h>
#include <vector>

namespace fcx {

struct SockAddr {
  sockaddr_storage ss;
  uint32_t len;
};

// What lives inside flagcxUniqueId.internal.
struct BootstrapHandle {
  uint64_t magic;
  SockAddr addr;
};
static_assert(sizeof(BootstrapHandle) <= FLAGCX_UNIQUE_ID_BYTES, "handle must fit the unique id");

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  Bootstrap(const Bootstrap &) = delete;

  // Creates the root listener + service thread and fills `out`.
  // With FLAGCX_COMM_ID=ip:port the address is fixed and only rank 0's
  // process actually starts the root thread (in init()).
  static flagcxResult_t createId(BootstrapHandle *out, bool allowFixedAddress = true);

  flagcxResult_t init(const BootstrapHandle &h, int rank, int nranks);
  void close();

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  void setAbortFlag(std::atomic<uint32_t> *f) { abort_ = f; }

  // Tagged point-to-point messages (blocking, deadline-bounded).
  flagcxResult_t send(int peer, int tag, const void *buf, size_t bytes);
  flagcxResult_t recv(int peer, int tag, void *buf, size_t bytes);
  // Full-duplex step: send to one peer while receiving from another.
  // Either direction can be disabled by passing peer -1.
  flagcxResult_t sendrecv(int sendPeer, int sendTag, const void *sbuf, size_t sbytes,
                          int recvPeer, int recvTag, void *rbuf, size_t rbytes);

  // Collectives over the rank set (host memory).
  flagcxResult_t allGather(void *buf, size_t bytesPerRank);  // in place, slot r = rank r
  flagcxResult_t barrier();
  flagcxResult_t broadcast(void *buf, size_t bytes, int root);

  // Counters for tests and the failure detector.
  uint64_t messagesSent() const { return nSent_; }

 private:
  flagcxResult_t ensureConn(int peer);
  bool takeUnexpected(int peer, int tag, void *buf, size_t bytes, flagcxResult_t *res);
  int64_t deadline() const;
  bool aborted() const { return abort_ && abort_->load(std::memory_order_relaxed); }
  void maybeInjectFault();

  int rank_ = -1, nranks_ = 0;
  uint64_t magic_ = 0;
  int listenFd_ = -1;
  std::vector<SockAddr> addrs_;
  std::vector<int> conns_;
  struct Stash { int peer; int tag; std::vector<char> data; };
  std::deque<Stash> unexpected_;
  std::deque<Stash> selfQueue_;
  std::recursive_mutex mu_;
  std::atomic<uint32_t> *abort_ = nullptr;
  int64_t timeoutMs_ = 120000;
  uint64_t nSent_ = 0;
  int barrierEpoch_ = 0;
  // fault injection (host side only)
  int faultKind_ = 0;
  int64_t faultArg_ = 0;
};

// Low-level helpers shared with the symmetric-heap fd exchange.
int64_t nowMs();
flagcxResult_t sockListen(int *fd, SockAddr *addr, const SockAddr *fixed);
flagcxResult_t sockConnect(int *fd, const SockAddr &addr, int64_t deadlineMs, std::atomic<uint32_t> *abortFlag);
flagcxResult_t sockAccept(int listenFd, int *fd, int64_t deadlineMs, std::atomic<uint32_t> *abortFlag);
flagcxResult_t sockSendAll(int fd, const void *buf, size_t n, int64_t deadlineMs, std::atomic<uint32_t> *abortFlag);
flagcxResult_t sockRecvAll(int fd, void *buf, size_t n, int64_t deadlineMs, std::atomic<uint32_t> *abortFlag);
bool parseIpPort(const char *s, SockAddr *out);
uint64_t hostHash();  // honours FLAGCX_HOSTID

}  // namespace fcx
