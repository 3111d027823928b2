#include "bootstrap.h"
#include "log.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <random>
#include <string>
#include <thread>
#include <time.h>
#include <unistd.h>

namespace fcx {

// ------------------------------------------------------------------ sockets

int64_t nowMs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

static void setNonBlocking(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof one);
}

bool parseIpPort(const char *s, SockAddr *out) {
  std::string str(s);
  size_t colon = str.rfind(':');
  if (colon == std::string::npos) return false;
  std::string ip = str.substr(0, colon);
  int port = atoi(str.c_str() + colon + 1);
  if (!ip.empty() && ip.front() == '[' && ip.back() == ']') ip = ip.substr(1, ip.size() - 2);
  memset(out, 0, sizeof *out);
  sockaddr_in *a4 = (sockaddr_in *)&out->ss;
  sockaddr_in6 *a6 = (sockaddr_in6 *)&out->ss;
  if (inet_pton(AF_INET, ip.c_str(), &a4->sin_addr) == 1) {
    a4->sin_family = AF_INET;
    a4->sin_port = htons(port);
    out->len = sizeof(sockaddr_in);
    return true;
  }
  if (inet_pton(AF_INET6, ip.c_str(), &a6->sin6_addr) == 1) {
    a6->sin6_family = AF_INET6;
    a6->sin6_port = htons(port);
    out->len = sizeof(sockaddr_in6);
    return true;
  }
  return false;
}

// Pick the local address that peers should dial.  FLAGCX_SOCKET_IFNAME is a
// comma list of interface-name prefixes ("=name" exact, leading "^" excludes);
// FLAGCX_SOCKET_FAMILY restricts to AF_INET or AF_INET6.
static bool pickInterface(SockAddr *out) {
  std::string want = envStr("SOCKET_IFNAME", "");
  std::string fam = envStr("SOCKET_FAMILY", "");
  int family = fam == "AF_INET6" ? AF_INET6 : (fam == "AF_INET" ? AF_INET : 0);
  bool exclude = !want.empty() && want[0] == '^';
  if (exclude) want = want.substr(1);
  std::vector<std::string> pats;
  for (size_t pos = 0; pos < want.size();) {
    size_t c = want.find(',', pos);
    pats.push_back(want.substr(pos, c == std::string::npos ? std::string::npos : c - pos));
    if (c == std::string::npos) break;
    pos = c + 1;
  }
  auto matches = [&](const char *name) {
    for (auto &p : pats) {
      if (p.empty()) continue;
      if (p[0] == '=') { if (p.substr(1) == name) return true; }
      else if (strncmp(name, p.c_str(), p.size()) == 0) return true;
    }
    return false;
  };
  ifaddrs *ifs = nullptr;
  if (getifaddrs(&ifs) != 0) return false;
  ifaddrs *best = nullptr, *loop = nullptr;
  for (ifaddrs *i = ifs; i; i = i->ifa_next) {
    if (!i->ifa_addr || !(i->ifa_flags & IFF_UP)) continue;
    int f = i->ifa_addr->sa_family;
    if (f != AF_INET && f != AF_INET6) continue;
    if (family && f != family) continue;
    if (!family && f == AF_INET6) continue;  // prefer IPv4 unless asked
    if (!pats.empty()) {
      bool m = matches(i->ifa_name);
      if (m == exclude) continue;
      best = i;
      break;
    }
    if (i->ifa_flags & IFF_LOOPBACK) { if (!loop) loop = i; continue; }
    if (strncmp(i->ifa_name, "docker", 6) == 0) continue;
    if (!best) best = i;
  }
  if (!best) best = loop;
  bool ok = false;
  if (best) {
    memset(out, 0, sizeof *out);
    out->len = best->ifa_addr->sa_family == AF_INET ? sizeof(sockaddr_in) : sizeof(sockaddr_in6);
    memcpy(&out->ss, best->ifa_addr, out->len);
    FCX_INFO(SUB_BOOTSTRAP | SUB_INIT, "bootstrap: using interface %s", best->ifa_name);
    ok = true;
  }
  freeifaddrs(ifs);
  return ok;
}

flagcxResult_t sockListen(int *fdOut, SockAddr *addr, const SockAddr *fixed) {
  SockAddr a;
  if (fixed) a = *fixed;
  else if (!pickInterface(&a)) {
    FCX_WARN("bootstrap: no usable network interface");
    return flagcxSystemError;
  }
  int fd = socket(a.ss.ss_family, SOCK_STREAM, 0);
  if (fd < 0) return flagcxSystemError;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  if (!fixed) {
    if (a.ss.ss_family == AF_INET) ((sockaddr_in *)&a.ss)->sin_port = 0;
    else ((sockaddr_in6 *)&a.ss)->sin6_port = 0;
  }
  if (bind(fd, (sockaddr *)&a.ss, a.len) != 0 || listen(fd, 4096) != 0) {
    FCX_WARN("bootstrap: bind/listen failed: %s", strerror(errno));
    ::close(fd);
    return flagcxSystemError;
  }
  socklen_t l = sizeof a.ss;
  getsockname(fd, (sockaddr *)&a.ss, &l);
  a.len = l;
  setNonBlocking(fd);
  *fdOut = fd;
  *addr = a;
  return flagcxSuccess;
}

static bool expired(int64_t deadlineMs) { return deadlineMs > 0 && nowMs() > deadlineMs; }

flagcxResult_t sockConnect(int *fdOut, const SockAddr &addr, int64_t deadlineMs, std::atomic<uint32_t> *ab) {
  // A refused connection is retried (the peer may not be listening yet);
  // any other error, the deadline or the abort flag end the attempt.
  for (;;) {
    int fd = socket(addr.ss.ss_family, SOCK_STREAM, 0);
    if (fd < 0) return flagcxSystemError;
    setNonBlocking(fd);
    int rc = connect(fd, (const sockaddr *)&addr.ss, addr.len);
    if (rc != 0 && errno == EINPROGRESS) {
      for (;;) {
        pollfd p{fd, POLLOUT, 0};
        int pr = poll(&p, 1, 50);
        if (pr > 0) break;
        if (expired(deadlineMs) || (ab && ab->load())) { ::close(fd); return flagcxRemoteError; }
      }
      int err = 0;
      socklen_t el = sizeof err;
      getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &el);
      rc = err ? -1 : 0;
      errno = err;
    }
    if (rc == 0) { *fdOut = fd; return flagcxSuccess; }
    int e = errno;
    ::close(fd);
    if (e != ECONNREFUSED && e != ETIMEDOUT && e != EAGAIN) {
      FCX_WARN("bootstrap: connect failed: %s", strerror(e));
      return flagcxSystemError;
    }
    if (expired(deadlineMs) || (ab && ab->load())) {
      FCX_WARN("bootstrap: connect gave up (%s)", strerror(e));
      return flagcxRemoteError;
    }
    usleep(1000);
  }
}

flagcxResult_t sockAccept(int listenFd, int *fdOut, int64_t deadlineMs, std::atomic<uint32_t> *ab) {
  for (;;) {
    int fd = accept(listenFd, nullptr, nullptr);
    if (fd >= 0) { setNonBlocking(fd); *fdOut = fd; return flagcxSuccess; }
    if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return flagcxSystemError;
    pollfd p{listenFd, POLLIN, 0};
    poll(&p, 1, 50);
    if (expired(deadlineMs) || (ab && ab->load())) return flagcxRemoteError;
  }
}

flagcxResult_t sockSendAll(int fd, const void *buf, size_t n, int64_t deadlineMs, std::atomic<uint32_t> *ab) {
  const char *p = (const char *)buf;
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w > 0) { p += w; n -= w; continue; }
    if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return flagcxRemoteError;
    pollfd pf{fd, POLLOUT, 0};
    poll(&pf, 1, 50);
    if (expired(deadlineMs) || (ab && ab->load())) return flagcxRemoteError;
  }
  return flagcxSuccess;
}

flagcxResult_t sockRecvAll(int fd, void *buf, size_t n, int64_t deadlineMs, std::atomic<uint32_t> *ab) {
  char *p = (char *)buf;
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r > 0) { p += r; n -= r; continue; }
    if (r == 0) return flagcxRemoteError;  // peer closed
    if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return flagcxRemoteError;
    pollfd pf{fd, POLLIN, 0};
    poll(&pf, 1, 50);
    if (expired(deadlineMs) || (ab && ab->load())) return flagcxRemoteError;
  }
  return flagcxSuccess;
}

uint64_t hostHash() {
  // FLAGCX_HOSTID lets one machine pose as several hosts in tests.
  std::string id = envStr("HOSTID", "");
  if (id.empty()) {
    char h[256] = "";
    gethostname(h, sizeof h - 1);
    id = h;
    if (FILE *f = fopen("/proc/sys/kernel/random/boot_id", "r")) {
      char b[64] = "";
      if (fgets(b, sizeof b, f)) id += b;
      fclose(f);
    }
  }
  uint64_t x = 1469598103934665603ull;  // FNV-1a
  for (unsigned char c : id) { x ^= c; x *= 1099511628211ull; }
  return x;
}

// ------------------------------------------------------------------ root

namespace {

constexpr uint64_t kHelloMagic = 0xf1a9c0ffee5eedull;

struct CheckIn {
  uint64_t magic;
  int32_t rank, nranks;
  SockAddr listenAddr;
};

struct PeerHello {
  uint64_t magic;
  int32_t rank;
  int32_t pad;
};

struct MsgHeader {
  int32_t tag;
  int32_t pad;
  uint64_t bytes;
};

// Root service: collect one check-in per rank, then send the full table.
void rootThread(int listenFd, uint64_t magic) {
  nameThisThread("flagcx-root");
  int64_t dl = nowMs() + envInt("BOOTSTRAP_TIMEOUT_MS", 600000);
  std::vector<int> fds;
  std::vector<SockAddr> table;
  int nranks = -1, got = 0;
  bool bad = false;
  while (nranks < 0 || got < nranks) {
    int fd;
    if (sockAccept(listenFd, &fd, dl, nullptr) != flagcxSuccess) { bad = true; break; }
    CheckIn ci;
    if (sockRecvAll(fd, &ci, sizeof ci, dl, nullptr) != flagcxSuccess || ci.magic != magic) {
      // A stranger (port scanner, stale rank of another job): drop it.
      FCX_INFO(SUB_BOOTSTRAP, "bootstrap root: rejected a connection with a wrong magic");
      ::close(fd);
      continue;
    }
    if (nranks < 0) {
      nranks = ci.nranks;
      fds.assign(nranks, -1);
      table.resize(nranks);
    }
    if (ci.nranks != nranks || ci.rank < 0 || ci.rank >= nranks) {
      FCX_WARN("bootstrap root: rank %d reports %d ranks, expected %d", ci.rank, ci.nranks, nranks);
      ::close(fd);
      bad = true;
      break;
    }
    if (fds[ci.rank] >= 0) {
      FCX_WARN("bootstrap root: rank %d checked in twice", ci.rank);
      ::close(fd);
      bad = true;
      break;
    }
    fds[ci.rank] = fd;
    table[ci.rank] = ci.listenAddr;
    got++;
  }
  for (int r = 0; r < (int)fds.size(); r++) {
    if (fds[r] < 0) continue;
    int32_t ok = bad ? 0 : 1;
    sockSendAll(fds[r], &ok, sizeof ok, dl, nullptr);
    if (!bad) sockSendAll(fds[r], table.data(), table.size() * sizeof(SockAddr), dl, nullptr);
    ::close(fds[r]);
  }
  ::close(listenFd);
}

}  // namespace

static constexpr uint64_t kFixedIdMagic = 0x464c41474358ull;

flagcxResult_t Bootstrap::createId(BootstrapHandle *out, bool allowFixedAddress) {
  memset(out, 0, sizeof *out);
  const char *fixed = allowFixedAddress ? getEnv("FLAGCX_COMM_ID") : nullptr;
  if (fixed) {
    // Static rendezvous: every rank derives the same handle; rank 0 opens it.
    if (!parseIpPort(fixed, &out->addr)) {
      FCX_WARN("FLAGCX_COMM_ID must be ip:port, got '%s'", fixed);
      return flagcxInvalidArgument;
    }
    out->magic = kFixedIdMagic;  // constant: all ranks must agree without talking
    return flagcxSuccess;
  }
  std::random_device rd;
  out->magic = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 17);
  int fd;
  FCX_CHECK(sockListen(&fd, &out->addr, nullptr));
  std::thread(rootThread, fd, out->magic).detach();
  return flagcxSuccess;
}

// ------------------------------------------------------------------ member functions

Bootstrap::~Bootstrap() { close(); }

void Bootstrap::close() {
  std::lock_guard<std::recursive_mutex> lk(mu_);
  for (int &fd : conns_)
    if (fd >= 0) { ::close(fd); fd = -1; }
  if (listenFd_ >= 0) { ::close(listenFd_); listenFd_ = -1; }
}

int64_t Bootstrap::deadline() const { return timeoutMs_ > 0 ? nowMs() + timeoutMs_ : 0; }

flagcxResult_t Bootstrap::init(const BootstrapHandle &h, int rank, int nranks) {
  rank_ = rank;
  nranks_ = nranks;
  magic_ = h.magic;
  timeoutMs_ = envInt("BOOTSTRAP_TIMEOUT_MS", 600000);
  conns_.assign(nranks, -1);

  // Host-side fault injector: "<kind>[:<arg>]", optionally limited to one
  // rank by FLAGCX_FAULT_RANK.  Kinds: bad_magic, close_after:N, delay_ms:N,
  // exit_after:N.  Nothing here touches a GPU.
  std::string fi = envStr("FAULT_INJECT", "");
  int64_t onlyRank = envInt("FAULT_RANK", -1);
  if (!fi.empty() && (onlyRank < 0 || onlyRank == rank)) {
    size_t c = fi.find(':');
    std::string kind = fi.substr(0, c);
    faultArg_ = c == std::string::npos ? 0 : atoll(fi.c_str() + c + 1);
    faultKind_ = kind == "bad_magic" ? 1 : kind == "close_after" ? 2 : kind == "delay_ms" ? 3 : kind == "exit_after" ? 4 : 0;
  }

  if (getEnv("FLAGCX_COMM_ID") && rank == 0 && h.magic == kFixedIdMagic) {
    int fd;
    SockAddr a;
    FCX_CHECK(sockListen(&fd, &a, &h.addr));
    std::thread(rootThread, fd, h.magic).detach();
  }

  SockAddr mine;
  FCX_CHECK(sockListen(&listenFd_, &mine, nullptr));

  int rootFd;
  int64_t dl = deadline();
  FCX_CHECK(sockConnect(&rootFd, h.addr, dl, abort_));
  CheckIn ci{};
  ci.magic = faultKind_ == 1 ? ~h.magic : h.magic;
  ci.rank = rank;
  ci.nranks = nranks;
  ci.listenAddr = mine;
  flagcxResult_t r = sockSendAll(rootFd, &ci, sizeof ci, dl, abort_);
  int32_t ok = 0;
  if (r == flagcxSuccess) r = sockRecvAll(rootFd, &ok, sizeof ok, dl, abort_);
  addrs_.resize(nranks);
  if (r == flagcxSuccess && ok) r = sockRecvAll(rootFd, addrs_.data(), nranks * sizeof(SockAddr), dl, abort_);
  ::close(rootFd);
  if (r != flagcxSuccess || !ok) {
    FCX_WARN("bootstrap: rank %d could not complete the rendezvous", rank);
    return r != flagcxSuccess ? r : flagcxInvalidUsage;
  }
  FCX_INFO(SUB_BOOTSTRAP | SUB_INIT, "bootstrap: rank %d/%d ready", rank, nranks);
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::ensureConn(int peer) {
  if (conns_[peer] >= 0) return flagcxSuccess;
  int64_t dl = deadline();
  if (rank_ < peer) {
    int fd;
    FCX_CHECK(sockConnect(&fd, addrs_[peer], dl, abort_));
    PeerHello hi{kHelloMagic ^ magic_, rank_, 0};
    flagcxResult_t r = sockSendAll(fd, &hi, sizeof hi, dl, abort_);
    if (r != flagcxSuccess) { ::close(fd); return r; }
    conns_[peer] = fd;
    return flagcxSuccess;
  }
  // The lower rank dials; accept until that peer has shown up, keeping any
  // other peers that arrive in the meantime.
  while (conns_[peer] < 0) {
    int fd;
    flagcxResult_t r = sockAccept(listenFd_, &fd, dl, abort_);
    if (r != flagcxSuccess) {
      FCX_WARN("bootstrap: rank %d never heard from rank %d", rank_, peer);
      return r;
    }
    PeerHello hi;
    r = sockRecvAll(fd, &hi, sizeof hi, dl, abort_);
    if (r != flagcxSuccess || hi.magic != (kHelloMagic ^ magic_) || hi.rank < 0 || hi.rank >= nranks_ || conns_[hi.rank] >= 0) {
      ::close(fd);
      continue;
    }
    conns_[hi.rank] = fd;
  }
  return flagcxSuccess;
}

void Bootstrap::maybeInjectFault() {
  if (!faultKind_) return;
  if (faultKind_ == 3) usleep(faultArg_ * 1000);
  if (faultKind_ == 2 && (int64_t)nSent_ >= faultArg_) {
    for (int &fd : conns_)
      if (fd >= 0) { ::shutdown(fd, SHUT_RDWR); }
  }
  if (faultKind_ == 4 && (int64_t)nSent_ >= faultArg_) _exit(17);
}

bool Bootstrap::takeUnexpected(int peer, int tag, void *buf, size_t bytes, flagcxResult_t *res) {
  for (auto it = unexpected_.begin(); it != unexpected_.end(); ++it) {
    if (it->peer == peer && it->tag == tag) {
      if (it->data.size() != bytes) {
        FCX_WARN("bootstrap: message from %d tag %d has %zu bytes, expected %zu", peer, tag, it->data.size(), bytes);
        *res = flagcxInternalError;
      } else {
        memcpy(buf, it->data.data(), bytes);
        *res = flagcxSuccess;
      }
      unexpected_.erase(it);
      return true;
    }
  }
  return false;
}

flagcxResult_t Bootstrap::sendrecv(int sp, int stag, const void *sbuf, size_t sbytes,
                                   int rp, int rtag, void *rbuf, size_t rbytes) {
  std::lock_guard<std::recursive_mutex> lk(mu_);
  maybeInjectFault();
  // Messages to self go through a local queue.
  if (sp == rank_) {
    selfQueue_.push_back({rank_, stag, std::vector<char>((const char *)sbuf, (const char *)sbuf + sbytes)});
    sp = -1;
    nSent_++;
  }
  if (rp == rank_) {
    for (auto it = selfQueue_.begin(); it != selfQueue_.end(); ++it)
      if (it->tag == rtag) {
        if (it->data.size() != rbytes) return flagcxInternalError;
        memcpy(rbuf, it->data.data(), rbytes);
        selfQueue_.erase(it);
        rp = -1;
        break;
      }
    if (rp == rank_) {
      FCX_WARN("bootstrap: receive from self with nothing queued (tag %d)", rtag);
      return flagcxInvalidUsage;
    }
  }
  if (sp >= 0) FCX_CHECK(ensureConn(sp));
  bool recvDone = rp < 0;
  if (!recvDone) {
    flagcxResult_t r;
    if (takeUnexpected(rp, rtag, rbuf, rbytes, &r)) {
      if (r != flagcxSuccess) return r;
      recvDone = true;
    } else {
      FCX_CHECK(ensureConn(rp));
    }
  }

  // Send side state.
  MsgHeader sh{stag, 0, (uint64_t)sbytes};
  size_t sHdrLeft = sp >= 0 ? sizeof sh : 0, sLeft = sp >= 0 ? sbytes : 0;
  const char *sHdrP = (const char *)&sh, *sP = (const char *)sbuf;
  // Receive side state: header, then payload into rbuf or into a stash.
  MsgHeader rh{};
  size_t rHdrLeft = sizeof rh, rLeft = 0;
  char *rHdrP = (char *)&rh, *rP = nullptr;
  bool inPayload = false, toStash = false;
  Stash stash;

  int64_t dl = deadline();
  while (sHdrLeft || sLeft || !recvDone) {
    pollfd pf[2];
    int np = 0, si = -1, ri = -1;
    if (sHdrLeft || sLeft) { pf[np] = {conns_[sp], POLLOUT, 0}; si = np++; }
    if (!recvDone) { pf[np] = {conns_[rp], POLLIN, 0}; ri = np++; }
    int pr = poll(pf, np, 50);
    if (pr < 0 && errno != EINTR) return flagcxSystemError;
    if (expired(dl) || aborted()) {
      FCX_WARN("bootstrap: rank %d timed out (send to %d, recv from %d)", rank_, sp, rp);
      return flagcxRemoteError;
    }
    if (si >= 0 && (pf[si].revents & (POLLOUT | POLLERR | POLLHUP))) {
      const char *&p = sHdrLeft ? sHdrP : sP;
      size_t &left = sHdrLeft ? sHdrLeft : sLeft;
      ssize_t w = ::send(conns_[sp], p, left, MSG_NOSIGNAL);
      if (w > 0) { p += w; left -= w; dl = deadline(); }
      else if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) {
        FCX_WARN("bootstrap: send to rank %d failed: %s", sp, strerror(errno));
        return flagcxRemoteError;
      }
      if (!sHdrLeft && !sLeft) nSent_++;
    }
    if (ri >= 0 && (pf[ri].revents & (POLLIN | POLLERR | POLLHUP))) {
      char *&p = inPayload ? rP : rHdrP;
      size_t &left = inPayload ? rLeft : rHdrLeft;
      ssize_t r = left ? ::recv(conns_[rp], p, left, 0) : 0;
      if (left && r == 0) {
        FCX_WARN("bootstrap: rank %d closed the connection", rp);
        return flagcxRemoteError;
      }
      if (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) {
        FCX_WARN("bootstrap: recv from rank %d failed: %s", rp, strerror(errno));
        return flagcxRemoteError;
      }
      if (r > 0) { p += r; left -= r; dl = deadline(); }
      if (!inPayload && rHdrLeft == 0) {
        inPayload = true;
        rLeft = rh.bytes;
        if (rh.tag == rtag) {
          if (rh.bytes != rbytes) {
            FCX_WARN("bootstrap: message from %d tag %d has %llu bytes, expected %zu", rp, rtag,
                     (unsigned long long)rh.bytes, rbytes);
            return flagcxInternalError;
          }
          toStash = false;
          rP = (char *)rbuf;
        } else {
          toStash = true;
          stash = {rp, rh.tag, std::vector<char>(rh.bytes)};
          rP = stash.data.data();
        }
      }
      if (inPayload && rLeft == 0) {
        if (toStash) {
          unexpected_.push_back(std::move(stash));
          inPayload = false;
          rHdrLeft = sizeof rh;
          rHdrP = (char *)&rh;
        } else {
          recvDone = true;
        }
      }
    }
  }
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::send(int peer, int tag, const void *buf, size_t bytes) {
  return sendrecv(peer, tag, buf, bytes, -1, 0, nullptr, 0);
}

flagcxResult_t Bootstrap::recv(int peer, int tag, void *buf, size_t bytes) {
  return sendrecv(-1, 0, nullptr, 0, peer, tag, buf, bytes);
}

flagcxResult_t Bootstrap::allGather(void *buf, size_t bytes) {
  // Ring: in step s forward the slot received in step s-1.
  if (nranks_ == 1) return flagcxSuccess;
  char *b = (char *)buf;
  int next = (rank_ + 1) % nranks_, prev = (rank_ + nranks_ - 1) % nranks_;
  for (int s = 0; s < nranks_ - 1; s++) {
    int sendSlot = (rank_ - s + nranks_) % nranks_;
    int recvSlot = (rank_ - s - 1 + nranks_) % nranks_;
    FCX_CHECK(sendrecv(next, 0x7a000 + s, b + sendSlot * bytes, bytes, prev, 0x7a000 + s, b + recvSlot * bytes, bytes));
  }
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::barrier() {
  // Dissemination barrier: log2(n) rounds of one-byte messages.
  char tok = 1, in;
  int e = barrierEpoch_++ & 0xff;
  for (int d = 1, round = 0; d < nranks_; d <<= 1, round++) {
    int to = (rank_ + d) % nranks_, from = (rank_ - d + nranks_) % nranks_;
    int tag = 0x7b0000 + (e << 8) + round;
    FCX_CHECK(sendrecv(to, tag, &tok, 1, from, tag, &in, 1));
  }
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::broadcast(void *buf, size_t bytes, int root) {
  if (nranks_ == 1) return flagcxSuccess;
  // Binomial tree rooted at `root`.
  int vr = (rank_ - root + nranks_) % nranks_;
  int mask = 1;
  while (mask < nranks_) {
    if (vr & mask) {
      int src = (rank_ - mask + nranks_) % nranks_;
      FCX_CHECK(recv(src, 0x7c000, buf, bytes));
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < nranks_) {
      int dst = (rank_ + mask) % nranks_;
      FCX_CHECK(send(dst, 0x7c000, buf, bytes));
    }
    mask >>= 1;
  }
  return flagcxSuccess;
}

}  // namespace fcx
