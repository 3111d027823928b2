// TCP implementation of the network transport table (flagcx_net.h).
// Requests are progressed inside test(), without helper threads; one message
// per request, framed by a 16-byte header {size, tag}.
#include "flagcx_net.h"
#include "bootstrap.h"
#include "log.h"

#include <cerrno>
#include <cstring>
#include <poll.h>
#include <unistd.h>

using namespace fcx;

namespace {

struct ListenComm { int fd; };
struct Conn { int fd; };
struct Hdr { uint64_t size; int32_t tag; int32_t pad; };
struct Req {
  int fd;
  bool isSend;
  Hdr hdr;
  size_t hdrDone = 0, dataDone = 0, cap = 0;
  char *data = nullptr;
  bool failed = false;
};

flagcxResult_t sInit() { return flagcxSuccess; }
flagcxResult_t sDevices(int *n) { *n = 1; return flagcxSuccess; }
flagcxResult_t sProps(int, flagcxNetProperties_t *p) {
  memset(p, 0, sizeof *p);
  snprintf(p->name, sizeof p->name, "socket");
  p->ptrSupport = FLAGCX_PTR_HOST;
  p->speedMbps = 10000;
  p->latencyUs = 30.f;
  p->maxComms = 65536;
  p->maxRecvs = 1;
  return flagcxSuccess;
}
flagcxResult_t sListen(int, void *handle, void **lc) {
  SockAddr a;
  int fd;
  FCX_CHECK(sockListen(&fd, &a, nullptr));
  // handle = {address length, address bytes}; IPv4/IPv6 socket addresses take at most 28 bytes
  memset(handle, 0, FLAGCX_NET_HANDLE_MAXSIZE);
  memcpy(handle, &a.len, sizeof a.len);
  memcpy((char *)handle + sizeof a.len, &a.ss, std::min<size_t>(a.len, FLAGCX_NET_HANDLE_MAXSIZE - sizeof a.len));
  *lc = new ListenComm{fd};
  return flagcxSuccess;
}
flagcxResult_t sConnect(int, void *handle, void **sc) {
  SockAddr a;
  memset(&a, 0, sizeof a);
  memcpy(&a.len, handle, sizeof a.len);
  if (a.len > FLAGCX_NET_HANDLE_MAXSIZE - sizeof a.len) return flagcxInvalidArgument;
  memcpy(&a.ss, (const char *)handle + sizeof a.len, a.len);
  int fd;
  FCX_CHECK(sockConnect(&fd, a, nowMs() + 60000, nullptr));
  *sc = new Conn{fd};
  return flagcxSuccess;
}
flagcxResult_t sAccept(void *lc, void **rc) {
  int fd;
  FCX_CHECK(sockAccept(((ListenComm *)lc)->fd, &fd, nowMs() + 60000, nullptr));
  *rc = new Conn{fd};
  return flagcxSuccess;
}
flagcxResult_t sCloseConn(void *c) { if (c) { ::close(((Conn *)c)->fd); delete (Conn *)c; } return flagcxSuccess; }
flagcxResult_t sCloseListen(void *c) { if (c) { ::close(((ListenComm *)c)->fd); delete (ListenComm *)c; } return flagcxSuccess; }
flagcxResult_t sRegMr(void *, void *, size_t, int type, void **mh) {
  if (type != FLAGCX_PTR_HOST) return flagcxNotSupported;  // TCP moves host memory only
  *mh = nullptr;
  return flagcxSuccess;
}
flagcxResult_t sRegMrDmaBuf(void *, void *, size_t, int, uint64_t, int, void **) { return flagcxNotSupported; }
flagcxResult_t sDeregMr(void *, void *) { return flagcxSuccess; }
flagcxResult_t sIsend(void *sc, void *data, size_t size, int tag, void *, void **request) {
  Req *r = new Req;
  r->fd = ((Conn *)sc)->fd;
  r->isSend = true;
  r->hdr = {size, tag, 0};
  r->data = (char *)data;
  r->cap = size;
  *request = r;
  return flagcxSuccess;
}
flagcxResult_t sIrecv(void *rc, int n, void **data, size_t *sizes, int *tags, void **, void **request) {
  if (n != 1) return flagcxInvalidArgument;
  Req *r = new Req;
  r->fd = ((Conn *)rc)->fd;
  r->isSend = false;
  r->hdr = {0, tags ? tags[0] : 0, 0};
  r->data = (char *)data[0];
  r->cap = sizes[0];
  *request = r;
  return flagcxSuccess;
}
flagcxResult_t sIflush(void *, int, void **, int *, void **, void **request) { *request = nullptr; return flagcxSuccess; }

// Move as many bytes as the socket takes right now.
bool pump(Req *r, char *buf, size_t want, size_t *done) {
  while (*done < want) {
    ssize_t k = r->isSend ? ::send(r->fd, buf + *done, want - *done, MSG_NOSIGNAL) : ::recv(r->fd, buf + *done, want - *done, 0);
    if (k > 0) { *done += k; continue; }
    if (k == 0 && !r->isSend) { r->failed = true; return false; }
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return false;
    r->failed = true;
    return false;
  }
  return true;
}

flagcxResult_t sTest(void *request, int *done, int *sizes) {
  *done = 0;
  if (!request) { *done = 1; return flagcxSuccess; }
  Req *r = (Req *)request;
  if (pump(r, (char *)&r->hdr, sizeof(Hdr), &r->hdrDone)) {
    if (!r->isSend && r->hdr.size > r->cap) { delete r; return flagcxInvalidArgument; }
    if (pump(r, r->data, r->hdr.size, &r->dataDone)) {
      *done = 1;
      if (sizes) sizes[0] = (int)r->hdr.size;
      delete r;
      return flagcxSuccess;
    }
  }
  if (r->failed) { delete r; return flagcxRemoteError; }
  return flagcxSuccess;
}
flagcxResult_t sGetDevFromName(const char *, int *dev) { *dev = 0; return flagcxSuccess; }

}  // namespace

extern "C" {
struct flagcxNetAdaptor flagcxNetSocket = {"socket", sInit, sDevices, sProps, sListen, sConnect, sAccept, sCloseConn, sCloseConn,
                                           sCloseListen, sRegMr, sRegMrDmaBuf, sDeregMr, sIsend, sIrecv, sIflush, sTest,
                                           nullptr, nullptr, nullptr, sGetDevFromName};
const struct flagcxNetAdaptor *flagcxGetNetAdaptor(void) { return &flagcxNetSocket; }
}
