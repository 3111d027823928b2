#include "hostcoll.h"
#include "hosttypes.h"
#include "log.h"

#include <algorithm>
#include <cstring>
#include <vector>

namespace fcx {

namespace {

enum : int { TAG_RS = 0x100000, TAG_AG = 0x110000, TAG_BC = 0x120000, TAG_RD = 0x130000,
             TAG_GA = 0x140000, TAG_SC = 0x150000, TAG_A2A = 0x160000, TAG_P2P = 0x170000 };

// Element range of chunk c when `count` elements are cut into n near-equal parts.
inline void chunkRange(size_t count, int n, int c, size_t *off, size_t *len) {
  size_t base = count / n, rem = count % n;
  *off = c * base + std::min<size_t>(c, rem);
  *len = base + ((size_t)c < rem ? 1 : 0);
}

// In-place ring reduce-scatter over `work`, which holds n chunks described by
// off[]/len[] (elements).  After n-1 steps rank r holds the finished chunk
// (r + ownerShift) mod n.
flagcxResult_t ringReduceScatter(Bootstrap &bs, char *work, const std::vector<size_t> &off, const std::vector<size_t> &len,
                                 flagcxDataType_t t, flagcxRedOp_t op, int ownerShift) {
  int n = bs.nranks(), r = bs.rank();
  size_t es = dtypeSize(t);
  size_t maxLen = *std::max_element(len.begin(), len.end());
  std::vector<char> tmp(maxLen * es);
  int next = (r + 1) % n, prev = (r + n - 1) % n;
  for (int s = 0; s < n - 1; s++) {
    int sc = ((r + ownerShift - 1 - s) % n + n) % n;
    int rc = ((r + ownerShift - 2 - s) % n + n) % n;
    FCX_CHECK(bs.sendrecv(next, TAG_RS + s, work + off[sc] * es, len[sc] * es, prev, TAG_RS + s, tmp.data(), len[rc] * es));
    hostReduceInto(work + off[rc] * es, tmp.data(), len[rc], t, op);
  }
  return flagcxSuccess;
}

// Ring all-gather of chunks; rank r starts owning chunk (r + ownerShift) mod n.
flagcxResult_t ringAllGather(Bootstrap &bs, char *work, const std::vector<size_t> &off, const std::vector<size_t> &len,
                             size_t es, int ownerShift) {
  int n = bs.nranks(), r = bs.rank();
  int next = (r + 1) % n, prev = (r + n - 1) % n;
  for (int s = 0; s < n - 1; s++) {
    int sc = ((r + ownerShift - s) % n + n) % n;
    int rc = ((r + ownerShift - 1 - s) % n + n) % n;
    FCX_CHECK(bs.sendrecv(next, TAG_AG + s, work + off[sc] * es, len[sc] * es, prev, TAG_AG + s, work + off[rc] * es, len[rc] * es));
  }
  return flagcxSuccess;
}

bool reducible(flagcxRedOp_t op) { return op >= flagcxSum && op <= flagcxAvg; }

}  // namespace

flagcxResult_t hostAllReduce(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, flagcxRedOp_t op) {
  size_t es = dtypeSize(t);
  if (!es || !reducible(op)) return flagcxInvalidArgument;
  int n = bs.nranks();
  if (send != recv) memmove(recv, send, count * es);
  if (n > 1) {
    std::vector<size_t> off(n), len(n);
    for (int c = 0; c < n; c++) chunkRange(count, n, c, &off[c], &len[c]);
    FCX_CHECK(ringReduceScatter(bs, (char *)recv, off, len, t, op, 0));
    FCX_CHECK(ringAllGather(bs, (char *)recv, off, len, es, 0));
  }
  if (op == flagcxAvg) hostDivide(recv, count, t, n);
  return flagcxSuccess;
}

flagcxResult_t hostReduceScatter(Bootstrap &bs, const void *send, void *recv, size_t recvcount, flagcxDataType_t t, flagcxRedOp_t op) {
  size_t es = dtypeSize(t);
  if (!es || !reducible(op)) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  std::vector<char> work((const char *)send, (const char *)send + (size_t)n * recvcount * es);
  if (n > 1) {
    std::vector<size_t> off(n), len(n, recvcount);
    for (int c = 0; c < n; c++) off[c] = c * recvcount;
    FCX_CHECK(ringReduceScatter(bs, work.data(), off, len, t, op, 0));
  }
  memcpy(recv, work.data() + (size_t)r * recvcount * es, recvcount * es);
  if (op == flagcxAvg) hostDivide(recv, recvcount, t, n);
  return flagcxSuccess;
}

flagcxResult_t hostAllGather(Bootstrap &bs, const void *send, void *recv, size_t sendcount, flagcxDataType_t t) {
  size_t es = dtypeSize(t);
  if (!es) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  char *mine = (char *)recv + (size_t)r * sendcount * es;
  if (send != mine) memmove(mine, send, sendcount * es);
  if (n == 1) return flagcxSuccess;
  std::vector<size_t> off(n), len(n, sendcount);
  for (int c = 0; c < n; c++) off[c] = c * sendcount;
  return ringAllGather(bs, (char *)recv, off, len, es, 0);
}

flagcxResult_t hostBroadcast(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root) {
  size_t es = dtypeSize(t);
  if (!es || root < 0 || root >= bs.nranks()) return flagcxInvalidArgument;
  if (bs.rank() == root && send != recv) memmove(recv, send, count * es);
  return bs.broadcast(recv, count * es, root);
}

flagcxResult_t hostReduce(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, flagcxRedOp_t op, int root) {
  size_t es = dtypeSize(t);
  if (!es || !reducible(op) || root < 0 || root >= bs.nranks()) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  // Reduce-scatter, then each rank ships its finished chunk to the root.
  std::vector<char> work((const char *)send, (const char *)send + count * es);
  std::vector<size_t> off(n), len(n);
  for (int c = 0; c < n; c++) chunkRange(count, n, c, &off[c], &len[c]);
  if (n > 1) FCX_CHECK(ringReduceScatter(bs, work.data(), off, len, t, op, 0));
  if (r == root) {
    memcpy((char *)recv + off[r] * es, work.data() + off[r] * es, len[r] * es);
    for (int p = 0; p < n; p++)
      if (p != root) FCX_CHECK(bs.recv(p, TAG_RD, (char *)recv + off[p] * es, len[p] * es));
    if (op == flagcxAvg) hostDivide(recv, count, t, n);
  } else {
    FCX_CHECK(bs.send(root, TAG_RD, work.data() + off[r] * es, len[r] * es));
  }
  return flagcxSuccess;
}

flagcxResult_t hostGather(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root) {
  size_t es = dtypeSize(t);
  if (!es || root < 0 || root >= bs.nranks()) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  if (r == root) {
    char *mine = (char *)recv + (size_t)r * count * es;
    if (send != mine) memmove(mine, send, count * es);
    for (int p = 0; p < n; p++)
      if (p != root) FCX_CHECK(bs.recv(p, TAG_GA, (char *)recv + (size_t)p * count * es, count * es));
  } else {
    FCX_CHECK(bs.send(root, TAG_GA, send, count * es));
  }
  return flagcxSuccess;
}

flagcxResult_t hostScatter(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root) {
  size_t es = dtypeSize(t);
  if (!es || root < 0 || root >= bs.nranks()) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  if (r == root) {
    for (int p = 0; p < n; p++)
      if (p != root) FCX_CHECK(bs.send(p, TAG_SC, (const char *)send + (size_t)p * count * es, count * es));
    const char *mine = (const char *)send + (size_t)r * count * es;
    if (recv != mine) memmove(recv, mine, count * es);
  } else {
    FCX_CHECK(bs.recv(root, TAG_SC, recv, count * es));
  }
  return flagcxSuccess;
}

flagcxResult_t hostAlltoAllv(Bootstrap &bs, const void *send, const size_t *scounts, const size_t *sdispls, void *recv,
                             const size_t *rcounts, const size_t *rdispls, flagcxDataType_t t) {
  size_t es = dtypeSize(t);
  if (!es) return flagcxInvalidArgument;
  int n = bs.nranks(), r = bs.rank();
  // Step d pairs every rank with (r+d) as destination and (r-d) as source,
  // so each step is a permutation and the full-duplex exchange cannot block.
  for (int d = 0; d < n; d++) {
    int to = (r + d) % n, from = (r - d + n) % n;
    const char *sp = (const char *)send + sdispls[to] * es;
    char *rp = (char *)recv + rdispls[from] * es;
    if (d == 0) {
      if (scounts[r] != rcounts[r]) return flagcxInvalidArgument;
      if (sp != rp) memmove(rp, sp, scounts[r] * es);
      continue;
    }
    FCX_CHECK(bs.sendrecv(to, TAG_A2A + d, sp, scounts[to] * es, from, TAG_A2A + d, rp, rcounts[from] * es));
  }
  return flagcxSuccess;
}

flagcxResult_t hostAlltoAll(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t) {
  int n = bs.nranks();
  std::vector<size_t> cnt(n, count), dsp(n);
  for (int i = 0; i < n; i++) dsp[i] = i * count;
  if (send == recv) {
    // In place: stage a copy of the outgoing blocks first.
    size_t es = dtypeSize(t);
    std::vector<char> tmp((const char *)send, (const char *)send + (size_t)n * count * es);
    return hostAlltoAllv(bs, tmp.data(), cnt.data(), dsp.data(), recv, cnt.data(), dsp.data(), t);
  }
  return hostAlltoAllv(bs, send, cnt.data(), dsp.data(), recv, cnt.data(), dsp.data(), t);
}

flagcxResult_t hostSend(Bootstrap &bs, const void *send, size_t count, flagcxDataType_t t, int peer) {
  size_t es = dtypeSize(t);
  if (!es || peer < 0 || peer >= bs.nranks()) return flagcxInvalidArgument;
  return bs.send(peer, TAG_P2P, send, count * es);
}

flagcxResult_t hostRecv(Bootstrap &bs, void *recv, size_t count, flagcxDataType_t t, int peer) {
  size_t es = dtypeSize(t);
  if (!es || peer < 0 || peer >= bs.nranks()) return flagcxInvalidArgument;
  return bs.recv(peer, TAG_P2P, recv, count * es);
}

}  // namespace fcx
