#include "planner.h"
#include "../core/hosttypes.h"
#include "../core/log.h"

#include <algorithm>
#include <cstring>
#include <cuda_runtime.h>
#include <functional>
#include <numeric>

namespace fcx {

// ------------------------------------------------------------------ XML

namespace {

void wr(FILE *f, int indent, const char *tag, long long v) { fprintf(f, "%*s<%s>%lld</%s>\n", indent, "", tag, v, tag); }

void writeHomo(FILE *f, const C2cHomoFunc &h, size_t cs, int ind) {
  fprintf(f, "%*s<HomoFunc>\n", ind, "");
  wr(f, ind + 2, "rootRank", h.rootRank);
  wr(f, ind + 2, "sendType", h.sendType);
  wr(f, ind + 2, "recvType", h.recvType);
  wr(f, ind + 2, "sendOffset", (long long)(h.sendOffset / cs));
  wr(f, ind + 2, "recvOffset", (long long)(h.recvOffset / cs));
  wr(f, ind + 2, "count", (long long)(h.count / cs));
  wr(f, ind + 2, "homoType", h.homoType);
  wr(f, ind + 2, "commOp", h.commOp);
  fprintf(f, "%*s</HomoFunc>\n", ind, "");
}

void writeHetero(FILE *f, const C2cHeteroFunc &h, size_t cs, int ind) {
  fprintf(f, "%*s<HeteroFunc>\n", ind, "");
  for (auto &o : h.p2pOps) {
    fprintf(f, "%*s<P2pOp>\n", ind + 2, "");
    wr(f, ind + 4, "rank", o.rank);
    wr(f, ind + 4, "peerRank", o.peerRank);
    wr(f, ind + 4, "offset", (long long)(o.offset / cs));
    wr(f, ind + 4, "count", (long long)(o.count / cs));
    wr(f, ind + 4, "isRecv", o.isRecv);
    if (o.buffType != 1) wr(f, ind + 4, "buffType", o.buffType);  // absent = receive buffer, as in the reference's files
    fprintf(f, "%*s</P2pOp>\n", ind + 2, "");
  }
  fprintf(f, "%*s</HeteroFunc>\n", ind, "");
}

template <typename T, typename W>
void writeSteps(FILE *f, const std::vector<std::vector<T>> &steps, const char *tag, W writer) {
  fprintf(f, "  <%s>\n", tag);
  for (auto &st : steps) {
    if (st.empty()) { fprintf(f, "    <Step/>\n"); continue; }
    fprintf(f, "    <Step>\n");
    for (auto &fn : st) writer(fn);
    fprintf(f, "    </Step>\n");
  }
  fprintf(f, "  </%s>\n", tag);
}

// A very small pull parser: tokens are <tag>, </tag>, <tag/> and text.
struct Tok { int kind; std::string s; };  // 0 open, 1 close, 2 empty, 3 text, 4 end
struct Lexer {
  std::string buf;
  size_t pos = 0;
  Tok next() {
    while (pos < buf.size() && isspace((unsigned char)buf[pos])) pos++;
    if (pos >= buf.size()) return {4, ""};
    if (buf[pos] == '<') {
      size_t e = buf.find('>', pos);
      if (e == std::string::npos) return {4, ""};
      std::string t = buf.substr(pos + 1, e - pos - 1);
      pos = e + 1;
      if (!t.empty() && (t[0] == '?' || t[0] == '!')) return next();  // declaration or comment
      if (!t.empty() && t[0] == '/') return {1, t.substr(1)};
      if (!t.empty() && t.back() == '/') { t.pop_back(); while (!t.empty() && isspace((unsigned char)t.back())) t.pop_back(); return {2, t}; }
      return {0, t};
    }
    size_t e = buf.find('<', pos);
    std::string t = buf.substr(pos, e == std::string::npos ? std::string::npos : e - pos);
    pos = e == std::string::npos ? buf.size() : e;
    while (!t.empty() && isspace((unsigned char)t.back())) t.pop_back();
    return {3, t};
  }
};

// Reads <tag>value</tag> pairs until </until>; calls set(tag, value) for each leaf.
bool readLeaves(Lexer &lx, const std::string &until, const std::function<bool(const std::string &, Lexer &)> &onOpen,
                const std::function<void(const std::string &, long long)> &set) {
  for (;;) {
    Tok t = lx.next();
    if (t.kind == 4) return false;
    if (t.kind == 1) { if (t.s == until) return true; continue; }
    if (t.kind == 2) { if (onOpen) { Lexer dummy; (void)dummy; } continue; }
    if (t.kind == 0) {
      if (onOpen && onOpen(t.s, lx)) continue;
      Tok v = lx.next();
      if (v.kind == 3) {
        set(t.s, strtoll(v.s.c_str(), nullptr, 10));
        lx.next();  // closing tag
      } else if (v.kind != 1) {
        return false;
      }
    }
  }
}

bool readHomo(Lexer &lx, C2cHomoFunc *h, size_t cs) {
  return readLeaves(lx, "HomoFunc", nullptr, [&](const std::string &k, long long v) {
    if (k == "rootRank") h->rootRank = (int)v;
    else if (k == "sendType") h->sendType = (int)v;
    else if (k == "recvType") h->recvType = (int)v;
    else if (k == "sendOffset") h->sendOffset = (size_t)v * cs;
    else if (k == "recvOffset") h->recvOffset = (size_t)v * cs;
    else if (k == "count") h->count = (size_t)v * cs;
    else if (k == "homoType") h->homoType = (int)v;
    else if (k == "commOp") h->commOp = (int)v;
  });
}

bool readHetero(Lexer &lx, C2cHeteroFunc *h, size_t cs) {
  for (;;) {
    Tok t = lx.next();
    if (t.kind == 4) return false;
    if (t.kind == 1 && t.s == "HeteroFunc") return true;
    if (t.kind == 0 && t.s == "P2pOp") {
      C2cP2pOp o;
      if (!readLeaves(lx, "P2pOp", nullptr, [&](const std::string &k, long long v) {
            if (k == "rank") o.rank = (int)v;
            else if (k == "peerRank") o.peerRank = (int)v;
            else if (k == "offset") o.offset = (size_t)v * cs;
            else if (k == "count") o.count = (size_t)v * cs;
            else if (k == "isRecv") o.isRecv = (int)v;
            else if (k == "buffType") o.buffType = (int)v;
          }))
        return false;
      h->p2pOps.push_back(o);
    }
  }
}

template <typename T, typename R>
bool readSteps(Lexer &lx, const std::string &tag, const char *fnTag, std::vector<std::vector<T>> *out, R reader) {
  for (;;) {
    Tok t = lx.next();
    if (t.kind == 4) return false;
    if (t.kind == 1 && t.s == tag) return true;
    if (t.kind == 2 && t.s == "Step") { out->emplace_back(); continue; }
    if (t.kind == 0 && t.s == "Step") {
      out->emplace_back();
      for (;;) {
        Tok u = lx.next();
        if (u.kind == 4) return false;
        if (u.kind == 1 && u.s == "Step") break;
        if (u.kind == 0 && u.s == fnTag) {
          T fn;
          if (!reader(lx, &fn)) return false;
          out->back().push_back(fn);
        }
      }
    }
  }
}

}  // namespace

size_t c2cAlgoHash(size_t sendCount, size_t recvCount, size_t rootCluster, int commOp, int redOp) {
  // same combination as the reference (flagcx/core/c2c_ir.h:19-28) so that plan files are interchangeable
  size_t h1 = std::hash<size_t>()(sendCount), h2 = std::hash<size_t>()(recvCount), h3 = std::hash<size_t>()(rootCluster);
  size_t h4 = std::hash<size_t>()((size_t)commOp), h5 = std::hash<size_t>()((size_t)redOp);
  return h1 ^ (h2 << 1) ^ (h3 << 2) ^ (h4 << 3) ^ (h5 << 4);
}

flagcxResult_t c2cExportXml(const C2cPlan &p, const std::string &prefix, int rank) {
  std::string fn = prefix + "_" + std::to_string(rank) + ".xml";
  FILE *f = fopen(fn.c_str(), "w");
  if (!f) { FCX_WARN("cannot write plan file %s", fn.c_str()); return flagcxSystemError; }
  // chunk size: the largest unit that divides every offset and count of the plan
  size_t g = p.totalCount;
  auto fold = [&](size_t v) { if (v) g = std::gcd(g, v); };
  for (auto *steps : {&p.preHomoFuncSteps, &p.homoInterFuncSteps, &p.postHomoFuncSteps})
    for (auto &st : *steps)
      for (auto &h : st) { fold(h.sendOffset); fold(h.recvOffset); fold(h.count); }
  for (auto &st : p.heteroFuncSteps)
    for (auto &h : st)
      for (auto &o : h.p2pOps) { fold(o.offset); fold(o.count); }
  fold(p.refresh.start); fold(p.refresh.offset); fold(p.refresh.count); fold(p.refresh.totalCount);
  if (!g) g = 1;
  size_t nChunks = p.totalCount ? p.totalCount / g : 1;
  fprintf(f, "<FlagcxC2cPlanner>\n");
  wr(f, 2, "nChunks", (long long)nChunks);
  wr(f, 2, "nSeqPreSteps", p.nSeqPreSteps);
  wr(f, 2, "nPipePreSteps", p.nPipePreSteps);
  wr(f, 2, "nSeqInterSteps", p.nSeqInterSteps);
  wr(f, 2, "nPipePostSteps", p.nPipePostSteps);
  wr(f, 2, "nSeqPostSteps", p.nSeqPostSteps);
  fprintf(f, "  <RefreshFunc>\n");
  wr(f, 4, "buffType", p.refresh.buffType);
  wr(f, 4, "start", (long long)(p.refresh.start / g));
  wr(f, 4, "offset", (long long)(p.refresh.offset / g));
  wr(f, 4, "count", (long long)(p.refresh.count / g));
  wr(f, 4, "totalCount", (long long)(p.refresh.totalCount / g));
  wr(f, 4, "redOp", p.refresh.redOp);
  fprintf(f, "  </RefreshFunc>\n");
  writeSteps(f, p.preHomoFuncSteps, "PreHomoFuncSteps", [&](const C2cHomoFunc &h) { writeHomo(f, h, g, 6); });
  writeSteps(f, p.heteroFuncSteps, "HeteroFuncSteps", [&](const C2cHeteroFunc &h) { writeHetero(f, h, g, 6); });
  writeSteps(f, p.homoInterFuncSteps, "HomoInterFuncSteps", [&](const C2cHomoFunc &h) { writeHomo(f, h, g, 6); });
  writeSteps(f, p.postHomoFuncSteps, "PostHomoFuncSteps", [&](const C2cHomoFunc &h) { writeHomo(f, h, g, 6); });
  fprintf(f, "</FlagcxC2cPlanner>\n");
  fclose(f);
  return flagcxSuccess;
}

flagcxResult_t c2cImportXml(C2cPlan *p, const std::string &prefix, int rank, size_t totalCount) {
  std::string fn = prefix + "_" + std::to_string(rank) + ".xml";
  FILE *f = fopen(fn.c_str(), "r");
  if (!f) { FCX_WARN("cannot read plan file %s", fn.c_str()); return flagcxSystemError; }
  Lexer lx;
  char tmp[4096];
  size_t n;
  while ((n = fread(tmp, 1, sizeof tmp, f)) > 0) lx.buf.append(tmp, n);
  fclose(f);
  *p = C2cPlan();
  p->totalCount = totalCount;
  Tok t = lx.next();
  if (t.kind != 0 || t.s != "FlagcxC2cPlanner") { FCX_WARN("%s: not a plan file", fn.c_str()); return flagcxInvalidArgument; }
  size_t cs = 1;
  bool ok = true;
  for (;;) {
    t = lx.next();
    if (t.kind == 4) { ok = false; break; }
    if (t.kind == 1 && t.s == "FlagcxC2cPlanner") break;
    if (t.kind != 0) continue;
    if (t.s == "RefreshFunc") {
      ok = readLeaves(lx, "RefreshFunc", nullptr, [&](const std::string &k, long long v) {
        if (k == "buffType") p->refresh.buffType = (int)v;
        else if (k == "start") p->refresh.start = (size_t)v * cs;
        else if (k == "offset") p->refresh.offset = (size_t)v * cs;
        else if (k == "count") p->refresh.count = (size_t)v * cs;
        else if (k == "totalCount") p->refresh.totalCount = (size_t)v * cs;
        else if (k == "redOp") p->refresh.redOp = (int)v;
      });
    } else if (t.s == "PreHomoFuncSteps") {
      ok = readSteps<C2cHomoFunc>(lx, t.s, "HomoFunc", &p->preHomoFuncSteps, [&](Lexer &l, C2cHomoFunc *h) { return readHomo(l, h, cs); });
    } else if (t.s == "HomoInterFuncSteps") {
      ok = readSteps<C2cHomoFunc>(lx, t.s, "HomoFunc", &p->homoInterFuncSteps, [&](Lexer &l, C2cHomoFunc *h) { return readHomo(l, h, cs); });
    } else if (t.s == "PostHomoFuncSteps") {
      ok = readSteps<C2cHomoFunc>(lx, t.s, "HomoFunc", &p->postHomoFuncSteps, [&](Lexer &l, C2cHomoFunc *h) { return readHomo(l, h, cs); });
    } else if (t.s == "HeteroFuncSteps") {
      ok = readSteps<C2cHeteroFunc>(lx, t.s, "HeteroFunc", &p->heteroFuncSteps, [&](Lexer &l, C2cHeteroFunc *h) { return readHetero(l, h, cs); });
    } else {
      Tok v = lx.next();
      long long val = v.kind == 3 ? strtoll(v.s.c_str(), nullptr, 10) : 0;
      if (v.kind == 3) lx.next();
      if (t.s == "nChunks") {
        p->nChunks = (size_t)std::max<long long>(1, val);
        if (totalCount % p->nChunks != 0) { FCX_WARN("%s: %zu elements are not divisible into %zu chunks", fn.c_str(), totalCount, p->nChunks); return flagcxInvalidArgument; }
        cs = totalCount / p->nChunks;
      } else if (t.s == "nSeqPreSteps") p->nSeqPreSteps = (int)val;
      else if (t.s == "nPipePreSteps") p->nPipePreSteps = (int)val;
      else if (t.s == "nSeqInterSteps") p->nSeqInterSteps = (int)val;
      else if (t.s == "nPipePostSteps") p->nPipePostSteps = (int)val;
      else if (t.s == "nSeqPostSteps") p->nSeqPostSteps = (int)val;
    }
    if (!ok) break;
  }
  if (!ok) { FCX_WARN("%s: malformed plan file", fn.c_str()); return flagcxInvalidArgument; }
  // scratch: the furthest element any function touches in buffer type 2
  size_t sc = 0;
  for (auto *steps : {&p->preHomoFuncSteps, &p->homoInterFuncSteps, &p->postHomoFuncSteps})
    for (auto &st : *steps)
      for (auto &h : st) {
        size_t mult = (h.commOp == flagcxCommOpAllGather || h.commOp == flagcxCommOpGather) ? 64 : 1;  // generous for gathers
        if (h.sendType == 2) sc = std::max(sc, h.sendOffset + h.count * ((h.commOp == flagcxCommOpReduceScatter || h.commOp == flagcxCommOpScatter) ? 64 : 1));
        if (h.recvType == 2) sc = std::max(sc, h.recvOffset + h.count * mult);
      }
  if (p->refresh.buffType == 2) sc = std::max(sc, p->refresh.start + p->refresh.totalCount);
  p->scratchCount = sc;
  p->pipelined = p->nPipePreSteps > 1;
  return flagcxSuccess;
}

// ------------------------------------------------------------------ default plans

// Stage tables of the hierarchical collectives (the reference's op -> stage table is
// flagcx/core/c2c_algo.cc:749-971, its chunk scheduling and cross-cluster send/recv search :1089-1394).
// World rank = cluster * L + local index.  "intra" = the ranks of one cluster, "inter" = the ranks that hold
// the same local index in every cluster.
bool c2cBuildPlan(C2cPlan *p, flagcxCommOp_t op, size_t count, int root, int C, int L, int myCluster, int myLocal, bool pipelined,
                  int interRanks, bool heteroP2p, const size_t *tables) {
  *p = C2cPlan();
  auto homo = [](int commOp, int sendType, size_t so, int recvType, size_t ro, size_t cnt, int homoType, int rootRank = -1) {
    C2cHomoFunc h;
    h.commOp = commOp; h.sendType = sendType; h.sendOffset = so; h.recvType = recvType; h.recvOffset = ro; h.count = cnt;
    h.homoType = homoType; h.rootRank = rootRank;
    return h;
  };
  auto p2p = [&](int peer, int buffType, size_t off, size_t cnt, int isRecv) {
    C2cP2pOp o;
    o.rank = myCluster * L + myLocal; o.peerRank = peer; o.buffType = buffType; o.offset = off; o.count = cnt; o.isRecv = isRecv;
    return o;
  };
  const int rootCluster = root / L, rootLocal = root % L;
  const int K = (interRanks >= 1 && interRanks <= L && L % interRanks == 0) ? interRanks : L;  // inter ranks per cluster
  const bool iAmInter = myLocal < K;
  const size_t n = (size_t)C * L;
  switch (op) {
    case flagcxCommOpAllReduce: {
      if (count == 0) return false;
      if (K < L) {
        // Few network ports per cluster: piece j of the vector is reduced onto inter rank j of every cluster,
        // all-reduced among the inter ranks j, and broadcast inside each cluster (the reference's
        // "all-gather by broadcasts" post stage).
        if (count % K != 0) return false;
        const size_t pc = count / K;
        p->totalCount = count;
        std::vector<C2cHomoFunc> pre, post;
        for (int j = 0; j < K; j++) {
          pre.push_back(homo(flagcxCommOpReduce, 0, j * pc, 1, j * pc, pc, 0, j));
          post.push_back(homo(flagcxCommOpBroadcast, 1, j * pc, 1, j * pc, pc, 2, j));
        }
        p->preHomoFuncSteps.push_back(pre);
        if (iAmInter) p->homoInterFuncSteps.push_back({homo(flagcxCommOpAllReduce, 1, myLocal * pc, 1, myLocal * pc, pc, 1)});
        else p->homoInterFuncSteps.push_back({});
        p->postHomoFuncSteps.push_back(post);
        p->nSeqPreSteps = p->nSeqInterSteps = p->nSeqPostSteps = 1;
        return true;
      }
      if (count % L != 0) return false;
      int pieces = 1;
      if (pipelined)
        for (int cand : {4, 2})
          if (count % ((size_t)L * cand) == 0 && count / cand >= (size_t)L * 4096) { pieces = cand; break; }
      size_t per = count / pieces, chunk = per / L;
      p->totalCount = count;
      for (int i = 0; i < pieces; i++) {
        p->preHomoFuncSteps.push_back({homo(flagcxCommOpReduceScatter, 0, i * per, 2, i * chunk, chunk, 0)});
        p->homoInterFuncSteps.push_back({homo(flagcxCommOpAllReduce, 2, i * chunk, 2, i * chunk, chunk, 1)});
        p->postHomoFuncSteps.push_back({homo(flagcxCommOpAllGather, 2, i * chunk, 1, i * per, chunk, 2)});
      }
      p->scratchCount = (size_t)pieces * chunk;
      p->pipelined = pieces > 1;
      p->nSeqPreSteps = pieces > 1 ? 0 : 1;
      p->nPipePreSteps = pieces > 1 ? pieces : 0;
      p->nSeqInterSteps = pieces > 1 ? 0 : 1;
      p->nPipePostSteps = pieces > 1 ? pieces : 0;
      p->nSeqPostSteps = pieces > 1 ? 0 : 1;
      return true;
    }
    case flagcxCommOpReduceScatter: {
      if (count == 0) return false;
      p->totalCount = count * n;
      std::vector<C2cHomoFunc> pre;
      for (int c = 0; c < C; c++) pre.push_back(homo(flagcxCommOpReduceScatter, 0, (size_t)c * L * count, 2, (size_t)c * count, count, 0));
      p->preHomoFuncSteps.push_back(pre);
      p->homoInterFuncSteps.push_back({homo(flagcxCommOpReduceScatter, 2, 0, 1, 0, count, 1)});
      p->scratchCount = (size_t)C * count;
      p->nSeqPreSteps = p->nSeqInterSteps = 1;
      return true;
    }
    case flagcxCommOpAllGather: {
      if (count == 0) return false;
      p->totalCount = count * n;
      if (K < L || heteroP2p) {
        // The cluster's pieces are gathered onto inter rank 0 at their place in the receive buffer; the inter
        // ranks 0 of all clusters swap their cluster blocks with point-to-point transfers (the planner-built
        // cross-cluster stage); each broadcasts the complete buffer inside its cluster.
        const size_t block = (size_t)L * count;
        p->preHomoFuncSteps.push_back({homo(flagcxCommOpGather, 0, 0, 1, (size_t)myCluster * block, count, 0, 0)});
        C2cHeteroFunc het;
        if (myLocal == 0)
          for (int k = 1; k < C; k++) {
            const int to = (myCluster + k) % C, from = (myCluster - k + C) % C;
            het.p2pOps.push_back(p2p(to * L, 1, (size_t)myCluster * block, block, 0));
            het.p2pOps.push_back(p2p(from * L, 1, (size_t)from * block, block, 1));
          }
        p->heteroFuncSteps.push_back({het});
        p->postHomoFuncSteps.push_back({homo(flagcxCommOpBroadcast, 1, 0, 1, 0, n * count, 2, 0)});
        p->nSeqPreSteps = p->nSeqPostSteps = 1;
        return true;
      }
      p->homoInterFuncSteps.push_back({homo(flagcxCommOpAllGather, 0, 0, 2, 0, count, 1)});
      std::vector<C2cHomoFunc> post;
      for (int c = 0; c < C; c++) post.push_back(homo(flagcxCommOpAllGather, 2, (size_t)c * count, 1, (size_t)c * L * count, count, 2));
      p->postHomoFuncSteps.push_back(post);
      p->scratchCount = (size_t)C * count;
      p->nSeqInterSteps = p->nSeqPostSteps = 1;
      return true;
    }
    case flagcxCommOpBroadcast: {
      if (count == 0) return false;
      p->totalCount = count;
      bool isRoot = myCluster == rootCluster && myLocal == rootLocal;
      if (heteroP2p) {
        // the root sends to its counterpart in every other cluster, which then broadcasts inside its cluster
        C2cHeteroFunc het;
        if (isRoot)
          for (int c = 0; c < C; c++)
            if (c != myCluster) het.p2pOps.push_back(p2p(c * L + rootLocal, 0, 0, count, 0));
        if (!isRoot && myLocal == rootLocal) het.p2pOps.push_back(p2p(root, 1, 0, count, 1));
        p->heteroFuncSteps.push_back({het});
        p->postHomoFuncSteps.push_back({homo(flagcxCommOpBroadcast, (isRoot ? 0 : 1), 0, 1, 0, count, 2, rootLocal)});
        p->nSeqPostSteps = 1;
        return true;
      }
      if (myLocal == rootLocal)
        p->homoInterFuncSteps.push_back({homo(flagcxCommOpBroadcast, isRoot ? 0 : 1, 0, 1, 0, count, 1, rootCluster)});
      else
        p->homoInterFuncSteps.push_back({});
      p->postHomoFuncSteps.push_back({homo(flagcxCommOpBroadcast, 1, 0, 1, 0, count, 2, rootLocal)});
      p->nSeqInterSteps = p->nSeqPostSteps = 1;
      return true;
    }
    case flagcxCommOpReduce: {
      if (count == 0) return false;
      p->totalCount = count;
      bool isRoot = myCluster == rootCluster && myLocal == rootLocal;
      p->preHomoFuncSteps.push_back({homo(flagcxCommOpReduce, 0, 0, 2, 0, count, 0, rootLocal)});
      if (myLocal == rootLocal)
        p->homoInterFuncSteps.push_back({homo(flagcxCommOpReduce, 2, 0, isRoot ? 1 : 2, isRoot ? 0 : count, count, 1, rootCluster)});
      else
        p->homoInterFuncSteps.push_back({});
      p->scratchCount = 2 * count;
      p->nSeqPreSteps = p->nSeqInterSteps = 1;
      return true;
    }
    case flagcxCommOpGather: {
      // every cluster gathers onto the root's counterpart (scratch: L pieces), the counterparts gather their
      // cluster blocks onto the root, where block c lands at c * L * count: rank order
      if (count == 0) return false;
      p->totalCount = count * n;
      const size_t block = (size_t)L * count;
      p->preHomoFuncSteps.push_back({homo(flagcxCommOpGather, 0, 0, 2, 0, count, 0, rootLocal)});
      if (myLocal == rootLocal) p->homoInterFuncSteps.push_back({homo(flagcxCommOpGather, 2, 0, 1, 0, block, 1, rootCluster)});
      else p->homoInterFuncSteps.push_back({});
      p->scratchCount = block;
      p->nSeqPreSteps = p->nSeqInterSteps = 1;
      return true;
    }
    case flagcxCommOpScatter: {
      // the mirror image: the root scatters cluster blocks to its counterparts, each scatters inside its cluster
      if (count == 0) return false;
      p->totalCount = count * n;
      const size_t block = (size_t)L * count;
      if (myLocal == rootLocal) p->homoInterFuncSteps.push_back({homo(flagcxCommOpScatter, 0, 0, 2, 0, block, 1, rootCluster)});
      else p->homoInterFuncSteps.push_back({});
      p->postHomoFuncSteps.push_back({homo(flagcxCommOpScatter, 2, 0, 1, 0, count, 2, rootLocal)});
      p->scratchCount = block;
      p->nSeqInterSteps = p->nSeqPostSteps = 1;
      return true;
    }
    case flagcxCommOpAlltoAll: {
      // Stage 1, inside the cluster, once per destination cluster c': rank (c,l) hands rank (c,l') the block it
      // addresses to (c',l'); scratch of (c,l') then holds [c'][l].  Stage 2, among the ranks of equal local
      // index: (c,l') sends (c',l') the L blocks scratch[c'][*]; what arrives from cluster c'' are the blocks of
      // the sources (c'',0..L-1), which is exactly the order of the all-to-all's receive buffer.
      if (count == 0) return false;
      p->totalCount = count * n;
      const size_t block = (size_t)L * count;
      std::vector<C2cHomoFunc> pre;
      for (int c = 0; c < C; c++) pre.push_back(homo(flagcxCommOpAlltoAll, 0, (size_t)c * block, 2, (size_t)c * block, count, 0));
      p->preHomoFuncSteps.push_back(pre);
      p->homoInterFuncSteps.push_back({homo(flagcxCommOpAlltoAll, 2, 0, 1, 0, block, 1)});
      p->scratchCount = n * count;
      p->nSeqPreSteps = p->nSeqInterSteps = 1;
      return true;
    }
    case flagcxCommOpAlltoAllv: {
      // Variable blocks: a list of point-to-point transfers on the world communicator, the local block as a
      // transfer to self (the reference's cross-cluster path is the same all-pairs send/recv,
      // flagcx/flagcx.cc:1376-1387).  Built per call: it depends on the counts.
      if (!tables) return false;
      const size_t *sc = tables, *sd = tables + n, *rc = tables + 2 * n, *rd = tables + 3 * n;
      C2cHeteroFunc het;
      const int me = myCluster * L + myLocal;
      for (size_t k = 0; k < n; k++) {
        const int to = (int)((me + k) % n), from = (int)((me + n - k) % n);
        if (sc[to]) het.p2pOps.push_back(p2p(to, 0, sd[to], sc[to], 0));
        if (rc[from]) het.p2pOps.push_back(p2p(from, 1, rd[from], rc[from], 1));
      }
      p->totalCount = 1;
      p->heteroFuncSteps.push_back({het});
      return true;
    }
    default:
      return false;  // send/recv and the barrier run on the world communicator as they are
  }
}

// ------------------------------------------------------------------ execution

namespace {

flagcxResult_t ensureState(flagcxComm *c) {
  if (!c->c2c) c->c2c = new C2cState();
  C2cState *s = c->c2c;
  if (s->ready || s->unusable) return flagcxSuccess;
  // clusters must be contiguous and of equal size for the hierarchical plans
  std::vector<int> sizes(c->nclusters, 0);
  for (int r = 0; r < c->nranks; r++) sizes[c->clusterOf[r]]++;
  bool equal = true;
  for (int v : sizes) equal = equal && v == sizes[0];
  for (int r = 1; r < c->nranks; r++) equal = equal && c->clusterOf[r] >= c->clusterOf[r - 1];
  if (!equal) {
    FCX_INFO(SUB_INIT, "C2C: clusters differ in size or are interleaved; collectives stay flat");
    s->unusable = true;
    return flagcxSuccess;
  }
  s->clusterSize = sizes[0];
  int first = 0;
  while (c->clusterOf[first] != c->myCluster) first++;
  s->myLocal = c->rank - first;
  FCX_CHECK(flagcxCommSplit(c, c->myCluster, c->rank, &s->intra));
  FCX_CHECK(flagcxCommSplit(c, s->myLocal, c->rank, &s->inter));
  if (!c->hostOnly && !c->hostFallback) {
    FCX_CHECK(cudaToResult(cudaStreamCreateWithFlags(&s->sideStream, cudaStreamNonBlocking), "C2C stream"));
    FCX_CHECK(cudaToResult(cudaEventCreateWithFlags(&s->evA, cudaEventDisableTiming), "C2C event"));
    FCX_CHECK(cudaToResult(cudaEventCreateWithFlags(&s->evB, cudaEventDisableTiming), "C2C event"));
  }
  // How many ranks of a cluster talk across clusters (the reference's single-NIC / multi-NIC / NIC-per-rank
  // modes, flagcx/core/c2c_algo.cc:637-672): FLAGCX_C2C_INTER_RANKS, else the number of distinct network ports
  // that FLAGCX_TOPO_FILE gives the GPUs of this cluster, else every rank.
  int k = (int)envInt("C2C_INTER_RANKS", 0);
  if (k <= 0 && !c->netOfRank.empty()) {
    std::vector<std::string> nets;
    for (int r = first; r < first + s->clusterSize; r++)
      if (!c->netOfRank[r].empty() && std::find(nets.begin(), nets.end(), c->netOfRank[r]) == nets.end()) nets.push_back(c->netOfRank[r]);
    k = (int)nets.size();
  }
  if (k <= 0 || k > s->clusterSize || s->clusterSize % k != 0) k = s->clusterSize;
  // every rank must use the same mode: agree on the smallest
  std::vector<int> ks(c->nranks, k);
  FCX_CHECK(c->bs.allGather(ks.data(), sizeof(int)));
  for (int v : ks) k = std::min(k, v);
  s->interRanks = k;
  s->heteroP2p = envInt("C2C_HETERO_P2P", 0) != 0;
  s->ready = true;
  FCX_INFO(SUB_INIT, "C2C: rank %d is local %d of cluster %d (%d clusters x %d ranks, %d inter ranks per cluster%s)", c->rank, s->myLocal,
           c->myCluster, c->nclusters, s->clusterSize, s->interRanks, s->heteroP2p ? ", point-to-point cross-cluster stage" : "");
  return flagcxSuccess;
}

flagcxResult_t ensureScratch(flagcxComm *c, size_t bytes) {
  C2cState *s = c->c2c;
  if (bytes <= s->scratchBytes) return flagcxSuccess;
  bytes = (bytes + (1 << 20) - 1) & ~(size_t)((1 << 20) - 1);
  if (c->hostOnly) {
    free(s->scratch);
    s->scratch = malloc(bytes);
    if (!s->scratch) return flagcxSystemError;
  } else {
    if (s->scratch) { cudaDeviceSynchronize(); cudaFree(s->scratch); }
    FCX_CHECK(cudaToResult(cudaMalloc(&s->scratch, bytes), "C2C scratch"));
  }
  s->scratchBytes = bytes;
  return flagcxSuccess;
}

flagcxResult_t runHomo(flagcxComm *c, const C2cHomoFunc &h, const PendingOp &o, cudaStream_t st) {
  C2cState *s = c->c2c;
  flagcxComm *sub = h.homoType == 1 ? s->inter : s->intra;
  const size_t es = dtypeSize(o.dt);
  char *bufs[3] = {(char *)o.send, (char *)o.recv, (char *)s->scratch};
  const char *send = bufs[h.sendType] ? bufs[h.sendType] + h.sendOffset * es : nullptr;
  char *recv = bufs[h.recvType == 1 ? 1 : 2] ? bufs[h.recvType == 1 ? 1 : 2] + h.recvOffset * es : nullptr;
  flagcxStream fs{st};
  int root = h.rootRank >= 0 ? h.rootRank : o.root;
  InternalCallScope internal;  // stage buffers are cut out of the user's buffers and may overlap
  switch (h.commOp) {
    case flagcxCommOpReduce: return flagcxReduce(send, recv, h.count, o.dt, o.red, root, sub, &fs);
    case flagcxCommOpAllReduce: return flagcxAllReduce(send, recv, h.count, o.dt, o.red, sub, &fs);
    case flagcxCommOpReduceScatter: return flagcxReduceScatter(send, recv, h.count, o.dt, o.red, sub, &fs);
    case flagcxCommOpAllGather: return flagcxAllGather(send, recv, h.count, o.dt, sub, &fs);
    case flagcxCommOpBroadcast: return flagcxBroadcast(send, recv, h.count, o.dt, root, sub, &fs);
    case flagcxCommOpGather: return flagcxGather(send, recv, h.count, o.dt, root, sub, &fs);
    case flagcxCommOpScatter: return flagcxScatter(send, recv, h.count, o.dt, root, sub, &fs);
    case flagcxCommOpAlltoAll: return flagcxAlltoAll(send, recv, h.count, o.dt, sub, &fs);
    default: FCX_WARN("C2C: plan uses unsupported stage operation %d", h.commOp); return flagcxInvalidArgument;
  }
}

// Point-to-point lists run on the world communicator as one fused group.
flagcxResult_t runHetero(flagcxComm *c, const C2cHeteroFunc &h, const PendingOp &o, cudaStream_t st) {
  if (h.p2pOps.empty()) return flagcxSuccess;
  const size_t es = dtypeSize(o.dt);
  flagcxStream fs{st};
  FCX_CHECK(flagcxGroupStart(c));
  flagcxResult_t r = flagcxSuccess;
  for (auto &p : h.p2pOps) {
    char *base = p.buffType == 0 ? (char *)o.send : p.buffType == 2 ? (char *)c->c2c->scratch : (char *)o.recv;
    char *buf = base + p.offset * es;
    r = p.isRecv ? flagcxRecv(buf, p.count, o.dt, p.peerRank, c, &fs) : flagcxSend(buf, p.count, o.dt, p.peerRank, c, &fs);
    if (r != flagcxSuccess) break;
  }
  flagcxResult_t e = flagcxGroupEnd(c);
  return r != flagcxSuccess ? r : e;
}

flagcxResult_t runRefresh(flagcxComm *c, const C2cRefreshFunc &f, const PendingOp &o, cudaStream_t st) {
  if (f.buffType < 0 || f.redOp != flagcxSum || f.totalCount == 0) return flagcxSuccess;
  const size_t es = dtypeSize(o.dt);
  char *buf = (f.buffType == 1 ? (char *)o.recv : (char *)c->c2c->scratch) + f.start * es;
  size_t tail = f.totalCount - f.offset - f.count;
  if (c->hostOnly) {
    memset(buf, 0, f.offset * es);
    memset(buf + (f.offset + f.count) * es, 0, tail * es);
    return flagcxSuccess;
  }
  if (f.offset) FCX_CHECK(cudaToResult(cudaMemsetAsync(buf, 0, f.offset * es, st), "C2C refresh"));
  if (tail) FCX_CHECK(cudaToResult(cudaMemsetAsync(buf + (f.offset + f.count) * es, 0, tail * es, st), "C2C refresh"));
  return flagcxSuccess;
}

}  // namespace

void c2cDestroy(flagcxComm *c) {
  if (!c->c2c) return;
  C2cState *s = c->c2c;
  if (s->scratch) {
    if (c->hostOnly) free(s->scratch);
    else { cudaDeviceSynchronize(); cudaFree(s->scratch); }
  }
  if (s->sideStream) cudaStreamDestroy(s->sideStream);
  if (s->evA) cudaEventDestroy(s->evA);
  if (s->evB) cudaEventDestroy(s->evB);
  for (auto e : s->pieceEvents) cudaEventDestroy(e);
  cudaGetLastError();
  delete s;  // intra / inter are children of the communicator and are freed with it
  c->c2c = nullptr;
}

flagcxResult_t c2cExecute(flagcxComm *c, const PendingOp &o, bool *handled) {
  *handled = false;
  static const bool disabled = envInt("C2C_DISABLE", 0) != 0;
  if (disabled) return flagcxSuccess;
  switch (o.op) {
    case flagcxCommOpAllReduce: case flagcxCommOpReduceScatter: case flagcxCommOpAllGather: case flagcxCommOpBroadcast:
    case flagcxCommOpReduce: case flagcxCommOpGather: case flagcxCommOpScatter: case flagcxCommOpAlltoAll:
    case flagcxCommOpAlltoAllv: break;
    default: return flagcxSuccess;
  }
  if (o.outDt != o.dt || o.scale != 1.0f) return flagcxSuccess;
  if (o.red == flagcxProd && false) return flagcxSuccess;
  FCX_CHECK(ensureState(c));
  C2cState *s = c->c2c;
  if (s->unusable) return flagcxSuccess;
  const int C = c->nclusters, L = s->clusterSize;
  const std::string algo = envStr("C2C_ALGO", "");
  const bool fromXml = algo == "XML_INPUT";
  const bool pipelined = algo == "RING_PIPELINED";

  size_t sendTotal = o.count, recvTotal = o.count;
  if (o.op == flagcxCommOpReduceScatter || o.op == flagcxCommOpScatter) sendTotal = o.count * c->nranks;
  if (o.op == flagcxCommOpAllGather || o.op == flagcxCommOpGather) recvTotal = o.count * c->nranks;
  if (o.op == flagcxCommOpAlltoAll) sendTotal = recvTotal = o.count * c->nranks;
  const bool rooted = o.op == flagcxCommOpBroadcast || o.op == flagcxCommOpReduce || o.op == flagcxCommOpGather || o.op == flagcxCommOpScatter;
  const size_t rootCluster = rooted ? (size_t)(o.root / L) : (size_t)-1;
  const size_t fileHash = c2cAlgoHash(sendTotal, recvTotal, rootCluster, o.op, o.red);
  const size_t key = fileHash ^ ((size_t)o.dt << 40) ^ ((size_t)o.root << 48) ^ (pipelined ? 1ull << 63 : 0);
  const bool perCall = o.op == flagcxCommOpAlltoAllv;  // the plan depends on this call's counts: never cached

  C2cPlan *plan = nullptr;
  C2cPlan fresh;
  for (auto it = s->cache.begin(); !perCall && it != s->cache.end(); ++it)
    if (it->key == key) {
      s->cache.splice(s->cache.begin(), s->cache, it);
      plan = &s->cache.front().plan;
      break;
    }
  if (!plan) {
    C2cPlan p;
    if (fromXml) {
      std::string prefix = envStr("ALGO_IMPORT_PREFIX", "");
      std::string path = envStr("ALGO_IMPORT_PATH", "");
      if (prefix.empty() && !path.empty()) prefix = path + "/" + std::to_string(fileHash);
      if (prefix.empty()) { FCX_WARN("FLAGCX_C2C_ALGO=XML_INPUT needs FLAGCX_ALGO_IMPORT_PREFIX or FLAGCX_ALGO_IMPORT_PATH"); return flagcxInvalidUsage; }
      FCX_CHECK(c2cImportXml(&p, prefix, c->rank, std::max(sendTotal, recvTotal)));
    } else if (!c2cBuildPlan(&p, o.op, o.count, o.root, C, L, c->myCluster, s->myLocal, pipelined, s->interRanks, s->heteroP2p,
                             o.tables.empty() ? nullptr : o.tables.data())) {
      return flagcxSuccess;  // not planned hierarchically: run flat
    }
    std::string ex = envStr("ALGO_EXPORT_PREFIX", "");
    std::string exPath = envStr("ALGO_EXPORT_PATH", "");
    if (ex.empty() && !exPath.empty()) ex = exPath + "/" + std::to_string(fileHash);
    if (!ex.empty() && !fromXml) c2cExportXml(p, ex, c->rank);
    if (perCall) {
      fresh = std::move(p);
      plan = &fresh;
    } else {
      s->cache.push_front({key, std::move(p)});
      if (s->cache.size() > 16) s->cache.pop_back();
      plan = &s->cache.front().plan;
    }
  }

  FCX_CHECK(ensureScratch(c, plan->scratchCount * dtypeSize(o.dt)));
  cudaStream_t st = o.stream;
  const bool gpu = !c->hostOnly && !c->hostFallback;
  FCX_CHECK(runRefresh(c, plan->refresh, o, st));
  const size_t nPre = plan->preHomoFuncSteps.size(), nHet = plan->heteroFuncSteps.size(), nInter = plan->homoInterFuncSteps.size(),
               nPost = plan->postHomoFuncSteps.size();
  if (plan->pipelined && gpu && nPre == nInter && nInter == nPost && nHet == 0 && nPre <= 8) {
    // Software pipeline over the pieces.  Intra-cluster work stays on the
    // caller's stream, inter-cluster work goes to the side stream:
    //   main: pre0 pre1 [wait inter0] post0 pre2 [wait inter1] post1 ...
    //   side:      [wait pre0] inter0 [wait pre1] inter1 ...
    // so the inter-cluster stage of piece i overlaps the intra-cluster stages
    // of its neighbours.  Both communicators see the same order on every rank.
    while (s->pieceEvents.size() < 2 * nPre) {
      cudaEvent_t e;
      FCX_CHECK(cudaToResult(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "C2C event"));
      s->pieceEvents.push_back(e);
    }
    auto issuePreAndInter = [&](size_t i) -> flagcxResult_t {
      for (auto &h : plan->preHomoFuncSteps[i]) FCX_CHECK(runHomo(c, h, o, st));
      cudaEventRecord(s->pieceEvents[2 * i], st);
      cudaStreamWaitEvent(s->sideStream, s->pieceEvents[2 * i], 0);
      for (auto &h : plan->homoInterFuncSteps[i]) FCX_CHECK(runHomo(c, h, o, s->sideStream));
      cudaEventRecord(s->pieceEvents[2 * i + 1], s->sideStream);
      return flagcxSuccess;
    };
    FCX_CHECK(issuePreAndInter(0));
    for (size_t i = 0; i < nPre; i++) {
      if (i + 1 < nPre) FCX_CHECK(issuePreAndInter(i + 1));
      cudaStreamWaitEvent(st, s->pieceEvents[2 * i + 1], 0);
      for (auto &h : plan->postHomoFuncSteps[i]) FCX_CHECK(runHomo(c, h, o, st));
    }
  } else {
    for (auto &step : plan->preHomoFuncSteps)
      for (auto &h : step) FCX_CHECK(runHomo(c, h, o, st));
    for (auto &step : plan->heteroFuncSteps)
      for (auto &h : step) FCX_CHECK(runHetero(c, h, o, st));
    for (auto &step : plan->homoInterFuncSteps)
      for (auto &h : step) FCX_CHECK(runHomo(c, h, o, st));
    for (auto &step : plan->postHomoFuncSteps)
      for (auto &h : step) FCX_CHECK(runHomo(c, h, o, st));
  }
  *handled = true;
  return flagcxSuccess;
}

}  // namespace fcx

using namespace fcx;

static flagcxResult_t commSplitImpl(flagcxComm_t comm, int color, int key, size_t stageBytes, size_t userBytes, flagcxComm_t *newcomm);

extern "C" flagcxResult_t flagcxCommSplit(flagcxComm_t comm, int color, int key, flagcxComm_t *newcomm) {
  return commSplitImpl(comm, color, key, 0, 0, newcomm);
}
extern "C" flagcxResult_t flagcxCommSplitSized(flagcxComm_t comm, int color, int key, size_t stageBytes, size_t userBytes,
                                               flagcxComm_t *newcomm) {
  return commSplitImpl(comm, color, key, stageBytes, userBytes, newcomm);
}

static flagcxResult_t commSplitImpl(flagcxComm_t comm, int color, int key, size_t stageBytes, size_t userBytes, flagcxComm_t *newcomm) {
  if (!validComm(comm) || !newcomm) return flagcxInvalidArgument;
  *newcomm = nullptr;
  const int n = comm->nranks, me = comm->rank;
  struct CK { int color, key; };
  std::vector<CK> all(n);
  all[me] = {color, key};
  FCX_CHECK(comm->bs.allGather(all.data(), sizeof(CK)));
  static std::atomic<int> splitSeq{0};
  const int tag = 0x5b1700 + (splitSeq++ & 0xff);
  // every colour group elects its first member (by key, then rank) as the one that opens the rendezvous
  std::vector<int> members;
  for (int r = 0; r < n; r++)
    if (all[r].color == color) members.push_back(r);
  std::stable_sort(members.begin(), members.end(), [&](int a, int b) { return all[a].key < all[b].key; });
  if (color < 0) return flagcxSuccess;
  int newRank = (int)(std::find(members.begin(), members.end(), me) - members.begin());
  BootstrapHandle h;
  if (newRank == 0) {
    FCX_CHECK(Bootstrap::createId(&h, /*allowFixedAddress=*/false));
    for (size_t i = 1; i < members.size(); i++) FCX_CHECK(comm->bs.send(members[i], tag, &h, sizeof h));
  } else {
    FCX_CHECK(comm->bs.recv(members[0], tag, &h, sizeof h));
  }
  flagcxComm *child = nullptr;
  unsigned flags = comm->hostOnly ? FLAGCX_INIT_HOST_ONLY : 0u;
  const char *savedSplit = getenv("FLAGCX_CLUSTER_SPLIT_LIST");
  std::string saved = savedSplit ? savedSplit : "";
  if (savedSplit) unsetenv("FLAGCX_CLUSTER_SPLIT_LIST");  // a sub-communicator is one cluster
  flagcxResult_t r = commCreate(&child, (int)members.size(), h, newRank, envInt("SUBCOMM_HEAP_SCALE_PCT", 25) / 100.0, flags, stageBytes, userBytes);
  if (savedSplit) setenv("FLAGCX_CLUSTER_SPLIT_LIST", saved.c_str(), 1);
  FCX_CHECK(r);
  child->hostFallback = comm->hostFallback;
  child->parent = comm;
  comm->children.push_back(child);
  *newcomm = child;
  return flagcxSuccess;
}
