// flagcx_perf - collective benchmark with the reference's command line,
// without MPI.
//
//   flagcx_perf -o allreduce -g 8 -b 8 -e 4G -f 2 -w 5 -n 20 [-L path/to/libflagcx.so]
//
// The reference's perf programs (test/perf/test_*.cpp, options parsed in
// test/perf/tools.cc:80-199) are launched with mpirun, one rank per GPU, and
// ship the unique id with MPI_Bcast.  This tool forks the ranks itself and
// passes the id through pipes; the library under test is loaded with dlopen,
// so the very same binary measures this library or the reference's
// libflagcx.so through the common C ABI.
//
// Options: -o op (allreduce allgather reducescatter alltoall alltoallv broadcast reduce gather scatter sendrecv)
//   -g ranks  -b min bytes  -e max bytes  -f factor  -w warm-up iterations  -n timed iterations
//   -p 1 print the first values  -r root (-1: every root in turn)  -R 1 buffers from flagcxMemAlloc + flagcxCommRegister
//   -d dtype (float bf16 half fp8 uint8)  -O reduction (sum max min avg)  -c 1 check results against a host computation
//   -J file append JSON lines  -T 1 tune: time every kernel variant of every (op, size) first and record the fastest
//   (this repository's library only)  -S file write the tuned table there (load it with FLAGCX_TUNER_CACHE)
// Sizes follow the reference: the size is the whole buffer; all-gather, reduce-scatter, all-to-all, gather and scatter
// move size/ranks per rank.  Reported: device time (CUDA events around the -n calls), MAX over ranks, and the
// reference-style host-timed mean over ranks; bus-bandwidth factors as in the reference's tests.
#include <algorithm>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "flagcx.h"

namespace {

struct Api {
  flagcxResult_t (*HandleInit)(flagcxHandlerGroup_t *);
  flagcxResult_t (*GetUniqueId)(flagcxUniqueId_t *);
  flagcxResult_t (*CommInitRank)(flagcxComm_t *, int, flagcxUniqueId_t, int);
  flagcxResult_t (*CommDestroy)(flagcxComm_t);
  flagcxResult_t (*MemAlloc)(void **, size_t, flagcxComm_t);
  flagcxResult_t (*MemFree)(void *, flagcxComm_t);
  flagcxResult_t (*CommRegister)(const flagcxComm_t, void *, size_t, void **);
  flagcxResult_t (*CommDeregister)(const flagcxComm_t, void *);
  flagcxResult_t (*Barrier)(flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*AllReduce)(const void *, void *, size_t, flagcxDataType_t, flagcxRedOp_t, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Reduce)(const void *, void *, size_t, flagcxDataType_t, flagcxRedOp_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*AllGather)(const void *, void *, size_t, flagcxDataType_t, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*ReduceScatter)(const void *, void *, size_t, flagcxDataType_t, flagcxRedOp_t, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Broadcast)(const void *, void *, size_t, flagcxDataType_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Gather)(const void *, void *, size_t, flagcxDataType_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Scatter)(const void *, void *, size_t, flagcxDataType_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*AlltoAll)(const void *, void *, size_t, flagcxDataType_t, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*AlltoAllv)(const void *, size_t *, size_t *, void *, size_t *, size_t *, flagcxDataType_t, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Send)(const void *, size_t, flagcxDataType_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*Recv)(void *, size_t, flagcxDataType_t, int, flagcxComm_t, flagcxStream_t);
  flagcxResult_t (*GroupStart)(flagcxComm_t);
  flagcxResult_t (*GroupEnd)(flagcxComm_t);
  // extensions of this repository's library (absent from the reference's): needed by the tune mode only
  flagcxResult_t (*TunerCandidates)(flagcxComm_t, flagcxCommOp_t, size_t, flagcxDataType_t, flagcxRedOp_t, int, int, int *, int *, int *) = nullptr;
  const char *(*KindName)(int) = nullptr;
  flagcxResult_t (*TunerPinEx)(flagcxComm_t, const char *, int, unsigned int) = nullptr;
  flagcxResult_t (*TunerRecordEx)(flagcxComm_t, flagcxCommOp_t, size_t, const char *, int, unsigned int, double) = nullptr;
  flagcxResult_t (*TunerSave)(flagcxComm_t, const char *) = nullptr;
};

template <typename F>
bool sym(void *h, const char *name, F *fn) {
  *fn = (F)dlsym(h, name);
  if (!*fn) fprintf(stderr, "missing symbol %s\n", name);
  return *fn != nullptr;
}

bool loadApi(const char *path, Api *a) {
  void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "dlopen(%s): %s\n", path, dlerror()); return false; }
  bool ok = true;
  ok &= sym(h, "flagcxHandleInit", &a->HandleInit);
  ok &= sym(h, "flagcxGetUniqueId", &a->GetUniqueId);
  ok &= sym(h, "flagcxCommInitRank", &a->CommInitRank);
  ok &= sym(h, "flagcxCommDestroy", &a->CommDestroy);
  ok &= sym(h, "flagcxMemAlloc", &a->MemAlloc);
  ok &= sym(h, "flagcxMemFree", &a->MemFree);
  ok &= sym(h, "flagcxCommRegister", &a->CommRegister);
  ok &= sym(h, "flagcxCommDeregister", &a->CommDeregister);
  ok &= sym(h, "flagcxBarrier", &a->Barrier);
  ok &= sym(h, "flagcxAllReduce", &a->AllReduce);
  ok &= sym(h, "flagcxReduce", &a->Reduce);
  ok &= sym(h, "flagcxAllGather", &a->AllGather);
  ok &= sym(h, "flagcxReduceScatter", &a->ReduceScatter);
  ok &= sym(h, "flagcxBroadcast", &a->Broadcast);
  ok &= sym(h, "flagcxGather", &a->Gather);
  ok &= sym(h, "flagcxScatter", &a->Scatter);
  ok &= sym(h, "flagcxAlltoAll", &a->AlltoAll);
  ok &= sym(h, "flagcxAlltoAllv", &a->AlltoAllv);
  ok &= sym(h, "flagcxSend", &a->Send);
  ok &= sym(h, "flagcxRecv", &a->Recv);
  ok &= sym(h, "flagcxGroupStart", &a->GroupStart);
  ok &= sym(h, "flagcxGroupEnd", &a->GroupEnd);
  a->TunerCandidates = (decltype(a->TunerCandidates))dlsym(h, "flagcxTunerCandidates");
  a->KindName = (decltype(a->KindName))dlsym(h, "flagcxKindName");
  a->TunerPinEx = (decltype(a->TunerPinEx))dlsym(h, "flagcxTunerPinEx");
  a->TunerRecordEx = (decltype(a->TunerRecordEx))dlsym(h, "flagcxTunerRecordEx");
  a->TunerSave = (decltype(a->TunerSave))dlsym(h, "flagcxTunerSave");
  return ok;
}

size_t parseSize(const char *s) {
  char *end;
  double v = strtod(s, &end);
  switch (*end) {
    case 'K': case 'k': v *= 1024; break;
    case 'M': case 'm': v *= 1024 * 1024; break;
    case 'G': case 'g': v *= 1024.0 * 1024 * 1024; break;
  }
  return (size_t)v;
}

struct Opts {
  std::string op = "allreduce", lib, dtype = "float", json, redop = "sum", tuneOut;
  int ranks = 0, warm = 5, iters = 20, print = 0, root = 0, reg = 0, check = 0, splitMask = 0, tune = 0;
  size_t minB = 8, maxB = 128u << 20;
  double factor = 2;
};

struct Row { size_t bytes; double devUs, hostUs; int bad; int op; };

// "-o a,b,c": several operations on one communicator (one process start-up for the whole list)
std::vector<std::string> splitOps(const std::string &s) {
  std::vector<std::string> v;
  size_t a = 0;
  while (a <= s.size()) {
    size_t b = s.find(',', a);
    if (b == std::string::npos) b = s.size();
    if (b > a) v.push_back(s.substr(a, b - a));
    a = b + 1;
  }
  return v;
}

#define CK(call)                                                             \
  do {                                                                       \
    flagcxResult_t _r = (call);                                              \
    if (_r != flagcxSuccess) {                                               \
      fprintf(stderr, "rank %d: %s failed with %d\n", rank, #call, (int)_r); \
      _exit(2);                                                              \
    }                                                                        \
  } while (0)

float bf16ToF(uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; }

int worker(const Opts &o, int rank, int n, int idRead, int idWrite[], int outFd) {
  Api api;
  if (!loadApi(o.lib.c_str(), &api)) return 3;
  cudaSetDevice(rank);  // before the split: one GPU per world rank
  cudaFree(0);
  flagcxHandlerGroup_t hg;
  CK(api.HandleInit(&hg));
  // -s mask: the ranks with the same (rank & mask) form one communicator, like the reference's harness
  // (test/perf/tools.cc:16-20); world rank stays the device index.
  const int worldRank = rank, worldSize = n, color = worldRank & o.splitMask;
  std::vector<int> members;
  for (int r = 0; r < worldSize; r++)
    if ((r & o.splitMask) == color) members.push_back(r);
  n = (int)members.size();
  rank = (int)(std::find(members.begin(), members.end(), worldRank) - members.begin());
  flagcxUniqueId id;
  if (rank == 0) {
    // the reference allocates the id itself and overwrites the pointer
    flagcxUniqueId_t q = nullptr;
    CK(api.GetUniqueId(&q));
    memcpy(&id, q, sizeof id);
    for (int r = 1; r < n; r++)
      if (write(idWrite[members[r]], &id, sizeof id) != (ssize_t)sizeof id) return 4;
  } else if (read(idRead, &id, sizeof id) != (ssize_t)sizeof id) {
    return 4;
  }
  flagcxComm_t comm;
  CK(api.CommInitRank(&comm, n, &id, rank));
  flagcxStream_t st;
  if (hg->devHandle->streamCreate(&st) != flagcxSuccess) return 5;
  cudaStream_t cs = *(cudaStream_t *)st;  // the wrapper's only member
  cudaStream_t cs_ = cs;

  const bool isBf16 = o.dtype == "bf16", isHalf = o.dtype == "half", isFp8 = o.dtype == "fp8", isU8 = o.dtype == "uint8" || isFp8;
  // fp8 (e4m3) is data type 10 of this library; the reference has no such type and moves fp8 as bytes
  const flagcxDataType_t dt = isBf16 ? flagcxBfloat16 : isHalf ? flagcxHalf : isFp8 ? (flagcxDataType_t)10 : isU8 ? flagcxUint8 : flagcxFloat;
  const flagcxRedOp_t red = o.redop == "max" ? flagcxMax : o.redop == "min" ? flagcxMin : o.redop == "avg" ? flagcxAvg : flagcxSum;
  const size_t es = (isBf16 || isHalf) ? 2 : isU8 ? 1 : 4;
  void *send = nullptr, *recv = nullptr, *hs = nullptr, *hr = nullptr;
  const size_t cap = std::max<size_t>(o.maxB, 64);
  if (o.reg) {
    CK(api.MemAlloc(&send, cap, comm));
    CK(api.MemAlloc(&recv, cap, comm));
    CK(api.CommRegister(comm, send, cap, &hs));
    CK(api.CommRegister(comm, recv, cap, &hr));
  } else {
    cudaMalloc(&send, cap);
    cudaMalloc(&recv, cap);
  }
  // data: element i of rank r is ((i + r) % 10) for floats (exact in bf16 too), bytes for uint8
  {
    size_t ne = cap / es;
    std::vector<char> host(cap);
    for (size_t i = 0; i < ne; i++) {
      float v = (float)((i + rank) % 10);
      if (es == 4) ((float *)host.data())[i] = v;
      else if (isBf16) { uint32_t u; memcpy(&u, &v, 4); ((uint16_t *)host.data())[i] = (uint16_t)(u >> 16); }
      else if (isHalf) ((uint16_t *)host.data())[i] = v == 0 ? 0 : (uint16_t)0;  // half only times; values unused
      else if (isFp8) host[i] = (char)(0x30 + ((i + rank) % 8));  // e4m3 codes of 0.5 .. 0.9375: sums stay finite
      else host[i] = (char)((i + rank) % 10);
    }
    cudaMemcpy(send, host.data(), cap, cudaMemcpyHostToDevice);
    cudaMemset(recv, 0, cap);
  }
  std::vector<Row> rows;
  const std::vector<std::string> ops = splitOps(o.op);
  for (size_t oi = 0; oi < ops.size(); oi++) {
  const std::string &opn = ops[oi];
  const bool whole = opn == "allreduce" || opn == "broadcast" || opn == "reduce" || opn == "sendrecv";
  for (size_t size = o.minB; size <= o.maxB;) {
    size_t count = std::max<size_t>(whole ? size / es : size / es / n, 1);
    size_t nbytes = count * es * (whole ? 1 : n);
    std::vector<int> roots;
    const bool rooted = opn == "broadcast" || opn == "reduce" || opn == "gather" || opn == "scatter";
    if (rooted && o.root < 0) for (int r = 0; r < n; r++) roots.push_back(r);
    else roots.push_back(std::max(o.root, 0));
    std::vector<size_t> cnt(n, count), dsp(n);
    for (int i = 0; i < n; i++) dsp[i] = i * count;
    auto call = [&](int root) {
      if (opn == "allreduce") CK(api.AllReduce(send, recv, count, dt, red, comm, st));
      else if (opn == "allgather") CK(api.AllGather(send, recv, count, dt, comm, st));
      else if (opn == "reducescatter") CK(api.ReduceScatter(send, recv, count, dt, red, comm, st));
      else if (opn == "alltoall") CK(api.AlltoAll(send, recv, count, dt, comm, st));
      else if (opn == "alltoallv") CK(api.AlltoAllv(send, cnt.data(), dsp.data(), recv, cnt.data(), dsp.data(), dt, comm, st));
      else if (opn == "broadcast") CK(api.Broadcast(send, recv, count, dt, root, comm, st));
      else if (opn == "reduce") CK(api.Reduce(send, recv, count, dt, red, root, comm, st));
      else if (opn == "gather") CK(api.Gather(send, recv, count, dt, root, comm, st));
      else if (opn == "scatter") CK(api.Scatter(send, recv, count, dt, root, comm, st));
      else if (opn == "sendrecv") {
        CK(api.GroupStart(comm));
        CK(api.Send(send, count, dt, (rank + 1) % n, comm, st));
        CK(api.Recv(recv, count, dt, (rank + n - 1) % n, comm, st));
        CK(api.GroupEnd(comm));
      } else { fprintf(stderr, "unknown op %s\n", opn.c_str()); _exit(2); }
    };
    int iters = size <= (256u << 20) ? o.iters : std::max(5, o.iters / 4);
    double devUs = 0, hostUs = 0;
    int bad = 0;
    if (o.tune && api.TunerCandidates && api.TunerPinEx && api.TunerRecordEx && api.KindName && opn != "sendrecv" && opn != "alltoallv") {
      // Tune mode: time every legal variant of this call (kind x CTA count, then sub-chunk sizes for the best
      // staged kind), let the ranks agree on the slowest rank's time per variant, record the fastest.
      const flagcxCommOp_t cop = opn == "allreduce" ? flagcxCommOpAllReduce : opn == "allgather" ? flagcxCommOpAllGather
                                 : opn == "reducescatter" ? flagcxCommOpReduceScatter : opn == "alltoall" ? flagcxCommOpAlltoAll
                                 : opn == "broadcast" ? flagcxCommOpBroadcast : opn == "reduce" ? flagcxCommOpReduce
                                 : opn == "gather" ? flagcxCommOpGather : flagcxCommOpScatter;
      const size_t keyBytes = count * es;
      int kinds[64], ctas[64], nc = 0;
      CK(api.TunerCandidates(comm, cop, keyBytes, dt, red, o.reg, 64, kinds, ctas, &nc));
      struct Cand { int kind, ctas; unsigned pipe; };
      std::vector<Cand> cands;
      for (int i = 0; i < nc; i++) cands.push_back({kinds[i], ctas[i], 0u});
      static float *agree = nullptr;  // device scratch for the cross-rank agreement
      if (!agree) cudaMalloc(&agree, 256 * sizeof(float));
      const int tIters = std::max(3, std::min(o.iters, size <= (64u << 20) ? 10 : 4));
      auto timeAll = [&](std::vector<Cand> &cs, std::vector<float> &us) {
        us.assign(cs.size(), 0.f);
        for (size_t i = 0; i < cs.size(); i++) {
          CK(api.TunerPinEx(comm, api.KindName(cs[i].kind), cs[i].ctas, cs[i].pipe));
          for (int w = 0; w < 2; w++) call(roots[0]);
          cudaEvent_t e0, e1;
          cudaEventCreate(&e0);
          cudaEventCreate(&e1);
          cudaEventRecord(e0, cs_);
          for (int k = 0; k < tIters; k++) call(roots[0]);
          cudaEventRecord(e1, cs_);
          cudaStreamSynchronize(cs_);
          float ms = 0;
          cudaEventElapsedTime(&ms, e0, e1);
          us[i] = ms * 1e3f / tIters;
          cudaEventDestroy(e0);
          cudaEventDestroy(e1);
        }
        CK(api.TunerPinEx(comm, nullptr, 0, 0));
        // the slowest rank's time decides (max over ranks), computed by the library itself
        cudaMemcpyAsync(agree, us.data(), us.size() * sizeof(float), cudaMemcpyHostToDevice, cs_);
        CK(api.AllReduce(agree, agree, us.size(), flagcxFloat, flagcxMax, comm, st));
        cudaMemcpyAsync(us.data(), agree, us.size() * sizeof(float), cudaMemcpyDeviceToHost, cs_);
        cudaStreamSynchronize(cs_);
      };
      std::vector<float> us;
      timeAll(cands, us);
      size_t best = 0;
      for (size_t i = 1; i < cands.size(); i++) if (us[i] < us[best]) best = i;
      Cand win = cands[best];
      float winUs = us[best];
      if (keyBytes >= (32u << 20)) {
        // sub-chunk size only matters to the staged, pipelined kinds: try two more sizes on the best of them
        size_t bs = cands.size();
        for (size_t i = 0; i < cands.size(); i++) {
          std::string kn = api.KindName(cands[i].kind);
          bool staged = kn.find("_zc") == std::string::npos && kn.find("_ll") == std::string::npos && kn != "ar_oneshot";
          if (staged && (bs == cands.size() || us[i] < us[bs])) bs = i;
        }
        if (bs < cands.size()) {
          std::vector<Cand> more = {{cands[bs].kind, cands[bs].ctas, 4u << 20}, {cands[bs].kind, cands[bs].ctas, 64u << 20}};
          std::vector<float> us2;
          timeAll(more, us2);
          for (size_t i = 0; i < more.size(); i++) {
            CK(api.TunerRecordEx(comm, cop, keyBytes, api.KindName(more[i].kind), more[i].ctas, more[i].pipe, us2[i]));
            if (us2[i] < winUs) { win = more[i]; winUs = us2[i]; }
          }
        }
      }
      for (size_t i = 0; i < cands.size(); i++)
        CK(api.TunerRecordEx(comm, cop, keyBytes, api.KindName(cands[i].kind), cands[i].ctas, cands[i].pipe, us[i]));
      if (rank == 0) {
        printf("tune %-13s %12zu B  -> %-10s x%-3d pipe %-9u %9.2f us   (prior's pick %s x%d: %.2f us; %d variants)\n", opn.c_str(), nbytes,
               api.KindName(win.kind), win.ctas, win.pipe, winUs, api.KindName(cands[0].kind), cands[0].ctas, us[0], (int)cands.size());
        fflush(stdout);
      }
    }
    for (int root : roots) {
      for (int i = 0; i < o.warm; i++) call(root);
      cudaStreamSynchronize(cs);
      CK(api.Barrier(comm, st));
      cudaEvent_t e0, e1;
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      auto t0 = std::chrono::steady_clock::now();
      cudaEventRecord(e0, cs);
      for (int i = 0; i < iters; i++) call(root);
      cudaEventRecord(e1, cs);
      cudaStreamSynchronize(cs);
      auto t1 = std::chrono::steady_clock::now();
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      devUs += ms * 1e3 / iters / roots.size();
      hostUs += std::chrono::duration<double, std::micro>(t1 - t0).count() / iters / roots.size();
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      if (o.check && es != 1 && !isHalf && red == flagcxSum && (opn == "allreduce" || opn == "allgather" || opn == "reducescatter" || opn == "alltoall")) {
        size_t outElems = opn == "allreduce" ? count : opn == "reducescatter" ? count : count * n;
        outElems = std::min<size_t>(outElems, 1 << 20);
        std::vector<char> h(outElems * es);
        cudaMemcpy(h.data(), recv, outElems * es, cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < outElems; i++) {
          float got = es == 4 ? ((float *)h.data())[i] : bf16ToF(((uint16_t *)h.data())[i]);
          float want = 0;
          if (opn == "allreduce") for (int r = 0; r < n; r++) want += (float)((i + r) % 10);
          else if (opn == "reducescatter") for (int r = 0; r < n; r++) want += (float)((rank * count + i + r) % 10);
          else if (opn == "allgather") want = (float)((i % count + i / count) % 10);
          else want = (float)((rank * count + i % count + i / count) % 10);
          if (std::fabs(got - want) > (es == 2 ? 0.51f : 1e-3f)) { bad++; if (bad < 4) fprintf(stderr, "rank %d %s[%zu] = %g, expected %g\n", rank, opn.c_str(), i, got, want); }
        }
      }
    }
    if (o.print && rank == 0) {
      float h[10] = {};
      cudaMemcpy(h, recv, std::min<size_t>(40, nbytes), cudaMemcpyDeviceToHost);
      printf("recv:");
      for (int i = 0; i < 10; i++) printf(" %g", h[i]);
      printf("\n");
    }
    rows.push_back({nbytes, devUs, hostUs, bad, (int)oi});
    size_t next = (size_t)(size * o.factor);
    size = next > size ? next : size + 1;
  }
  }
  CK(api.Barrier(comm, st));
  if (o.tune && !o.tuneOut.empty() && api.TunerSave && rank == 0) CK(api.TunerSave(comm, o.tuneOut.c_str()));
  if (o.reg) {
    api.CommDeregister(comm, hs);
    api.CommDeregister(comm, hr);
    api.MemFree(send, comm);
    api.MemFree(recv, comm);
  } else {
    cudaFree(send);
    cudaFree(recv);
  }
  CK(api.CommDestroy(comm));
  size_t nrows = rows.size();
  if (write(outFd, &nrows, sizeof nrows) < 0 || write(outFd, rows.data(), nrows * sizeof(Row)) < 0) return 6;
  return 0;
}

double busFactor(const std::string &op, int n) {
  if (op == "allreduce") return 2.0 * (n - 1) / n;
  if (op == "allgather" || op == "reducescatter" || op == "alltoall" || op == "alltoallv" || op == "gather" || op == "scatter") return (double)(n - 1) / n;
  return 1.0;
}

}  // namespace

int main(int argc, char **argv) {
  Opts o;
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    const char *v = argv[i + 1];
    if (k == "-o") o.op = v;
    else if (k == "-g") o.ranks = atoi(v);
    else if (k == "-b") o.minB = parseSize(v);
    else if (k == "-e") o.maxB = parseSize(v);
    else if (k == "-f") o.factor = atof(v);
    else if (k == "-w") o.warm = atoi(v);
    else if (k == "-n") o.iters = atoi(v);
    else if (k == "-p") o.print = atoi(v);
    else if (k == "-r") o.root = atoi(v);
    else if (k == "-R") o.reg = atoi(v);
    else if (k == "-s") o.splitMask = (int)strtol(v, nullptr, 0);
    else if (k == "-L") o.lib = v;
    else if (k == "-d") o.dtype = v;
    else if (k == "-c") o.check = atoi(v);
    else if (k == "-J") o.json = v;
    else if (k == "-O") o.redop = v;
    else if (k == "-T") o.tune = atoi(v);
    else if (k == "-S") o.tuneOut = v;
    else { fprintf(stderr, "unknown option %s\n", k.c_str()); return 1; }
  }
  if (o.lib.empty()) {
    // default: this repository's library
    char self[4096];
    ssize_t k = readlink("/proc/self/exe", self, sizeof self - 1);
    std::string dir = k > 0 ? std::string(self, k) : std::string(".");
    dir = dir.substr(0, dir.rfind('/'));
    o.lib = dir + "/../../flagcx_b200/lib/libflagcx.so";  // build/bin -> repository root
  }
  setenv("FLAGCX_SOCKET_IFNAME", "lo", 0);
  int n = o.ranks;
  if (n <= 0) {
    // count GPUs in a child so that this process never creates a CUDA context before forking
    int pfd[2];
    if (pipe(pfd)) return 1;
    if (fork() == 0) { int c = 0; cudaGetDeviceCount(&c); if (write(pfd[1], &c, sizeof c) < 0) _exit(1); _exit(0); }
    if (read(pfd[0], &n, sizeof n) != (ssize_t)sizeof n) n = 1;
    wait(nullptr);
  }
  std::vector<int> idR(n, -1), idW(n, -1), outR(n), pids(n);
  for (int r = 1; r < n; r++) { int p[2]; if (pipe(p)) return 1; idR[r] = p[0]; idW[r] = p[1]; }
  for (int r = 0; r < n; r++) {
    int p[2];
    if (pipe(p)) return 1;
    outR[r] = p[0];
    pid_t pid = fork();
    if (pid == 0) _exit(worker(o, r, n, idR[r], idW.data(), p[1]));
    pids[r] = pid;
    close(p[1]);
  }
  std::vector<std::vector<Row>> all(n);
  bool fail = false;
  for (int r = 0; r < n; r++) {
    size_t nrows = 0;
    if (read(outR[r], &nrows, sizeof nrows) == (ssize_t)sizeof nrows && nrows < 4096) {
      all[r].resize(nrows);
      size_t got = 0;
      while (got < nrows * sizeof(Row)) {
        ssize_t k = read(outR[r], (char *)all[r].data() + got, nrows * sizeof(Row) - got);
        if (k <= 0) break;
        got += k;
      }
    }
    int status = 0;
    waitpid(pids[r], &status, 0);
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) { fprintf(stderr, "rank %d exited abnormally (%d)\n", r, status); fail = true; }
  }
  if (fail) return 1;
  const std::vector<std::string> ops = splitOps(o.op);
  FILE *jf = o.json.empty() ? nullptr : fopen(o.json.c_str(), "a");
  int lastOp = -1;
  for (size_t i = 0; i < all[0].size(); i++) {
    const std::string &opn = ops[all[0][i].op];
    int groupSize = 0;
    for (int r = 0; r < n; r++) groupSize += ((r & o.splitMask) == 0);
    const double f = busFactor(opn, groupSize);
    if (all[0][i].op != lastOp) {
      lastOp = all[0][i].op;
      printf("# %s, %d ranks%s, %s, library %s\n", opn.c_str(), groupSize, o.splitMask ? " per communicator" : "", o.dtype.c_str(), o.lib.c_str());
      printf("# %12s %12s %12s %12s %14s %6s\n", "bytes", "time_us", "algbw_GB/s", "busbw_GB/s", "host_mean_us", "wrong");
    }
    double dev = 0, host = 0;
    int bad = 0;
    for (int r = 0; r < n; r++) { dev = std::max(dev, all[r][i].devUs); host += all[r][i].hostUs / n; bad += all[r][i].bad; }
    double alg = all[0][i].bytes / dev / 1e3;
    printf("  %12zu %12.2f %12.2f %12.2f %14.2f %6d\n", all[0][i].bytes, dev, alg, alg * f, host, bad);
    if (jf)
      fprintf(jf, "{\"op\": \"%s\", \"lib\": \"%s\", \"dtype\": \"%s\", \"ranks\": %d, \"bytes\": %zu, \"time_us\": %.3f, \"algbw_gbs\": %.3f, "
                  "\"busbw_gbs\": %.3f, \"host_mean_us\": %.3f, \"wrong\": %d, \"registered\": %d}\n",
              opn.c_str(), o.lib.c_str(), o.dtype.c_str(), n, all[0][i].bytes, dev, alg, alg * f, host, bad, o.reg);
  }
  if (jf) fclose(jf);
  return 0;
}
