// Internal definition of a communicator and of the opaque handle types.
#pragma once
#include "bootstrap.h"
#include "flagcx.h"
#include "flagcx_ext.h"
#include "symheap.h"
#include "tuner.h"
#include "../kernels/devcomm.h"

#include <atomic>
#include <cuda_runtime_api.h>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

struct flagcxStream { cudaStream_t base; };
struct flagcxEvent { cudaEvent_t base; };
struct flagcxIpcMemHandle { cudaIpcMemHandle_t base; };

namespace fcx {

struct PeerInfo {
  uint64_t hostHash;
  int32_t pid, cudaDev, hostOnly, pad;
  char vendor[32];
  char busId[32];
};

// An operation queued between flagcxGroupStart and flagcxGroupEnd.
struct PendingOp {
  flagcxCommOp_t op;
  const void *send;
  void *recv;
  size_t count;
  flagcxDataType_t dt, outDt;
  flagcxRedOp_t red;
  int root;  // peer for send/recv
  float scale;
  std::vector<size_t> tables;  // all-to-all-v: scounts, sdispls, rcounts, rdispls
  cudaStream_t stream;
};

struct Segment {  // a registered user buffer
  char *localBase = nullptr;
  size_t bytes = 0;
  char *peer[FCX_MAX_RANKS] = {};
  bool used = false;
};

class C2cState;   // cross-cluster planner state (c2c/planner.h)
class FifoService;  // device->host request queue service (core/fifo.h)

}  // namespace fcx

struct flagcxComm {
  uint32_t magic = 0xF1A6C0DE;
  int rank = 0, nranks = 1;
  fcx::Bootstrap bs;
  std::atomic<uint32_t> abortFlag{0};
  bool hostOnly = false;     // no GPU behind this communicator: buffers are host memory
  bool hostFallback = false;  // FLAGCX_USE_HOST_COMM=1 with a GPU: copy to host, combine there, copy back
  int cudaDev = -1;
  std::vector<fcx::PeerInfo> peers;

  // cluster view (FLAGCX_CLUSTER_SPLIT_LIST)
  std::vector<int> clusterOf;
  int nclusters = 1, myCluster = 0;
  // network port each rank's GPU is attached to, from FLAGCX_TOPO_FILE (empty without one)
  std::vector<std::string> netOfRank;

  // device side
  fcx::SymHeap heap;
  FcxDevComm dev{};
  FcxDevError *errHost = nullptr;
  uint32_t *abortHost = nullptr;
  char *(*segsDev)[FCX_MAX_RANKS] = nullptr;
  fcx::Arena arena;
  std::vector<fcx::Segment> segs;
  uint64_t seq = 0;
  uint64_t sendChunks[FCX_MAX_RANKS] = {}, recvChunks[FCX_MAX_RANKS] = {};
  int nextSignal = 0;
  // zero-copy kinds through the switch: 0 never, 1 from three ranks on, 2 whenever the box has a multicast alias
  int zcMcMode = 1, zcAgMcMode = 1;

  std::unique_ptr<fcx::Tuner> tuner;
  flagcxCommCounters counters{};
  std::mutex mu;

  // group state (per communicator; depth is per thread, see group.cc)
  std::vector<fcx::PendingOp> pending;

  // hybrid (multi-cluster) machinery, created on first use
  fcx::C2cState *c2c = nullptr;
  // device->host request queue
  fcx::FifoService *fifo = nullptr;
  // communicators split off this one, destroyed with it (a child destroyed on its own leaves this list)
  std::vector<flagcxComm *> children;
  flagcxComm *parent = nullptr;
  bool destroyed = false;
  // Heap memory handed to owners that may outlive the communicator (tensors): while any is outstanding a
  // destroyed communicator keeps its heap mapped and is only freed by the last release.
  std::atomic<int> heapRefs{0};
};

namespace fcx {

bool validComm(flagcxComm_t c);
flagcxResult_t cudaToResult(cudaError_t e, const char *what);

// Direct (non-grouped, single-cluster) launches; implemented in coll.cc.
flagcxResult_t launchCollective(flagcxComm *c, const PendingOp &op);
flagcxResult_t launchP2pBatch(flagcxComm *c, const std::vector<PendingOp> &ops);
flagcxResult_t hostCollective(flagcxComm *c, const PendingOp &op);
int groupDepth();
// While an object of this type lives on a thread, the overlap rule of the argument check is off for that
// thread's calls: the hierarchical planner cuts user buffers into stage buffers that may legitimately overlap.
struct InternalCallScope {
  InternalCallScope();
  ~InternalCallScope();
};

// comm.cc
// stageOverride / userOverride: bytes of one staging half and of the flagcxMemAlloc area (0: FLAGCX_STAGE_BYTES /
// FLAGCX_HEAP_USER_BYTES times heapScale).
flagcxResult_t commCreate(flagcxComm **out, int nranks, const BootstrapHandle &h, int rank, double heapScale, unsigned flags,
                          size_t stageOverride = 0, size_t userOverride = 0);
flagcxResult_t commFree(flagcxComm *c);
flagcxResult_t commHeapRetain(flagcxComm *c);
flagcxResult_t commHeapRelease(flagcxComm *c, void *ptr);

}  // namespace fcx
