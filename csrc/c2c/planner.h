// Cross-cluster ("C2C") hierarchical collectives.
//
// When a communicator spans more than one cluster (different vendors in the
// reference; here the box cut into sub-clusters by FLAGCX_CLUSTER_SPLIT_LIST)
// a collective runs as a plan of stages, exactly the structure of the
// reference's planner (flagcx/core/c2c_algo.h:198-270, c2c_algo.cc:610-2301):
//
//   RefreshFunc         zero the parts of a buffer this rank does not own
//   PreHomoFuncSteps    collectives inside each cluster
//   HeteroFuncSteps     point-to-point lists between clusters
//   HomoInterFuncSteps  collectives among the ranks that hold the same local
//                       index in every cluster (the "inter" communicator)
//   PostHomoFuncSteps   collectives inside each cluster
//
// The plan is data (struct C2cPlan) and can be written to / read from the same
// per-rank XML files as the reference (flagcx/core/c2c_ir.h:1-178), which is
// what the InterOp DSL (flagcx_b200/tools) emits.  What differs is execution:
// every stage is enqueued on the caller's stream as this library's own
// kernels over sub-communicators, with no host synchronisation between stages
// (the reference synchronises the stream three to six times per call), and the
// pipelined algorithm overlaps the inter-cluster stage of one piece with the
// intra-cluster stage of the next on a second stream joined by events.
#pragma once
#include "../core/comm.h"

#include <list>
#include <string>
#include <vector>

namespace fcx {

struct C2cHomoFunc {
  int rootRank = -1;   // -1: the call's root
  int sendType = 0;    // 0 user send buffer, 1 user receive buffer, 2 scratch
  int recvType = 1;    // 1 user receive buffer, 2 scratch
  size_t sendOffset = 0, recvOffset = 0, count = 0;  // elements
  int homoType = 0;    // 0 pre (intra), 1 inter, 2 post (intra)
  int commOp = flagcxCommNoOp;
};

struct C2cP2pOp {
  int rank = 0, peerRank = 0;
  size_t offset = 0, count = 0;  // elements, relative to the buffer named by buffType
  int isRecv = 0;
  int buffType = 1;              // 0 user send buffer, 1 user receive buffer (the reference's only choice), 2 scratch
};

struct C2cHeteroFunc {
  std::vector<C2cP2pOp> p2pOps;
};

struct C2cRefreshFunc {
  int buffType = -1;  // -1 none, 1 receive buffer, 2 scratch
  size_t start = 0, offset = 0, count = 0, totalCount = 0;
  int redOp = flagcxSum;
};

struct C2cPlan {
  size_t nChunks = 1;       // offsets in the XML are in units of totalCount / nChunks
  size_t totalCount = 0;    // elements that nChunks refers to
  int nSeqPreSteps = 0, nPipePreSteps = 0, nSeqInterSteps = 0, nPipePostSteps = 0, nSeqPostSteps = 0;
  C2cRefreshFunc refresh;
  std::vector<std::vector<C2cHomoFunc>> preHomoFuncSteps, homoInterFuncSteps, postHomoFuncSteps;
  std::vector<std::vector<C2cHeteroFunc>> heteroFuncSteps;
  size_t scratchCount = 0;  // elements of scratch the plan needs
  bool pipelined = false;   // overlap inter stage of piece i with pre stage of piece i+1
};

flagcxResult_t c2cExportXml(const C2cPlan &p, const std::string &prefix, int rank);
flagcxResult_t c2cImportXml(C2cPlan *p, const std::string &prefix, int rank, size_t totalCount);

// File name component used by FLAGCX_ALGO_EXPORT_PATH / FLAGCX_ALGO_IMPORT_PATH.
size_t c2cAlgoHash(size_t sendCount, size_t recvCount, size_t rootCluster, int commOp, int redOp);

// Build the default plan of a collective for a communicator of nclusters x clusterSize ranks.
// Returns false when the operation is not planned hierarchically (the caller runs it flat).
// interRanks: how many ranks of a cluster talk to the other clusters - the reference's three modes: 1 = one
// network port per cluster ("single NIC"), k dividing clusterSize = several ("multi NIC"), clusterSize = every
// rank has its own ("each NIC per rank", the natural mode inside one NVSwitch domain).  The inter ranks are
// the local indices 0 .. interRanks-1.  heteroP2p: move data between clusters with point-to-point lists on the
// world communicator (the reference's hetero stage) instead of collectives on the inter communicator, where
// the operation allows it (no reduction across clusters).  tables: all-to-all-v counts and displacements
// (scounts, sdispls, rcounts, rdispls; nranks entries each), else null.
bool c2cBuildPlan(C2cPlan *p, flagcxCommOp_t op, size_t count, int root, int nclusters, int clusterSize, int myCluster,
                  int myLocal, bool pipelined, int interRanks = 0, bool heteroP2p = false, const size_t *tables = nullptr);

class C2cState {
 public:
  flagcxComm *intra = nullptr, *inter = nullptr;
  int clusterSize = 0, myLocal = 0;
  int interRanks = 0;       // ranks per cluster that talk across clusters (see c2cBuildPlan)
  bool heteroP2p = false;   // cross-cluster stage as point-to-point lists where the operation allows it
  bool ready = false, unusable = false;
  void *scratch = nullptr;
  size_t scratchBytes = 0;
  cudaStream_t sideStream = nullptr;
  cudaEvent_t evA = nullptr, evB = nullptr;
  std::vector<cudaEvent_t> pieceEvents;  // two per pipeline piece
  struct Cached {
    size_t key;
    C2cPlan plan;
  };
  std::list<Cached> cache;  // most recent first, at most 16 entries like the reference (flagcx/flagcx.cc:24-26)
};

}  // namespace fcx
