// Variant selection for the collective kernels.
//
// The reference's tuner searches NCCL environment knobs by tearing the NCCL
// communicator down and re-creating it per candidate, and times candidates
// with CUDA events on the caller's stream (flagcx/core/flagcx_tuner.cc:160-449,
// candidates in flagcx/adaptor/tuner/nccl_tuner.cc:5-16).  This one searches
// over the library's own kernel variants (kind x CTA count) with no
// communicator re-creation: a candidate is just different launch arguments.
//
//   * prior: an alpha-beta cost model (launch + barriers + NVLink bytes +
//     local HBM bytes), the counterpart of the reference's unused
//     flagcx/core/cost_model.cc, seeded with measured link/HBM rates;
//   * online search (FLAGCX_USE_TUNER=1): for each (op, size bucket) the first
//     nLoops x nCandidates calls cycle through the candidates, timed with
//     events; ranks then average their times over the bootstrap network and
//     adopt the fastest (with 5% hysteresis in favour of the prior's pick);
//   * persistence (FLAGCX_TUNER_CACHE=<file>): decisions are saved at
//     communicator destruction and loaded at creation;
//   * pinning (FLAGCX_USE_COMM_TAG="<kind>:<nctas>") forces one variant.
#pragma once
#include "bootstrap.h"
#include "flagcx.h"
#include "../kernels/devcomm.h"
#include <cuda_runtime_api.h>
#include <functional>
#include <map>
#include <string>
#include <vector>

namespace fcx {

struct Plan {
  int kind = 0;   // FcxKind
  int nctas = 1;
  unsigned int pipeBytes = 0;  // bytes a rank sends per pipeline sub-chunk of a staged kind (0: the communicator's setting)
};

struct TunerCaps {
  int nranks = 1;
  bool multicast = false;
  size_t stageBytes = 0;
  int maxCtas = 64;
  size_t pipeBytes = 0;  // bytes a rank sends per pipeline sub-chunk (0: 16 MiB)
};

// Estimated duration in microseconds of one launch (cost-model prior).
double estimateUs(const Plan &p, flagcxCommOp_t op, size_t bytes, int esize, const TunerCaps &caps);

const char *kindName(int kind);
int kindFromName(const std::string &s);

class Tuner {
 public:
  Tuner(Bootstrap *bs, const TunerCaps &caps);
  ~Tuner();

  // All variants that can legally run this call.
  // `zc`: every rank's buffers are peer-visible (symmetric heap or registered), so the zero-copy kinds may run.
  std::vector<Plan> candidates(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast,
                               bool zc = false) const;

  // Pick the plan for this call.  When the online search is active and the
  // returned `timed` is true the caller brackets the launch with
  // beginTiming/endTiming.
  // `maySearch` false (a stream that is being captured into a graph, for one) keeps the online search out of
  // this call: closing a timed call synchronises on an event, which a capture forbids.
  Plan choose(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast, bool *timed, bool zc = false,
              bool maySearch = true);
  void beginTiming(cudaStream_t s);
  void endTiming(cudaStream_t s);

  // Offline interface: record a measured time for a plan, adopt the best.
  void record(flagcxCommOp_t op, size_t bytes, const Plan &p, double us);
  // Upper bound on the CTAs of any plan handed out (0: none).  A caller that overlaps collectives with
  // compute kernels sets it so that a collective leaves most SMs to the compute stream.
  void setCtaBudget(int n) { budget_ = n > 0 ? n : 0; fast_.clear(); }
  int ctaBudget() const { return budget_; }
  flagcxResult_t load(const std::string &path);
  flagcxResult_t save(const std::string &path) const;
  std::string describe() const;  // one line per decided key

  bool searching() const { return search_; }
  // The plan that would run, without advancing the online search.
  Plan peek(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast, bool zc = false) const;
  double estimate(const Plan &p, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt) const;
  // Force one variant for every call it can legally serve; nullptr clears.
  void pin(const Plan *p);

 private:
  // Decisions are kept per (op, size bucket, zero-copy or staged).  A decision is only ever applied to a call
  // whose own candidate list holds its kind; the online search is keyed by the call's full signature `sig`
  // (element type, reduction, cast) as well, because the candidate list depends on all of them.
  struct Key {
    int op, log2b, zc, sig;
    bool operator<(const Key &o) const {
      if (op != o.op) return op < o.op;
      if (log2b != o.log2b) return log2b < o.log2b;
      if (zc != o.zc) return zc < o.zc;
      return sig < o.sig;
    }
  };
  struct Search {
    std::vector<Plan> cands;
    std::vector<double> sumUs;
    std::vector<int> nSamples;
    long calls = 0;
    bool decided = false;
  };
  static int bucket(size_t bytes);
  void decide(const Key &k, Search &s);
  bool lookup(const Key &k, const std::function<bool(const Plan &)> &legal, Plan *out) const;

  Bootstrap *bs_;
  TunerCaps caps_;
  bool search_ = false;
  int nLoops_ = 5;
  bool pinned_ = false;
  Plan pin_;
  int budget_ = 0;
  Plan clamp(Plan p) const { if (budget_ > 0 && p.nctas > budget_) p.nctas = budget_; return p; }
  // decisions of earlier calls, keyed by everything that can change the answer
  std::map<uint64_t, Plan> fast_;
  std::map<Key, Plan> best_;
  std::map<Key, double> bestUs_;
  std::map<Key, Search> searches_;
  // timing state of the call in flight
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
  Search *cur_ = nullptr;
  int curIdx_ = -1;
  Key curKey_{};
};

}  // namespace fcx
