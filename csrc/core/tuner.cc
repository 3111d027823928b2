#include "tuner.h"
#include "hosttypes.h"
#include "log.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <sstream>

namespace fcx {

// The copy-engine form of the movers has passed its multi-GPU test on two GPUs only: from three ranks on the tuner offers
// it (and accepts it from a measured table) when FLAGCX_COPY_ENGINE=1; a pinned plan still reaches it.
static bool ceOffered(int n) {
  static const bool on = envInt("COPY_ENGINE", 0) != 0;
  return n == 2 || (n > 2 && on);
}

static const char *kKindNames[FCX_K_NUM] = {"barrier", "ar_ll", "ar_oneshot", "ar_twoshot", "ar_nvls", "rs", "rs_nvls", "ag",
                                            "ag_nvls", "bcast", "reduce", "gather", "scatter", "a2a", "a2av", "move_ll", "rs_ll", "reduce_ll",
                                            "ar_zc", "rs_zc", "reduce_zc", "move_zc", "move_ce"};

const char *kindName(int kind) { return kind >= 0 && kind < FCX_K_NUM ? kKindNames[kind] : "?"; }

int kindFromName(const std::string &s) {
  for (int i = 0; i < FCX_K_NUM; i++)
    if (s == kKindNames[i]) return i;
  return -1;
}

// ------------------------------------------------------------------ cost model

// Rates in bytes per microsecond.  Link and HBM figures are the measured
// ones for this class of machine (peer copy ~770 GB/s per direction, device
// copy ~6.5 TB/s read+write); per-CTA figures bound what few CTAs can move.
namespace {
// Per-CTA figures come from a copy probe on two B200s: one CTA of 512 threads moves about 45 GB/s to a peer
// with plain loads and stores and sixteen CTAs saturate a direction of NVLink at about 685 GB/s, both
// directions at once; a CTA copies about 60 GB/s inside its own memory.  Large messages run as a software
// pipeline over sub-chunks in which about half of the CTAs are on the link and half on local memory.
constexpr double kLaunchUs = 2.2, kBarrierUs = 1.8, kLLUs = 1.6, kPipeBarrierUs = 0.4;
constexpr double kLinkRate = 680e3, kCtaPushRate = 40e3, kCtaMmRate = 3.5e3;  // multimem: 64-128 CTAs reached 430-490 GB/s on four GPUs
constexpr double kHbmRate = 5500e3, kCtaLocalRate = 60e3;

// Zero-copy kinds: a CTA keeps 8 switch reductions of 16 bytes per thread in flight (about 20 GB/s per CTA at
// the switch's round-trip time), pulls about 30 GB/s from peers with plain loads, and stores through the
// multicast alias at about the plain push rate.
constexpr double kCtaZcMmRate = 20e3, kCtaPullRate = 30e3;

double pushUs(double bytes, double nctas) { return bytes / std::min(kLinkRate, std::max(1.0, nctas) * kCtaPushRate); }
double mmUs(double bytes, double nctas) { return bytes / std::min(kLinkRate, std::max(1.0, nctas) * kCtaMmRate); }
double localUs(double bytes, double nctas) { return bytes / std::min(kHbmRate, std::max(1.0, nctas) * kCtaLocalRate); }

// A kind with `depth` phases that moves linkBytes over NVLink and localBytes inside the GPU, cut into
// sub-chunks of pipeBytes / (n-1) per piece.
double pipelinedUs(double linkBytes, double localBytes, double pieceBytes, int depth, bool mm, int c, const TunerCaps &caps) {
  const double n = caps.nranks, sub = std::max(16384.0, (double)(caps.pipeBytes ? caps.pipeBytes : (16u << 20)) / std::max(1.0, n - 1));
  const double chunks = std::max(1.0, std::ceil(pieceBytes / sub));
  auto link = [&](double ctas) { return mm ? mmUs(linkBytes, ctas) : pushUs(linkBytes, ctas); };
  if (chunks <= 1.0) return kLaunchUs + (depth - 1) * kBarrierUs + link(c) + localUs(localBytes, c);
  const double l = link(c * 0.5), h = localUs(localBytes, c * 0.5);
  return kLaunchUs + kBarrierUs + (chunks + depth - 2) * kPipeBarrierUs + std::max(l, h) + (link(c) + localUs(localBytes, c)) / chunks;
}
}  // namespace

double estimateUs(const Plan &p, flagcxCommOp_t op, size_t bytesIn, int, const TunerCaps &caps) {
  const double b = (double)bytesIn, n = caps.nranks;
  const int c = p.nctas;
  const bool mc = caps.multicast && caps.nranks > 2;  // with two ranks the zero-copy kinds use plain loads and stores
  const double zcFixed = kLaunchUs + 2 * kBarrierUs;
  switch (p.kind) {
    // zero-copy kinds: two barriers, one pass; bound by the link or by what `c` CTAs keep in flight
    case FCX_K_AR_ZC:
      if (mc) return zcFixed + std::max(b * (1 + 1 / n) / kLinkRate, b / n / (c * kCtaZcMmRate));
      return zcFixed + std::max(b * (n - 1) / n / kLinkRate, b * (n - 1) / n / (c * kCtaPullRate));
    case FCX_K_RS_ZC:  // b: per-rank piece
      if (mc) return zcFixed + std::max(b * (n - 1) / kLinkRate, b / (c * kCtaZcMmRate));
      return zcFixed + std::max(b * (n - 1) / kLinkRate, b * (n - 1) / (c * kCtaPullRate));
    case FCX_K_REDUCE_ZC:
      if (mc) return zcFixed + std::max(b / kLinkRate, b / (c * kCtaZcMmRate));
      return zcFixed + std::max(b * (n - 1) / kLinkRate, b * (n - 1) / (c * kCtaPullRate));
    case FCX_K_MOVE_CE: {
      // two one-CTA kernels around copy-engine transfers queued by the host: a few microseconds per copy to
      // start, then the link rate; no SM moves data
      const double copies = (op == flagcxCommOpBroadcast || op == flagcxCommOpScatter) ? n - 1 : n;
      return 2 * kLaunchUs + 2 * kBarrierUs + 4.0 * copies + b * (n - 1) / kLinkRate;
    }
    case FCX_K_MOVE_ZC:
      switch (op) {
        case flagcxCommOpBroadcast:
          return zcFixed + (mc ? std::max(b / kLinkRate, b / (c * kCtaPushRate)) : std::max(b * (n - 1) / kLinkRate, b * (n - 1) / (c * kCtaPushRate)));
        case flagcxCommOpAllGather:
          return zcFixed + std::max(b * (n - 1) / kLinkRate, (mc ? b : b * (n - 1)) / (c * kCtaPushRate));
        case flagcxCommOpGather:
        case flagcxCommOpAlltoAllv:
          return zcFixed + std::max(b * (n - 1) / kLinkRate, b * (n - 1) / (c * kCtaPullRate));
        default:
          return zcFixed + std::max(b * (n - 1) / kLinkRate, b * (n - 1) / (c * kCtaPushRate));
      }
    case FCX_K_BARRIER: return kLaunchUs + kBarrierUs;
    case FCX_K_AR_LL: return kLaunchUs + kLLUs + pushUs(2 * (n - 1) * b, c) + localUs(2 * n * b, c);
    case FCX_K_AR_ONESHOT: return kLaunchUs + kBarrierUs + pushUs((n - 1) * b, c) + localUs((n + 1) * b, c);
    case FCX_K_AR_TWOSHOT: return pipelinedUs(2 * (n - 1) / n * b, 4 * b, b / n, 3, false, c, caps);
    case FCX_K_AR_NVLS: return pipelinedUs(2 * b / n, 4 * b, b / n, 3, true, c, caps);
    case FCX_K_REDUCE: return pipelinedUs(2 * (n - 1) / n * b, 3 * b, b / n, 3, false, c, caps);
    // below, b is the per-rank piece
    case FCX_K_RS: return pipelinedUs((n - 1) * b, (n + 1) * b, b, 2, false, c, caps);
    case FCX_K_RS_NVLS: return pipelinedUs(b, 2 * n * b, b, 2, true, c, caps);
    case FCX_K_AG: return pipelinedUs((n - 1) * b, 2 * n * b, b, 2, false, c, caps);
    case FCX_K_AG_NVLS: return pipelinedUs(b, 2 * n * b, b, 2, true, c, caps);
    case FCX_K_BCAST: return pipelinedUs(caps.multicast ? b : (n - 1) * b, 2 * b, b, 2, caps.multicast, c, caps);
    case FCX_K_GATHER:
    case FCX_K_SCATTER: return pipelinedUs((n - 1) * b, 2 * b, b, 2, false, c, caps);
    case FCX_K_A2A: return pipelinedUs((n - 1) * b, 2 * n * b, b, 2, false, c, caps);
    case FCX_K_A2AV: return kLaunchUs + 2 * kBarrierUs + pushUs((n - 1) * b, c) + localUs(2 * n * b, c);
    // LL forms (b: per-rank piece, whole vector for reduce): every payload byte travels with a flag byte, no barrier
    case FCX_K_MOVE_LL:
    case FCX_K_RS_LL: return kLaunchUs + kLLUs + pushUs(2 * (n - 1) * b, c) + localUs(2 * n * b, c);
    case FCX_K_REDUCE_LL: return kLaunchUs + kLLUs + pushUs(2 * b, c) + localUs(2 * n * b, c);
    default: return 1e9;
  }
}

// ------------------------------------------------------------------ tuner

Tuner::Tuner(Bootstrap *bs, const TunerCaps &caps) : bs_(bs), caps_(caps) {
  search_ = envInt("USE_TUNER", 0) != 0;
  nLoops_ = (int)envInt("TUNER_SEARCH_NLOOPS", 5);
  std::string tag = envStr("USE_COMM_TAG", "");
  if (!tag.empty()) {
    size_t c = tag.find(':');
    int k = kindFromName(tag.substr(0, c));
    if (k >= 0) {
      pinned_ = true;
      pin_.kind = k;
      pin_.nctas = c == std::string::npos ? 16 : std::max(1, atoi(tag.c_str() + c + 1));
    } else {
      FCX_WARN("FLAGCX_USE_COMM_TAG='%s' names no kernel variant", tag.c_str());
    }
  }
  std::string cache = envStr("TUNER_CACHE", "");
  if (!cache.empty()) load(cache);
}

Tuner::~Tuner() {
  if (ev0_) cudaEventDestroy(ev0_);
  if (ev1_) cudaEventDestroy(ev1_);
}

int Tuner::bucket(size_t bytes) {
  int l = 0;
  while (((size_t)1 << l) < bytes && l < 62) l++;
  return l;
}

static void addCtas(std::vector<Plan> &out, int kind, std::initializer_list<int> cs, size_t units, int maxCtas) {
  int cap = (int)std::min<size_t>((units + 511) / 512, (size_t)maxCtas);
  cap = std::max(cap, 1);
  int last = -1;
  for (int c : cs) {
    int cc = std::min(c, cap);
    if (cc != last) out.push_back({kind, cc});
    last = cc;
  }
}

std::vector<Plan> Tuner::candidates(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast, bool zc) const {
  std::vector<Plan> out;
  const int n = caps_.nranks;
  const size_t units = (bytes + 15) / 16;
  const int mx = caps_.maxCtas;
  const bool mmType = dt == flagcxFloat32 || dt == flagcxBfloat16 || dt == flagcxFloat16;
  const bool mmOp = dt == flagcxFloat32 ? (red == flagcxSum || red == flagcxAvg) : (red != flagcxProd);
  const bool nvls = caps_.multicast && mmType && mmOp && !cast && n > 1;
  switch (op) {
    case flagcxCommOpAllReduce:
      if (!cast && bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_AR_LL, {1, 2, 4}, units, mx);
      if ((bytes + 64) * n <= caps_.stageBytes && bytes <= (8u << 20)) addCtas(out, FCX_K_AR_ONESHOT, {2, 8, 16, 32, 64}, units, mx);
      if (bytes > 2048 || out.empty()) addCtas(out, FCX_K_AR_TWOSHOT, {8, 16, 32, 64, 128}, units / n + 1, mx);
      if (nvls && bytes >= 4096) addCtas(out, FCX_K_AR_NVLS, {8, 16, 32, 64, 128}, units / n + 1, mx);
      if (zc && n > 1) addCtas(out, FCX_K_AR_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units / n + 1, mx);
      break;
    case flagcxCommOpReduceScatter:
      if (!cast && bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_RS_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_RS, {2, 8, 16, 32, 64, 128}, units, mx);
      if (nvls && bytes >= 4096) addCtas(out, FCX_K_RS_NVLS, {8, 16, 32, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_RS_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      break;
    case flagcxCommOpAllGather:
      if (bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_MOVE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_AG, {2, 8, 16, 32, 64, 128}, units, mx);
      if (caps_.multicast && n > 1 && bytes >= 4096) addCtas(out, FCX_K_AG_NVLS, {8, 16, 32, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      if (zc && ceOffered(n) && bytes >= (256u << 10)) out.push_back({FCX_K_MOVE_CE, 1});
      break;
    case flagcxCommOpReduce:
      if (!cast && bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_REDUCE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_REDUCE, {2, 8, 16, 32, 64, 128}, units / n + 1, mx);
      if (zc && n > 1 && nvls) addCtas(out, FCX_K_REDUCE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      break;
    case flagcxCommOpBroadcast:
      if (bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_MOVE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_BCAST, {1, 4, 16, 32, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      if (zc && ceOffered(n) && bytes >= (256u << 10)) out.push_back({FCX_K_MOVE_CE, 1});
      break;
    case flagcxCommOpGather:
      if (bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_MOVE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_GATHER, {1, 4, 16, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      break;
    case flagcxCommOpScatter:
      if (bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_MOVE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_SCATTER, {1, 4, 16, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      if (zc && ceOffered(n) && bytes >= (256u << 10)) out.push_back({FCX_K_MOVE_CE, 1});
      break;
    case flagcxCommOpAlltoAll:
      if (bytes <= FCX_LL_MAX_PAYLOAD) addCtas(out, FCX_K_MOVE_LL, {1, 2, 4}, units, mx);
      addCtas(out, FCX_K_A2A, {2, 8, 16, 32, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {1, 2, 4, 8, 16, 24, 32, 48, 64, 96}, units, mx);
      if (zc && ceOffered(n) && bytes >= (256u << 10)) out.push_back({FCX_K_MOVE_CE, 1});
      break;
    case flagcxCommOpAlltoAllv:
      addCtas(out, FCX_K_A2AV, {2, 8, 16, 32, 64, 128}, units, mx);
      if (zc && n > 1) addCtas(out, FCX_K_MOVE_ZC, {8, 16, 32, 64}, units, mx);
      break;
    default: out.push_back({FCX_K_BARRIER, 1}); break;
  }
  return out;
}

// The decision for a call: the entry of its exact signature, else the generic entry of its bucket.  A call
// that may run zero-copy also looks at the staged table of the bucket and takes the faster of the two, since a
// staged kind serves peer-visible buffers just as well.
bool Tuner::lookup(const Key &k, const std::function<bool(const Plan &)> &legalIn, Plan *out) const {
  // Under a CTA budget a decision that was measured with more CTAs than the budget allows says nothing about
  // the clamped launch (a staged kind that wins with 128 CTAs loses badly with 16): such entries are skipped and
  // the cost model, evaluated at the budget, decides.
  auto legal = [&](const Plan &p) { return legalIn(p) && (budget_ <= 0 || p.nctas <= budget_); };
  auto it = best_.find(k);
  if (it != best_.end() && legal(it->second)) { *out = it->second; return true; }
  bool have = false;
  double bestUs = 0;
  for (int zc = k.zc; zc >= 0; zc--) {
    const Key g{k.op, k.log2b, zc, -1};
    auto b = best_.find(g);
    if (b == best_.end() || !legal(b->second)) continue;
    auto u = bestUs_.find(g);
    const double us = u == bestUs_.end() ? 0.0 : u->second;
    if (!have || us < bestUs) { *out = b->second; bestUs = us; have = true; }
  }
  return have;
}

static int sigOf(flagcxDataType_t dt, flagcxRedOp_t red, bool cast) { return ((int)dt << 8) | ((int)red << 4) | (cast ? 1 : 0); }

void Tuner::decide(const Key &k, Search &s) {
  // Average every candidate's mean time over the ranks, then take the minimum.
  const int nc = (int)s.cands.size(), n = bs_ ? bs_->nranks() : 1;
  std::vector<double> all((size_t)n * nc, 0.0);
  int me = bs_ ? bs_->rank() : 0;
  for (int i = 0; i < nc; i++) all[(size_t)me * nc + i] = s.nSamples[i] ? s.sumUs[i] / s.nSamples[i] : 1e12;
  if (bs_ && n > 1) bs_->allGather(all.data(), nc * sizeof(double));
  std::vector<double> mean(nc, 0.0);
  for (int r = 0; r < n; r++)
    for (int i = 0; i < nc; i++) mean[i] += all[(size_t)r * nc + i] / n;
  int bestI = 0;  // candidate 0 is the prior's pick (candidates are sorted by the cost model)
  for (int i = 1; i < nc; i++)
    if (mean[i] < mean[bestI] * 0.95) bestI = i;
  best_[k] = s.cands[bestI];
  bestUs_[k] = mean[bestI];
  // the same answer serves calls of other signatures in this bucket as long as their own candidate list holds it
  Key generic{k.op, k.log2b, k.zc, -1};
  if (!best_.count(generic)) { best_[generic] = s.cands[bestI]; bestUs_[generic] = mean[bestI]; }
  s.decided = true;
  FCX_INFO(SUB_TUNING, "tuner: op %d, <=2^%d bytes%s -> %s with %d CTAs (%.2f us)", k.op, k.log2b, k.zc ? " (zero-copy)" : "",
           kindName(s.cands[bestI].kind), s.cands[bestI].nctas, mean[bestI]);
}

Plan Tuner::choose(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast, bool *timed, bool zc,
                   bool maySearch) {
  if (timed) *timed = false;
  // FLAGCX_FORCE_CTAS overrides the CTA count of whatever variant is chosen (for experiments)
  static const int forceCtas = (int)envInt("FORCE_CTAS", 0);
  if (forceCtas > 0) {
    Plan p = peek(op, bytes, dt, red, cast, zc);
    p.nctas = forceCtas;
    return p;
  }
  // Close the timing of the previous searched call.
  if (cur_ && maySearch) {
    cudaEventSynchronize(ev1_);
    float ms = 0;
    if (cudaEventElapsedTime(&ms, ev0_, ev1_) == cudaSuccess) {
      cur_->sumUs[curIdx_] += ms * 1e3;
      cur_->nSamples[curIdx_]++;
    }
    cudaGetLastError();
    Search *s = cur_;
    cur_ = nullptr;
    if (!s->decided && s->calls >= (long)nLoops_ * (long)s->cands.size()) decide(curKey_, *s);
  }
  const bool searching = search_ && maySearch;
  // Hot path: the answer for this exact (op, bytes, type, reduction, cast, zero-copy) was computed before.
  const uint64_t fkey = ((uint64_t)bytes << 16) ^ ((uint64_t)op << 12) ^ ((uint64_t)dt << 8) ^ ((uint64_t)red << 4) ^ (cast ? 1u : 0u) ^
                        (zc ? 2u : 0u) ^ ((uint64_t)bucket(bytes) << 56);
  if (!searching) {
    auto f = fast_.find(fkey);
    if (f != fast_.end()) return f->second;
  }
  std::vector<Plan> cands = candidates(op, bytes, dt, red, cast, zc);
  auto legal = [&](const Plan &p) {
    for (auto &c : cands)
      if (c.kind == p.kind) return true;
    return false;
  };
  auto remember = [&](Plan p) {
    p = clamp(p);
    if (!searching && !pinned_ && fast_.size() < 4096) fast_[fkey] = p;
    return p;
  };
  if (pinned_ && legal(pin_)) return clamp(pin_);
  const Key k{(int)op, bucket(bytes), zc ? 1 : 0, sigOf(dt, red, cast)};
  {
    Plan found;
    if (lookup(k, legal, &found)) return remember(found);
  }
  // order by the prior
  std::sort(cands.begin(), cands.end(), [&](const Plan &a, const Plan &b) {
    return estimateUs(clamp(a), op, bytes, (int)dtypeSize(dt), caps_) < estimateUs(clamp(b), op, bytes, (int)dtypeSize(dt), caps_);
  });
  if (!searching || cands.size() < 2) return remember(cands[0]);
  Search &s = searches_[k];  // keyed by the full signature: every candidate in it is legal for this call
  if (s.cands.empty()) {
    s.cands = cands;
    s.sumUs.assign(cands.size(), 0.0);
    s.nSamples.assign(cands.size(), 0);
  }
  if (s.decided) {
    auto it = best_.find(k);
    return clamp(it != best_.end() && legal(it->second) ? it->second : cands[0]);
  }
  int idx = (int)(s.calls % (long)s.cands.size());
  s.calls++;
  cur_ = &s;
  curIdx_ = idx;
  curKey_ = k;
  if (timed) *timed = true;
  return clamp(s.cands[idx]);
}

Plan Tuner::peek(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red, bool cast, bool zc) const {
  std::vector<Plan> cands = candidates(op, bytes, dt, red, cast, zc);
  auto legal = [&](const Plan &p) {
    for (auto &c : cands)
      if (c.kind == p.kind) return true;
    return false;
  };
  if (pinned_ && legal(pin_)) return clamp(pin_);
  const Key k{(int)op, bucket(bytes), zc ? 1 : 0, sigOf(dt, red, cast)};
  {
    Plan found;
    if (lookup(k, legal, &found)) return clamp(found);
  }
  Plan best = cands[0];
  double bestUs = 1e30;
  for (auto &c : cands) {
    double us = estimateUs(clamp(c), op, bytes, (int)dtypeSize(dt), caps_);
    if (us < bestUs) { bestUs = us; best = c; }
  }
  return clamp(best);
}

double Tuner::estimate(const Plan &p, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt) const {
  return estimateUs(p, op, bytes, (int)dtypeSize(dt), caps_);
}

void Tuner::pin(const Plan *p) {
  fast_.clear();
  pinned_ = p != nullptr;
  if (p) pin_ = *p;
}

void Tuner::beginTiming(cudaStream_t st) {
  if (!ev0_) { cudaEventCreate(&ev0_); cudaEventCreate(&ev1_); }
  cudaEventRecord(ev0_, st);
}

void Tuner::endTiming(cudaStream_t st) { cudaEventRecord(ev1_, st); }

static bool isZcKind(int k) { return k == FCX_K_AR_ZC || k == FCX_K_RS_ZC || k == FCX_K_REDUCE_ZC || k == FCX_K_MOVE_ZC || k == FCX_K_MOVE_CE; }

void Tuner::record(flagcxCommOp_t op, size_t bytes, const Plan &p, double us) {
  Key k{(int)op, bucket(bytes), isZcKind(p.kind) ? 1 : 0, -1};
  auto it = bestUs_.find(k);
  if (it == bestUs_.end() || us < it->second) {
    best_[k] = p;
    bestUs_[k] = us;
    fast_.clear();
  }
}

flagcxResult_t Tuner::load(const std::string &path) {
  FILE *f = fopen(path.c_str(), "r");
  if (!f) return flagcxSystemError;
  char line[512];
  int loaded = 0;
  while (fgets(line, sizeof line, f)) {
    int op, l2, nr, nctas;
    char kind[64];
    double us;
    if (sscanf(line, " {\"op\": %d, \"log2_bytes\": %d, \"nranks\": %d, \"kind\": \"%63[^\"]\", \"nctas\": %d, \"us\": %lf", &op, &l2,
               &nr, kind, &nctas, &us) == 6) {
      int k = kindFromName(kind);
      if (nr != caps_.nranks || k < 0) continue;
      if (k == FCX_K_MOVE_CE && !ceOffered(caps_.nranks)) continue;
      if ((k == FCX_K_AR_NVLS || k == FCX_K_RS_NVLS || k == FCX_K_AG_NVLS) && !caps_.multicast) continue;
      Key key{op, l2, isZcKind(k) ? 1 : 0, -1};
      unsigned int pipe = 0;
      if (const char *pb = strstr(line, "\"pipe_bytes\":")) pipe = (unsigned int)strtoul(pb + 13, nullptr, 10);
      best_[key] = {k, nctas, pipe};
      bestUs_[key] = us;
      loaded++;
    }
  }
  fclose(f);
  fast_.clear();
  FCX_INFO(SUB_TUNING, "tuner: loaded %d decisions from %s", loaded, path.c_str());
  return flagcxSuccess;
}

flagcxResult_t Tuner::save(const std::string &path) const {
  FILE *f = fopen(path.c_str(), "w");
  if (!f) return flagcxSystemError;
  fprintf(f, "[\n");
  bool first = true;
  for (auto &kv : best_) {
    if (kv.first.sig != -1) continue;  // the per-signature entries live for the process only
    auto us = bestUs_.find(kv.first);
    fprintf(f, "%s {\"op\": %d, \"log2_bytes\": %d, \"nranks\": %d, \"kind\": \"%s\", \"nctas\": %d, \"us\": %.3f", first ? "" : ",\n",
            kv.first.op, kv.first.log2b, caps_.nranks, kindName(kv.second.kind), kv.second.nctas, us == bestUs_.end() ? 0.0 : us->second);
    if (kv.second.pipeBytes) fprintf(f, ", \"pipe_bytes\": %u", kv.second.pipeBytes);
    fprintf(f, "}");
    first = false;
  }
  fprintf(f, "\n]\n");
  fclose(f);
  return flagcxSuccess;
}

std::string Tuner::describe() const {
  std::ostringstream os;
  for (auto &kv : best_)
    if (kv.first.sig == -1)
      os << "op " << kv.first.op << " <=2^" << kv.first.log2b << " B" << (kv.first.zc ? " zc" : "") << ": " << kindName(kv.second.kind) << " x"
         << kv.second.nctas << "\n";
  return os.str();
}

}  // namespace fcx
