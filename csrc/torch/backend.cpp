// PyTorch ProcessGroup backend "flagcx" on top of the C API.
//
// Same override set as the reference plugin
// (plugin/torch/flagcx/include/backend_flagcx.hpp:75-172,
// plugin/torch/flagcx/src/backend_flagcx.cpp) plus allreduce_coalesced, the
// coalesced all-gather / reduce-scatter forms and a real time-out.  What is
// different underneath:
//   * CUDA tensors run on an internal high-priority stream ordered after the
//     caller's current stream by an event; Work::wait() orders the caller's
//     stream after the collective (no host blocking);
//   * every tensor that an operation touches is recorded on the internal
//     stream with the caching allocator, so it cannot be recycled while the
//     kernel still runs (the reference leaves this as a TODO, :378-379);
//   * CPU tensors are served too, by the library's TCP host path, so the one
//     backend can be registered for both device types;
//   * Work::wait(timeout) polls the event and the communicator's async error,
//     and turns a device-side time-out into an exception instead of a hang.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Utils.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include <chrono>
#include <memory>
#include <thread>

#include "flagcx.h"
#include "flagcx_ext.h"

namespace fcxt {

#define FCX_TORCH_CHECK(call)                                                                        \
  do {                                                                                               \
    flagcxResult_t _r = (call);                                                                      \
    TORCH_CHECK(_r == flagcxSuccess, "flagcx: ", flagcxGetErrorString(_r), " (", #call, "): ",       \
                flagcxGetLastError(nullptr));                                                        \
  } while (0)

struct flagcxStreamLayout { cudaStream_t base; };  // same layout as the library's flagcxStream

static flagcxDataType_t toDtype(at::ScalarType t) {
  switch (t) {
    case at::kChar: return flagcxInt8;
    case at::kByte: return flagcxUint8;
    case at::kBool: return flagcxUint8;
    case at::kInt: return flagcxInt32;
    case at::kLong: return flagcxInt64;
    case at::kHalf: return flagcxFloat16;
    case at::kFloat: return flagcxFloat32;
    case at::kDouble: return flagcxFloat64;
    case at::kBFloat16: return flagcxBfloat16;
    case at::kFloat8_e4m3fn: return flagcxFloat8e4m3;
    case at::kFloat8_e5m2: return flagcxFloat8e5m2;
    case at::kUInt32: return flagcxUint32;
    case at::kUInt64: return flagcxUint64;
    default: TORCH_CHECK(false, "flagcx: unsupported tensor dtype ", t);
  }
}

static flagcxRedOp_t toRedOp(const c10d::ReduceOp &op, at::ScalarType t) {
  switch (op) {
    case c10d::ReduceOp::SUM: return t == at::kBool ? flagcxMax : flagcxSum;  // logical or
    case c10d::ReduceOp::PRODUCT: return t == at::kBool ? flagcxMin : flagcxProd;
    case c10d::ReduceOp::MIN: return flagcxMin;
    case c10d::ReduceOp::MAX: return flagcxMax;
    case c10d::ReduceOp::AVG: return flagcxAvg;
    default: TORCH_CHECK(false, "flagcx: unsupported reduce op");
  }
}

class FlagcxWork : public c10d::Work {
 public:
  FlagcxWork(c10d::OpType op, int rank, flagcxComm_t comm, bool cuda, c10::DeviceIndex dev, std::chrono::milliseconds timeout)
      : c10d::Work(rank, op), comm_(comm), cuda_(cuda), timeout_(timeout) {
    if (cuda_) {
      event_ = std::make_unique<at::cuda::CUDAEvent>(cudaEventDisableTiming);
      dev_ = dev;
    }
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                       cuda_ ? std::vector<c10::Device>{c10::Device(c10::kCUDA, dev)}
                                                             : std::vector<c10::Device>{});
  }

  void record(const c10::cuda::CUDAStream &s) { event_->record(s); }
  void stash(const std::vector<at::Tensor> &ts) { stashed_.insert(stashed_.end(), ts.begin(), ts.end()); }
  void setOutputs(std::vector<at::Tensor> outs) { outputs_ = std::move(outs); }
  void markBarrier() { barrier_ = true; }
  void finishHost() {
    future_->markCompleted(c10::IValue(outputs_));
    done_ = true;
  }
  void finishCudaEnqueue(const c10::cuda::CUDAStream &s) {
    // A device-aware future records its events on the streams that are current when it is completed, and
    // whoever waits on it synchronises with those events: the communication stream must be current here.
    c10::cuda::CUDAStreamGuard g(s);
    future_->markCompleted(c10::IValue(outputs_));
  }

  bool isCompleted() override {
    if (!cuda_) return done_;
    return event_->query();
  }
  bool isSuccess() const override { return true; }

  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override {
    if (!cuda_) return true;
    auto cur = c10::cuda::getCurrentCUDAStream(dev_);
    event_->block(cur);
    if (barrier_ || timeout != kNoTimeout) {
      // host-blocking forms: poll, so that a device-side give-up or the deadline surface as an error
      auto limit = timeout != kNoTimeout ? timeout : timeout_;
      auto t0 = std::chrono::steady_clock::now();
      while (!event_->query()) {
        flagcxResult_t async = flagcxSuccess;
        flagcxCommGetAsyncError(comm_, &async);
        TORCH_CHECK(async == flagcxSuccess, "flagcx: a device wait gave up (peer missing or too slow)");
        if (limit.count() > 0 && std::chrono::steady_clock::now() - t0 > limit)
          TORCH_CHECK(false, "flagcx: operation timed out after ", limit.count(), " ms");
        std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
    }
    stashed_.clear();
    return true;
  }
  void synchronize() override { wait(); }
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
  flagcxComm_t comm_;
  bool cuda_, done_ = false, barrier_ = false;
  c10::DeviceIndex dev_ = 0;
  std::unique_ptr<at::cuda::CUDAEvent> event_;
  std::vector<at::Tensor> stashed_, outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  std::chrono::milliseconds timeout_;
};

class FlagcxBackend : public c10d::Backend {
 public:
  FlagcxBackend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, std::chrono::milliseconds timeout)
      : c10d::Backend(rank, size), store_(store), timeout_(timeout) {}

  ~FlagcxBackend() override {
    for (auto &kv : comms_)
      if (kv.second) flagcxCommDestroy(kv.second);
  }

  const std::string getBackendName() const override { return "flagcx"; }
  bool supportsCoalescing() const override { return true; }
  void setTimeout(std::chrono::milliseconds t) override { timeout_ = t; }

  // ---- communicator management: one per device type ("cpu" or "cuda:N"), created on first use
  flagcxComm_t comm(const at::Device &dev) {
    std::string key = dev.is_cuda() ? "cuda" : "cpu";
    auto it = comms_.find(key);
    if (it != comms_.end()) return it->second;
    c10::cuda::OptionalCUDAGuard guard;
    if (dev.is_cuda()) guard.set_device(dev);
    std::string storeKey = "flagcx/unique_id/" + key + "/" + std::to_string(commCounter_++);
    flagcxUniqueId id;
    if (getRank() == 0) {
      flagcxUniqueId_t p = &id;
      FCX_TORCH_CHECK(flagcxGetUniqueId(&p));
      std::vector<uint8_t> v((uint8_t *)id.internal, (uint8_t *)id.internal + FLAGCX_UNIQUE_ID_BYTES);
      store_->set(storeKey, v);
    } else {
      auto v = store_->get(storeKey);
      TORCH_CHECK(v.size() == FLAGCX_UNIQUE_ID_BYTES, "flagcx: bad unique id in the store");
      memcpy(id.internal, v.data(), FLAGCX_UNIQUE_ID_BYTES);
    }
    flagcxComm_t c = nullptr;
    flagcxResult_t r = flagcxCommInitRankEx(&c, getSize(), &id, getRank(), dev.is_cuda() ? 0u : FLAGCX_INIT_HOST_ONLY);
    FCX_TORCH_CHECK(r);
    flagcxCommSetTimeoutMs(c, (int)std::max<int64_t>(1000, timeout_.count()));
    // FLAGCX_TORCH_CTAS=n caps the CTAs of this backend's collectives: for trainers whose collectives overlap
    // compute (DistributedDataParallel's buckets during the backward pass)
    if (dev.is_cuda()) {
      if (const char *cap = getenv("FLAGCX_TORCH_CTAS")) {
        int n = atoi(cap);
        if (n > 0) flagcxCommSetCtaBudget(c, n);
      }
    }
    comms_[key] = c;
    if (dev.is_cuda()) {
      stream_ = std::make_unique<c10::cuda::CUDAStream>(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, dev.index()));
      wrapped_.base = stream_->stream();
    }
    return c;
  }

  flagcxStream_t fstream() { return reinterpret_cast<flagcxStream_t>(&wrapped_); }

  // Order the internal stream after the caller's stream.
  void syncStream(const at::Device &dev) {
    if (coalescing_ && syncedInGroup_) return;
    at::cuda::CUDAEvent ev(cudaEventDisableTiming);
    ev.record(c10::cuda::getCurrentCUDAStream(dev.index()));
    ev.block(*stream_);
    syncedInGroup_ = true;
  }

  template <typename F>
  c10::intrusive_ptr<c10d::Work> run(c10d::OpType type, const at::Device &dev, std::vector<at::Tensor> touched,
                                     std::vector<at::Tensor> outputs, F &&fn) {
    flagcxComm_t c = comm(dev);
    seq_++;
    auto work = c10::make_intrusive<FlagcxWork>(type, getRank(), c, dev.is_cuda(), dev.is_cuda() ? dev.index() : 0, timeout_);
    work->setOutputs(std::move(outputs));
    if (!dev.is_cuda()) {
      fn(c, nullptr);
      if (coalescing_) hostPending_.push_back(work);
      else work->finishHost();
      return work;
    }
    c10::cuda::CUDAGuard guard(dev);
    syncStream(dev);
    for (auto &t : touched)
      if (t.defined() && t.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *stream_);
    {
      c10::cuda::CUDAStreamGuard sg(*stream_);
      fn(c, fstream());
    }
    work->stash(touched);
    if (coalescing_) {
      cudaPending_.push_back(work);
      coalescedDev_ = dev;
    } else {
      work->record(*stream_);
      work->finishCudaEnqueue(*stream_);
    }
    return work;
  }

  static void checkSingle(const std::vector<at::Tensor> &ts) {
    TORCH_CHECK(ts.size() == 1, "flagcx: expected exactly one tensor, got ", ts.size());
    TORCH_CHECK(ts[0].is_contiguous(), "flagcx: tensors must be contiguous");
  }

  // ---- collectives
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor> &tensors, const c10d::BroadcastOptions &opts) override {
    checkSingle(tensors);
    auto t = tensors[0];
    int root = (int)opts.rootRank;
    return run(c10d::OpType::BROADCAST, t.device(), {t}, {t}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), toDtype(t.scalar_type()), root, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor> &tensors, const c10d::AllreduceOptions &opts) override {
    checkSingle(tensors);
    auto t = tensors[0];
    auto op = toRedOp(opts.reduceOp, t.scalar_type());
    return run(c10d::OpType::ALLREDUCE, t.device(), {t}, {t}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toDtype(t.scalar_type()), op, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor> &tensors,
                                                      const c10d::AllreduceCoalescedOptions &opts) override {
    TORCH_CHECK(!tensors.empty(), "flagcx: empty tensor list");
    auto ts = tensors;
    auto dev = ts[0].device();
    auto redop = opts.reduceOp;
    return run(c10d::OpType::ALLREDUCE_COALESCED, dev, ts, ts, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxGroupStart(c));
      for (auto &t : ts) {
        TORCH_CHECK(t.is_contiguous(), "flagcx: tensors must be contiguous");
        FCX_TORCH_CHECK(flagcxAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toDtype(t.scalar_type()),
                                        toRedOp(redop, t.scalar_type()), c, s));
      }
      FCX_TORCH_CHECK(flagcxGroupEnd(c));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor> &tensors, const c10d::ReduceOptions &opts) override {
    checkSingle(tensors);
    auto t = tensors[0];
    auto op = toRedOp(opts.reduceOp, t.scalar_type());
    int root = (int)opts.rootRank;
    return run(c10d::OpType::REDUCE, t.device(), {t}, {t}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxReduce(t.data_ptr(), t.data_ptr(), t.numel(), toDtype(t.scalar_type()), op, root, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor &out, at::Tensor &in, const c10d::AllgatherOptions &) override {
    TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "flagcx: tensors must be contiguous");
    TORCH_CHECK(out.numel() == in.numel() * getSize(), "flagcx: output must hold world_size inputs");
    auto o = out, i = in;
    return run(c10d::OpType::_ALLGATHER_BASE, in.device(), {i, o}, {o}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxAllGather(i.data_ptr(), o.data_ptr(), i.numel(), toDtype(i.scalar_type()), c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>> &outputs, std::vector<at::Tensor> &inputs,
                                           const c10d::AllgatherOptions &) override {
    checkSingle(inputs);
    TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == getSize(), "flagcx: need world_size output tensors");
    auto in = inputs[0];
    auto outs = outputs[0];
    auto flat = at::empty({getSize() * in.numel()}, in.options());
    std::vector<at::Tensor> touched = outs;
    touched.push_back(in);
    touched.push_back(flat);
    auto work = run(c10d::OpType::ALLGATHER, in.device(), touched, outs, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxAllGather(in.data_ptr(), flat.data_ptr(), in.numel(), toDtype(in.scalar_type()), c, s));
      scatterFlat(flat, outs, in.device());
    });
    return work;
  }

  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor> &outputs, std::vector<at::Tensor> &inputs,
                                                                  const c10d::AllgatherOptions &) override {
    TORCH_CHECK(outputs.size() == inputs.size() && !inputs.empty(), "flagcx: mismatched tensor lists");
    auto outs = outputs, ins = inputs;
    std::vector<at::Tensor> touched = outs;
    touched.insert(touched.end(), ins.begin(), ins.end());
    return run(c10d::OpType::COALESCED, ins[0].device(), touched, outs, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxGroupStart(c));
      for (size_t k = 0; k < ins.size(); k++)
        FCX_TORCH_CHECK(flagcxAllGather(ins[k].data_ptr(), outs[k].data_ptr(), ins[k].numel(), toDtype(ins[k].scalar_type()), c, s));
      FCX_TORCH_CHECK(flagcxGroupEnd(c));
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>> &outputLists,
                                                      std::vector<at::Tensor> &inputs, const c10d::AllgatherOptions &opts) override {
    c10::intrusive_ptr<c10d::Work> last;
    for (size_t k = 0; k < inputs.size(); k++) {
      std::vector<std::vector<at::Tensor>> o{outputLists[k]};
      std::vector<at::Tensor> i{inputs[k]};
      last = allgather(o, i, opts);
    }
    return last;
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor &out, at::Tensor &in, const c10d::ReduceScatterOptions &opts) override {
    TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "flagcx: tensors must be contiguous");
    TORCH_CHECK(in.numel() == out.numel() * getSize(), "flagcx: input must hold world_size outputs");
    auto o = out, i = in;
    auto op = toRedOp(opts.reduceOp, in.scalar_type());
    return run(c10d::OpType::_REDUCE_SCATTER_BASE, in.device(), {i, o}, {o}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxReduceScatter(i.data_ptr(), o.data_ptr(), o.numel(), toDtype(i.scalar_type()), op, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor> &outputs, std::vector<std::vector<at::Tensor>> &inputs,
                                                const c10d::ReduceScatterOptions &opts) override {
    checkSingle(outputs);
    TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == getSize(), "flagcx: need world_size input tensors");
    auto out = outputs[0];
    auto ins = inputs[0];
    auto op = toRedOp(opts.reduceOp, out.scalar_type());
    auto flat = at::empty({getSize() * out.numel()}, out.options());
    std::vector<at::Tensor> touched = ins;
    touched.push_back(out);
    touched.push_back(flat);
    return run(c10d::OpType::REDUCE_SCATTER, out.device(), touched, {out}, [=](flagcxComm_t c, flagcxStream_t s) {
      gatherFlat(ins, flat, out.device());
      FCX_TORCH_CHECK(flagcxReduceScatter(flat.data_ptr(), out.data_ptr(), out.numel(), toDtype(out.scalar_type()), op, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor> &outputs, std::vector<at::Tensor> &inputs,
                                                                  const c10d::ReduceScatterOptions &opts) override {
    TORCH_CHECK(outputs.size() == inputs.size() && !inputs.empty(), "flagcx: mismatched tensor lists");
    auto outs = outputs, ins = inputs;
    auto redop = opts.reduceOp;
    std::vector<at::Tensor> touched = outs;
    touched.insert(touched.end(), ins.begin(), ins.end());
    return run(c10d::OpType::COALESCED, ins[0].device(), touched, outs, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxGroupStart(c));
      for (size_t k = 0; k < ins.size(); k++)
        FCX_TORCH_CHECK(flagcxReduceScatter(ins[k].data_ptr(), outs[k].data_ptr(), outs[k].numel(), toDtype(ins[k].scalar_type()),
                                            toRedOp(redop, ins[k].scalar_type()), c, s));
      FCX_TORCH_CHECK(flagcxGroupEnd(c));
    });
  }

  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>> &outputs, std::vector<at::Tensor> &inputs,
                                        const c10d::GatherOptions &opts) override {
    checkSingle(inputs);
    auto in = inputs[0];
    int root = (int)opts.rootRank;
    std::vector<at::Tensor> outs;
    at::Tensor flat;
    if (getRank() == root) {
      TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == getSize(), "flagcx: root needs world_size output tensors");
      outs = outputs[0];
      flat = at::empty({getSize() * in.numel()}, in.options());
    }
    std::vector<at::Tensor> touched = outs;
    touched.push_back(in);
    if (flat.defined()) touched.push_back(flat);
    bool isRoot = getRank() == root;
    return run(c10d::OpType::GATHER, in.device(), touched, outs, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxGather(in.data_ptr(), isRoot ? flat.data_ptr() : nullptr, in.numel(), toDtype(in.scalar_type()), root, c, s));
      if (isRoot) scatterFlat(flat, outs, in.device());
    });
  }

  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor> &outputs, std::vector<std::vector<at::Tensor>> &inputs,
                                         const c10d::ScatterOptions &opts) override {
    checkSingle(outputs);
    auto out = outputs[0];
    int root = (int)opts.rootRank;
    bool isRoot = getRank() == root;
    std::vector<at::Tensor> ins;
    at::Tensor flat;
    if (isRoot) {
      TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == getSize(), "flagcx: root needs world_size input tensors");
      ins = inputs[0];
      flat = at::empty({getSize() * out.numel()}, out.options());
    }
    std::vector<at::Tensor> touched = ins;
    touched.push_back(out);
    if (flat.defined()) touched.push_back(flat);
    return run(c10d::OpType::SCATTER, out.device(), touched, {out}, [=](flagcxComm_t c, flagcxStream_t s) {
      if (isRoot) gatherFlat(ins, flat, out.device());
      FCX_TORCH_CHECK(flagcxScatter(isRoot ? flat.data_ptr() : nullptr, out.data_ptr(), out.numel(), toDtype(out.scalar_type()), root, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor &out, at::Tensor &in, std::vector<int64_t> &outSplits,
                                               std::vector<int64_t> &inSplits, const c10d::AllToAllOptions &) override {
    TORCH_CHECK(in.is_contiguous() && out.is_contiguous(), "flagcx: tensors must be contiguous");
    auto o = out, i = in;
    const int n = getSize();
    if (outSplits.empty() && inSplits.empty()) {
      TORCH_CHECK(in.numel() % n == 0 && out.numel() == in.numel(), "flagcx: all_to_all_single needs sizes divisible by world_size");
      return run(c10d::OpType::ALLTOALL_BASE, in.device(), {i, o}, {o}, [=](flagcxComm_t c, flagcxStream_t s) {
        FCX_TORCH_CHECK(flagcxAlltoAll(i.data_ptr(), o.data_ptr(), i.numel() / n, toDtype(i.scalar_type()), c, s));
      });
    }
    TORCH_CHECK((int)outSplits.size() == n && (int)inSplits.size() == n, "flagcx: split lists must have world_size entries");
    int64_t rowIn = in.dim() > 0 && in.size(0) > 0 ? in.numel() / in.size(0) : 1;
    int64_t rowOut = out.dim() > 0 && out.size(0) > 0 ? out.numel() / out.size(0) : 1;
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    for (int k = 0; k < n; k++) {
      sc[k] = inSplits[k] * rowIn; sd[k] = so; so += sc[k];
      rc[k] = outSplits[k] * rowOut; rd[k] = ro; ro += rc[k];
    }
    return run(c10d::OpType::ALLTOALL_BASE, in.device(), {i, o}, {o}, [=](flagcxComm_t c, flagcxStream_t s) mutable {
      FCX_TORCH_CHECK(flagcxAlltoAllv(i.data_ptr(), sc.data(), sd.data(), o.data_ptr(), rc.data(), rd.data(), toDtype(i.scalar_type()), c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor> &outputs, std::vector<at::Tensor> &inputs,
                                          const c10d::AllToAllOptions &) override {
    const int n = getSize();
    TORCH_CHECK((int)outputs.size() == n && (int)inputs.size() == n, "flagcx: need world_size tensors on both sides");
    auto outs = outputs, ins = inputs;
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    for (int k = 0; k < n; k++) {
      sc[k] = ins[k].numel(); sd[k] = so; so += sc[k];
      rc[k] = outs[k].numel(); rd[k] = ro; ro += rc[k];
    }
    auto fin = at::empty({(int64_t)so}, ins[0].options());
    auto fout = at::empty({(int64_t)ro}, outs[0].options());
    std::vector<at::Tensor> touched = outs;
    touched.insert(touched.end(), ins.begin(), ins.end());
    touched.push_back(fin);
    touched.push_back(fout);
    return run(c10d::OpType::ALLTOALL, ins[0].device(), touched, outs, [=](flagcxComm_t c, flagcxStream_t s) mutable {
      for (int k = 0; k < n; k++) fin.narrow(0, sd[k], sc[k]).copy_(ins[k].reshape({-1}), true);
      FCX_TORCH_CHECK(flagcxAlltoAllv(fin.data_ptr(), sc.data(), sd.data(), fout.data_ptr(), rc.data(), rd.data(),
                                      toDtype(fin.scalar_type()), c, s));
      for (int k = 0; k < n; k++) outs[k].copy_(fout.narrow(0, rd[k], rc[k]).view_as(outs[k]), true);
    });
  }

  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor> &tensors, int dst, int) override {
    checkSingle(tensors);
    auto t = tensors[0];
    return run(c10d::OpType::SEND, t.device(), {t}, {}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxSend(t.data_ptr(), t.numel(), toDtype(t.scalar_type()), dst, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor> &tensors, int src, int) override {
    checkSingle(tensors);
    auto t = tensors[0];
    return run(c10d::OpType::RECV, t.device(), {t}, {t}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxRecv(t.data_ptr(), t.numel(), toDtype(t.scalar_type()), src, c, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor> &, int) override {
    TORCH_CHECK(false, "flagcx: recvAnysource is not supported (neither by the reference backend)");
  }

  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions &opts) override {
    at::Device dev(at::kCPU);
    if (!opts.device_ids.empty()) dev = at::Device(at::kCUDA, (c10::DeviceIndex)opts.device_ids[0]);
    else if (opts.device.has_value()) dev = *opts.device;
    else if (comms_.count("cuda")) dev = at::Device(at::kCUDA, c10::cuda::current_device());
    else if (!comms_.count("cpu") && at::cuda::is_available()) dev = at::Device(at::kCUDA, c10::cuda::current_device());
    if (dev.is_cuda() && !dev.has_index()) dev = at::Device(at::kCUDA, c10::cuda::current_device());
    if (!dev.is_cuda()) {
      return run(c10d::OpType::BARRIER, dev, {}, {}, [=](flagcxComm_t c, flagcxStream_t) { FCX_TORCH_CHECK(flagcxBarrier(c, nullptr)); });
    }
    // device barrier: a one-element all-reduce keeps it asynchronous; wait() then blocks the host
    auto t = at::zeros({1}, at::TensorOptions().device(dev).dtype(at::kInt));
    auto work = run(c10d::OpType::BARRIER, dev, {t}, {}, [=](flagcxComm_t c, flagcxStream_t s) {
      FCX_TORCH_CHECK(flagcxAllReduce(t.data_ptr(), t.data_ptr(), 1, flagcxInt32, flagcxSum, c, s));
    });
    static_cast<FlagcxWork *>(work.get())->markBarrier();
    return work;
  }

  // ---- coalescing: GroupStart at start, GroupEnd + one event at end
  void startCoalescing() override {
    coalescing_ = true;
    syncedInGroup_ = false;
    FCX_TORCH_CHECK(flagcxGroupStart(nullptr));
  }

  c10::intrusive_ptr<c10d::Work> endCoalescing() override {
    TORCH_CHECK(coalescing_, "flagcx: endCoalescing without startCoalescing");
    coalescing_ = false;
    c10::intrusive_ptr<FlagcxWork> work;
    if (!cudaPending_.empty()) {
      c10::cuda::CUDAGuard guard(coalescedDev_);
      {
        c10::cuda::CUDAStreamGuard sg(*stream_);
        FCX_TORCH_CHECK(flagcxGroupEnd(nullptr));
      }
      work = c10::make_intrusive<FlagcxWork>(c10d::OpType::COALESCED, getRank(), comms_["cuda"], true, coalescedDev_.index(), timeout_);
      work->record(*stream_);
      work->finishCudaEnqueue(*stream_);
      for (auto &w : cudaPending_) {
        w->record(*stream_);
        w->finishCudaEnqueue(*stream_);
      }
    } else {
      FCX_TORCH_CHECK(flagcxGroupEnd(nullptr));
      auto it = comms_.find("cpu");
      work = c10::make_intrusive<FlagcxWork>(c10d::OpType::COALESCED, getRank(), it == comms_.end() ? nullptr : it->second, false, 0,
                                             timeout_);
      work->finishHost();
    }
    for (auto &w : hostPending_) w->finishHost();
    cudaPending_.clear();
    hostPending_.clear();
    return work;
  }

  // ---- extras used by the Python side
  uint64_t commHandle(const std::string &key) {
    auto it = comms_.find(key);
    return it == comms_.end() ? 0 : (uint64_t)(uintptr_t)it->second;
  }
  uint64_t ensureComm(const at::Device &dev) { return (uint64_t)(uintptr_t)comm(dev); }

  // ---- group health and bookkeeping (the reference plugin has none of these)

  // Collectives issued so far on this group; equal on every rank of a healthy group.
  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }

  // A barrier over the store that names the ranks which did not arrive before the time-out.
  void monitoredBarrier(const c10d::BarrierOptions &opts, bool waitAllRanks = false) override {
    const auto limit = opts.timeout.count() > 0 ? opts.timeout : (timeout_.count() > 0 ? timeout_ : std::chrono::milliseconds(300000));
    const std::string base = "flagcx/monitored_barrier/" + std::to_string(monitored_++) + "/";
    store_->set(base + std::to_string(getRank()), std::vector<uint8_t>{1});
    if (getRank() != 0) {
      // rank 0 publishes the verdict; everybody else waits for it
      try {
        store_->wait({base + "done"}, limit + std::chrono::milliseconds(1000));
      } catch (const std::exception &) {
        TORCH_CHECK(false, "flagcx: monitoredBarrier: rank ", getRank(), " did not hear from rank 0 within ", limit.count(), " ms");
      }
      auto v = store_->get(base + "done");
      TORCH_CHECK(!v.empty() && v[0] == 1, "flagcx: monitoredBarrier failed: some ranks did not arrive (see rank 0)");
      return;
    }
    std::vector<int> missing;
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 1; r < getSize(); r++) {
      auto left = limit - std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0);
      if (left.count() < 1) left = std::chrono::milliseconds(1);
      try {
        store_->wait({base + std::to_string(r)}, left);
      } catch (const std::exception &) {
        missing.push_back(r);
        if (!waitAllRanks) break;
      }
    }
    store_->set(base + "done", std::vector<uint8_t>{(uint8_t)(missing.empty() ? 1 : 0)});
    if (!missing.empty()) {
      std::string who;
      for (int r : missing) who += (who.empty() ? "" : ", ") + std::to_string(r);
      TORCH_CHECK(false, "flagcx: monitoredBarrier: rank(s) ", who, " did not arrive within ", limit.count(), " ms");
    }
  }

  // Block the host until everything this backend enqueued has run.
  void waitForPendingWorks() override {
    if (stream_) stream_->synchronize();
  }

  // What the library's bounded device waits and the host path have recorded.
  c10d::ErrorType getError() override {
    for (auto &kv : comms_) {
      if (!kv.second) continue;
      flagcxResult_t async = flagcxSuccess;
      flagcxCommGetAsyncError(kv.second, &async);
      if (async == flagcxRemoteError) return c10d::ErrorType::REMOTE_ERROR;
      if (async != flagcxSuccess && async != flagcxInProgress) return c10d::ErrorType::COMM_ERROR;
    }
    return c10d::ErrorType::SUCCESS;
  }

  // Tensors in the communicator's symmetric heap: collectives on them need no staging copy on the NVLS path and
  // the fused kernels can address them on every peer.
  bool supportsTensorAlloc(c10::DeviceIndex) override { return true; }
  at::Tensor allocateTensor(long size, at::TensorOptions options = {}) override {
    TORCH_CHECK(options.device().is_cuda(), "flagcx: allocateTensor needs a CUDA device in its options");
    flagcxComm_t c = comm(options.device());
    const size_t bytes = std::max<size_t>((size_t)size * c10::elementSize(c10::typeMetaToScalarType(options.dtype())), 16);
    void *p = nullptr;
    FCX_TORCH_CHECK(flagcxMemAlloc(&p, bytes, c));
    return at::from_blob(p, {size}, [c](void *q) { flagcxMemFree(q, c); }, options);
  }

  void abort() override {
    for (auto &kv : comms_)
      if (kv.second) { flagcxCommAbort(kv.second); kv.second = nullptr; }
  }
  void shutdown() override {
    for (auto &kv : comms_)
      if (kv.second) { flagcxCommDestroy(kv.second); kv.second = nullptr; }
  }

 private:
  void scatterFlat(const at::Tensor &flat, const std::vector<at::Tensor> &outs, const at::Device &) {
    int64_t per = flat.numel() / (int64_t)outs.size();
    for (size_t k = 0; k < outs.size(); k++) outs[k].copy_(flat.narrow(0, k * per, per).view_as(outs[k]), true);
  }
  void gatherFlat(const std::vector<at::Tensor> &ins, const at::Tensor &flat, const at::Device &) {
    int64_t per = flat.numel() / (int64_t)ins.size();
    for (size_t k = 0; k < ins.size(); k++) flat.narrow(0, k * per, per).copy_(ins[k].reshape({-1}), true);
  }

  c10::intrusive_ptr<c10d::Store> store_;
  std::chrono::milliseconds timeout_;
  std::map<std::string, flagcxComm_t> comms_;
  int commCounter_ = 0;
  uint64_t seq_ = 0, monitored_ = 0;
  std::unique_ptr<c10::cuda::CUDAStream> stream_;
  flagcxStreamLayout wrapped_{};
  bool coalescing_ = false, syncedInGroup_ = false;
  std::vector<c10::intrusive_ptr<FlagcxWork>> cudaPending_, hostPending_;
  at::Device coalescedDev_{at::kCPU};
};

c10::intrusive_ptr<c10d::Backend> createBackend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size,
                                                const std::chrono::duration<float> &timeout) {
  return c10::make_intrusive<FlagcxBackend>(store, rank, size, std::chrono::duration_cast<std::chrono::milliseconds>(timeout));
}

void bindBackend(py::module &m) {
  py::class_<FlagcxBackend, c10::intrusive_ptr<FlagcxBackend>, c10d::Backend>(m, "FlagcxBackend")
      .def("comm_handle", &FlagcxBackend::commHandle, "raw flagcxComm_t of the 'cuda' or 'cpu' communicator (0 if not created yet)")
      .def("ensure_comm", [](FlagcxBackend &b, const py::object &dev) { return b.ensureComm(torch::python::detail::py_object_to_device(dev)); });
  m.def("create_backend", &createBackend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"));
}

}  // namespace fcxt
