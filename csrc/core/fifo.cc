// Host side of the device->host request queue (flagcx_kernel.h).
//
// The reference runs this service inside its proxy (flagcx/core/proxy.cc:1074-1182,
// queue set-up in flagcx/core/flagcx_kernel_host.cc:31-45).  Here it is a
// small thread per communicator, started the first time the queue is asked
// for; it turns Send/Recv requests into one grouped launch per Term and
// answers Wait after its private stream has drained.
#include "comm.h"
#include "flagcx_kernel.h"
#include "log.h"

#include <chrono>
#include <cstring>
#include <cuda_runtime.h>
#include <thread>

namespace fcx {

class FifoService {
 public:
  uint64_t *host = nullptr;
  void *dev = nullptr;
  std::thread th;
  std::atomic<bool> stop{false};
  cudaStream_t stream = nullptr;
  int cudaDev = 0;
};

static void serve(flagcxComm *c, FifoService *f) {
  nameThisThread("flagcx-fifo");
  cudaSetDevice(f->cudaDev);
  volatile uint64_t *buf = f->host;
  flagcxStream fs{f->stream};
  bool open = false;
  while (!f->stop.load()) {
    uint64_t consumed = buf[1], produced = buf[2];
    if (consumed >= produced) {
      std::this_thread::sleep_for(std::chrono::microseconds(20));
      continue;
    }
    const uint64_t cap = buf[0], slot = consumed % cap;
    flagcxDeviceTrigger t{buf[3 + 2 * slot], buf[4 + 2 * slot]};
    flagcxResult_t r = flagcxSuccess;
    switch (t.getType()) {
      case flagcxDevicePrimSend:
        if (!open) { flagcxGroupStart(c); open = true; }
        r = flagcxSend((const void *)t.getAddr(), t.getCount(), (flagcxDataType_t)t.getDatatype(), (int)t.getPeerRank(), c, &fs);
        break;
      case flagcxDevicePrimRecv:
        if (!open) { flagcxGroupStart(c); open = true; }
        r = flagcxRecv((void *)t.getAddr(), t.getCount(), (flagcxDataType_t)t.getDatatype(), (int)t.getPeerRank(), c, &fs);
        break;
      case flagcxDevicePrimTerm:
        if (open) { r = flagcxGroupEnd(c); open = false; }
        break;
      case flagcxDevicePrimWait:
        if (open) { r = flagcxGroupEnd(c); open = false; }
        cudaStreamSynchronize(f->stream);
        break;
      default:
        FCX_WARN("request queue: unknown primitive %llu", (unsigned long long)t.getType());
    }
    if (r != flagcxSuccess) FCX_WARN("request queue: request failed with %d", (int)r);
    __sync_synchronize();
    buf[1] = consumed + 1;
  }
  if (open) flagcxGroupEnd(c);
}

void fifoStop(flagcxComm *c) {
  if (!c->fifo) return;
  FifoService *f = c->fifo;
  f->stop.store(true);
  if (f->th.joinable()) f->th.join();
  if (f->stream) cudaStreamDestroy(f->stream);
  if (f->host) cudaFreeHost(f->host);
  cudaGetLastError();
  delete f;
  c->fifo = nullptr;
}

}  // namespace fcx

using namespace fcx;

extern "C" flagcxResult_t flagcxCommFifoBuffer(const flagcxComm_t comm, void **buffer) {
  if (!validComm(comm) || !buffer) return flagcxInvalidArgument;
  if (comm->hostOnly || !comm->heap.bytes) return flagcxNotSupported;
  std::lock_guard<std::mutex> lk(comm->mu);
  if (!comm->fifo) {
    FifoService *f = new FifoService();
    size_t words = 3 + 2 * FLAGCX_KERNEL_FIFO_CAPACITY;
    FCX_CHECK(cudaToResult(cudaHostAlloc((void **)&f->host, words * sizeof(uint64_t), cudaHostAllocMapped), "request queue"));
    memset(f->host, 0, words * sizeof(uint64_t));
    f->host[0] = FLAGCX_KERNEL_FIFO_CAPACITY;
    FCX_CHECK(cudaToResult(cudaHostGetDevicePointer(&f->dev, f->host, 0), "request queue"));
    FCX_CHECK(cudaToResult(cudaStreamCreateWithFlags(&f->stream, cudaStreamNonBlocking), "request queue stream"));
    f->cudaDev = comm->cudaDev;
    comm->fifo = f;
    f->th = std::thread(serve, comm, f);
  }
  *buffer = comm->fifo->dev;
  return flagcxSuccess;
}
