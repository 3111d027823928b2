// Symmetric heap: one device allocation per rank that every rank of the
// communicator maps, plus (when the box supports it) an NVSwitch multicast
// alias that addresses the same offset on all ranks at once.
//
// Two back ends:
//   vmm - cuMemCreate + POSIX file descriptors passed over a unix socket,
//         cuMemMap in every process, optional cuMulticast* object.
//   ipc - cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle (no multicast).
// The reference's CUDA adaptor only has the second mechanism, for its 64 MiB
// staging FIFO (flagcx/adaptor/device/cuda_adaptor.cc:292-333; a VMM allocator
// is left disabled at :106-141).
#pragma once
#include "bootstrap.h"
#include "flagcx.h"
#include <cstddef>
#include <map>
#include <mutex>
#include <vector>

namespace fcx {

struct SymHeap {
  int nranks = 0, rank = 0;
  size_t bytes = 0;
  char *base[8] = {};     // base[r] = this process's mapping of rank r's heap
  char *mcBase = nullptr;  // multicast alias or null
  bool vmm = false;
  // opaque driver handles (CUmemGenericAllocationHandle are 64-bit integers)
  unsigned long long localHandle = 0, peerHandle[8] = {}, mcHandle = 0;
  size_t mappedBytes = 0;

  // Collective over `bs`.  mode: 0 = auto (vmm, fall back to ipc), 1 = vmm, 2 = ipc.
  flagcxResult_t create(Bootstrap &bs, int cudaDev, size_t wantBytes, int mode, bool wantMulticast);
  void destroy();
};

// First-fit allocator over the user part of the heap (host-side metadata only).
class Arena {
 public:
  void reset(size_t base, size_t bytes);
  // returns offset or ~0 on failure
  size_t alloc(size_t bytes, size_t align = 512);
  bool free(size_t off);
  size_t bytesFree() const;
 private:
  std::map<size_t, size_t> free_;   // offset -> length
  std::map<size_t, size_t> used_;
  mutable std::mutex mu_;
};

// Driver entry points resolved through the runtime (the library does not link libcuda).
bool driverReady();

}  // namespace fcx
