#include "symheap.h"
#include "log.h"

#include <cerrno>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace fcx {

// ------------------------------------------------------------------ driver entry points

namespace {

struct Drv {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
  CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
  CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
  CUresult (*DeviceGet)(CUdevice *, int);
  CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char **);
  bool ok = false, mcOk = false;
};

Drv gDrv;
std::once_flag gDrvOnce;

template <typename F>
bool resolve(const char *name, F *fn, int version) {
  void *p = nullptr;
  cudaDriverEntryPointQueryResult st;
  cudaError_t e = cudaGetDriverEntryPointByVersion(name, &p, version, cudaEnableDefault, &st);
  if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *fn = (F)p;
  return true;
}

void loadDriver() {
  Drv &d = gDrv;
  bool ok = true;
  ok &= resolve("cuMemCreate", &d.MemCreate, 12000);
  ok &= resolve("cuMemRelease", &d.MemRelease, 12000);
  ok &= resolve("cuMemAddressReserve", &d.MemAddressReserve, 12000);
  ok &= resolve("cuMemAddressFree", &d.MemAddressFree, 12000);
  ok &= resolve("cuMemMap", &d.MemMap, 12000);
  ok &= resolve("cuMemUnmap", &d.MemUnmap, 12000);
  ok &= resolve("cuMemSetAccess", &d.MemSetAccess, 12000);
  ok &= resolve("cuMemExportToShareableHandle", &d.MemExportToShareableHandle, 12000);
  ok &= resolve("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle, 12000);
  ok &= resolve("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity, 12000);
  ok &= resolve("cuDeviceGet", &d.DeviceGet, 12000);
  ok &= resolve("cuDeviceGetAttribute", &d.DeviceGetAttribute, 12000);
  ok &= resolve("cuGetErrorString", &d.GetErrorString, 12000);
  d.ok = ok;
  bool mc = ok;
  mc &= resolve("cuMulticastCreate", &d.MulticastCreate, 12010);
  mc &= resolve("cuMulticastAddDevice", &d.MulticastAddDevice, 12010);
  mc &= resolve("cuMulticastBindMem", &d.MulticastBindMem, 12010);
  mc &= resolve("cuMulticastUnbind", &d.MulticastUnbind, 12010);
  mc &= resolve("cuMulticastGetGranularity", &d.MulticastGetGranularity, 12010);
  d.mcOk = mc;
}

const char *cuErr(CUresult r) {
  const char *s = nullptr;
  if (gDrv.GetErrorString) gDrv.GetErrorString(r, &s);
  return s ? s : "unknown";
}

#define CU_TRY(call, what)                                              \
  do {                                                                  \
    CUresult _r = (call);                                               \
    if (_r != CUDA_SUCCESS) {                                           \
      FCX_INFO(SUB_INIT | SUB_ALLOC, "symheap: %s failed: %s", what, cuErr(_r)); \
      return flagcxUnhandledDeviceError;                                \
    }                                                                   \
  } while (0)

// ---- file-descriptor passing over abstract unix datagram sockets ----------

void udsAddr(sockaddr_un *a, socklen_t *len, uint64_t key, int rank) {
  memset(a, 0, sizeof *a);
  a->sun_family = AF_UNIX;
  int n = snprintf(a->sun_path + 1, sizeof a->sun_path - 1, "flagcx-%016llx-%d", (unsigned long long)key, rank);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

flagcxResult_t udsSendFd(int sock, uint64_t key, int toRank, int fd, int fromRank) {
  sockaddr_un a;
  socklen_t al;
  udsAddr(&a, &al, key, toRank);
  int payload = fromRank;
  iovec iov{&payload, sizeof payload};
  char ctl[CMSG_SPACE(sizeof(int))] = {};
  msghdr m{};
  m.msg_name = &a;
  m.msg_namelen = al;
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctl;
  m.msg_controllen = sizeof ctl;
  cmsghdr *c = CMSG_FIRSTHDR(&m);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  int64_t dl = nowMs() + 60000;
  for (;;) {
    if (sendmsg(sock, &m, 0) >= 0) return flagcxSuccess;
    if (errno != EAGAIN && errno != ECONNREFUSED && errno != ENOENT && errno != EINTR) break;
    if (nowMs() > dl) break;
    usleep(1000);
  }
  FCX_WARN("symheap: sendmsg(fd) to rank %d failed: %s", toRank, strerror(errno));
  return flagcxSystemError;
}

flagcxResult_t udsRecvFd(int sock, int *fd, int *fromRank) {
  int payload = -1;
  iovec iov{&payload, sizeof payload};
  char ctl[CMSG_SPACE(sizeof(int))] = {};
  msghdr m{};
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctl;
  m.msg_controllen = sizeof ctl;
  timeval tv{60, 0};
  setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  ssize_t r;
  do { r = recvmsg(sock, &m, 0); } while (r < 0 && errno == EINTR);
  if (r < 0) {
    FCX_WARN("symheap: recvmsg(fd) failed: %s", strerror(errno));
    return flagcxSystemError;
  }
  cmsghdr *c = CMSG_FIRSTHDR(&m);
  if (!c || c->cmsg_type != SCM_RIGHTS) return flagcxSystemError;
  memcpy(fd, CMSG_DATA(c), sizeof(int));
  *fromRank = payload;
  return flagcxSuccess;
}

// All ranks agree (logical AND) on a local success flag.
flagcxResult_t agree(Bootstrap &bs, bool mine, bool *all) {
  std::vector<int> v(bs.nranks(), 0);
  v[bs.rank()] = mine ? 1 : 0;
  FCX_CHECK(bs.allGather(v.data(), sizeof(int)));
  *all = true;
  for (int x : v) *all = *all && x;
  return flagcxSuccess;
}

}  // namespace

bool driverReady() {
  std::call_once(gDrvOnce, loadDriver);
  return gDrv.ok;
}

// ------------------------------------------------------------------ heap

static flagcxResult_t createVmm(SymHeap &h, Bootstrap &bs, int dev, size_t want, bool wantMc, uint64_t key) {
  Drv &d = gDrv;
  const int n = bs.nranks(), me = bs.rank();
  CUdevice cuDev;
  CU_TRY(d.DeviceGet(&cuDev, dev), "cuDeviceGet");
  int vmmOk = 0, fdOk = 0, mcOk = 0;
  d.DeviceGetAttribute(&vmmOk, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cuDev);
  d.DeviceGetAttribute(&fdOk, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cuDev);
  if (d.mcOk) d.DeviceGetAttribute(&mcOk, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cuDev);
  if (!vmmOk || !fdOk) return flagcxNotSupported;
  bool useMc = wantMc && mcOk && n > 1;
  bool allMc;
  FCX_CHECK(agree(bs, useMc, &allMc));
  useMc = allMc;

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CU_TRY(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  CUmulticastObjectProp mcProp{};
  if (useMc) {
    mcProp.numDevices = n;
    mcProp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcProp.size = want;
    size_t mg = 0;
    if (d.MulticastGetGranularity(&mg, &mcProp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  size_t bytes = (want + gran - 1) / gran * gran;
  mcProp.size = bytes;

  CUmemGenericAllocationHandle local;
  CU_TRY(d.MemCreate(&local, bytes, &prop, 0), "cuMemCreate");
  h.localHandle = local;
  h.mappedBytes = bytes;
  int myFd = -1;
  CU_TRY(d.MemExportToShareableHandle(&myFd, local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");

  // unix socket for fd passing
  int us = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (us < 0) return flagcxSystemError;
  sockaddr_un a;
  socklen_t al;
  udsAddr(&a, &al, key, me);
  if (bind(us, (sockaddr *)&a, al) != 0) {
    FCX_WARN("symheap: bind of the fd-passing socket failed: %s", strerror(errno));
    ::close(us);
    return flagcxSystemError;
  }
  flagcxResult_t res = bs.barrier();  // every rank is bound before anyone sends
  std::vector<int> fds(n, -1);
  for (int step = 1; step < n && res == flagcxSuccess; step++) {
    int to = (me + step) % n;
    res = udsSendFd(us, key, to, myFd, me);
    if (res != flagcxSuccess) break;
    int fd, from;
    res = udsRecvFd(us, &fd, &from);
    if (res == flagcxSuccess) {
      if (from < 0 || from >= n || fds[from] >= 0) res = flagcxInternalError;
      else fds[from] = fd;
    }
  }
  ::close(myFd);
  if (res != flagcxSuccess) { ::close(us); return res; }
  // Nobody moves on to the multicast hand-off (which reuses the socket)
  // before every rank has collected all heap descriptors.
  res = bs.barrier();
  if (res != flagcxSuccess) { ::close(us); return res; }

  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < n; r++) {
    CUmemGenericAllocationHandle hd = local;
    if (r != me) {
      CUresult ir = d.MemImportFromShareableHandle(&hd, (void *)(uintptr_t)fds[r], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fds[r]);
      if (ir != CUDA_SUCCESS) {
        FCX_INFO(SUB_INIT, "symheap: import of rank %d's heap failed: %s", r, cuErr(ir));
        ::close(us);
        return flagcxUnhandledDeviceError;
      }
      h.peerHandle[r] = hd;
    }
    CUdeviceptr va = 0;
    CU_TRY(d.MemAddressReserve(&va, bytes, gran, 0, 0), "cuMemAddressReserve");
    CU_TRY(d.MemMap(va, bytes, 0, hd, 0), "cuMemMap");
    CU_TRY(d.MemSetAccess(va, bytes, &acc, 1), "cuMemSetAccess");
    h.base[r] = (char *)va;
  }

  if (useMc) {
    // Rank 0 creates the multicast object; all add their device; only after
    // everyone has been added may memory be bound.
    CUmemGenericAllocationHandle mc = 0;
    bool ok = true;
    if (me == 0) {
      ok = d.MulticastCreate(&mc, &mcProp) == CUDA_SUCCESS;
      int mcFd = -1;
      if (ok) ok = d.MemExportToShareableHandle(&mcFd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
      int flag = ok ? 1 : 0;
      bs.broadcast(&flag, sizeof flag, 0);
      if (ok) {
        for (int r = 1; r < n; r++) udsSendFd(us, key, r, mcFd, 0);
        ::close(mcFd);
      }
    } else {
      int flag = 0;
      bs.broadcast(&flag, sizeof flag, 0);
      ok = flag != 0;
      if (ok) {
        int fd = -1, from;
        ok = udsRecvFd(us, &fd, &from) == flagcxSuccess &&
             d.MemImportFromShareableHandle(&mc, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
        if (fd >= 0) ::close(fd);
      }
    }
    if (ok) ok = d.MulticastAddDevice(mc, cuDev) == CUDA_SUCCESS;
    bool all;
    FCX_CHECK(agree(bs, ok, &all));
    if (all) {
      ok = d.MulticastBindMem(mc, 0, local, 0, bytes, 0) == CUDA_SUCCESS;
      CUdeviceptr va = 0;
      if (ok) ok = d.MemAddressReserve(&va, bytes, gran, 0, 0) == CUDA_SUCCESS;
      if (ok) ok = d.MemMap(va, bytes, 0, mc, 0) == CUDA_SUCCESS;
      if (ok) ok = d.MemSetAccess(va, bytes, &acc, 1) == CUDA_SUCCESS;
      FCX_CHECK(agree(bs, ok, &all));
      if (all) {
        h.mcBase = (char *)va;
        h.mcHandle = mc;
        FCX_INFO(SUB_INIT | SUB_NVLS, "symheap: NVSwitch multicast alias mapped (%zu MiB)", bytes >> 20);
      } else {
        FCX_INFO(SUB_INIT | SUB_NVLS, "symheap: multicast bind/map failed on some rank; continuing without it");
      }
    } else {
      FCX_INFO(SUB_INIT | SUB_NVLS, "symheap: multicast object could not be set up; continuing without it");
    }
  }
  ::close(us);
  h.bytes = bytes;
  h.vmm = true;
  return flagcxSuccess;
}

static flagcxResult_t createIpc(SymHeap &h, Bootstrap &bs, size_t want) {
  const int n = bs.nranks(), me = bs.rank();
  size_t bytes = (want + (2u << 20) - 1) & ~(size_t)((2u << 20) - 1);
  void *p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    FCX_WARN("symheap: cudaMalloc of %zu bytes failed", bytes);
    return flagcxUnhandledDeviceError;
  }
  std::vector<cudaIpcMemHandle_t> hs(n);
  if (n > 1 && cudaIpcGetMemHandle(&hs[me], p) != cudaSuccess) {
    cudaGetLastError();
    return flagcxUnhandledDeviceError;
  }
  FCX_CHECK(bs.allGather(hs.data(), sizeof(cudaIpcMemHandle_t)));
  for (int r = 0; r < n; r++) {
    if (r == me) { h.base[r] = (char *)p; continue; }
    void *q = nullptr;
    if (cudaIpcOpenMemHandle(&q, hs[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      FCX_WARN("symheap: cannot open rank %d's heap through CUDA IPC", r);
      return flagcxUnhandledDeviceError;
    }
    h.base[r] = (char *)q;
  }
  h.bytes = bytes;
  h.vmm = false;
  return flagcxSuccess;
}

flagcxResult_t SymHeap::create(Bootstrap &bs, int cudaDev, size_t wantBytes, int mode, bool wantMulticast) {
  nranks = bs.nranks();
  rank = bs.rank();
  if (nranks > 8) return flagcxNotSupported;
  // A key all ranks share, to name the fd-passing sockets.
  uint64_t key = 0;
  if (rank == 0) key = ((uint64_t)getpid() << 32) ^ (uint64_t)nowMs() ^ (uint64_t)(uintptr_t)this;
  FCX_CHECK(bs.broadcast(&key, sizeof key, 0));
  bool tryVmm = mode != 2 && driverReady();
  if (tryVmm) {
    flagcxResult_t r = createVmm(*this, bs, cudaDev, wantBytes, wantMulticast, key);
    bool all;
    FCX_CHECK(agree(bs, r == flagcxSuccess, &all));
    if (all) return flagcxSuccess;
    if (mode == 1) {
      FCX_WARN("symheap: the VMM back end was requested but is not usable on every rank");
      return flagcxUnhandledDeviceError;
    }
    FCX_INFO(SUB_INIT, "symheap: falling back to CUDA IPC");
    destroy();
  }
  flagcxResult_t r = createIpc(*this, bs, wantBytes);
  bool all;
  FCX_CHECK(agree(bs, r == flagcxSuccess, &all));
  return all ? flagcxSuccess : flagcxUnhandledDeviceError;
}

void SymHeap::destroy() {
  Drv &d = gDrv;
  if (vmm || localHandle) {
    if (mcBase) {
      d.MemUnmap((CUdeviceptr)mcBase, mappedBytes);
      d.MemAddressFree((CUdeviceptr)mcBase, mappedBytes);
      mcBase = nullptr;
    }
    if (mcHandle) {
      int dev = 0;
      cudaGetDevice(&dev);
      CUdevice cuDev;
      if (d.DeviceGet(&cuDev, dev) == CUDA_SUCCESS) d.MulticastUnbind(mcHandle, cuDev, 0, mappedBytes);
      d.MemRelease(mcHandle);
      mcHandle = 0;
    }
    for (int r = 0; r < nranks; r++) {
      if (base[r]) {
        d.MemUnmap((CUdeviceptr)base[r], mappedBytes);
        d.MemAddressFree((CUdeviceptr)base[r], mappedBytes);
        base[r] = nullptr;
      }
      if (peerHandle[r]) { d.MemRelease(peerHandle[r]); peerHandle[r] = 0; }
    }
    if (localHandle) { d.MemRelease(localHandle); localHandle = 0; }
  } else {
    for (int r = 0; r < nranks; r++) {
      if (!base[r]) continue;
      if (r == rank) cudaFree(base[r]);
      else cudaIpcCloseMemHandle(base[r]);
      base[r] = nullptr;
    }
  }
  cudaGetLastError();
  vmm = false;
  bytes = 0;
}

// ------------------------------------------------------------------ arena

void Arena::reset(size_t base, size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  free_.clear();
  used_.clear();
  if (bytes) free_[base] = bytes;
}

size_t Arena::alloc(size_t bytes, size_t align) {
  std::lock_guard<std::mutex> lk(mu_);
  if (!bytes) bytes = align;
  bytes = (bytes + align - 1) / align * align;
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    size_t off = it->first, len = it->second;
    size_t start = (off + align - 1) / align * align;
    if (start + bytes > off + len) continue;
    free_.erase(it);
    if (start > off) free_[off] = start - off;
    if (start + bytes < off + len) free_[start + bytes] = off + len - start - bytes;
    used_[start] = bytes;
    return start;
  }
  return ~(size_t)0;
}

bool Arena::free(size_t off) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = used_.find(off);
  if (it == used_.end()) return false;
  size_t len = it->second;
  used_.erase(it);
  auto nx = free_.lower_bound(off);
  if (nx != free_.end() && off + len == nx->first) { len += nx->second; nx = free_.erase(nx); }
  if (nx != free_.begin()) {
    auto pv = std::prev(nx);
    if (pv->first + pv->second == off) { pv->second += len; return true; }
  }
  free_[off] = len;
  return true;
}

size_t Arena::bytesFree() const {
  std::lock_guard<std::mutex> lk(mu_);
  size_t s = 0;
  for (auto &kv : free_) s += kv.second;
  return s;
}

}  // namespace fcx
