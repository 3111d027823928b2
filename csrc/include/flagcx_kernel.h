/*
 * flagcx_kernel.h - device-initiated, host-executed point-to-point requests.
 *
 * Compatibility layer for programs written against the reference's device
 * API (flagcx/include/flagcx_kernel.h:103-110, flagcx/kernels/flagcx_kernel_device.cu):
 * a kernel enqueues 16-byte requests into a small queue in mapped host
 * memory; a host thread of the communicator executes them as grouped
 * send/recv on a private stream.  The native way to communicate from a kernel
 * in this library needs no host thread at all: see flagcx_device.cuh
 * (put / get / signal / wait on the symmetric heap).
 *
 * Queue layout (flagcxCommFifoBuffer returns its device address), 64-bit words:
 *   [0] capacity   [1] consumed   [2] produced   [3 + 2*i], [4 + 2*i] request i
 * Request encoding: word0 = buffer address; word1 = count (32 bits) |
 * peer rank (20 bits) << 32 | data type (4 bits) << 52 | primitive (4 bits) << 56.
 * One producer thread per queue, as in the reference.
 */
#ifndef FLAGCX_KERNEL_H_
#define FLAGCX_KERNEL_H_

#include "flagcx.h"
#include <stdint.h>

#define FLAGCX_KERNEL_FIFO_CAPACITY 16

typedef enum {
  flagcxDevicePrimSend = 0,
  flagcxDevicePrimRecv = 1,
  flagcxDevicePrimTerm = 2,
  flagcxDevicePrimWait = 3
} flagcxDevicePrim;

#define FLAGCX_TRIGGER_OFF_PEER 32
#define FLAGCX_TRIGGER_OFF_DTYPE 52
#define FLAGCX_TRIGGER_OFF_PRIM 56

struct flagcxDeviceTrigger {
  uint64_t fst, snd;
#ifdef __cplusplus
  uint64_t getAddr() const { return fst; }
  uint64_t getCount() const { return snd & 0xffffffffull; }
  uint64_t getPeerRank() const { return (snd >> FLAGCX_TRIGGER_OFF_PEER) & 0xfffffull; }
  uint64_t getDatatype() const { return (snd >> FLAGCX_TRIGGER_OFF_DTYPE) & 0xfull; }
  uint64_t getType() const { return (snd >> FLAGCX_TRIGGER_OFF_PRIM) & 0xfull; }
#endif
};
typedef struct flagcxDeviceTrigger *flagcxDeviceTrigger_t;

#ifdef __cplusplus
extern "C" {
#endif
/* Host-launched demo of the request queue: one device thread asks for a send
 * to sendPeer and a receive from recvPeer, closes the group and waits. */
void flagcxP2pDemo(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int sendPeer, int recvPeer,
                   flagcxComm_t comm, flagcxStream_t stream);
#ifdef __cplusplus
}
#endif

#ifdef __CUDACC__
/* A bounded spin: gives up (returning flagcxRemoteError) instead of hanging
 * the GPU when the host side never answers. */
#ifndef FLAGCX_FIFO_MAX_SPINS
#define FLAGCX_FIFO_MAX_SPINS (1u << 26)
#endif

__device__ __forceinline__ flagcxResult_t flagcxFifoEnqueue(void *fifoBuffer, uint64_t addr, uint64_t count, uint64_t peerRank,
                                                           uint64_t datatype, uint64_t type) {
  volatile uint64_t *buf = (volatile uint64_t *)fifoBuffer;
  const uint64_t cap = buf[0];
  const uint64_t produced = buf[2];
  unsigned spins = 0;
  while (produced - buf[1] >= cap) {  // queue full: wait for the host to consume
    if (++spins > FLAGCX_FIFO_MAX_SPINS) return flagcxRemoteError;
    __nanosleep(200);
  }
  const uint64_t slot = produced % cap;
  buf[3 + 2 * slot] = addr;
  buf[4 + 2 * slot] = (count & 0xffffffffull) | ((peerRank & 0xfffffull) << FLAGCX_TRIGGER_OFF_PEER) |
                      ((datatype & 0xfull) << FLAGCX_TRIGGER_OFF_DTYPE) | ((type & 0xfull) << FLAGCX_TRIGGER_OFF_PRIM);
  __threadfence_system();
  buf[2] = produced + 1;
  __threadfence_system();
  return flagcxSuccess;
}
__device__ __forceinline__ flagcxResult_t flagcxDeviceSend(const void *sendbuff, size_t count, flagcxDataType_t datatype, int peer,
                                                          void *fifoBuffer) {
  return flagcxFifoEnqueue(fifoBuffer, (uint64_t)sendbuff, count, (uint64_t)peer, (uint64_t)datatype, flagcxDevicePrimSend);
}
__device__ __forceinline__ flagcxResult_t flagcxDeviceRecv(void *recvbuff, size_t count, flagcxDataType_t datatype, int peer,
                                                          void *fifoBuffer) {
  return flagcxFifoEnqueue(fifoBuffer, (uint64_t)recvbuff, count, (uint64_t)peer, (uint64_t)datatype, flagcxDevicePrimRecv);
}
__device__ __forceinline__ flagcxResult_t flagcxDeviceTerm(void *fifoBuffer) {
  return flagcxFifoEnqueue(fifoBuffer, 0, 0, 0, 0, flagcxDevicePrimTerm);
}
__device__ __forceinline__ flagcxResult_t flagcxDeviceWait(void *fifoBuffer) {
  flagcxResult_t r = flagcxFifoEnqueue(fifoBuffer, 0, 0, 0, 0, flagcxDevicePrimWait);
  if (r != flagcxSuccess) return r;
  volatile uint64_t *buf = (volatile uint64_t *)fifoBuffer;
  unsigned spins = 0;
  while (buf[1] < buf[2]) {
    if (++spins > FLAGCX_FIFO_MAX_SPINS) return flagcxRemoteError;
    __nanosleep(spins < 64 ? 100 : 1000);
  }
  return flagcxSuccess;
}
#endif /* __CUDACC__ */

#endif /* FLAGCX_KERNEL_H_ */
