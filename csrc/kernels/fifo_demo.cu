// flagcxP2pDemo: the reference's demonstration of device-initiated requests
// (flagcx/kernels/device_collective_demo.cu:5-34): one device thread asks the
// host for a send and a receive, closes the group and waits for completion.
#include "flagcx_kernel.h"
#include <cuda_runtime.h>

struct flagcxStreamView { cudaStream_t base; };

__global__ void fcxP2pDemoKernel(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t dt, int sendPeer, int recvPeer,
                                 void *fifo) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    flagcxDeviceSend(sendbuff, count, dt, sendPeer, fifo);
    flagcxDeviceRecv(recvbuff, count, dt, recvPeer, fifo);
    flagcxDeviceTerm(fifo);
    flagcxDeviceWait(fifo);
  }
}

extern "C" void flagcxP2pDemo(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int sendPeer, int recvPeer,
                              flagcxComm_t comm, flagcxStream_t stream) {
  void *fifo = nullptr;
  if (flagcxCommFifoBuffer(comm, &fifo) != flagcxSuccess) return;
  cudaStream_t s = stream ? ((flagcxStreamView *)stream)->base : (cudaStream_t)0;
  fcxP2pDemoKernel<<<1, 1, 0, s>>>(sendbuff, recvbuff, count, datatype, sendPeer, recvPeer, fifo);
}
