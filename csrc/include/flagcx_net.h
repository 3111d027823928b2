/*
 * flagcx_net.h - network transport interface (the multi-node seam).
 *
 * A communicator of this build spans one NVSwitch domain, where every byte
 * moves by NVLink loads and stores; nothing on that path touches a NIC.  The
 * reference also carries inter-node transports behind a table of function
 * pointers (flagcx/adaptor/include/adaptor.h:235-293: IB verbs RC/UC, UCX and
 * TCP sockets).  The same table is declared here, with a TCP implementation
 * (core/net_socket.cc) used by tests and as the starting point of a multi-node
 * transport; the verbs/UCX back ends are not part of this build.
 */
#ifndef FLAGCX_NET_H_
#define FLAGCX_NET_H_

#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FLAGCX_NET_HANDLE_MAXSIZE 128
#define FLAGCX_PTR_HOST 1
#define FLAGCX_PTR_CUDA 2

typedef struct {
  char name[64];
  char pciPath[128];
  int ptrSupport;      /* FLAGCX_PTR_* mask */
  int speedMbps;
  int port;
  float latencyUs;
  int maxComms;
  int maxRecvs;
} flagcxNetProperties_t;

struct flagcxNetAdaptor {
  const char *name;
  flagcxResult_t (*init)(void);
  flagcxResult_t (*devices)(int *ndev);
  flagcxResult_t (*getProperties)(int dev, flagcxNetProperties_t *props);
  flagcxResult_t (*listen)(int dev, void *handle /* FLAGCX_NET_HANDLE_MAXSIZE bytes out */, void **listenComm);
  flagcxResult_t (*connect)(int dev, void *handle, void **sendComm);
  flagcxResult_t (*accept)(void *listenComm, void **recvComm);
  flagcxResult_t (*closeSend)(void *sendComm);
  flagcxResult_t (*closeRecv)(void *recvComm);
  flagcxResult_t (*closeListen)(void *listenComm);
  flagcxResult_t (*regMr)(void *comm, void *data, size_t size, int type, void **mhandle);
  flagcxResult_t (*regMrDmaBuf)(void *comm, void *data, size_t size, int type, uint64_t offset, int fd, void **mhandle);
  flagcxResult_t (*deregMr)(void *comm, void *mhandle);
  flagcxResult_t (*isend)(void *sendComm, void *data, size_t size, int tag, void *mhandle, void **request);
  flagcxResult_t (*irecv)(void *recvComm, int n, void **data, size_t *sizes, int *tags, void **mhandles, void **request);
  flagcxResult_t (*iflush)(void *recvComm, int n, void **data, int *sizes, void **mhandles, void **request);
  flagcxResult_t (*test)(void *request, int *done, int *sizes);
  /* one-sided operations: no implementation provides them (the reference's are NULL as well) */
  flagcxResult_t (*write)(void *sendComm, void *local, uint64_t remote, size_t size, void **request);
  flagcxResult_t (*read)(void *sendComm, void *local, uint64_t remote, size_t size, void **request);
  flagcxResult_t (*signal)(void *sendComm, uint64_t remote, uint64_t value, void **request);
  flagcxResult_t (*getDevFromName)(const char *name, int *dev);
};

/* The TCP implementation. */
extern struct flagcxNetAdaptor flagcxNetSocket;
/* Selected transport: "socket" is the only one in this build (FLAGCX_FORCE_NET_SOCKET is implied). */
const struct flagcxNetAdaptor *flagcxGetNetAdaptor(void);

#ifdef __cplusplus
}
#endif
#endif
