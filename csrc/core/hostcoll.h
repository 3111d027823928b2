// CPU implementations of the eleven collectives plus send/recv over the
// bootstrap TCP mesh.  They serve communicators created without a GPU and
// the FLAGCX_USE_HOST_COMM=1 fallback (reference behaviour:
// flagcx/flagcx.cc:1177-1229 with flagcx/adaptor/ccl/bootstrap_adaptor.cc),
// and they are the independent oracle that GPU results are compared with.
#pragma once
#include "bootstrap.h"

namespace fcx {

flagcxResult_t hostAllReduce(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, flagcxRedOp_t op);
flagcxResult_t hostReduceScatter(Bootstrap &bs, const void *send, void *recv, size_t recvcount, flagcxDataType_t t, flagcxRedOp_t op);
flagcxResult_t hostAllGather(Bootstrap &bs, const void *send, void *recv, size_t sendcount, flagcxDataType_t t);
flagcxResult_t hostBroadcast(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root);
flagcxResult_t hostReduce(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, flagcxRedOp_t op, int root);
flagcxResult_t hostGather(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root);
flagcxResult_t hostScatter(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t, int root);
flagcxResult_t hostAlltoAll(Bootstrap &bs, const void *send, void *recv, size_t count, flagcxDataType_t t);
flagcxResult_t hostAlltoAllv(Bootstrap &bs, const void *send, const size_t *scounts, const size_t *sdispls, void *recv,
                             const size_t *rcounts, const size_t *rdispls, flagcxDataType_t t);
flagcxResult_t hostSend(Bootstrap &bs, const void *send, size_t count, flagcxDataType_t t, int peer);
flagcxResult_t hostRecv(Bootstrap &bs, void *recv, size_t count, flagcxDataType_t t, int peer);

}  // namespace fcx
