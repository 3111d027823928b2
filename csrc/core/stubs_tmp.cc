#include "comm.h"
namespace fcx {
void fifoStop(flagcxComm *) {}
void c2cDestroy(flagcxComm *) {}
flagcxResult_t c2cExecute(flagcxComm *, const PendingOp &, bool *handled) { *handled = false; return flagcxSuccess; }
}
extern "C" flagcxResult_t flagcxCommFifoBuffer(const flagcxComm_t, void **b) { *b = nullptr; return flagcxNotSupported; }
extern "C" flagcxResult_t flagcxCommSplit(flagcxComm_t, int, int, flagcxComm_t *) { return flagcxNotSupported; }
