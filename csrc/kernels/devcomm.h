// Structures shared by the host runtime and the device kernels.
//
// Memory model.  Every rank owns one "heap": a device allocation that all
// other ranks of the communicator map into their own address space, so
// heap[p] + x on rank r is a valid pointer to byte x of rank p's heap.  Where
// the box has an NVSwitch multicast object, mcHeap + x addresses byte x of
// *every* rank's heap at once (multimem instructions).  The reference has
// nothing comparable: its intra-node path stages data through a 64 MiB IPC
// FIFO with two CPU-driven copies per chunk (flagcx/core/p2p.cc:73-205).
//
// The head of each heap is a control block with fixed offsets (below); the
// rest is staging space for buffers the peers cannot see, and the user heap
// that flagcxMemAlloc hands out.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define FCX_MAX_RANKS 8     // one NVSwitch domain
#define FCX_MAX_CTAS 128    // upper bound on CTAs of one collective launch
#define FCX_MAX_SEGS 64     // registered user buffers per communicator
#define FCX_MAX_GROUP_OPS 64

// Where a user buffer lives, as seen by the peers.
#define FCX_SEG_NONE (-1)     // not peer-visible
#define FCX_SEG_HEAP 0        // inside the symmetric heap: peer p reaches it at heap[p] + offset
#define FCX_SEG_ABS 0x7fff    // the offset is an address every rank can use as it is (single-GPU emulation)
                              // 1 .. FCX_MAX_SEGS-1: registered segment, peer p reaches it at segs[seg][p] + offset

// ---- control block layout (byte offsets inside a heap) -------------------
#define FCX_OFF_FLAGS 0                      // u64 [FCX_MAX_CTAS][FCX_MAX_RANKS]
#define FCX_OFF_DONE (8 * 1024)              // u64 [FCX_MAX_RANKS]: last finished collective of each peer
#define FCX_OFF_MAIL (8 * 1024 + 256)        // FcxMail [2][FCX_MAX_RANKS]
#define FCX_OFF_P2P (16 * 1024)              // FcxP2pCtl [2 dirs][FCX_MAX_RANKS]
#define FCX_OFF_LOCAL (32 * 1024)            // counters only this rank touches
#define FCX_OFF_DEVAPI (40 * 1024)           // u64 [64][FCX_MAX_RANKS]: user-visible signals of the device API
#define FCX_OFF_LL (64 * 1024)               // LL lines [2][FCX_MAX_RANKS][FCX_LL_SLOT_BYTES]
#define FCX_LL_SLOT_BYTES (64 * 1024)        // holds 32 KiB of payload
#define FCX_LL_MAX_PAYLOAD (FCX_LL_SLOT_BYTES / 2)
#define FCX_OFF_STAGE (2 * 1024 * 1024)      // stage[2][stageBytes], then p2p staging, then user heap
#define FCX_DEVAPI_SIGNALS 64

struct FcxMail {  // 64 bytes, written by the source rank before it raises its flag
  uint64_t a, b, c, d, e, f, g, h;
};

struct FcxP2pCtl {  // one per (direction, peer); all counters only ever grow
  uint64_t ready;     // sender -> receiver: chunks made available so far
  uint64_t consumed;  // receiver -> sender: chunks fully read so far
  uint64_t srcOff;    // sender -> receiver: offset of the data inside its segment when it is peer-visible, else ~0
  uint64_t srcSeg;    // sender -> receiver: that segment (FCX_SEG_*)
};

// Why a kernel gave up waiting.  Lives in page-locked host memory so the host
// can read it while the context stays healthy.
struct FcxDevError {
  uint32_t code;       // 0 = none, 1 = timeout, 2 = abort requested, 3 = bad argument
  uint32_t peer;       // rank that was waited for
  uint32_t where;      // FCX_WAIT_* site
  uint32_t cta;
  uint64_t expected, seen;
  uint64_t seq;
};
#define FCX_ERR_NONE 0
#define FCX_ERR_TIMEOUT 1
#define FCX_ERR_ABORT 2
#define FCX_ERR_BADARG 3

#define FCX_WAIT_BARRIER 1
#define FCX_WAIT_DONE 2
#define FCX_WAIT_LL 3
#define FCX_WAIT_P2P_READY 4
#define FCX_WAIT_P2P_CONSUMED 5
#define FCX_WAIT_DEVAPI 6
#define FCX_WAIT_TEST 7

struct FcxDevComm {
  int rank, nranks;
  char *heap[FCX_MAX_RANKS];
  char *mcHeap;                  // multicast alias of the heaps, or null
  size_t heapBytes;
  size_t stageBytes;             // bytes of one staging half
  unsigned int pipeBytes;        // bytes a rank sends per pipeline sub-chunk of a large collective (0: 16 MiB)
  size_t p2pOff, p2pChunkBytes;  // per-peer send staging: [peer][2][p2pChunkBytes]
  size_t userOff;                // start of the flagcxMemAlloc area
  FcxDevError *err;              // host-mapped
  volatile uint32_t *abortWord;  // host-mapped; nonzero asks every waiter to leave
  uint64_t timeoutNs;
  char *(*segs)[FCX_MAX_RANKS];  // device table: registered segment -> peer base pointers
};

// ---- one collective launch ------------------------------------------------
enum FcxKind : int {
  FCX_K_BARRIER = 0,
  FCX_K_AR_LL,        // one-shot all-reduce, flags travel inside the data lines
  FCX_K_AR_ONESHOT,   // push whole vector to every peer, one barrier, reduce locally
  FCX_K_AR_TWOSHOT,   // push slices, barrier, reduce, push results, barrier, copy out
  FCX_K_AR_NVLS,      // multimem.ld_reduce + multimem.st through the switch
  FCX_K_RS,           // reduce-scatter: push slices, barrier, reduce locally
  FCX_K_RS_NVLS,
  FCX_K_AG,           // all-gather: push own part to every peer, barrier, copy out
  FCX_K_AG_NVLS,      // multimem.st of own part
  FCX_K_BCAST,
  FCX_K_REDUCE,
  FCX_K_GATHER,
  FCX_K_SCATTER,
  FCX_K_A2A,
  FCX_K_A2AV,
  FCX_K_MOVE_LL,      // small all-gather / broadcast / gather / scatter / all-to-all: flags travel inside the data lines
  FCX_K_RS_LL,        // small reduce-scatter, same idea
  FCX_K_REDUCE_LL,    // small reduce to the root, same idea
  // Zero-copy kinds: every rank's buffer is peer-visible (symmetric heap or a registered segment), so the
  // kernel reads and writes the peers' user buffers directly and nothing is staged.  When the offsets agree on
  // all ranks and the box has a multicast alias, the reducing kinds go through the switch (multimem).
  FCX_K_AR_ZC,        // owner of a slice reduces it out of all send buffers and stores it into all recv buffers
  FCX_K_RS_ZC,        // every rank reduces its piece out of all send buffers into its own recv buffer
  FCX_K_REDUCE_ZC,    // the root reduces the whole vector out of all send buffers
  FCX_K_MOVE_ZC,      // all-gather / broadcast / gather / scatter / all-to-all(v) straight between user buffers
  // Copy-engine form of the push movers on symmetric-heap buffers: a one-CTA kernel opens (barrier + check that
  // every rank's receive buffer sits at the same heap offset), the host queues one peer copy per destination on
  // the same stream (the copy engines move the bytes, no SM does), a one-CTA barrier kernel closes.
  FCX_K_MOVE_CE,
  FCX_K_NUM
};

struct FcxCollArgs {
  int kind;
  int dtype, redop, root;
  int elemSize;          // bytes per element (the byte-moving kinds only look at this)
  int ceOpen;            // FCX_K_MOVE_ZC launched as the opening step of FCX_K_MOVE_CE: exchange and check, move nothing
  int useMc;             // broadcast: root stores through the multicast alias
  int moveOp;            // FCX_K_MOVE_LL: which byte mover it stands for (FCX_K_AG, _BCAST, _GATHER, _SCATTER, _A2A)
  int outDtype;          // all-reduce with fused cast: element type of recv (== dtype when unused)
  float scale;           // multiplied into the result before the final rounding (1 = off)
  uint64_t seq;          // unused by the kernels (they count in device memory); kept for logs
  const void *send;
  void *recv;
  size_t count;          // elements of the piece handled by this launch (per-rank piece for AG/RS/A2A/gather/scatter)
  size_t sendStride;     // elements between consecutive rank pieces in the user send buffer
  size_t recvStride;     // same for the receive buffer
  // zero-copy description: segment (FCX_SEG_*) and byte offset inside it of send/recv when they are
  // peer-visible; segment FCX_SEG_NONE otherwise
  uint64_t sendHeapOff, recvHeapOff;
  int sendSeg, recvSeg;
  // all-to-all-v tables (elements), valid for FCX_K_A2AV
  uint64_t scounts[FCX_MAX_RANKS], sdispls[FCX_MAX_RANKS], rcounts[FCX_MAX_RANKS], rdispls[FCX_MAX_RANKS];
};

// ---- grouped point-to-point launch -------------------------------------------
struct FcxP2pOp {
  int isRecv, peer;
  void *buf;
  size_t bytes;
  uint64_t firstChunk;   // running chunk counter of this (direction, peer) before the op
  uint64_t heapOff;      // send only: offset inside its segment when the buffer is peer-visible, else ~0
  int seg;               // send only: that segment (FCX_SEG_*)
};

struct FcxP2pArgs {
  int nops, ctasPerOp;
  FcxP2pOp ops[FCX_MAX_GROUP_OPS];
};
