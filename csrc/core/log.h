// Logging, environment parameters and error bookkeeping.
//
// Environment names and their meaning follow the reference
// (flagcx/service/debug.cc:54-229, flagcx/service/param.cc:25-94):
//   FLAGCX_DEBUG        = NONE|VERSION|WARN|INFO|ABORT|TRACE
//   FLAGCX_DEBUG_SUBSYS = comma list of INIT,COLL,P2P,SHM,NET,GRAPH,TUNING,
//                         ENV,ALLOC,CALL,PROXY,NVLS,BOOTSTRAP,REG,KERNEL,ALL
//                         (a leading '^' inverts the set)
//   FLAGCX_DEBUG_FILE   = path, with %h -> host name and %p -> pid
// Values may also come from ~/.flagcx.conf and /etc/flagcx.conf
// (KEY=VALUE lines); the process environment wins over both files.
#pragma once
#include "flagcx.h"
#include <cstdint>
#include <string>

namespace fcx {

enum LogLevel { LOG_NONE = 0, LOG_VERSION, LOG_WARN, LOG_INFO, LOG_ABORT, LOG_TRACE };

enum LogSubsys : uint32_t {
  SUB_INIT = 1u << 0, SUB_COLL = 1u << 1, SUB_P2P = 1u << 2, SUB_SHM = 1u << 3,
  SUB_NET = 1u << 4, SUB_GRAPH = 1u << 5, SUB_TUNING = 1u << 6, SUB_ENV = 1u << 7,
  SUB_ALLOC = 1u << 8, SUB_CALL = 1u << 9, SUB_PROXY = 1u << 10, SUB_NVLS = 1u << 11,
  SUB_BOOTSTRAP = 1u << 12, SUB_REG = 1u << 13, SUB_KERNEL = 1u << 14, SUB_ALL = ~0u
};

// printf-style logger; cheap when the level/subsystem is filtered out.
void logMsg(LogLevel lvl, uint32_t subsys, const char *file, int line, const char *fmt, ...)
    __attribute__((format(printf, 5, 6)));
bool logEnabled(LogLevel lvl, uint32_t subsys);
// Text of the most recent WARN on this thread (flagcxGetLastError).
const char *lastErrorText();

// Environment access: loads the conf files once, then getenv.
const char *getEnv(const char *name);
int64_t envInt(const char *name, int64_t dflt);          // "FLAGCX_" prefix is added
std::string envStr(const char *name, const char *dflt);  // "FLAGCX_" prefix is added
void setLogRank(int rank, int dev);
void nameThisThread(const char *name);  // honours FLAGCX_SET_THREAD_NAME

}  // namespace fcx

#define FCX_WARN(...) ::fcx::logMsg(::fcx::LOG_WARN, ::fcx::SUB_ALL, __FILE__, __LINE__, __VA_ARGS__)
#define FCX_INFO(sub, ...)                                                        \
  do {                                                                            \
    if (::fcx::logEnabled(::fcx::LOG_INFO, sub))                                  \
      ::fcx::logMsg(::fcx::LOG_INFO, sub, __FILE__, __LINE__, __VA_ARGS__);       \
  } while (0)
#define FCX_TRACE(sub, ...)                                                       \
  do {                                                                            \
    if (::fcx::logEnabled(::fcx::LOG_TRACE, sub))                                 \
      ::fcx::logMsg(::fcx::LOG_TRACE, sub, __FILE__, __LINE__, __VA_ARGS__);      \
  } while (0)

// Propagate a non-success result, logging where it passed through.
#define FCX_CHECK(call)                                                           \
  do {                                                                            \
    flagcxResult_t _r = (call);                                                   \
    if (_r != flagcxSuccess && _r != flagcxInProgress) {                          \
      FCX_INFO(::fcx::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)_r);       \
      return _r;                                                                  \
    }                                                                             \
  } while (0)
