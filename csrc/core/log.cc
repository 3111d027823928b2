#include "log.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <pthread.h>
#include <cstdlib>
#include <string>
#include <sys/syscall.h>
#include <sys/time.h>
#include <unistd.h>

namespace fcx {

namespace {

std::once_flag gConfOnce, gLogOnce;
int gLevel = LOG_NONE;
uint32_t gMask = SUB_INIT | SUB_ENV;
FILE *gOut = nullptr;
int gRank = -1, gDev = -1;
char gHost[128] = "";
thread_local char tLastError[1024] = "";
std::mutex gWriteMu;

void loadConfFile(const char *path) {
  FILE *f = fopen(path, "r");
  if (!f) return;
  char line[1024];
  while (fgets(line, sizeof line, f)) {
    char *p = line;
    while (*p == ' ' || *p == '\t') p++;
    if (*p == '#' || *p == '\n' || *p == 0) continue;
    char *eq = strchr(p, '=');
    if (!eq) continue;
    *eq = 0;
    char *val = eq + 1;
    size_t n = strlen(val);
    while (n && (val[n - 1] == '\n' || val[n - 1] == '\r' || val[n - 1] == ' ')) val[--n] = 0;
    size_t k = strlen(p);
    while (k && (p[k - 1] == ' ' || p[k - 1] == '\t')) p[--k] = 0;
    if (k) setenv(p, val, /*overwrite=*/0);
  }
  fclose(f);
}

void loadConf() {
  const char *home = getenv("HOME");
  if (home) loadConfFile((std::string(home) + "/.flagcx.conf").c_str());
  loadConfFile("/etc/flagcx.conf");
}

struct SubName { const char *name; uint32_t bit; };
const SubName kSubs[] = {
    {"INIT", SUB_INIT}, {"COLL", SUB_COLL}, {"P2P", SUB_P2P}, {"SHM", SUB_SHM},
    {"NET", SUB_NET}, {"GRAPH", SUB_GRAPH}, {"TUNING", SUB_TUNING}, {"ENV", SUB_ENV},
    {"ALLOC", SUB_ALLOC}, {"CALL", SUB_CALL}, {"PROXY", SUB_PROXY}, {"NVLS", SUB_NVLS},
    {"BOOTSTRAP", SUB_BOOTSTRAP}, {"REG", SUB_REG}, {"KERNEL", SUB_KERNEL}, {"ALL", SUB_ALL}};

void initLog() {
  gethostname(gHost, sizeof gHost - 1);
  if (char *dot = strchr(gHost, '.')) *dot = 0;
  const char *lv = getEnv("FLAGCX_DEBUG");
  if (lv) {
    if (!strcasecmp(lv, "VERSION")) gLevel = LOG_VERSION;
    else if (!strcasecmp(lv, "WARN")) gLevel = LOG_WARN;
    else if (!strcasecmp(lv, "INFO")) gLevel = LOG_INFO;
    else if (!strcasecmp(lv, "ABORT")) gLevel = LOG_ABORT;
    else if (!strcasecmp(lv, "TRACE")) gLevel = LOG_TRACE;
  }
  if (const char *ss = getEnv("FLAGCX_DEBUG_SUBSYS")) {
    bool invert = ss[0] == '^';
    if (invert) ss++;
    uint32_t m = 0;
    std::string s(ss);
    size_t pos = 0;
    while (pos <= s.size()) {
      size_t c = s.find(',', pos);
      std::string tok = s.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
      for (auto &sn : kSubs)
        if (!strcasecmp(tok.c_str(), sn.name)) m |= sn.bit;
      if (c == std::string::npos) break;
      pos = c + 1;
    }
    gMask = invert ? ~m : m;
  }
  gOut = stdout;
  if (const char *fn = getEnv("FLAGCX_DEBUG_FILE")) {
    std::string path;
    for (const char *p = fn; *p; p++) {
      if (p[0] == '%' && p[1] == 'h') { path += gHost; p++; }
      else if (p[0] == '%' && p[1] == 'p') { path += std::to_string(getpid()); p++; }
      else path += *p;
    }
    if (FILE *f = fopen(path.c_str(), "w")) { gOut = f; setvbuf(f, nullptr, _IOLBF, 0); }
  }
}

}  // namespace

const char *getEnv(const char *name) {
  std::call_once(gConfOnce, loadConf);
  return getenv(name);
}

int64_t envInt(const char *name, int64_t dflt) {
  std::string full = std::string("FLAGCX_") + name;
  const char *v = getEnv(full.c_str());
  if (!v || !*v) return dflt;
  char *end = nullptr;
  long long x = strtoll(v, &end, 0);
  if (end == v) {
    if (!strcasecmp(v, "true")) return 1;
    if (!strcasecmp(v, "false")) return 0;
    return dflt;
  }
  // Size suffixes so that heap sizes can be written as 2G / 512M / 64K.
  if (*end == 'K' || *end == 'k') x <<= 10;
  else if (*end == 'M' || *end == 'm') x <<= 20;
  else if (*end == 'G' || *end == 'g') x <<= 30;
  return x;
}

std::string envStr(const char *name, const char *dflt) {
  std::string full = std::string("FLAGCX_") + name;
  const char *v = getEnv(full.c_str());
  return v ? std::string(v) : std::string(dflt ? dflt : "");
}

void setLogRank(int rank, int dev) { gRank = rank; gDev = dev; }

bool logEnabled(LogLevel lvl, uint32_t subsys) {
  std::call_once(gLogOnce, initLog);
  return gLevel >= lvl && (subsys & gMask);
}

const char *lastErrorText() { return tLastError; }

void logMsg(LogLevel lvl, uint32_t subsys, const char *file, int line, const char *fmt, ...) {
  std::call_once(gLogOnce, initLog);
  char body[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(body, sizeof body, fmt, ap);
  va_end(ap);
  if (lvl == LOG_WARN) {
    snprintf(tLastError, sizeof tLastError, "%s", body);
    // FLAGCX_WARN_ENABLE_DEBUG_INFO=1: after the first warning, log INFO of every subsystem
    // (reference: flagcx/service/debug.cc:157)
    static const bool escalate = getEnv("FLAGCX_WARN_ENABLE_DEBUG_INFO") && atoi(getEnv("FLAGCX_WARN_ENABLE_DEBUG_INFO")) != 0;
    if (escalate && gLevel < LOG_INFO) {
      gLevel = LOG_INFO;
      gMask = ~0u;
    }
  }
  if (gLevel < lvl) return;
  if (lvl != LOG_WARN && !(subsys & gMask)) return;
  const char *base = strrchr(file, '/');
  base = base ? base + 1 : file;
  long tid = syscall(SYS_gettid);
  std::lock_guard<std::mutex> lk(gWriteMu);
  if (lvl == LOG_WARN) {
    fprintf(gOut, "\n%s:%d:%ld [%d] %s:%d FLAGCX WARN %s\n", gHost, getpid(), tid, gDev, base, line, body);
  } else if (lvl == LOG_TRACE) {
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    double ms = tv.tv_sec * 1e3 + tv.tv_usec * 1e-3;
    fprintf(gOut, "%s:%d:%ld [%d] %.3f %s:%d FLAGCX TRACE %s\n", gHost, getpid(), tid, gDev, ms, base, line, body);
  } else {
    fprintf(gOut, "%s:%d:%ld [%d] FLAGCX INFO %s\n", gHost, getpid(), tid, gDev, body);
  }
  fflush(gOut);
}

// FLAGCX_SET_THREAD_NAME=1: helper threads carry a name ("flagcx-root", "flagcx-fifo") visible in ps/top/gdb
// (reference: flagcx/service/debug.cc:231).
void nameThisThread(const char *name) {
  static const bool on = getEnv("FLAGCX_SET_THREAD_NAME") && atoi(getEnv("FLAGCX_SET_THREAD_NAME")) != 0;
  if (on) pthread_setname_np(pthread_self(), name);
}

}  // namespace fcx
