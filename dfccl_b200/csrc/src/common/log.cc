#include "log.h"
#include "param.h"
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unistd.h>
#include <sys/time.h>
#include <execinfo.h>
#include <signal.h>

namespace dfccl {
namespace {
std::once_flag g_once;
int g_level = LOG_NONE;
uint64_t g_mask = SUB_INIT | SUB_ENV;
FILE* g_out = nullptr;
std::mutex g_mu;
thread_local int t_rank = -1;
thread_local char t_last[512];
char g_host[64] = "?";

struct Name { const char* n; uint64_t v; };
const Name kSubsys[] = {{"INIT", SUB_INIT}, {"COLL", SUB_COLL}, {"P2P", SUB_P2P}, {"SHM", SUB_SHM},
  {"NET", SUB_NET}, {"GRAPH", SUB_GRAPH}, {"TUNING", SUB_TUNING}, {"ENV", SUB_ENV}, {"ALLOC", SUB_ALLOC},
  {"CALL", SUB_CALL}, {"DAEMON", SUB_DAEMON}, {"QUEUE", SUB_QUEUE}, {"BOOT", SUB_BOOT},
  {"LEARN", SUB_LEARN}, {"ALL", SUB_ALL}};

void segvHandler(int sig) {
  void* frames[64];
  int n = backtrace(frames, 64);
  const char msg[] = "\nDFCCL: fatal signal, native backtrace:\n";
  (void)!write(2, msg, sizeof(msg) - 1);
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}

void setup() {
  if (const char* bt = envGet("DEBUG_BACKTRACE")) if (bt[0] == '1') { signal(SIGSEGV, segvHandler); signal(SIGBUS, segvHandler); signal(SIGABRT, segvHandler); }
  const char* lv = envGet("DEBUG");
  g_level = LOG_NONE;
  if (lv) {
    if (!strcasecmp(lv, "VERSION")) g_level = LOG_VERSION;
    else if (!strcasecmp(lv, "WARN")) g_level = LOG_WARN;
    else if (!strcasecmp(lv, "INFO")) g_level = LOG_INFO;
    else if (!strcasecmp(lv, "ABORT")) g_level = LOG_ABORT;
    else if (!strcasecmp(lv, "TRACE")) g_level = LOG_TRACE;
  }
  g_mask = SUB_INIT | SUB_ENV;
  if (const char* ss = envGet("DEBUG_SUBSYS")) {
    bool invert = ss[0] == '^';
    std::string s(ss + (invert ? 1 : 0));
    uint64_t m = 0;
    size_t pos = 0;
    while (pos <= s.size()) {
      size_t c = s.find(',', pos);
      std::string tok = s.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
      for (auto& k : kSubsys) if (!strcasecmp(tok.c_str(), k.n)) m |= k.v;
      if (c == std::string::npos) break;
      pos = c + 1;
    }
    g_mask = invert ? ~m : m;
  }
  gethostname(g_host, sizeof(g_host) - 1);
  if (g_out && g_out != stdout) fclose(g_out);
  g_out = stdout;
  if (const char* f = envGet("DEBUG_FILE")) {
    std::string path;
    for (const char* p = f; *p; ++p) {
      if (p[0] == '%' && p[1] == 'h') { path += g_host; ++p; }
      else if (p[0] == '%' && p[1] == 'p') { path += std::to_string(getpid()); ++p; }
      else path += *p;
    }
    if (FILE* fp = fopen(path.c_str(), "w")) { setvbuf(fp, nullptr, _IOLBF, 0); g_out = fp; }
  }
}
void ensure() { std::call_once(g_once, setup); }
}  // namespace

int logLevel() { ensure(); return g_level; }
bool logEnabled(LogLevel lvl, uint64_t subsys) { ensure(); return g_level >= lvl && (g_mask & subsys); }
void logReset() { ensure(); std::lock_guard<std::mutex> l(g_mu); setup(); }
void logSetRank(int rank) { t_rank = rank; }
const char* lastError() { return t_last; }

void logWrite(LogLevel lvl, uint64_t subsys, const char* file, int line, const char* fmt, ...) {
  ensure();
  char body[768];
  va_list ap; va_start(ap, fmt); vsnprintf(body, sizeof(body), fmt, ap); va_end(ap);
  if (lvl == LOG_WARN) { strncpy(t_last, body, sizeof(t_last) - 1); t_last[sizeof(t_last) - 1] = 0; }
  if (g_level < lvl || !(g_mask & subsys)) return;
  char line_[1024];
  if (lvl == LOG_WARN)
    snprintf(line_, sizeof(line_), "\n%s:%d:%d [%d] %s:%d DFCCL WARN %s\n", g_host, (int)getpid(),
             (int)gettid(), t_rank, file ? file : "", line, body);
  else if (lvl == LOG_TRACE) {
    timeval tv; gettimeofday(&tv, nullptr);
    snprintf(line_, sizeof(line_), "%s:%d:%d [%d] %ld.%06ld %s:%d DFCCL TRACE %s\n", g_host, (int)getpid(),
             (int)gettid(), t_rank, (long)tv.tv_sec, (long)tv.tv_usec, file ? file : "", line, body);
  } else
    snprintf(line_, sizeof(line_), "%s:%d:%d [%d] DFCCL INFO %s\n", g_host, (int)getpid(), (int)gettid(),
             t_rank, body);
  std::lock_guard<std::mutex> l(g_mu);
  fputs(line_, g_out ? g_out : stdout);
  if (lvl == LOG_WARN) fflush(g_out ? g_out : stdout);
  if (g_level == LOG_ABORT && lvl == LOG_WARN) abort();
}

const char* resultString(ncclResult_t r) {
  switch ((int)r) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "unhandled system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case dfcclTimeout: return "bounded device wait timed out";
    case dfcclAborted: return "aborted";
    default: return "unknown result code";
  }
}
}  // namespace dfccl
