#include "param.h"
#include "log.h"
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <pwd.h>
#include <unistd.h>

namespace dfccl {
namespace {
std::once_flag g_conf_once;
void loadOne(const std::string& path) {
  std::ifstream in(path);
  if (!in) return;
  std::string line;
  while (std::getline(in, line)) {
    if (line.empty() || line[0] == '#') continue;
    size_t eq = line.find('=');
    if (eq == std::string::npos) continue;
    std::string k = line.substr(0, eq), v = line.substr(eq + 1);
    while (!v.empty() && (v.back() == '\r' || v.back() == ' ')) v.pop_back();
    setenv(k.c_str(), v.c_str(), 0);  // the real environment wins
  }
}
}  // namespace

void loadConfFiles() {
  std::call_once(g_conf_once, [] {
    const char* home = getenv("HOME");
    if (!home) { if (passwd* pw = getpwuid(getuid())) home = pw->pw_dir; }
    if (home) { loadOne(std::string(home) + "/.dfccl.conf"); loadOne(std::string(home) + "/.nccl.conf"); }
    loadOne("/etc/dfccl.conf");
    loadOne("/etc/nccl.conf");
  });
}

const char* envGet(const char* name) {
  loadConfFiles();
  char buf[160];
  snprintf(buf, sizeof(buf), "DFCCL_%s", name);
  if (const char* v = getenv(buf)) return v;
  snprintf(buf, sizeof(buf), "NCCL_%s", name);
  if (const char* v = getenv(buf)) return v;
  static const char* kBare[] = {"RECV_SUCCESS_FACTOR", "RECV_SUCCESS_THRESHOLD", "TOLERANT_UNPROGRESSED_CNT",
    "BASE_CTX_SWITCH_THRESHOLD", "NUM_TRY_TASKQ_HEAD", "NUM_ITER_ENV", "CHECK_REMAINING_SQE_INTERVAL",
    "SHOW_ALL_PREPARED_COLL", "DEBUG_FILE"};
  for (const char* b : kBare) if (!strcmp(b, name)) return getenv(name);
  return nullptr;
}

int64_t paramI64(const char* name, int64_t dflt) {
  const char* s = envGet(name);
  if (!s || !*s) return dflt;
  errno = 0;
  char* end = nullptr;
  long long v = strtoll(s, &end, 0);
  if (errno || end == s) { DF_INFO(SUB_ENV, "invalid value '%s' for %s, using %lld", s, name, (long long)dflt); return dflt; }
  // size suffixes for byte-valued parameters
  if (*end == 'k' || *end == 'K') v <<= 10; else if (*end == 'm' || *end == 'M') v <<= 20;
  else if (*end == 'g' || *end == 'G') v <<= 30;
  DF_INFO(SUB_ENV, "%s set by environment to %lld", name, v);
  return v;
}
double paramF64(const char* name, double dflt) {
  const char* s = envGet(name);
  if (!s || !*s) return dflt;
  char* end = nullptr;
  double v = strtod(s, &end);
  return end == s ? dflt : v;
}
std::string paramStr(const char* name, const char* dflt) {
  const char* s = envGet(name);
  return s ? std::string(s) : std::string(dflt ? dflt : "");
}
}  // namespace dfccl
