// Logging and error-check helpers.
//
// Levels and subsystem masks follow the reference's debug facility
// (src/debug.cc:18-125, src/include/debug.h:103-111): DFCCL_DEBUG (or NCCL_DEBUG)
// = VERSION | WARN | INFO | ABORT | TRACE, DFCCL_DEBUG_SUBSYS (or NCCL_DEBUG_SUBSYS)
// = comma list with optional leading ^ to invert, DFCCL_DEBUG_FILE with %h (host)
// and %p (pid) expansion.  The reference's ofccl code printed through raw printf
// macros into a hard-coded developer path (src/include/debug.h:19-58,
// src/enqueue_ofccl.cc:1297); here everything goes through one sink.
#pragma once
#include <cstdint>
#include <cstdio>
#include "dfccl.h"

namespace dfccl {

enum LogLevel { LOG_NONE = 0, LOG_VERSION = 1, LOG_WARN = 2, LOG_INFO = 3, LOG_ABORT = 4, LOG_TRACE = 5 };
enum LogSubsys : uint64_t {
  SUB_INIT = 1, SUB_COLL = 2, SUB_P2P = 4, SUB_SHM = 8, SUB_NET = 16, SUB_GRAPH = 32, SUB_TUNING = 64,
  SUB_ENV = 128, SUB_ALLOC = 256, SUB_CALL = 512, SUB_DAEMON = 1024, SUB_QUEUE = 2048, SUB_BOOT = 4096,
  SUB_LEARN = 8192, SUB_ALL = ~0ull
};

int  logLevel();
bool logEnabled(LogLevel lvl, uint64_t subsys);
void logWrite(LogLevel lvl, uint64_t subsys, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
void logReset();                 // re-read the environment (tests)
void logSetRank(int rank);       // shown in the prefix of this thread's lines
const char* lastError();         // text of the most recent WARN of this thread
const char* resultString(ncclResult_t r);

}  // namespace dfccl

#define DF_WARN(...)  ::dfccl::logWrite(::dfccl::LOG_WARN, ::dfccl::SUB_ALL, __FILE__, __LINE__, __VA_ARGS__)
#define DF_INFO(sub, ...) do { if (::dfccl::logEnabled(::dfccl::LOG_INFO, sub)) \
  ::dfccl::logWrite(::dfccl::LOG_INFO, sub, nullptr, 0, __VA_ARGS__); } while (0)
#define DF_TRACE(sub, ...) do { if (::dfccl::logEnabled(::dfccl::LOG_TRACE, sub)) \
  ::dfccl::logWrite(::dfccl::LOG_TRACE, sub, __FILE__, __LINE__, __VA_ARGS__); } while (0)

// Propagate a failing ncclResult_t.
#define DFCHECK(call) do { ncclResult_t r_ = (call); if (r_ != ncclSuccess) { \
  DF_INFO(::dfccl::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)r_); return r_; } } while (0)
#define DFCHECKGOTO(call, res, label) do { res = (call); if (res != ncclSuccess) { \
  DF_INFO(::dfccl::SUB_ALL, "%s:%d -> %d", __FILE__, __LINE__, (int)res); goto label; } } while (0)
// CUDA runtime call -> ncclUnhandledCudaError.
#define CUDACHECK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
  DF_WARN("CUDA failure '%s' at %s", cudaGetErrorString(e_), #call); (void)cudaGetLastError(); \
  return ncclUnhandledCudaError; } } while (0)
#define CUDACHECKGOTO(call, res, label) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
  DF_WARN("CUDA failure '%s' at %s", cudaGetErrorString(e_), #call); (void)cudaGetLastError(); \
  res = ncclUnhandledCudaError; goto label; } } while (0)
// errno-style system call (negative or -1 on failure).
#define SYSCHECK(call, name) do { long rv_; do { rv_ = (long)(call); } while (rv_ == -1 && errno == EINTR); \
  if (rv_ == -1) { DF_WARN("call to %s failed: %s", name, strerror(errno)); return ncclSystemError; } } while (0)
