// Environment parameters.
//
// envGet("X") looks up DFCCL_X, then NCCL_X, then (for the scheduler tunables the
// reference reads without a prefix, src/enqueue_ofccl.cc:1287-1297) plain X.
// Values may also come from ~/.dfccl.conf, ~/.nccl.conf, /etc/dfccl.conf or
// /etc/nccl.conf ("KEY=VALUE" lines), loaded once before the first lookup
// (reference: src/misc/param.cc:50-80).  paramI64 caches nothing: tests change
// the environment between contexts and expect the new value.
#pragma once
#include <cstdint>
#include <string>

namespace dfccl {
const char* envGet(const char* name);                  // nullptr if unset
int64_t paramI64(const char* name, int64_t dflt);
double  paramF64(const char* name, double dflt);
std::string paramStr(const char* name, const char* dflt);
void loadConfFiles();                                  // idempotent
}  // namespace dfccl
