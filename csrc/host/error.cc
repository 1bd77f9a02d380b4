#include "launch.h"
#include <atomic>

namespace mep {
std::string& last_error() { static thread_local std::string e; return e; }
int set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  last_error() = buf;
  return -1;
}
}  // namespace mep

namespace mep { std::atomic<long long> g_launches{0}; }

// Number of kernels this library has launched in this process (all streams).
extern "C" long long mep_launch_count() { return mep::g_launches.load(); }

extern "C" const char* mep_last_error() { return mep::last_error().c_str(); }
extern "C" int mep_abi_version() { return 1; }

MEP_EXPORT_SIZEOF(MepRankCtx, MepRankCtx)
MEP_EXPORT_SIZEOF(MepStatus, MepStatus)
