// Status names, platform helpers and the ABI canary.
#include "ss_core.h"

#include <cstring>
#include <ctime>
#include <thread>

extern "C" {

const char* ss_status_string(int status) {
  switch (status) {
    case SS_OK: return "ok";
    case SS_INVALID_ARGUMENT: return "invalid argument";
    case SS_OUT_OF_MEMORY: return "out of memory";
    case SS_NO_PROGRESS: return "no progress";
    case SS_BACKEND_FAILURE: return "backend failure";
    case SS_CLOSED: return "closed";
    case SS_FAILED: return "failure latched";
    case SS_TIMEOUT: return "timeout";
    case SS_INFEASIBLE: return "infeasible";
    case SS_INTERNAL: return "internal error";
    case SS_IO_ERROR: return "file pool i/o error";
    default: return "unknown status";
  }
}

int64_t ss_monotonic_ns(void) {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<int64_t>(ts.tv_sec) * 1000000000ll + ts.tv_nsec;
}

int ss_cpu_count(void) {
  const unsigned n = std::thread::hardware_concurrency();
  return n == 0 ? 1 : static_cast<int>(n);
}

uint32_t ss_abi_version(void) { return 1; }

size_t ss_struct_size(const char* name) {
#define SS_SIZE(T) if (std::strcmp(name, #T) == 0) return sizeof(T)
  SS_SIZE(ss_program); SS_SIZE(ss_device_config); SS_SIZE(ss_action); SS_SIZE(ss_interval);
  SS_SIZE(ss_sim_result); SS_SIZE(ss_search_options); SS_SIZE(ss_search_summary);
  SS_SIZE(ss_backend); SS_SIZE(ss_runtime_config); SS_SIZE(ss_failure); SS_SIZE(ss_trace_event);
  SS_SIZE(ss_runtime_stats); SS_SIZE(ss_plan_desc); SS_SIZE(ss_transfer_profile);
#undef SS_SIZE
  return 0;
}

}  // extern "C"
