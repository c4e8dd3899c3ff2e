// Shared internal helpers of the native core.
#pragma once
#include "ss_core.h"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace ssc {

// A program unpacked into per-task / per-object adjacency.
struct Use {
  int32_t task;
  int32_t object;
  int32_t mode;
};

struct ProgramView {
  int32_t n_tasks = 0, n_objects = 0;
  std::vector<int64_t> duration, workspace, bytes;
  std::vector<int32_t> flags;
  std::vector<Use> uses;                       // sorted by (task, object)
  std::vector<int32_t> task_use_begin;         // CSR into uses, n_tasks + 1
  std::vector<std::vector<int32_t>> object_uses;   // indices into uses, ascending task

  bool persistent(int o) const { return (flags[o] & SS_OBJ_PERSISTENT) != 0; }
  bool pinned_resident(int o) const { return (flags[o] & SS_OBJ_PINNED_RESIDENT) != 0; }
};

// Returns SS_OK or SS_INVALID_ARGUMENT.
int unpack_program(const ss_program* p, ProgramView& out);

inline int64_t align_up(int64_t v, int64_t a) { return a <= 1 ? v : (v + a - 1) / a * a; }

inline int64_t transfer_ns(int64_t bytes, double bps, int64_t latency) {
  if (bps <= 0) return latency;
  return latency + static_cast<int64_t>(static_cast<double>(bytes) / bps * 1e9 + 0.5);
}

struct SimOutput {
  ss_sim_result result{};
  std::vector<int64_t> task_start, task_end, action_start, action_end;
  std::vector<ss_interval> intervals;
};

int simulate(const ProgramView& pv, const ss_device_config& cfg, const ss_action* actions,
             int32_t n_actions, SimOutput& out);

int place_lifetimes(int32_t n, const int64_t* bytes, const int64_t* start, const int64_t* end,
                    int64_t alignment, int64_t* offsets, int64_t* span);

}  // namespace ssc
