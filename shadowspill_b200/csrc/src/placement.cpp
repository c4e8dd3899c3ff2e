// Fixed-offset placement of device leases and recovery of the reuse
// dependencies the layout implies.
//
// Placement: largest lease first (ties: earlier start, then input order); each
// lease takes the lowest aligned offset whose address range is clear of every
// already-placed lease that overlaps it in time. Sharing an address is safe
// only causally, so every shared byte yields a dependency "successor waits for
// the most recent earlier occupant", which the runtime enforces with an event.
//
// Behavioural model: packages/engine/csrc/src/planner/admission/placement.c:594
// and reuse.c (docs/architecture/fixed-placement.md:56-66,163-202).
#include "common.hpp"

#include <map>
#include <numeric>

namespace ssc {

int place_lifetimes(int32_t n, const int64_t* bytes, const int64_t* start, const int64_t* end,
                    int64_t alignment, int64_t* offsets, int64_t* span) {
  if (n < 0) return SS_INVALID_ARGUMENT;
  std::vector<int32_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) {
    if (bytes[a] != bytes[b]) return bytes[a] > bytes[b];
    if (start[a] != start[b]) return start[a] < start[b];
    return a < b;
  });
  std::vector<int32_t> placed;
  placed.reserve(n);
  int64_t extent = 0;
  std::vector<std::pair<int64_t, int64_t>> busy;   // [offset, end offset) of time-overlapping leases
  for (int32_t idx : order) {
    if (bytes[idx] < 0 || end[idx] < start[idx]) return SS_INVALID_ARGUMENT;
    busy.clear();
    for (int32_t j : placed) {
      // half-open lifetimes: a lease that ends exactly when another starts does not overlap
      if (start[j] < end[idx] && start[idx] < end[j] && bytes[j] > 0)
        busy.emplace_back(offsets[j], offsets[j] + bytes[j]);
    }
    std::sort(busy.begin(), busy.end());
    int64_t at = 0;
    for (auto& b : busy) {
      if (b.first - at >= bytes[idx]) break;      // gap before this busy range fits
      if (b.second > at) at = align_up(b.second, alignment);
    }
    offsets[idx] = at;
    extent = std::max(extent, at + bytes[idx]);
    placed.push_back(idx);
  }
  if (span) *span = extent;
  return SS_OK;
}

}  // namespace ssc

extern "C" {

int ss_place_lifetimes(int32_t n, const int64_t* bytes, const int64_t* start_ns,
                       const int64_t* end_ns, int64_t alignment, int64_t* offsets, int64_t* span) {
  if (n > 0 && (!bytes || !start_ns || !end_ns || !offsets)) return SS_INVALID_ARGUMENT;
  return ssc::place_lifetimes(n, bytes, start_ns, end_ns, alignment, offsets, span);
}

int ss_recover_layout_reuse(int32_t n, const int64_t* bytes, const int64_t* start_ns,
                            const int64_t* end_ns, const int64_t* offsets, int32_t* pred_begin,
                            int32_t* pred_index, int32_t max_preds) {
  if (n < 0 || !pred_begin) return SS_INVALID_ARGUMENT;
  std::vector<int32_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) {
    if (start_ns[a] != start_ns[b]) return start_ns[a] < start_ns[b];
    return end_ns[a] < end_ns[b];
  });
  // address -> (range end, most recent occupant); ranges are disjoint
  std::map<int64_t, std::pair<int64_t, int32_t>> owner;
  std::vector<std::vector<int32_t>> preds(n);
  for (int32_t idx : order) {
    const int64_t lo = offsets[idx], hi = offsets[idx] + bytes[idx];
    if (bytes[idx] <= 0) continue;
    auto it = owner.lower_bound(lo);
    if (it != owner.begin()) {
      auto prev = std::prev(it);
      if (prev->second.first > lo) it = prev;
    }
    std::vector<std::pair<int64_t, std::pair<int64_t, int32_t>>> keep;
    while (it != owner.end() && it->first < hi) {
      const int64_t a = it->first, b = it->second.first;
      const int32_t who = it->second.second;
      if (end_ns[who] > start_ns[idx]) return SS_INVALID_ARGUMENT;   // layout overlaps in time
      if (std::find(preds[idx].begin(), preds[idx].end(), who) == preds[idx].end())
        preds[idx].push_back(who);
      if (a < lo) keep.push_back({a, {lo, who}});
      if (b > hi) keep.push_back({hi, {b, who}});
      it = owner.erase(it);
    }
    for (auto& k : keep) owner[k.first] = k.second;
    owner[lo] = {hi, idx};
  }
  int32_t total = 0;
  for (int32_t i = 0; i < n; ++i) {
    pred_begin[i] = total;
    for (int32_t p : preds[i]) {
      if (pred_index && total < max_preds) pred_index[total] = p;
      ++total;
    }
  }
  pred_begin[n] = total;
  return total <= max_preds || !pred_index ? SS_OK : SS_OUT_OF_MEMORY;
}

}  // extern "C"
