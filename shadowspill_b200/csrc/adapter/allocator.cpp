// Allocation adapter: PyTorch's CUDA tensors inside a task come out of a workspace slice of
// the runtime's fixed device pool, under a checked per-task allocation contract.
//
// Installed as torch's pluggable CUDA allocator (ss_alloc / ss_free) before the process
// touches CUDA. Three kinds of memory leave it:
//   * inside a task (between ss_alloc_begin_task and ss_alloc_end_task) and with a slice
//     configured: a range of the slice (address-ordered first fit over a free list with
//     coalescing; every range is 512-byte aligned). No driver call on this path.
//   * outside tasks, on another stream than the slice's, or with no slice: blocks from the driver
//     (cudaMalloc), kept per stream in size buckets when freed, so set-up code does not pay a
//     driver call per tensor and a block is never handed to another stream than the one whose
//     work may still be using it.
// A task's allocations are its *contract*: in RECORD mode the sequence of request sizes is
// kept (the profiler runs a task three times and requires the sequences to agree); in CHECK
// mode every request is compared with the recorded sequence and a deviation is latched as a
// contract violation naming the task. Exhaustion of the slice is latched the same way; the request
// itself is then served by the driver (PyTorch does not check a pluggable allocator's result, so a
// null pointer would become a tensor that faults the GPU), and the executor, which reads the latch
// after every task, raises torch.OutOfMemoryError naming the task.
//
// Reference behaviour: packages/engine/csrc/adapter/pytorch/allocator/allocator.c:64,124,178
// (allocation callbacks, task scoping, typed failures) and docs/architecture/
// task-boundaries.md:147-151 (the allocation contract).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#ifdef SS_ALLOCATOR_WITH_CUDA
#include <cuda_runtime.h>
#endif

namespace {

constexpr size_t ALIGN = 512;
inline size_t round_up(size_t n) { return (n + ALIGN - 1) / ALIGN * ALIGN; }

enum Mode : int { MODE_OFF = 0, MODE_RECORD = 1, MODE_CHECK = 2 };

struct State {
  std::mutex mu;
  // ---- the slice
  uintptr_t base = 0;
  size_t bytes = 0;
  void* slice_stream = nullptr;                     // the one stream whose tasks use the slice
  std::map<uintptr_t, size_t> free_ranges;          // offset -> length
  std::unordered_map<uintptr_t, size_t> live;       // address -> length (slice allocations)
  size_t in_use = 0, peak = 0;
  size_t all_in_use = 0, task_peak = 0, task_base_use = 0;   // slice + driver bytes handed out
  // ---- task scope
  bool in_task = false;
  int mode = MODE_OFF;
  std::string task;
  std::vector<int64_t> sequence;                    // sizes requested by the running task
  std::vector<int64_t> expected;                    // CHECK mode: the recorded contract
  size_t cursor = 0;
  // ---- failures (first one wins)
  std::string error;
  int error_kind = 0;                               // 1 = exhausted, 2 = contract violation
  // ---- driver blocks
  std::unordered_map<uintptr_t, std::pair<size_t, void*>> driver_live;      // address -> (length, stream)
  std::multimap<std::pair<void*, size_t>, uintptr_t> driver_cache;          // (stream, length) -> address
  size_t driver_bytes = 0, driver_cached = 0;
  uint64_t n_slice = 0, n_driver = 0, n_cache_hits = 0;
};

State& S() {
  static State s;
  return s;
}

void latch(State& s, int kind, const std::string& msg) {
  if (s.error_kind == 0) { s.error_kind = kind; s.error = msg; }
}

uintptr_t carve(State& s, size_t need) {
  for (auto it = s.free_ranges.begin(); it != s.free_ranges.end(); ++it) {
    if (it->second < need) continue;
    const uintptr_t off = it->first;
    const size_t len = it->second;
    s.free_ranges.erase(it);
    if (len > need) s.free_ranges[off + need] = len - need;
    return off;
  }
  return UINTPTR_MAX;
}

void give_back(State& s, uintptr_t off, size_t len) {
  auto next = s.free_ranges.lower_bound(off);
  if (next != s.free_ranges.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) { off = prev->first; len += prev->second; s.free_ranges.erase(prev); }
  }
  if (next != s.free_ranges.end() && off + len == next->first) { len += next->second; s.free_ranges.erase(next); }
  s.free_ranges[off] = len;
}

void* driver_alloc(State& s, size_t need, void* stream) {
  auto hit = s.driver_cache.lower_bound({stream, need});
  if (hit != s.driver_cache.end() && hit->first.first == stream && hit->first.second <= need + need / 4) {
    const uintptr_t p = hit->second;
    s.driver_cached -= hit->first.second;
    s.driver_live[p] = {hit->first.second, stream};
    s.driver_cache.erase(hit);
    ++s.n_cache_hits;
    return reinterpret_cast<void*>(p);
  }
  void* p = nullptr;
#ifdef SS_ALLOCATOR_WITH_CUDA
  if (cudaMalloc(&p, need) != cudaSuccess) {
    cudaGetLastError();
    // give cached blocks back to the driver (after the device is idle) and try once more
    cudaDeviceSynchronize();
    for (auto& kv : s.driver_cache) cudaFree(reinterpret_cast<void*>(kv.second));
    s.driver_bytes -= s.driver_cached; s.driver_cached = 0; s.driver_cache.clear();
    if (cudaMalloc(&p, need) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  }
#else
  p = ::operator new(need, std::nothrow);            // host build: the test double of the driver
  if (!p) return nullptr;
#endif
  s.driver_live[reinterpret_cast<uintptr_t>(p)] = {need, stream};
  s.driver_bytes += need;
  ++s.n_driver;
  return p;
}

}  // namespace

extern "C" {

// ---- the two functions torch calls
void* ss_alloc(int64_t size, int device, void* stream) {
  (void)device;
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  const size_t need = round_up(size > 0 ? static_cast<size_t>(size) : 1);
  if (s.in_task && s.mode != MODE_OFF) {
    if (s.mode == MODE_CHECK) {
      if (s.cursor >= s.expected.size() || s.expected[s.cursor] != size) {
        char buf[512];
        std::snprintf(buf, sizeof buf,
                      "allocation contract of task %s violated: request %zu asks for %lld bytes, "
                      "the profiled task asked for %lld (%zu requests recorded)",
                      s.task.c_str(), s.cursor, static_cast<long long>(size),
                      s.cursor < s.expected.size() ? static_cast<long long>(s.expected[s.cursor]) : -1LL,
                      s.expected.size());
        latch(s, 2, buf);
      }
      ++s.cursor;
    }
    s.sequence.push_back(size);
  }
  if (s.in_task && s.bytes > 0 && stream == s.slice_stream) {
    const uintptr_t off = carve(s, need);
    if (off == UINTPTR_MAX) {
      char buf[512];
      std::snprintf(buf, sizeof buf,
                    "task %s: workspace exhausted: %lld bytes requested, %zu of %zu bytes in use "
                    "(largest free range %zu)", s.task.c_str(), static_cast<long long>(size), s.in_use, s.bytes,
                    s.free_ranges.empty() ? size_t{0}
                        : std::max_element(s.free_ranges.begin(), s.free_ranges.end(),
                                           [](auto& a, auto& b) { return a.second < b.second; })->second);
      latch(s, 1, buf);
      void* spill = driver_alloc(s, need, stream);    // never a null tensor: see the header
      if (!spill) throw std::bad_alloc();
      s.all_in_use += s.driver_live[reinterpret_cast<uintptr_t>(spill)].first;
      return spill;
    }
    const uintptr_t addr = s.base + off;
    s.live[addr] = need;
    s.in_use += need;
    s.peak = std::max(s.peak, s.in_use);
    s.all_in_use += need;
    s.task_peak = std::max(s.task_peak, s.all_in_use - std::min(s.all_in_use, s.task_base_use));
    ++s.n_slice;
    return reinterpret_cast<void*>(addr);
  }
  void* p = driver_alloc(s, need, stream);
  if (!p) throw std::bad_alloc();                     // reaches Python as MemoryError
  s.all_in_use += s.driver_live[reinterpret_cast<uintptr_t>(p)].first;
  if (s.in_task)
    s.task_peak = std::max(s.task_peak, s.all_in_use - std::min(s.all_in_use, s.task_base_use));
  return p;
}

void ss_free(void* ptr, int64_t size, int device, void* stream) {
  (void)size; (void)device; (void)stream;
  if (!ptr) return;
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  const uintptr_t addr = reinterpret_cast<uintptr_t>(ptr);
  auto it = s.live.find(addr);
  if (it != s.live.end()) {
    give_back(s, addr - s.base, it->second);
    s.in_use -= it->second;
    s.all_in_use -= std::min(s.all_in_use, it->second);
    s.live.erase(it);
    return;
  }
  auto d = s.driver_live.find(addr);
  if (d == s.driver_live.end()) return;               // not ours (a range of a slice since re-configured)
  s.driver_cache.emplace(std::make_pair(d->second.second, d->second.first), addr);
  s.driver_cached += d->second.first;
  s.all_in_use -= std::min(s.all_in_use, d->second.first);
  s.driver_live.erase(d);
}

// ---- control
// The slice [base, base + bytes), used by tasks that run on `stream`. Re-configuring with live slice allocations is refused (-1).
int ss_alloc_configure(void* base, int64_t bytes, void* stream) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  if (!s.live.empty()) return -1;
  s.slice_stream = stream;
  s.base = reinterpret_cast<uintptr_t>(base);
  s.bytes = bytes > 0 ? static_cast<size_t>(bytes) / ALIGN * ALIGN : 0;
  s.free_ranges.clear();
  if (s.bytes) s.free_ranges[0] = s.bytes;
  s.in_use = s.peak = 0;
  return 0;
}

// mode 0: scope only; 1: record the contract; 2: check against `expected[0..n)`.
int ss_alloc_begin_task(const char* name, int mode, const int64_t* expected, int64_t n) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  if (s.in_task) return -1;
  s.in_task = true;
  s.mode = mode;
  s.task = name ? name : "?";
  s.sequence.clear();
  s.expected.assign(expected, expected + (expected && n > 0 ? n : 0));
  s.cursor = 0;
  s.task_base_use = s.all_in_use;
  s.task_peak = 0;
  return 0;
}

// Ends the task scope. Returns the number of requests the task made; in CHECK mode a task that
// made fewer requests than recorded is a violation too.
int64_t ss_alloc_end_task(void) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  if (!s.in_task) return -1;
  if (s.mode == MODE_CHECK && s.cursor < s.expected.size()) {
    char buf[256];
    std::snprintf(buf, sizeof buf, "allocation contract of task %s violated: %zu requests made, %zu recorded",
                  s.task.c_str(), s.cursor, s.expected.size());
    latch(s, 2, buf);
  }
  s.in_task = false;
  return static_cast<int64_t>(s.sequence.size());
}

int64_t ss_alloc_sequence(int64_t* out, int64_t capacity) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  const int64_t n = static_cast<int64_t>(s.sequence.size());
  for (int64_t i = 0; i < n && i < capacity; ++i) out[i] = s.sequence[i];
  return n;
}

// 0 = none, 1 = workspace exhausted, 2 = contract violation; the message goes to `out`. Clears the latch.
int ss_alloc_take_error(char* out, int64_t capacity) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  const int kind = s.error_kind;
  if (out && capacity > 0) {
    std::strncpy(out, s.error.c_str(), static_cast<size_t>(capacity) - 1);
    out[capacity - 1] = 0;
  }
  s.error_kind = 0;
  s.error.clear();
  return kind;
}

// [slice bytes, in use, peak, peak of the last task above its starting level, driver bytes held,
//  driver bytes cached, slice allocations, driver allocations, cache hits]
void ss_alloc_stats(int64_t* out) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  out[0] = static_cast<int64_t>(s.bytes); out[1] = static_cast<int64_t>(s.in_use);
  out[2] = static_cast<int64_t>(s.peak); out[3] = static_cast<int64_t>(s.task_peak);
  out[4] = static_cast<int64_t>(s.driver_bytes); out[5] = static_cast<int64_t>(s.driver_cached);
  out[6] = static_cast<int64_t>(s.n_slice); out[7] = static_cast<int64_t>(s.n_driver);
  out[8] = static_cast<int64_t>(s.n_cache_hits);
}

void ss_alloc_reset_peak(void) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  s.peak = s.in_use;
}

// Returns cached driver blocks to the driver (torch.cuda.empty_cache has no hook into us).
void ss_alloc_trim(void) {
  State& s = S();
  std::lock_guard<std::mutex> lk(s.mu);
  for (auto& kv : s.driver_cache) {
#ifdef SS_ALLOCATOR_WITH_CUDA
    cudaFree(reinterpret_cast<void*>(kv.second));
#else
    ::operator delete(reinterpret_cast<void*>(kv.second));
#endif
  }
  s.driver_bytes -= s.driver_cached;
  s.driver_cached = 0;
  s.driver_cache.clear();
}

}  // extern "C"
