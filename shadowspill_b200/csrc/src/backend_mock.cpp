// Mock device backend: host memory stands in for device memory, every stream is
// a real thread draining an ordered queue, copies can take simulated time, and
// the n-th operation of a kind can be made to fail once. It lets the whole
// runtime (lanes, worker, reuse dependencies, failure latch) run and be tested
// with no GPU, and it is the execution backend of the CPU plumbing path.
//
// Role model: packages/engine/csrc/backends/mock/src/backend_mock.c
// (failure injection: backend_mock.h:82-91).
#include "ss_core.h"

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <dlfcn.h>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct MockEvent {
  std::mutex m;
  std::condition_variable cv;
  uint64_t record_gen = 0;   // records enqueued
  uint64_t done_gen = 0;     // records completed
  int64_t done_ns = 0;
};

struct MockStream {
  std::mutex m;
  std::condition_variable cv;
  std::deque<std::function<void()>> q;
  bool stop = false;
  bool busy = false;
  std::thread th;
  MockStream() {
    th = std::thread([this] {
      for (;;) {
        std::function<void()> op;
        {
          std::unique_lock<std::mutex> lk(m);
          cv.wait(lk, [&] { return stop || !q.empty(); });
          if (q.empty()) { if (stop) return; continue; }
          op = std::move(q.front());
          q.pop_front();
          busy = true;
        }
        op();
        {
          std::lock_guard<std::mutex> lk(m);
          busy = false;
        }
        cv.notify_all();
      }
    });
  }
  void push(std::function<void()> op) {
    { std::lock_guard<std::mutex> lk(m); q.push_back(std::move(op)); }
    cv.notify_all();
  }
  void drain() {
    std::unique_lock<std::mutex> lk(m);
    cv.wait(lk, [&] { return q.empty() && !busy; });
  }
  ~MockStream() {
    { std::lock_guard<std::mutex> lk(m); stop = true; }
    cv.notify_all();
    if (th.joinable()) th.join();
  }
};

struct Mock {
  double bps;
  int64_t latency_ns;
  std::atomic<int64_t> count[SS_OP_COUNT];
  std::atomic<int64_t> fail_at[SS_OP_COUNT];
  std::atomic<int64_t> device_bytes{0};
  Mock(double b, int64_t l) : bps(b), latency_ns(l) {
    for (int i = 0; i < SS_OP_COUNT; ++i) { count[i] = 0; fail_at[i] = 0; }
  }
  bool fails(int kind) {
    const int64_t n = ++count[kind];
    const int64_t at = fail_at[kind].load();
    if (at != 0 && n == at) { fail_at[kind] = 0; return true; }
    return false;
  }
};

Mock* M(void* self) { return static_cast<Mock*>(self); }

void signal_event(MockEvent* e, uint64_t gen) {
  {
    std::lock_guard<std::mutex> lk(e->m);
    if (gen > e->done_gen) { e->done_gen = gen; e->done_ns = ss_monotonic_ns(); }
  }
  e->cv.notify_all();
}

int device_alloc(void* self, size_t bytes, void** out) {
  if (M(self)->fails(SS_OP_DEVICE_ALLOC)) return SS_OUT_OF_MEMORY;
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes ? bytes : 1) != 0) return SS_OUT_OF_MEMORY;
  M(self)->device_bytes += static_cast<int64_t>(bytes);
  *out = p;
  return SS_OK;
}
int device_free(void*, void* p) { std::free(p); return SS_OK; }
int host_alloc(void* self, size_t bytes, int, void** out) {
  if (M(self)->fails(SS_OP_HOST_ALLOC)) return SS_OUT_OF_MEMORY;
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes ? bytes : 1) != 0) return SS_OUT_OF_MEMORY;
  *out = p;
  return SS_OK;
}
int host_free(void*, void* p, size_t) { std::free(p); return SS_OK; }
int stream_create(void* self, void** out) {
  if (M(self)->fails(SS_OP_STREAM_CREATE)) return SS_BACKEND_FAILURE;
  *out = new MockStream();
  return SS_OK;
}
int stream_destroy(void*, void* s) { delete static_cast<MockStream*>(s); return SS_OK; }
int event_create(void* self, int, void** out) {
  if (M(self)->fails(SS_OP_EVENT_CREATE)) return SS_BACKEND_FAILURE;
  *out = new MockEvent();
  return SS_OK;
}
int event_destroy(void*, void* e) { delete static_cast<MockEvent*>(e); return SS_OK; }
int event_record(void* self, void* ev, void* stream) {
  if (M(self)->fails(SS_OP_EVENT_RECORD)) return SS_BACKEND_FAILURE;
  auto* e = static_cast<MockEvent*>(ev);
  uint64_t gen;
  { std::lock_guard<std::mutex> lk(e->m); gen = ++e->record_gen; }
  if (stream == nullptr) { signal_event(e, gen); return SS_OK; }   // host-side work: done now
  static_cast<MockStream*>(stream)->push([e, gen] { signal_event(e, gen); });
  return SS_OK;
}
int event_query(void*, void* ev) {
  auto* e = static_cast<MockEvent*>(ev);
  std::lock_guard<std::mutex> lk(e->m);
  return e->done_gen >= e->record_gen ? SS_OK : SS_TIMEOUT;
}
int event_synchronize(void* self, void* ev) {
  if (M(self)->fails(SS_OP_SYNC)) return SS_BACKEND_FAILURE;
  auto* e = static_cast<MockEvent*>(ev);
  std::unique_lock<std::mutex> lk(e->m);
  const uint64_t target = e->record_gen;
  e->cv.wait(lk, [&] { return e->done_gen >= target; });
  return SS_OK;
}
int event_elapsed_ns(void*, void* a, void* b, int64_t* out) {
  *out = static_cast<MockEvent*>(b)->done_ns - static_cast<MockEvent*>(a)->done_ns;
  return SS_OK;
}
int stream_wait_event(void* self, void* stream, void* ev) {
  if (M(self)->fails(SS_OP_STREAM_WAIT)) return SS_BACKEND_FAILURE;
  auto* e = static_cast<MockEvent*>(ev);
  uint64_t target;
  { std::lock_guard<std::mutex> lk(e->m); target = e->record_gen; }
  if (target == 0) return SS_OK;   // never recorded: no-op, as on CUDA
  if (stream == nullptr) {         // host-synchronous compute waits right here
    std::unique_lock<std::mutex> lk(e->m);
    e->cv.wait(lk, [&] { return e->done_gen >= target; });
    return SS_OK;
  }
  static_cast<MockStream*>(stream)->push([e, target] {
    std::unique_lock<std::mutex> lk(e->m);
    e->cv.wait(lk, [&] { return e->done_gen >= target; });
  });
  return SS_OK;
}
int stream_synchronize(void* self, void* stream) {
  if (M(self)->fails(SS_OP_SYNC)) return SS_BACKEND_FAILURE;
  if (stream) static_cast<MockStream*>(stream)->drain();
  return SS_OK;
}
void simulated_delay(Mock* m, size_t bytes) {
  int64_t ns = m->latency_ns;
  if (m->bps > 0) ns += static_cast<int64_t>(static_cast<double>(bytes) / m->bps * 1e9);
  if (ns > 0) std::this_thread::sleep_for(std::chrono::nanoseconds(ns));
}
int copy_async(void* self, void* dst, const void* src, size_t bytes, int, void* stream) {
  Mock* m = M(self);
  if (m->fails(SS_OP_COPY)) return SS_BACKEND_FAILURE;
  auto op = [m, dst, src, bytes] { simulated_delay(m, bytes); std::memcpy(dst, src, bytes); };
  if (stream == nullptr) op(); else static_cast<MockStream*>(stream)->push(op);
  return SS_OK;
}
int memset_async(void* self, void* dst, int value, size_t bytes, void* stream) {
  if (M(self)->fails(SS_OP_MEMSET)) return SS_BACKEND_FAILURE;
  auto op = [dst, value, bytes] { std::memset(dst, value, bytes); };
  if (stream == nullptr) op(); else static_cast<MockStream*>(stream)->push(op);
  return SS_OK;
}
int device_memory_info(void*, size_t* f, size_t* t) {
  *f = static_cast<size_t>(1) << 40; *t = static_cast<size_t>(1) << 40;
  return SS_OK;
}
void destroy(void* self) { delete M(self); }

}  // namespace

extern "C" {

ss_backend* ss_mock_backend_create(double bytes_per_second, int64_t latency_ns) {
  auto* b = new ss_backend();
  b->self = new Mock(bytes_per_second, latency_ns);
  b->name = "mock";
  b->device_alloc = device_alloc; b->device_free = device_free;
  b->host_alloc = host_alloc; b->host_free = host_free;
  b->stream_create = stream_create; b->stream_destroy = stream_destroy;
  b->event_create = event_create; b->event_destroy = event_destroy;
  b->event_record = event_record; b->event_query = event_query;
  b->event_synchronize = event_synchronize; b->event_elapsed_ns = event_elapsed_ns;
  b->stream_wait_event = stream_wait_event; b->stream_synchronize = stream_synchronize;
  b->copy_async = copy_async; b->memset_async = memset_async;
  b->device_memory_info = device_memory_info;
  b->range_push = nullptr; b->range_pop = nullptr;
  b->destroy = destroy;
  return b;
}

int ss_mock_fail_operation(ss_backend* backend, int op_kind, int64_t nth) {
  if (!backend || std::strcmp(backend->name, "mock") != 0 || op_kind < 0 || op_kind >= SS_OP_COUNT)
    return SS_INVALID_ARGUMENT;
  Mock* m = M(backend->self);
  m->fail_at[op_kind] = nth == 0 ? 0 : m->count[op_kind].load() + nth;
  return SS_OK;
}

int64_t ss_mock_operation_count(ss_backend* backend, int op_kind) {
  if (!backend || op_kind < 0 || op_kind >= SS_OP_COUNT) return -1;
  return M(backend->self)->count[op_kind].load();
}

int ss_mock_enqueue_compute(ss_backend* backend, void* stream, int64_t duration_ns) {
  if (!backend || !stream) return SS_INVALID_ARGUMENT;
  static_cast<MockStream*>(stream)->push(
      [duration_ns] { std::this_thread::sleep_for(std::chrono::nanoseconds(duration_ns)); });
  return SS_OK;
}

ss_backend* ss_backend_dlopen(const char* path, int device, char* error, size_t error_len) {
  auto fail = [&](const std::string& msg) -> ss_backend* {
    if (error && error_len) { std::strncpy(error, msg.c_str(), error_len - 1); error[error_len - 1] = 0; }
    return nullptr;
  };
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return fail(std::string("dlopen: ") + dlerror());
  using open_fn = ss_backend* (*)(int, char*, size_t);
  auto fn = reinterpret_cast<open_fn>(dlsym(h, "ss_backend_open"));
  if (!fn) return fail("backend has no ss_backend_open entry");
  ss_backend* b = fn(device, error, error_len);
  return b;
}

}  // extern "C"
