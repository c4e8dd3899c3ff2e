// Execution runtime: device and spill pools, admitted plans with fixed-offset
// device stays, a fetch lane and an evict lane (one backend stream each), and a
// worker thread that turns the action batches published at task boundaries into
// stream work while honouring the layout's reuse dependencies.
//
// Division of labour (mirrors the reference's dispatcher / worker split,
// packages/engine/csrc/src/runtime/tasks/task_boundaries.c:778 and
// runtime/worker/worker.c:151):
//   dispatcher thread  ss_before_task: make the compute stream wait for the
//                      task's inputs and for the previous occupants of every
//                      range the task creates. ss_after_task: record the task
//                      fence and publish the actions the task triggers.
//   worker thread      issues published actions lane by lane in plan order. A
//                      fetch is held back (on the host) until the release of
//                      every predecessor of its destination range has been
//                      recorded, because a stream cannot wait for an event that
//                      has not been recorded yet.
// Objects whose home is the optional file pool move through staged lanes
// (staged_lane.hpp): the worker submits a job when the action's trigger is
// published and pumps the lanes; completion events are recorded when the last
// chunk's copy is enqueued, an evict is durable when its last chunk is written.
// Every host-side wait is bounded; on expiry the first-writer-wins failure
// latch is set and all entry points return SS_FAILED from then on.
#include "common.hpp"
#include "staged_lane.hpp"

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

namespace {

constexpr int64_t HOST_WAIT_NS = 60ll * 1000000000ll;

struct IntervalState {
  ss_interval iv;
  void* ready_event = nullptr;     // fetch completion (fetched stays)
  void* release_event = nullptr;   // what a successor must wait for
  std::atomic<int> ready_issued{0};
  std::atomic<int> released{0};
  bool release_on_compute = false; // release event is a compute-stream fence
};

struct PlanState {
  int32_t id = 0;
  int32_t n_tasks = 0, n_objects = 0;
  std::vector<int64_t> object_bytes, spill_offset, file_offset;
  std::vector<std::unique_ptr<ssc::StagedJob>> jobs;      // per action; null unless file-homed
  std::vector<std::atomic<int>> action_durable;           // evict to file: every chunk written
  std::atomic<int> staged_pending{0};                     // submitted staged jobs not yet complete
  std::vector<ss_action> actions;
  std::vector<std::unique_ptr<IntervalState>> intervals;
  std::vector<int32_t> pred_begin, pred_index;
  std::vector<ssc::Use> uses;
  std::vector<int32_t> task_use_begin;
  std::vector<int32_t> action_interval;        // fetch -> stay it opens; evict/release -> stay it ends
  std::vector<std::vector<int32_t>> task_creates;   // stays opened by each task
  std::vector<void*> task_fence;               // one event per task
  std::vector<uint8_t> task_side_stream;       // 1: the task's fence was recorded on a stream other than compute
  std::vector<void*> action_event;             // one event per transfer action
  std::vector<void*> action_begin_event;       // only with tracing configured: copy start
  void* step_begin_event = nullptr;            // only with tracing configured
  std::vector<int32_t> action_prev_evict;      // fetch -> earlier evict of the same object, or -1
  std::vector<std::atomic<int>> action_issued;
  // per step
  std::vector<int32_t> object_current;         // open stay per object, -1 if none
  std::vector<int32_t> fetch_order, evict_order, release_order;   // action indices by lane
  size_t next_fetch = 0, next_evict = 0, next_release = 0;
  std::atomic<int32_t> published_task{-2};     // highest task whose actions are published
  void* compute_stream = nullptr;
  bool active = false;
  void* step_event = nullptr;
};

}  // namespace

struct ss_runtime {
  ss_backend* be = nullptr;
  ss_runtime_config cfg{};
  void* device_base = nullptr;
  bool device_external = false;
  void* spill_base = nullptr;
  void* fetch_stream = nullptr;
  void* evict_stream = nullptr;
  ssc::FilePool local_file;
  ssc::RemotePool remote;
  ssc::ChunkStore* store = nullptr;        // whichever of the two is open
  std::unique_ptr<ssc::StagedLane> fetch_lane, evict_lane;
  std::mutex mu;                      // guards plans map and worker handoff
  std::condition_variable cv;
  std::map<int32_t, std::unique_ptr<PlanState>> plans;
  int32_t next_plan = 1;
  std::thread worker;
  std::atomic<bool> stop{false};
  std::atomic<bool> closed{false};
  // failure latch
  std::atomic<int> failed{0};
  std::mutex fail_mu;
  ss_failure failure{};
  // trace
  std::mutex trace_mu;
  std::vector<ss_trace_event> ring;
  size_t ring_head = 0, ring_count = 0;
  std::atomic<bool> tracing{false};
  // stats
  std::atomic<int64_t> st_steps{0}, st_tasks{0}, st_fetches{0}, st_fetch_bytes{0}, st_evicts{0},
      st_evict_bytes{0}, st_releases{0}, st_reuse_waits{0}, st_events{0}, st_host_allocs{0},
      st_wakeups{0};

  void trace(int kind, int a, int64_t bytes) {
    if (!tracing.load(std::memory_order_relaxed) || ring.empty()) return;
    std::lock_guard<std::mutex> lk(trace_mu);
    ss_trace_event& e = ring[(ring_head + ring_count) % ring.size()];
    e.kind = kind; e.a = a; e.host_ns = ss_monotonic_ns(); e.bytes = bytes;
    if (ring_count < ring.size()) ++ring_count; else ring_head = (ring_head + 1) % ring.size();
  }
  int latch(int reason, int status, int task, int object, int action, int pool, const char* msg) {
    int expected = 0;
    if (failed.compare_exchange_strong(expected, 1)) {
      std::lock_guard<std::mutex> lk(fail_mu);
      failure.status = status; failure.reason = reason; failure.task = task;
      failure.object = object; failure.action = action; failure.pool = pool;
      std::snprintf(failure.message, sizeof failure.message, "%s", msg ? msg : "");
      trace(SS_TRACE_FAILURE, action, 0);
    }
    cv.notify_all();
    return SS_FAILED;
  }
  char* dev(int64_t off) { return static_cast<char*>(device_base) + off; }
  char* spill(int64_t off) { return static_cast<char*>(spill_base) + off; }
};

namespace {

int new_event(ss_runtime* rt, void** out, int timing = 0) {
  int rc = rt->be->event_create(rt->be->self, timing, out);
  if (rc == SS_OK) rt->st_events++;
  return rc;
}

// ---- staged transfers of objects whose home is the file pool
bool file_homed(const PlanState& P, int32_t object) {
  return !P.file_offset.empty() && P.file_offset[object] >= 0;
}

void submit_staged_evict(ss_runtime* rt, PlanState& P, int32_t a) {
  const ss_action& A = P.actions[a];
  IntervalState* I = P.intervals[P.action_interval[a]].get();
  ssc::StagedJob& J = *P.jobs[a];
  J.to_device = false;
  J.file_off = P.file_offset[A.object];
  J.dev = rt->dev(I->iv.offset);
  J.bytes = P.object_bytes[A.object];
  J.tag = a;
  PlanState* Pp = &P;
  J.before_first_copy = [rt, Pp, I, a](ssc::StagedJob&) -> int {
    ss_backend* be = rt->be;
    const ss_action& A = Pp->actions[a];
    int rc = SS_OK;
    if (A.trigger_task >= 0) rc = be->stream_wait_event(be->self, rt->evict_stream, Pp->task_fence[A.trigger_task]);
    if (rc == SS_OK && I->ready_event && I->iv.begin_action >= 0)
      rc = be->stream_wait_event(be->self, rt->evict_stream, I->ready_event);
    if (rc == SS_OK && !Pp->action_begin_event.empty())
      rc = be->event_record(be->self, Pp->action_begin_event[a], rt->evict_stream);
    return rc == SS_OK ? 0 : -1;
  };
  J.after_last_copy = [rt, Pp, I, a](ssc::StagedJob& j) -> int {
    ss_backend* be = rt->be;
    if (be->event_record(be->self, Pp->action_event[a], rt->evict_stream) != SS_OK) return -1;
    I->release_event = Pp->action_event[a];      // the range is free once the last chunk left it
    I->release_on_compute = false;
    I->released.store(1, std::memory_order_release);
    Pp->action_issued[a].store(1, std::memory_order_release);
    rt->st_evicts++; rt->st_evict_bytes += j.bytes;
    rt->trace(SS_TRACE_EVICT_ISSUE, a, j.bytes);
    return 0;
  };
  J.on_durable = [rt, Pp, a](ssc::StagedJob& j) {
    Pp->action_durable[a].store(1, std::memory_order_release);
    Pp->staged_pending.fetch_sub(1, std::memory_order_acq_rel);
    rt->trace(SS_TRACE_EVICT_DONE, a, j.bytes);
  };
  P.staged_pending.fetch_add(1, std::memory_order_acq_rel);
  rt->evict_lane->submit(&J);
}

void submit_staged_fetch(ss_runtime* rt, PlanState& P, int32_t a) {
  const ss_action& A = P.actions[a];
  const int32_t ii = P.action_interval[a];
  IntervalState* I = P.intervals[ii].get();
  ssc::StagedJob& J = *P.jobs[a];
  J.to_device = true;
  J.file_off = P.file_offset[A.object];
  J.dev = rt->dev(I->iv.offset);
  J.bytes = P.object_bytes[A.object];
  J.tag = a;
  PlanState* Pp = &P;
  // reading ahead into the ring starts at once; the copies wait until every previous
  // occupant of the destination range has been released
  J.before_first_copy = [rt, Pp, ii, a](ssc::StagedJob&) -> int {
    ss_backend* be = rt->be;
    for (int32_t k = Pp->pred_begin[ii]; k < Pp->pred_begin[ii + 1]; ++k)
      if (!Pp->intervals[Pp->pred_index[k]]->released.load(std::memory_order_acquire)) {
        rt->st_reuse_waits++;
        return 1;
      }
    const ss_action& A = Pp->actions[a];
    int rc = SS_OK;
    if (A.trigger_task >= 0) rc = be->stream_wait_event(be->self, rt->fetch_stream, Pp->task_fence[A.trigger_task]);
    for (int32_t k = Pp->pred_begin[ii]; rc == SS_OK && k < Pp->pred_begin[ii + 1]; ++k) {
      IntervalState& Jv = *Pp->intervals[Pp->pred_index[k]];
      if (Jv.release_event) rc = be->stream_wait_event(be->self, rt->fetch_stream, Jv.release_event);
    }
    if (rc == SS_OK && !Pp->action_begin_event.empty())
      rc = be->event_record(be->self, Pp->action_begin_event[a], rt->fetch_stream);
    return rc == SS_OK ? 0 : -1;
  };
  J.after_last_copy = [rt, Pp, I, a](ssc::StagedJob& j) -> int {
    ss_backend* be = rt->be;
    if (be->event_record(be->self, Pp->action_event[a], rt->fetch_stream) != SS_OK) return -1;
    I->ready_event = Pp->action_event[a];
    I->ready_issued.store(1, std::memory_order_release);
    Pp->action_issued[a].store(1, std::memory_order_release);
    rt->st_fetches++; rt->st_fetch_bytes += j.bytes;
    rt->trace(SS_TRACE_FETCH_ISSUE, a, j.bytes);
    Pp->staged_pending.fetch_sub(1, std::memory_order_acq_rel);
    return 0;
  };
  J.on_durable = nullptr;
  P.staged_pending.fetch_add(1, std::memory_order_acq_rel);
  rt->fetch_lane->submit(&J);
}

// Issues every published action it can, lane by lane. Returns true if anything moved.
bool pump_plan(ss_runtime* rt, PlanState& P) {
  bool moved = false;
  const int32_t pub = P.published_task.load(std::memory_order_acquire);
  ss_backend* be = rt->be;
  // ---- releases: the stay ends at the trigger task's fence
  while (P.next_release < P.release_order.size()) {
    const int32_t a = P.release_order[P.next_release];
    const ss_action& A = P.actions[a];
    if (A.trigger_task > pub) break;
    IntervalState& I = *P.intervals[P.action_interval[a]];
    I.release_event = A.trigger_task >= 0 ? P.task_fence[A.trigger_task] : nullptr;
    // a fence on the compute stream orders later compute work by itself; a fence of a task that
    // ran on a side stream (a collective) has to be waited for
    I.release_on_compute = !(A.trigger_task >= 0 && P.task_side_stream[A.trigger_task]);
    I.released.store(1, std::memory_order_release);
    P.action_issued[a].store(1, std::memory_order_release);
    rt->st_releases++;
    rt->trace(SS_TRACE_RELEASE, a, I.iv.bytes);
    ++P.next_release; moved = true;
  }
  // ---- evicts
  while (P.next_evict < P.evict_order.size()) {
    const int32_t a = P.evict_order[P.next_evict];
    const ss_action& A = P.actions[a];
    if (A.trigger_task > pub) break;
    if (file_homed(P, A.object)) {
      // a stay opened by a staged fetch has its ready event only once that fetch is complete
      const int32_t ii = P.action_interval[a];
      if (P.intervals[ii]->iv.begin_action >= 0 &&
          !P.intervals[ii]->ready_issued.load(std::memory_order_acquire)) break;
      submit_staged_evict(rt, P, a);
      ++P.next_evict; moved = true;
      continue;
    }
    IntervalState& I = *P.intervals[P.action_interval[a]];
    int rc = SS_OK;
    if (A.trigger_task >= 0) rc = be->stream_wait_event(be->self, rt->evict_stream, P.task_fence[A.trigger_task]);
    if (rc == SS_OK && I.ready_event && I.iv.begin_action >= 0)
      rc = be->stream_wait_event(be->self, rt->evict_stream, I.ready_event);
    if (rc == SS_OK && !P.action_begin_event.empty())
      rc = be->event_record(be->self, P.action_begin_event[a], rt->evict_stream);
    if (rc == SS_OK)
      rc = be->copy_async(be->self, rt->spill(P.spill_offset[A.object]), rt->dev(I.iv.offset),
                          static_cast<size_t>(P.object_bytes[A.object]), SS_COPY_D2H, rt->evict_stream);
    if (rc == SS_OK) rc = be->event_record(be->self, P.action_event[a], rt->evict_stream);
    if (rc != SS_OK) {
      rt->latch(SS_FAIL_BACKEND_COPY, rc, A.trigger_task, A.object, a, 1, "evict failed to enqueue");
      return false;
    }
    I.release_event = P.action_event[a];
    I.release_on_compute = false;
    I.released.store(1, std::memory_order_release);
    P.action_issued[a].store(1, std::memory_order_release);
    rt->st_evicts++; rt->st_evict_bytes += P.object_bytes[A.object];
    rt->trace(SS_TRACE_EVICT_ISSUE, a, P.object_bytes[A.object]);
    ++P.next_evict; moved = true;
  }
  // ---- fetches: FIFO; the head may have to wait for predecessors of its range
  while (P.next_fetch < P.fetch_order.size()) {
    const int32_t a = P.fetch_order[P.next_fetch];
    const ss_action& A = P.actions[a];
    if (A.trigger_task > pub) break;
    const int32_t ii = P.action_interval[a];
    if (file_homed(P, A.object)) {
      const int32_t prev = P.action_prev_evict[a];
      if (prev >= 0 && !P.action_durable[prev].load(std::memory_order_acquire)) break;
      submit_staged_fetch(rt, P, a);
      ++P.next_fetch; moved = true;
      continue;
    }
    IntervalState& I = *P.intervals[ii];
    bool blocked = false;
    for (int32_t k = P.pred_begin[ii]; k < P.pred_begin[ii + 1]; ++k)
      if (!P.intervals[P.pred_index[k]]->released.load(std::memory_order_acquire)) { blocked = true; break; }
    const int32_t pe = P.action_prev_evict[a];
    if (!blocked && pe >= 0 && !P.action_issued[pe].load(std::memory_order_acquire)) blocked = true;
    if (blocked) { rt->st_reuse_waits++; break; }
    int rc = SS_OK;
    if (A.trigger_task >= 0) rc = be->stream_wait_event(be->self, rt->fetch_stream, P.task_fence[A.trigger_task]);
    for (int32_t k = P.pred_begin[ii]; rc == SS_OK && k < P.pred_begin[ii + 1]; ++k) {
      IntervalState& J = *P.intervals[P.pred_index[k]];
      if (J.release_event) rc = be->stream_wait_event(be->self, rt->fetch_stream, J.release_event);
    }
    if (rc == SS_OK && pe >= 0) rc = be->stream_wait_event(be->self, rt->fetch_stream, P.action_event[pe]);
    if (rc == SS_OK && !P.action_begin_event.empty())
      rc = be->event_record(be->self, P.action_begin_event[a], rt->fetch_stream);
    if (rc == SS_OK)
      rc = be->copy_async(be->self, rt->dev(I.iv.offset), rt->spill(P.spill_offset[A.object]),
                          static_cast<size_t>(P.object_bytes[A.object]), SS_COPY_H2D, rt->fetch_stream);
    if (rc == SS_OK) rc = be->event_record(be->self, P.action_event[a], rt->fetch_stream);
    if (rc != SS_OK) {
      rt->latch(SS_FAIL_BACKEND_COPY, rc, A.trigger_task, A.object, a, 0, "fetch failed to enqueue");
      return false;
    }
    I.ready_event = P.action_event[a];
    I.ready_issued.store(1, std::memory_order_release);
    P.action_issued[a].store(1, std::memory_order_release);
    rt->st_fetches++; rt->st_fetch_bytes += P.object_bytes[A.object];
    rt->trace(SS_TRACE_FETCH_ISSUE, a, P.object_bytes[A.object]);
    ++P.next_fetch; moved = true;
  }
  return moved;
}

void worker_main(ss_runtime* rt) {
#ifdef __linux__
  pthread_setname_np(pthread_self(), "ss.wkr");
#endif
  std::unique_lock<std::mutex> lk(rt->mu);
  while (!rt->stop.load()) {
    bool moved = false;
    if (!rt->failed.load()) {
      for (auto& kv : rt->plans)
        if (kv.second->active) moved |= pump_plan(rt, *kv.second);
      for (ssc::StagedLane* lane : {rt->evict_lane.get(), rt->fetch_lane.get()}) {
        if (!lane) continue;
        const int r = lane->pump();
        if (r < 0) {
          rt->latch(SS_FAIL_BACKEND_COPY, SS_IO_ERROR, -1, -1, -1, 2, lane->message().c_str());
          break;
        }
        moved |= r > 0;
      }
    }
    if (moved) { rt->cv.notify_all(); continue; }
    rt->st_wakeups++;
    // chunks in flight complete without anybody signalling this thread: poll them closely
    const bool staging = !rt->failed.load() && ((rt->fetch_lane && rt->fetch_lane->busy()) ||
                                                (rt->evict_lane && rt->evict_lane->busy()));
    const int64_t poll = std::max<int64_t>(rt->cfg.worker_poll_ns, 1000);
    rt->cv.wait_for(lk, std::chrono::nanoseconds(staging ? poll * 10 : poll * 200));
  }
}

PlanState* find_plan(ss_runtime* rt, int32_t id) {
  auto it = rt->plans.find(id);
  return it == rt->plans.end() ? nullptr : it->second.get();
}

// Bounded host wait for a flag the worker sets.
bool wait_flag(ss_runtime* rt, std::atomic<int>& flag) {
  if (flag.load(std::memory_order_acquire)) return true;
  const int64_t t0 = ss_monotonic_ns();
  rt->cv.notify_all();
  int spins = 0;
  while (!flag.load(std::memory_order_acquire)) {
    if (rt->failed.load()) return false;
    if (++spins < 2000) { std::this_thread::yield(); continue; }
    std::this_thread::sleep_for(std::chrono::microseconds(20));
    if (ss_monotonic_ns() - t0 > HOST_WAIT_NS) return false;
  }
  return true;
}

}  // namespace

extern "C" {

int ss_runtime_create(ss_backend* backend, const ss_runtime_config* config, ss_runtime** out) {
  if (!backend || !config || !out || config->device_bytes < 0 || config->spill_bytes < 0)
    return SS_INVALID_ARGUMENT;
  auto* rt = new ss_runtime();
  rt->be = backend;
  rt->cfg = *config;
  if (rt->cfg.worker_poll_ns <= 0) rt->cfg.worker_poll_ns = 1000;
  int rc = SS_OK;
  if (config->external_device_base != nullptr) {
    rt->device_base = config->external_device_base;
    rt->device_external = true;
  } else if (config->device_bytes > 0) {
    rc = backend->device_alloc(backend->self, static_cast<size_t>(config->device_bytes), &rt->device_base);
  }
  if (rc == SS_OK && config->spill_bytes > 0) {
    rc = backend->host_alloc(backend->self, static_cast<size_t>(config->spill_bytes),
                             config->numa_node, &rt->spill_base);
    rt->st_host_allocs++;
  }
  if (rc == SS_OK) rc = backend->stream_create(backend->self, &rt->fetch_stream);
  if (rc == SS_OK) rc = backend->stream_create(backend->self, &rt->evict_stream);
  if (rc == SS_OK && config->file_bytes > 0) {
    std::string error;
    if (config->remote_address && *config->remote_address) {
      rc = rt->remote.open(config->remote_address, config->file_bytes, error);
      rt->store = &rt->remote;
    } else {
      rc = rt->local_file.open(config->file_directory, config->file_image, config->file_create_image,
                               config->file_bytes, error);
      rt->store = &rt->local_file;
    }
    if (rc != SS_OK) std::fprintf(stderr, "ss runtime: %s\n", error.c_str());
    const int64_t chunk = config->file_chunk_bytes > 0 ? config->file_chunk_bytes : (2ll << 20);
    const int32_t depth = config->file_queue_depth > 0 ? config->file_queue_depth : 16;
    const int32_t io = config->file_io_threads > 0 ? config->file_io_threads : 4;
    if (rc == SS_OK) {
      rt->fetch_lane = std::make_unique<ssc::StagedLane>(backend, rt->fetch_stream, rt->store, true, chunk, depth, io);
      rt->evict_lane = std::make_unique<ssc::StagedLane>(backend, rt->evict_stream, rt->store, false, chunk, depth, io);
      rc = rt->fetch_lane->init(config->numa_node);
      if (rc == SS_OK) rc = rt->evict_lane->init(config->numa_node);
      rt->st_host_allocs += 2;
    }
    // the strings belong to the caller
    rt->cfg.file_directory = rt->cfg.file_image = rt->cfg.remote_address = nullptr;
  }
  if (rc != SS_OK) {
    rt->fetch_lane.reset(); rt->evict_lane.reset();
    rt->local_file.close(); rt->remote.close(); rt->store = nullptr;
    if (rt->evict_stream) backend->stream_destroy(backend->self, rt->evict_stream);
    if (rt->fetch_stream) backend->stream_destroy(backend->self, rt->fetch_stream);
    if (rt->device_base && !rt->device_external) backend->device_free(backend->self, rt->device_base);
    if (rt->spill_base) backend->host_free(backend->self, rt->spill_base, static_cast<size_t>(config->spill_bytes));
    delete rt;
    return rc;
  }
  if (config->trace_capacity > 0) rt->ring.resize(static_cast<size_t>(config->trace_capacity));
  rt->worker = std::thread(worker_main, rt);
  *out = rt;
  return SS_OK;
}

static void release_plan(ss_runtime* rt, PlanState& P) {
  for (void* e : P.task_fence) if (e) rt->be->event_destroy(rt->be->self, e);
  for (void* e : P.action_event) if (e) rt->be->event_destroy(rt->be->self, e);
  for (void* e : P.action_begin_event) if (e) rt->be->event_destroy(rt->be->self, e);
  if (P.step_event) rt->be->event_destroy(rt->be->self, P.step_event);
  if (P.step_begin_event) rt->be->event_destroy(rt->be->self, P.step_begin_event);
  P.task_fence.clear(); P.action_event.clear(); P.action_begin_event.clear();
  P.step_event = P.step_begin_event = nullptr;
}

int ss_runtime_close(ss_runtime* rt) {
  if (!rt) return SS_INVALID_ARGUMENT;
  if (rt->closed.exchange(true)) return SS_CLOSED;
  rt->stop = true;
  rt->cv.notify_all();
  if (rt->worker.joinable()) rt->worker.join();
  ss_backend* be = rt->be;
  be->stream_synchronize(be->self, rt->fetch_stream);
  be->stream_synchronize(be->self, rt->evict_stream);
  rt->fetch_lane.reset();            // joins the disk threads, frees the rings
  rt->evict_lane.reset();
  rt->local_file.close(); rt->remote.close(); rt->store = nullptr;
  for (auto& kv : rt->plans) release_plan(rt, *kv.second);
  rt->plans.clear();
  be->stream_destroy(be->self, rt->fetch_stream);
  be->stream_destroy(be->self, rt->evict_stream);
  if (rt->device_base && !rt->device_external) be->device_free(be->self, rt->device_base);
  if (rt->spill_base) be->host_free(be->self, rt->spill_base, static_cast<size_t>(rt->cfg.spill_bytes));
  rt->device_base = rt->spill_base = nullptr;
  return rt->failed.load() ? SS_FAILED : SS_OK;
}

void ss_runtime_abandon(ss_runtime* rt) {
  if (!rt || rt->closed.exchange(true)) return;
  rt->stop = true;
  rt->cv.notify_all();
  if (rt->worker.joinable()) rt->worker.detach();
  size_t open_plans = rt->plans.size();
  std::fprintf(stderr, "ss runtime abandoned: %zu plan(s) open, no drain\n", open_plans);
}

void ss_runtime_destroy(ss_runtime* rt) {
  if (!rt) return;
  if (!rt->closed.load()) ss_runtime_close(rt);
  delete rt;
}

void* ss_runtime_device_base(ss_runtime* rt) { return rt ? rt->device_base : nullptr; }
void* ss_runtime_spill_base(ss_runtime* rt) { return rt ? rt->spill_base : nullptr; }

int ss_runtime_failure(ss_runtime* rt, ss_failure* out) {
  if (!rt || !out) return SS_INVALID_ARGUMENT;
  if (!rt->failed.load()) { std::memset(out, 0, sizeof *out); return SS_TIMEOUT; }
  std::lock_guard<std::mutex> lk(rt->fail_mu);
  *out = rt->failure;
  return SS_OK;
}

int ss_runtime_latch_failure(ss_runtime* rt, int reason, int status, const char* message) {
  if (!rt) return SS_INVALID_ARGUMENT;
  rt->latch(reason, status, -1, -1, -1, -1, message);
  return SS_OK;
}

int ss_runtime_stats_read(ss_runtime* rt, ss_runtime_stats* out) {
  if (!rt || !out) return SS_INVALID_ARGUMENT;
  out->steps = rt->st_steps; out->tasks = rt->st_tasks; out->fetches = rt->st_fetches;
  out->fetch_bytes = rt->st_fetch_bytes; out->evicts = rt->st_evicts;
  out->evict_bytes = rt->st_evict_bytes; out->releases = rt->st_releases;
  out->reuse_waits = rt->st_reuse_waits; out->events_created = rt->st_events;
  out->host_allocations = rt->st_host_allocs; out->worker_wakeups = rt->st_wakeups;
  out->staged_read_chunks = rt->fetch_lane ? rt->fetch_lane->chunks_done() : 0;
  out->staged_read_bytes = rt->fetch_lane ? rt->fetch_lane->bytes_done() : 0;
  out->staged_write_chunks = rt->evict_lane ? rt->evict_lane->chunks_done() : 0;
  out->staged_write_bytes = rt->evict_lane ? rt->evict_lane->bytes_done() : 0;
  return SS_OK;
}

int ss_trace_begin(ss_runtime* rt) {
  if (!rt) return SS_INVALID_ARGUMENT;
  if (rt->ring.empty()) return SS_INVALID_ARGUMENT;
  { std::lock_guard<std::mutex> lk(rt->trace_mu); rt->ring_head = rt->ring_count = 0; }
  rt->tracing = true;
  return SS_OK;
}
int ss_trace_end(ss_runtime* rt) {
  if (!rt) return SS_INVALID_ARGUMENT;
  rt->tracing = false;
  return SS_OK;
}
int32_t ss_trace_read(ss_runtime* rt, ss_trace_event* out, int32_t capacity) {
  if (!rt || !out) return 0;
  std::lock_guard<std::mutex> lk(rt->trace_mu);
  const int32_t n = static_cast<int32_t>(std::min<size_t>(rt->ring_count, static_cast<size_t>(capacity)));
  for (int32_t i = 0; i < n; ++i) out[i] = rt->ring[(rt->ring_head + i) % rt->ring.size()];
  return n;
}

int ss_plan_admit(ss_runtime* rt, const ss_plan_desc* d, int32_t* plan_id) {
  if (!rt || !d || !plan_id) return SS_INVALID_ARGUMENT;
  if (rt->closed.load()) return SS_CLOSED;
  if (rt->failed.load()) return SS_FAILED;
  auto P = std::make_unique<PlanState>();
  P->n_tasks = d->n_tasks; P->n_objects = d->n_objects;
  P->object_bytes.assign(d->object_bytes, d->object_bytes + d->n_objects);
  P->spill_offset.assign(d->spill_offset, d->spill_offset + d->n_objects);
  if (d->file_offset) {
    P->file_offset.assign(d->file_offset, d->file_offset + d->n_objects);
    for (int32_t o = 0; o < d->n_objects; ++o) {
      if (P->file_offset[o] < 0) continue;
      if (!rt->store || P->spill_offset[o] >= 0 || d->object_bytes[o] <= 0 ||
          P->file_offset[o] + d->object_bytes[o] > rt->store->bytes())
        return SS_INVALID_ARGUMENT;      // no file pool, two homes, or outside the file
    }
  }
  P->actions.assign(d->actions, d->actions + d->n_actions);
  for (int32_t i = 0; i < d->n_intervals; ++i) {
    auto s = std::make_unique<IntervalState>();
    s->iv = d->intervals[i];
    const ss_interval& iv = s->iv;
    if (iv.object < 0 || iv.object >= d->n_objects || iv.offset < 0 ||
        iv.offset + d->object_bytes[iv.object] > rt->cfg.device_bytes) {
      return rt->latch(SS_FAIL_PLAN, SS_INVALID_ARGUMENT, -1, iv.object, -1, 0,
                       "stay outside the device pool"), SS_INVALID_ARGUMENT;
    }
    P->intervals.push_back(std::move(s));
  }
  P->pred_begin.assign(d->reuse_pred_begin, d->reuse_pred_begin + d->n_intervals + 1);
  P->pred_index.assign(d->reuse_pred_index, d->reuse_pred_index + P->pred_begin[d->n_intervals]);
  P->uses.resize(d->n_uses);
  P->task_use_begin.assign(d->n_tasks + 1, 0);
  for (int32_t i = 0; i < d->n_uses; ++i) {
    P->uses[i] = ssc::Use{d->use_task[i], d->use_object[i], d->use_mode[i]};
    if (d->use_task[i] < 0 || d->use_task[i] >= d->n_tasks) return SS_INVALID_ARGUMENT;
    P->task_use_begin[d->use_task[i] + 1]++;
  }
  for (int32_t t = 0; t < d->n_tasks; ++t) P->task_use_begin[t + 1] += P->task_use_begin[t];
  for (int32_t o = 0; o < d->n_objects; ++o) {
    if (d->spill_offset[o] >= 0 && d->spill_offset[o] + d->object_bytes[o] > rt->cfg.spill_bytes)
      return SS_OUT_OF_MEMORY;
  }
  // action <-> stay links
  P->action_interval.assign(d->n_actions, -1);
  P->task_creates.assign(d->n_tasks, {});
  for (int32_t i = 0; i < d->n_intervals; ++i) {
    const ss_interval& iv = P->intervals[i]->iv;
    if (iv.begin_action >= 0) {
      if (iv.begin_action >= d->n_actions) return SS_INVALID_ARGUMENT;
      P->action_interval[iv.begin_action] = i;
    } else if (iv.begin_task >= 0 && iv.begin_task < d->n_tasks) {
      P->task_creates[iv.begin_task].push_back(i);
    } else {
      return SS_INVALID_ARGUMENT;
    }
    if (iv.end_action >= 0) {
      if (iv.end_action >= d->n_actions) return SS_INVALID_ARGUMENT;
      P->action_interval[iv.end_action] = i;
    }
  }
  P->action_prev_evict.assign(d->n_actions, -1);
  {
    std::vector<int32_t> last_evict(d->n_objects, -1);
    for (int32_t a = 0; a < d->n_actions; ++a) {
      const ss_action& A = P->actions[a];
      if (P->action_interval[a] < 0) return SS_INVALID_ARGUMENT;   // every action touches a stay
      if (A.kind == SS_ACT_EVICT) {
        if (P->spill_offset[A.object] < 0 && !file_homed(*P, A.object)) return SS_INVALID_ARGUMENT;
        last_evict[A.object] = a; P->evict_order.push_back(a);
      } else if (A.kind == SS_ACT_FETCH) {
        if (P->spill_offset[A.object] < 0 && !file_homed(*P, A.object)) return SS_INVALID_ARGUMENT;
        P->action_prev_evict[a] = last_evict[A.object]; P->fetch_order.push_back(a);
      } else {
        P->release_order.push_back(a);
      }
    }
  }
  // events are created once here; steady-state steps create none
  P->task_fence.assign(d->n_tasks, nullptr);
  P->task_side_stream.assign(d->n_tasks, 0);
  P->action_event.assign(d->n_actions, nullptr);
  for (int32_t t = 0; t < d->n_tasks; ++t)
    if (int rc = new_event(rt, &P->task_fence[t])) { release_plan(rt, *P); return rc; }
  const int timed = rt->ring.empty() ? 0 : 1;   // tracing configured: events carry timestamps
  if (timed) P->action_begin_event.assign(d->n_actions, nullptr);
  for (int32_t a = 0; a < d->n_actions; ++a)
    if (P->actions[a].kind != SS_ACT_RELEASE) {
      if (int rc = new_event(rt, &P->action_event[a], timed)) { release_plan(rt, *P); return rc; }
      if (timed)
        if (int rc = new_event(rt, &P->action_begin_event[a], 1)) { release_plan(rt, *P); return rc; }
    }
  if (int rc = new_event(rt, &P->step_event)) { release_plan(rt, *P); return rc; }
  if (timed)
    if (int rc = new_event(rt, &P->step_begin_event, 1)) { release_plan(rt, *P); return rc; }
  P->action_issued = std::vector<std::atomic<int>>(d->n_actions);
  P->action_durable = std::vector<std::atomic<int>>(d->n_actions);
  P->jobs.resize(d->n_actions);
  for (int32_t a = 0; a < d->n_actions; ++a)
    if (P->actions[a].kind != SS_ACT_RELEASE && file_homed(*P, P->actions[a].object))
      P->jobs[a] = std::make_unique<ssc::StagedJob>();
  P->object_current.assign(d->n_objects, -1);
  std::lock_guard<std::mutex> lk(rt->mu);
  P->id = rt->next_plan++;
  *plan_id = P->id;
  rt->plans[P->id] = std::move(P);
  return SS_OK;
}

int ss_plan_close(ss_runtime* rt, int32_t plan_id) {
  if (!rt) return SS_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lk(rt->mu);
  PlanState* P = find_plan(rt, plan_id);
  if (!P) return SS_INVALID_ARGUMENT;
  if (P->active) return SS_INVALID_ARGUMENT;
  release_plan(rt, *P);
  rt->plans.erase(plan_id);
  return SS_OK;
}

int ss_step_begin(ss_runtime* rt, int32_t plan_id, void* compute_stream) {
  if (!rt) return SS_INVALID_ARGUMENT;
  if (rt->closed.load()) return SS_CLOSED;
  if (rt->failed.load()) return SS_FAILED;
  {
    std::lock_guard<std::mutex> lk(rt->mu);
    PlanState* P = find_plan(rt, plan_id);
    if (!P || P->active) return SS_INVALID_ARGUMENT;
    for (auto& I : P->intervals) {
      I->ready_event = nullptr; I->release_event = nullptr;
      I->ready_issued = 0; I->released = 0; I->release_on_compute = false;
    }
    for (auto& f : P->action_issued) f = 0;
    for (auto& f : P->action_durable) f = 0;
    std::fill(P->task_side_stream.begin(), P->task_side_stream.end(), 0);
    P->staged_pending.store(0);
    std::fill(P->object_current.begin(), P->object_current.end(), -1);
    P->next_fetch = P->next_evict = P->next_release = 0;
    P->compute_stream = compute_stream;
    P->published_task.store(-1, std::memory_order_release);
    if (P->step_begin_event)
      rt->be->event_record(rt->be->self, P->step_begin_event, compute_stream);
    P->active = true;
  }
  rt->st_steps++;
  rt->trace(SS_TRACE_STEP_BEGIN, plan_id, 0);
  rt->cv.notify_all();
  return SS_OK;
}

int ss_before_task(ss_runtime* rt, int32_t plan_id, int32_t task, void** ptrs, int32_t max_ptrs) {
  return ss_before_task_on(rt, plan_id, task, ptrs, max_ptrs, nullptr);
}

// `stream`: the stream the task's kernels will run on (null = the step's compute stream). The waits
// for fetched inputs and for the previous occupants of created ranges are enqueued there. A task on
// a side stream is ordered against compute work by its caller; the runtime orders it against
// transfers and range reuse.
int ss_before_task_on(ss_runtime* rt, int32_t plan_id, int32_t task, void** ptrs, int32_t max_ptrs,
                      void* stream) {
  if (!rt) return SS_INVALID_ARGUMENT;
  if (rt->failed.load()) return SS_FAILED;
  PlanState* P;
  { std::lock_guard<std::mutex> lk(rt->mu); P = find_plan(rt, plan_id); }
  if (!P || !P->active || task < 0 || task >= P->n_tasks) return SS_INVALID_ARGUMENT;
  ss_backend* be = rt->be;
  void* const task_stream = stream ? stream : P->compute_stream;
  const bool side = task_stream != P->compute_stream;
  // stays this task opens: wait for the previous occupants of their ranges
  for (int32_t ii : P->task_creates[task]) {
    IntervalState& I = *P->intervals[ii];
    for (int32_t k = P->pred_begin[ii]; k < P->pred_begin[ii + 1]; ++k) {
      IntervalState& J = *P->intervals[P->pred_index[k]];
      if (!wait_flag(rt, J.released))
        return rt->latch(SS_FAIL_CAPACITY, SS_NO_PROGRESS, task, I.iv.object, -1, 0,
                         "range predecessor never released");
      if (J.release_event && (side || !J.release_on_compute)) {
        int rc = be->stream_wait_event(be->self, task_stream, J.release_event);
        if (rc != SS_OK) return rt->latch(SS_FAIL_BACKEND_EVENT, rc, task, I.iv.object, -1, 0, "stream wait failed");
        rt->trace(SS_TRACE_REUSE_WAIT, task, I.iv.bytes);
      }
    }
    P->object_current[I.iv.object] = ii;
  }
  int32_t n = 0;
  for (int32_t i = P->task_use_begin[task]; i < P->task_use_begin[task + 1]; ++i, ++n) {
    const ssc::Use& u = P->uses[i];
    int32_t ii = P->object_current[u.object];
    if (u.mode != SS_USE_CREATE) {
      // the stay may be one a fetch opens: find it through the worker's issue flag
      if (ii < 0 || P->intervals[ii]->released.load(std::memory_order_acquire)) {
        ii = -1;
        for (int32_t f = 0; f < static_cast<int32_t>(P->fetch_order.size()); ++f) {
          const int32_t a = P->fetch_order[f];
          const int32_t cand = P->action_interval[a];
          if (P->actions[a].object == u.object && P->actions[a].trigger_task < task &&
              !(P->intervals[cand]->iv.end_action >= 0 &&
                P->actions[P->intervals[cand]->iv.end_action].trigger_task < task))
            ii = cand;
        }
        if (ii < 0)
          return rt->latch(SS_FAIL_OBJECT_STATE, SS_INVALID_ARGUMENT, task, u.object, -1, 0,
                           "task input has no device stay");
        P->object_current[u.object] = ii;
      }
      IntervalState& I = *P->intervals[ii];
      if (I.iv.begin_action >= 0) {
        if (!wait_flag(rt, I.ready_issued))
          return rt->latch(SS_FAIL_CAPACITY, SS_NO_PROGRESS, task, u.object, I.iv.begin_action, 0,
                           "fetch was never issued");
        int rc = be->stream_wait_event(be->self, task_stream, I.ready_event);
        if (rc != SS_OK) return rt->latch(SS_FAIL_BACKEND_EVENT, rc, task, u.object, -1, 0, "stream wait failed");
        rt->trace(SS_TRACE_INPUT_WAIT, task, I.iv.bytes);
      }
    }
    if (ptrs && n < max_ptrs) ptrs[n] = rt->dev(P->intervals[ii]->iv.offset);
  }
  rt->trace(SS_TRACE_TASK_BEGIN, task, 0);
  return SS_OK;
}

int ss_after_task(ss_runtime* rt, int32_t plan_id, int32_t task) {
  return ss_after_task_on(rt, plan_id, task, nullptr);
}

int ss_after_task_on(ss_runtime* rt, int32_t plan_id, int32_t task, void* stream) {
  if (!rt) return SS_INVALID_ARGUMENT;
  if (rt->failed.load()) return SS_FAILED;
  PlanState* P;
  { std::lock_guard<std::mutex> lk(rt->mu); P = find_plan(rt, plan_id); }
  if (!P || !P->active || task < 0 || task >= P->n_tasks) return SS_INVALID_ARGUMENT;
  void* const task_stream = stream ? stream : P->compute_stream;
  P->task_side_stream[task] = task_stream != P->compute_stream;
  int rc = rt->be->event_record(rt->be->self, P->task_fence[task], task_stream);
  if (rc != SS_OK) return rt->latch(SS_FAIL_BACKEND_EVENT, rc, task, -1, -1, 0, "fence record failed");
  rt->st_tasks++;
  rt->trace(SS_TRACE_TASK_END, task, 0);
  P->published_task.store(task, std::memory_order_release);
  rt->cv.notify_all();
  return SS_OK;
}

int ss_step_end(ss_runtime* rt, int32_t plan_id) {
  if (!rt) return SS_INVALID_ARGUMENT;
  PlanState* P;
  { std::lock_guard<std::mutex> lk(rt->mu); P = find_plan(rt, plan_id); }
  if (!P || !P->active) return SS_INVALID_ARGUMENT;
  const int64_t t0 = ss_monotonic_ns();
  int result = SS_OK;
  for (;;) {
    bool done;
    {
      std::lock_guard<std::mutex> lk(rt->mu);
      done = P->next_fetch == P->fetch_order.size() && P->next_evict == P->evict_order.size() &&
             P->next_release == P->release_order.size() && P->staged_pending.load() == 0;
    }
    if (done) break;
    if (rt->failed.load()) { result = SS_FAILED; break; }
    if (ss_monotonic_ns() - t0 > HOST_WAIT_NS) {
      result = rt->latch(SS_FAIL_PLAN, SS_NO_PROGRESS, -1, -1, -1, 0, "step never drained");
      break;
    }
    rt->cv.notify_all();
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  ss_backend* be = rt->be;
  if (result == SS_OK) {
    int rc = be->stream_synchronize(be->self, rt->fetch_stream);
    if (rc == SS_OK) rc = be->stream_synchronize(be->self, rt->evict_stream);
    if (rc == SS_OK && P->compute_stream) rc = be->stream_synchronize(be->self, P->compute_stream);
    if (rc != SS_OK) result = rt->latch(SS_FAIL_BACKEND_EVENT, rc, -1, -1, -1, 0, "drain failed");
  }
  {
    std::lock_guard<std::mutex> lk(rt->mu);
    P->active = false;
  }
  rt->trace(SS_TRACE_STEP_END, plan_id, 0);
  if (rt->failed.load()) return SS_FAILED;
  return result;
}

int ss_step_abandon(ss_runtime* rt, int32_t plan_id, const char* why) {
  if (!rt) return SS_INVALID_ARGUMENT;
  PlanState* P;
  { std::lock_guard<std::mutex> lk(rt->mu); P = find_plan(rt, plan_id); }
  if (!P) return SS_INVALID_ARGUMENT;
  if (!P->active) return SS_OK;
  rt->latch(SS_FAIL_EXTERNAL, SS_FAILED, -1, -1, -1, 0, why ? why : "step abandoned by the caller");
  rt->cv.notify_all();
  ss_backend* be = rt->be;
  be->stream_synchronize(be->self, rt->fetch_stream);
  be->stream_synchronize(be->self, rt->evict_stream);
  if (P->compute_stream) be->stream_synchronize(be->self, P->compute_stream);
  {
    std::lock_guard<std::mutex> lk(rt->mu);
    P->active = false;
  }
  rt->trace(SS_TRACE_STEP_END, plan_id, 1);
  return SS_OK;
}

int32_t ss_plan_transfer_times(ss_runtime* rt, int32_t plan_id, int64_t* begin_ns, int64_t* end_ns,
                               int32_t capacity) {
  if (!rt || !begin_ns || !end_ns) return -1;
  PlanState* P;
  { std::lock_guard<std::mutex> lk(rt->mu); P = find_plan(rt, plan_id); }
  if (!P || P->active || !P->step_begin_event) return -1;
  ss_backend* be = rt->be;
  be->stream_synchronize(be->self, rt->fetch_stream);
  be->stream_synchronize(be->self, rt->evict_stream);
  const int32_t n = std::min<int32_t>(capacity, static_cast<int32_t>(P->actions.size()));
  for (int32_t a = 0; a < n; ++a) {
    begin_ns[a] = end_ns[a] = -1;
    if (!P->action_event[a] || !P->action_issued[a].load(std::memory_order_acquire)) continue;
    int64_t b = 0, e = 0;
    if (be->event_elapsed_ns(be->self, P->step_begin_event, P->action_begin_event[a], &b) == SS_OK &&
        be->event_elapsed_ns(be->self, P->step_begin_event, P->action_event[a], &e) == SS_OK) {
      begin_ns[a] = b; end_ns[a] = e;
    }
  }
  return static_cast<int32_t>(P->actions.size());
}

int ss_runtime_wait_idle(ss_runtime* rt) {
  if (!rt) return SS_INVALID_ARGUMENT;
  ss_backend* be = rt->be;
  int rc = be->stream_synchronize(be->self, rt->fetch_stream);
  if (rc == SS_OK) rc = be->stream_synchronize(be->self, rt->evict_stream);
  return rc;
}

int ss_spill_write(ss_runtime* rt, int64_t off, const void* src, int64_t bytes) {
  if (!rt || off < 0 || bytes < 0 || off + bytes > rt->cfg.spill_bytes) return SS_INVALID_ARGUMENT;
  std::memcpy(rt->spill(off), src, static_cast<size_t>(bytes));
  return SS_OK;
}
int ss_spill_read(ss_runtime* rt, int64_t off, void* dst, int64_t bytes) {
  if (!rt || off < 0 || bytes < 0 || off + bytes > rt->cfg.spill_bytes) return SS_INVALID_ARGUMENT;
  std::memcpy(dst, rt->spill(off), static_cast<size_t>(bytes));
  return SS_OK;
}

int ss_calibrate_transfers(ss_runtime* rt, int64_t bytes, int32_t repeats, ss_transfer_profile* out) {
  if (!rt || !out || bytes <= 0 || bytes > rt->cfg.device_bytes / 2 || bytes > rt->cfg.spill_bytes / 2)
    return SS_INVALID_ARGUMENT;
  if (repeats <= 0) repeats = 3;
  ss_backend* be = rt->be;
  auto time_copy = [&](bool fetch, bool with_other, int64_t n) -> double {
    double best = 1e30;
    for (int r = 0; r < repeats; ++r) {
      be->stream_synchronize(be->self, rt->fetch_stream);
      be->stream_synchronize(be->self, rt->evict_stream);
      if (with_other) {
        if (fetch) be->copy_async(be->self, rt->spill(bytes), rt->dev(bytes), static_cast<size_t>(bytes), SS_COPY_D2H, rt->evict_stream);
        else be->copy_async(be->self, rt->dev(bytes), rt->spill(bytes), static_cast<size_t>(bytes), SS_COPY_H2D, rt->fetch_stream);
      }
      const int64_t t0 = ss_monotonic_ns();
      if (fetch) {
        be->copy_async(be->self, rt->dev(0), rt->spill(0), static_cast<size_t>(n), SS_COPY_H2D, rt->fetch_stream);
        be->stream_synchronize(be->self, rt->fetch_stream);
      } else {
        be->copy_async(be->self, rt->spill(0), rt->dev(0), static_cast<size_t>(n), SS_COPY_D2H, rt->evict_stream);
        be->stream_synchronize(be->self, rt->evict_stream);
      }
      best = std::min(best, static_cast<double>(ss_monotonic_ns() - t0));
    }
    return best;
  };
  const double lat_f = time_copy(true, false, 64), lat_e = time_copy(false, false, 64);
  const double f_solo = time_copy(true, false, bytes), e_solo = time_copy(false, false, bytes);
  const double f_conc = time_copy(true, true, bytes), e_conc = time_copy(false, true, bytes);
  auto rate = [&](double ns, double lat) { return static_cast<double>(bytes) / std::max(ns - lat, 1.0) * 1e9; };
  out->fetch_latency_ns = static_cast<int64_t>(lat_f);
  out->evict_latency_ns = static_cast<int64_t>(lat_e);
  out->fetch_solo_bps = rate(f_solo, lat_f);
  out->evict_solo_bps = rate(e_solo, lat_e);
  out->fetch_concurrent_bps = std::min(rate(f_conc, lat_f), out->fetch_solo_bps);
  out->evict_concurrent_bps = std::min(rate(e_conc, lat_e), out->evict_solo_bps);
  return SS_OK;
}

int ss_file_write(ss_runtime* rt, int64_t off, const void* src, int64_t bytes) {
  if (!rt || !rt->store) return SS_INVALID_ARGUMENT;
  return rt->store->write(off, src, bytes);
}
int ss_file_read(ss_runtime* rt, int64_t off, void* dst, int64_t bytes) {
  if (!rt || !rt->store) return SS_INVALID_ARGUMENT;
  return rt->store->read(off, dst, bytes);
}
int ss_runtime_file_info(ss_runtime* rt, int32_t* direct, int64_t* ring_bytes) {
  if (!rt || !rt->store) return SS_INVALID_ARGUMENT;
  if (direct) *direct = rt->local_file.direct() ? 1 : 0;
  if (ring_bytes) *ring_bytes = rt->fetch_lane ? rt->fetch_lane->ring_bytes() : 0;
  return SS_OK;
}

int ss_calibrate_file_transfers(ss_runtime* rt, int64_t bytes, int32_t repeats, ss_transfer_profile* out) {
  if (!rt || !out || !rt->store || bytes <= 0 || bytes > rt->cfg.device_bytes / 2 ||
      bytes > rt->store->bytes() / 2)
    return SS_INVALID_ARGUMENT;
  if (repeats <= 0) repeats = 3;
  ss_backend* be = rt->be;
  // the worker only pumps the lanes while it holds this mutex: keep it out for the duration
  std::lock_guard<std::mutex> lk(rt->mu);
  for (auto& kv : rt->plans) if (kv.second->active) return SS_INVALID_ARGUMENT;
  bool failed = false;
  auto time_job = [&](bool fetch, bool with_other, int64_t n) -> double {
    double best = 1e30;
    for (int r = 0; r < repeats && !failed; ++r) {
      be->stream_synchronize(be->self, rt->fetch_stream);
      be->stream_synchronize(be->self, rt->evict_stream);
      ssc::StagedJob main_job, other_job;
      main_job.to_device = fetch; main_job.file_off = 0; main_job.dev = rt->dev(0); main_job.bytes = n;
      other_job.to_device = !fetch; other_job.file_off = bytes; other_job.dev = rt->dev(bytes); other_job.bytes = bytes;
      ssc::StagedLane* main_lane = fetch ? rt->fetch_lane.get() : rt->evict_lane.get();
      ssc::StagedLane* other_lane = fetch ? rt->evict_lane.get() : rt->fetch_lane.get();
      if (with_other) other_lane->submit(&other_job);
      const int64_t t0 = ss_monotonic_ns();
      main_lane->submit(&main_job);
      int64_t t_done = 0;
      while (main_lane->busy() || (with_other && other_lane->busy())) {
        if (main_lane->pump() < 0 || (with_other && other_lane->pump() < 0)) { failed = true; break; }
        if (!t_done && !main_lane->busy()) {
          if (fetch) be->stream_synchronize(be->self, rt->fetch_stream);
          t_done = ss_monotonic_ns();
        }
        if (ss_monotonic_ns() - t0 > HOST_WAIT_NS) { failed = true; break; }
        std::this_thread::yield();
      }
      if (!t_done) {
        if (fetch) be->stream_synchronize(be->self, rt->fetch_stream);
        t_done = ss_monotonic_ns();
      }
      best = std::min(best, static_cast<double>(t_done - t0));
    }
    return best;
  };
  const int64_t small = ssc::DIRECT_ALIGN;
  const double lat_f = time_job(true, false, small), lat_e = time_job(false, false, small);
  const double e_solo = time_job(false, false, bytes), f_solo = time_job(true, false, bytes);
  const double f_conc = time_job(true, true, bytes), e_conc = time_job(false, true, bytes);
  be->stream_synchronize(be->self, rt->fetch_stream);
  be->stream_synchronize(be->self, rt->evict_stream);
  if (failed) {
    // the lanes may still hold this call's jobs: make sure nobody pumps them again
    rt->latch(SS_FAIL_BACKEND_COPY, SS_IO_ERROR, -1, -1, -1, 2, "calibration of the staged lanes failed");
    return SS_IO_ERROR;
  }
  auto rate = [&](double ns, double lat) { return static_cast<double>(bytes) / std::max(ns - lat, 1.0) * 1e9; };
  out->fetch_latency_ns = static_cast<int64_t>(lat_f);
  out->evict_latency_ns = static_cast<int64_t>(lat_e);
  out->fetch_solo_bps = rate(f_solo, lat_f);
  out->evict_solo_bps = rate(e_solo, lat_e);
  out->fetch_concurrent_bps = std::min(rate(f_conc, lat_f), out->fetch_solo_bps);
  out->evict_concurrent_bps = std::min(rate(e_conc, lat_e), out->evict_solo_bps);
  return SS_OK;
}

}  // extern "C"
