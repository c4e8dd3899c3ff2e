// Deterministic discrete-event replay of (program, schedule, device config).
//
// One compute resource runs the tasks in order. Two serial lanes move data:
// fetch (spill -> device) and evict (device -> spill); each lane's rate drops to
// its "concurrent" value while the other lane is moving bytes. A fetch reserves
// its destination when it reaches the head of its lane (it waits there for
// capacity, it does not fail); a created object and the task workspace are
// reserved when the task starts. The replay reports when every task and action
// ran, every device stay of every object, and where time was lost.
//
// Behavioural model: the reference's C simulator
// (packages/engine/csrc/src/simulator/simulator.c:27-88, transfers.c, memory.c).
#include "common.hpp"

#include <deque>
#include <limits>

namespace ssc {

int unpack_program(const ss_program* p, ProgramView& out) {
  if (!p || p->n_tasks < 0 || p->n_objects < 0 || p->n_uses < 0) return SS_INVALID_ARGUMENT;
  out.n_tasks = p->n_tasks;
  out.n_objects = p->n_objects;
  out.duration.assign(p->task_duration_ns, p->task_duration_ns + p->n_tasks);
  if (p->task_workspace_bytes)
    out.workspace.assign(p->task_workspace_bytes, p->task_workspace_bytes + p->n_tasks);
  else
    out.workspace.assign(p->n_tasks, 0);
  out.bytes.assign(p->object_bytes, p->object_bytes + p->n_objects);
  if (p->object_flags)
    out.flags.assign(p->object_flags, p->object_flags + p->n_objects);
  else
    out.flags.assign(p->n_objects, 0);
  out.uses.resize(p->n_uses);
  int32_t prev_task = 0;
  for (int32_t i = 0; i < p->n_uses; ++i) {
    Use u{p->use_task[i], p->use_object[i], p->use_mode[i]};
    if (u.task < 0 || u.task >= p->n_tasks || u.object < 0 || u.object >= p->n_objects ||
        u.mode < 0 || u.mode > 2 || u.task < prev_task)
      return SS_INVALID_ARGUMENT;
    prev_task = u.task;
    out.uses[i] = u;
  }
  out.task_use_begin.assign(p->n_tasks + 1, 0);
  for (auto& u : out.uses) out.task_use_begin[u.task + 1]++;
  for (int32_t t = 0; t < p->n_tasks; ++t) out.task_use_begin[t + 1] += out.task_use_begin[t];
  out.object_uses.assign(p->n_objects, {});
  for (int32_t i = 0; i < p->n_uses; ++i) out.object_uses[out.uses[i].object].push_back(i);
  for (int64_t b : out.bytes)
    if (b < 0) return SS_INVALID_ARGUMENT;
  return SS_OK;
}

namespace {

struct Lane {
  std::deque<int32_t> queue;   // action indices in issue order
  int32_t current = -1;
  int64_t latency_left = 0;
  double bytes_left = 0.0;
  int64_t busy_ns = 0;
  bool moving() const { return current >= 0 && latency_left == 0 && bytes_left > 0.0; }
};

struct ObjState {
  bool resident = false;   // device bytes reserved
  bool ready = false;      // device copy valid
  bool fetching = false;
  bool evicting = false;
  int32_t open_interval = -1;
};

}  // namespace

int simulate(const ProgramView& pv, const ss_device_config& cfg, const ss_action* actions,
             int32_t n_actions, SimOutput& out) {
  const int32_t nt = pv.n_tasks, no = pv.n_objects;
  out.task_start.assign(nt, -1);
  out.task_end.assign(nt, -1);
  out.action_start.assign(n_actions, -1);
  out.action_end.assign(n_actions, -1);
  out.intervals.clear();
  ss_sim_result& R = out.result;
  R = ss_sim_result{};
  R.stalled_task = -1;
  for (int32_t t = 0; t < nt; ++t) R.compute_ns += pv.duration[t];

  // actions grouped by trigger task (+1 so that -1 maps to slot 0)
  std::vector<std::vector<int32_t>> by_trigger(nt + 1);
  for (int32_t a = 0; a < n_actions; ++a) {
    const ss_action& A = actions[a];
    if (A.object < 0 || A.object >= no || A.trigger_task < -1 || A.trigger_task >= nt ||
        A.kind < 0 || A.kind > 2)
      return SS_INVALID_ARGUMENT;
    by_trigger[A.trigger_task + 1].push_back(a);
  }

  std::vector<ObjState> st(no);
  Lane fetch, evict;
  int64_t used = 0, now = 0;
  int32_t ti = 0;
  bool running = false;
  int64_t run_end = 0;
  const int64_t cap = cfg.capacity_bytes;

  auto open_interval = [&](int32_t o, int32_t begin_action, int32_t begin_task) {
    ss_interval iv{};
    iv.object = o; iv.begin_action = begin_action; iv.begin_task = begin_task; iv.end_action = -1;
    iv.bytes = pv.bytes[o]; iv.start_ns = now; iv.end_ns = -1; iv.offset = -1;
    st[o].open_interval = static_cast<int32_t>(out.intervals.size());
    out.intervals.push_back(iv);
  };
  auto free_object = [&](int32_t o, int32_t end_action) {
    ObjState& s = st[o];
    if (!s.resident) return;
    s.resident = false; s.ready = false;
    used -= pv.bytes[o];
    if (s.open_interval >= 0) {
      out.intervals[s.open_interval].end_ns = now;
      out.intervals[s.open_interval].end_action = end_action;
      s.open_interval = -1;
    }
  };
  auto fire = [&](int32_t slot) -> int {
    for (int32_t a : by_trigger[slot]) {
      const ss_action& A = actions[a];
      if (A.kind == SS_ACT_RELEASE) {
        if (!st[A.object].resident || st[A.object].evicting || st[A.object].fetching)
          return SS_INVALID_ARGUMENT;
        out.action_start[a] = out.action_end[a] = now;
        free_object(A.object, a);
      } else if (A.kind == SS_ACT_FETCH) {
        fetch.queue.push_back(a);
      } else {
        evict.queue.push_back(a);
      }
    }
    return SS_OK;
  };
  if (int rc = fire(0)) return rc;

  int64_t wait_since = -1;      // compute idle since, -1 = not waiting
  bool wait_capacity = false;

  const int64_t INF = std::numeric_limits<int64_t>::max();
  for (;;) {
    // ---- lanes: start the head transfer when possible
    if (fetch.current < 0 && !fetch.queue.empty()) {
      const int32_t a = fetch.queue.front();
      const int32_t o = actions[a].object;
      bool blocked = false;
      if (st[o].resident) {
        // the previous stay is still draining to spill: the fetch waits behind that evict
        bool draining = st[o].evicting;
        for (int32_t e : evict.queue) if (actions[e].object == o) { draining = true; break; }
        if (!draining) return SS_INVALID_ARGUMENT;   // fetched twice
        blocked = true;
      }
      if (!blocked && used + pv.bytes[o] <= cap) {
        fetch.queue.pop_front();
        fetch.current = a;
        fetch.latency_left = cfg.fetch_latency_ns;
        fetch.bytes_left = static_cast<double>(pv.bytes[o]);
        used += pv.bytes[o];
        R.peak_bytes = std::max(R.peak_bytes, used);
        st[o].resident = true; st[o].fetching = true;
        out.action_start[a] = now;
        open_interval(o, a, actions[a].trigger_task);
        R.fetch_bytes += pv.bytes[o];
      }
    }
    if (evict.current < 0 && !evict.queue.empty()) {
      const int32_t a = evict.queue.front();
      const int32_t o = actions[a].object;
      if (!st[o].resident || !st[o].ready) return SS_INVALID_ARGUMENT;
      evict.queue.pop_front();
      evict.current = a;
      evict.latency_left = cfg.evict_latency_ns;
      evict.bytes_left = static_cast<double>(pv.bytes[o]);
      st[o].evicting = true;
      out.action_start[a] = now;
      R.evict_bytes += pv.bytes[o];
    }
    // ---- compute: start the next task when its inputs and memory are there
    if (!running && ti < nt) {
      bool inputs_ok = true, impossible = false;
      int64_t need = pv.workspace[ti];
      for (int32_t i = pv.task_use_begin[ti]; i < pv.task_use_begin[ti + 1]; ++i) {
        const Use& u = pv.uses[i];
        const ObjState& s = st[u.object];
        if (u.mode == SS_USE_CREATE) {
          if (s.resident) { impossible = true; break; }
          need += pv.bytes[u.object];
        } else if (!(s.resident && s.ready) || s.evicting) {
          inputs_ok = false;
          if (!s.fetching) {
            // is a fetch for it still queued?
            bool queued = false;
            for (int32_t a : fetch.queue) if (actions[a].object == u.object) { queued = true; break; }
            if (!queued) impossible = true;
          }
        }
      }
      if (impossible) {
        R.status = SS_NO_PROGRESS; R.stalled_task = ti; R.makespan_ns = now;
        return SS_OK;
      }
      const bool mem_ok = used + need <= cap;
      if (inputs_ok && mem_ok) {
        if (wait_since >= 0) {
          (wait_capacity ? R.capacity_wait_ns : R.input_wait_ns) += now - wait_since;
          wait_since = -1;
        }
        for (int32_t i = pv.task_use_begin[ti]; i < pv.task_use_begin[ti + 1]; ++i) {
          const Use& u = pv.uses[i];
          if (u.mode == SS_USE_CREATE) {
            st[u.object].resident = true; st[u.object].ready = true;
            used += pv.bytes[u.object];
            open_interval(u.object, -1, ti);
          }
        }
        used += pv.workspace[ti];
        R.peak_bytes = std::max(R.peak_bytes, used);
        running = true;
        out.task_start[ti] = now;
        run_end = now + pv.duration[ti];
      } else if (wait_since < 0) {
        wait_since = now;
        wait_capacity = inputs_ok && !mem_ok;
      }
    }
    // ---- next event
    const double frate = evict.moving() ? cfg.fetch_concurrent_bps : cfg.fetch_solo_bps;
    const double erate = fetch.moving() ? cfg.evict_concurrent_bps : cfg.evict_solo_bps;
    auto lane_finish = [&](const Lane& L, double rate) -> int64_t {
      if (L.current < 0) return INF;
      const double ns = rate > 0 ? L.bytes_left / rate * 1e9 : 0.0;
      return now + L.latency_left + static_cast<int64_t>(ns + 0.999999);
    };
    // a lane leaving its latency phase changes the other lane's rate: stop there too
    auto lane_phase = [&](const Lane& L) -> int64_t {
      return (L.current >= 0 && L.latency_left > 0) ? now + L.latency_left : INF;
    };
    int64_t next = running ? run_end : INF;
    next = std::min(next, lane_finish(fetch, frate));
    next = std::min(next, lane_finish(evict, erate));
    next = std::min(next, lane_phase(fetch));
    next = std::min(next, lane_phase(evict));
    if (next == INF) {
      if (ti >= nt && fetch.queue.empty() && evict.queue.empty()) break;   // finished
      R.status = SS_NO_PROGRESS; R.stalled_task = ti < nt ? ti : -1; R.makespan_ns = now;
      return SS_OK;
    }
    const int64_t dt = next - now;
    auto advance = [&](Lane& L, double rate) {
      if (L.current < 0) return;
      L.busy_ns += dt;
      int64_t d = dt;
      if (L.latency_left > 0) {
        const int64_t c = std::min(L.latency_left, d);
        L.latency_left -= c; d -= c;
      }
      if (d > 0 && L.latency_left == 0) L.bytes_left -= rate * static_cast<double>(d) / 1e9;
    };
    advance(fetch, frate);
    advance(evict, erate);
    now = next;
    // ---- completions
    if (fetch.current >= 0 && fetch.latency_left == 0 && fetch.bytes_left <= 0.5) {
      const int32_t a = fetch.current, o = actions[a].object;
      st[o].fetching = false; st[o].ready = true;
      out.action_end[a] = now;
      fetch.current = -1;
    }
    if (evict.current >= 0 && evict.latency_left == 0 && evict.bytes_left <= 0.5) {
      const int32_t a = evict.current, o = actions[a].object;
      st[o].evicting = false;
      out.action_end[a] = now;
      evict.current = -1;
      free_object(o, a);
    }
    if (running && now >= run_end) {
      running = false;
      out.task_end[ti] = now;
      used -= pv.workspace[ti];
      if (int rc = fire(ti + 1)) return rc;
      ++ti;
    }
  }
  R.makespan_ns = now;
  R.fetch_busy_ns = fetch.busy_ns;
  R.evict_busy_ns = evict.busy_ns;
  // anything still resident at the end is a schedule defect for persistent objects
  for (int32_t o = 0; o < no; ++o) {
    if (st[o].resident) {
      if (pv.persistent(o) && !pv.pinned_resident(o)) { R.status = SS_INVALID_ARGUMENT; }
      out.intervals[st[o].open_interval].end_ns = now;
    }
  }
  return SS_OK;
}

}  // namespace ssc

extern "C" {

int ss_simulate(const ss_program* program, const ss_device_config* config,
                const ss_action* actions, int32_t n_actions, ss_sim_result* result,
                int64_t* task_start, int64_t* task_end, int64_t* action_start,
                int64_t* action_end, ss_interval* intervals, int32_t max_intervals,
                int32_t* n_intervals) {
  if (!program || !config || !result || (n_actions > 0 && !actions)) return SS_INVALID_ARGUMENT;
  ssc::ProgramView pv;
  if (int rc = ssc::unpack_program(program, pv)) return rc;
  ssc::SimOutput out;
  if (int rc = ssc::simulate(pv, *config, actions, n_actions, out)) return rc;
  *result = out.result;
  auto copy = [](int64_t* dst, const std::vector<int64_t>& src) {
    if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(int64_t));
  };
  copy(task_start, out.task_start); copy(task_end, out.task_end);
  copy(action_start, out.action_start); copy(action_end, out.action_end);
  if (n_intervals) *n_intervals = static_cast<int32_t>(out.intervals.size());
  if (intervals) {
    const int32_t n = std::min<int32_t>(max_intervals, static_cast<int32_t>(out.intervals.size()));
    if (n > 0) std::memcpy(intervals, out.intervals.data(), n * sizeof(ss_interval));
  }
  return SS_OK;
}

int ss_check_schedule(const ss_program* program, const ss_action* actions, int32_t n_actions,
                      int32_t* bad_action, int32_t* bad_task) {
  if (bad_action) *bad_action = -1;
  if (bad_task) *bad_task = -1;
  ssc::ProgramView pv;
  if (int rc = ssc::unpack_program(program, pv)) return rc;
  // order-only replay: residency by task index, transfers instantaneous
  std::vector<char> resident(pv.n_objects, 0), dirty(pv.n_objects, 0);
  std::vector<std::vector<int32_t>> by_trigger(pv.n_tasks + 1);
  for (int32_t a = 0; a < n_actions; ++a) {
    if (actions[a].trigger_task < -1 || actions[a].trigger_task >= pv.n_tasks ||
        actions[a].object < 0 || actions[a].object >= pv.n_objects) {
      if (bad_action) *bad_action = a;
      return SS_INVALID_ARGUMENT;
    }
    by_trigger[actions[a].trigger_task + 1].push_back(a);
  }
  auto apply = [&](int32_t slot) -> int32_t {
    for (int32_t a : by_trigger[slot]) {
      const int32_t o = actions[a].object;
      if (actions[a].kind == SS_ACT_FETCH) {
        // a transient object can only come back after an evict gave it a spill copy
        if (resident[o] || (!pv.persistent(o) && dirty[o] != 2)) return a;
        resident[o] = 1;
      } else if (actions[a].kind == SS_ACT_EVICT) {
        if (!resident[o]) return a;
        resident[o] = 0; dirty[o] = 2;   // 2 = has a spill copy
      } else {
        if (!resident[o]) return a;
        if (pv.persistent(o) && dirty[o] == 1) return a;   // would lose an update
        resident[o] = 0;
      }
    }
    return -1;
  };
  int32_t bad = apply(0);
  if (bad >= 0) { if (bad_action) *bad_action = bad; return SS_INVALID_ARGUMENT; }
  for (int32_t t = 0; t < pv.n_tasks; ++t) {
    for (int32_t i = pv.task_use_begin[t]; i < pv.task_use_begin[t + 1]; ++i) {
      const ssc::Use& u = pv.uses[i];
      if (u.mode == SS_USE_CREATE) {
        if (resident[u.object]) { if (bad_task) *bad_task = t; return SS_INVALID_ARGUMENT; }
        resident[u.object] = 1; dirty[u.object] = 1;
      } else {
        if (!resident[u.object]) { if (bad_task) *bad_task = t; return SS_INVALID_ARGUMENT; }
        if (u.mode == SS_USE_MUTATE) dirty[u.object] = 1;
      }
    }
    bad = apply(t + 1);
    if (bad >= 0) { if (bad_action) *bad_action = bad; return SS_INVALID_ARGUMENT; }
  }
  for (int32_t o = 0; o < pv.n_objects; ++o) {
    if (pv.persistent(o) && resident[o] && !pv.pinned_resident(o)) return SS_INVALID_ARGUMENT;
    if (pv.persistent(o) && dirty[o] == 1) return SS_INVALID_ARGUMENT;
  }
  return SS_OK;
}

int64_t ss_transfer_duration_ns(int64_t bytes, double bytes_per_second, int64_t latency_ns) {
  return ssc::transfer_ns(bytes, bytes_per_second, latency_ns);
}

}  // extern "C"
