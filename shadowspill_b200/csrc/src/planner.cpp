// Memory-schedule search: keep / spill / re-fetch decisions for one resolved
// program under a device capacity.
//
// Per candidate (residency strategy x fetch rule):
//   Reduce   start with every object resident from first to last use; while the
//            task-granular pressure profile exceeds capacity, cut the gap (the
//            stretch between two consecutive uses of one object) that covers
//            the peak and ranks best under the strategy. The peak comes from a
//            segment tree over task boundaries (range add, leftmost maximum),
//            the best covering gap from an index of heaps keyed by the
//            strategy's lexicographic rank; a plain scanning reducer with the
//            same decisions stays selectable (options.linear_reduce).
//            Objects under the eviction threshold are not part of the problem:
//            they live in a resident slice reserved before reduction.
//   Emit     turn the surviving residency segments into fetch / evict / release
//            actions; fetch triggers follow the rule (demand, latest-safe,
//            packed-fifo, packed-fit).
//   Simulate replay with the event simulator.
//   Repair   pull late fetches earlier while the makespan improves. A schedule the
//            simulator cannot finish names the boundary that starved: the
//            boundary-pressure repair adds a request at that boundary (doubled
//            when it fails again) and reduces again; only when that is used up
//            is the whole capacity tightened.
//   Place    fixed-offset placement of the simulated device stays, slice objects
//            at static homes behind them; if the layout overruns, give capacity
//            back (capacity refinement) and retry.
// The best placed candidate by simulated makespan wins. Candidates run on a
// small thread pool.
//
// Behavioural model: the reference's PressureFit
// (packages/engine/csrc/src/planner/search/algorithms/pressurefit/candidates/search.c:850,
// docs/architecture/pressurefit.md:291-361,421-498,548-568).
#include "common.hpp"

#include <atomic>
#include <mutex>
#include <sstream>
#include <thread>

namespace ssc {
namespace {

struct Gap {            // stretch between use k and use k+1 of an object
  int32_t object;
  int32_t k;            // index into object_uses[object]
  int32_t t_prev, t_next;
  bool cut = false;
};

struct Candidate {
  int strategy, rule;
  int status = SS_INFEASIBLE;
  std::vector<ss_action> actions;
  SimOutput sim;
  int64_t logical_capacity = 0;
  int64_t span = 0;
  int repairs = 0;
  std::string trace;
};

// Pressure over task boundaries: range add, global maximum and its leftmost position, all O(log n).
struct PressureTree {
  int32_t n = 0, size = 1;
  std::vector<int64_t> mx, lazy;
  void build(const std::vector<int64_t>& a) {
    n = static_cast<int32_t>(a.size());
    size = 1;
    while (size < std::max(n, 1)) size <<= 1;
    mx.assign(2 * size, std::numeric_limits<int64_t>::min() / 4);
    lazy.assign(2 * size, 0);
    for (int32_t i = 0; i < n; ++i) mx[size + i] = a[i];
    for (int32_t i = size - 1; i >= 1; --i) mx[i] = std::max(mx[2 * i], mx[2 * i + 1]);
  }
  void add(int32_t lo, int32_t hi, int64_t v) { if (lo <= hi) add(1, 0, size - 1, lo, hi, v); }
  void add(int32_t node, int32_t l, int32_t r, int32_t lo, int32_t hi, int64_t v) {
    if (hi < l || r < lo) return;
    if (lo <= l && r <= hi) { mx[node] += v; lazy[node] += v; return; }
    const int32_t m = (l + r) / 2;
    add(2 * node, l, m, lo, hi, v);
    add(2 * node + 1, m + 1, r, lo, hi, v);
    mx[node] = std::max(mx[2 * node], mx[2 * node + 1]) + lazy[node];
  }
  int64_t peak() const { return mx[1]; }
  int32_t leftmost_peak() const {     // the position a left-to-right scan with ">" would return
    int32_t node = 1;
    int64_t want = mx[1];
    while (node < size) {
      want -= lazy[node];
      node = (mx[2 * node] == want) ? 2 * node : 2 * node + 1;
    }
    return node - size;
  }
};

// Gaps indexed by the boundary range their cut would relieve: a gap is stored on the O(log n)
// canonical nodes of a segment tree that cover [lo, hi], each node a max-heap under the strategy's
// lexicographic key. The best gap covering a boundary is the best heap top on the root-to-leaf
// path; gaps already cut are dropped lazily when they surface.
struct CutIndex {
  struct Entry { double key[3]; int32_t gap; };
  static bool worse(const Entry& a, const Entry& b) {     // heap order: the top is the best
    for (int i = 0; i < 3; ++i) if (a.key[i] != b.key[i]) return a.key[i] < b.key[i];
    return a.gap > b.gap;                                  // ties: the gap found first by a scan
  }
  int32_t size = 1;
  std::vector<std::vector<Entry>> heap;
  void init(int32_t n) {
    size = 1;
    while (size < std::max(n, 1)) size <<= 1;
    heap.assign(2 * size, {});
  }
  void insert(int32_t lo, int32_t hi, const Entry& e) {
    for (int32_t l = lo + size, r = hi + size + 1; l < r; l >>= 1, r >>= 1) {
      if (l & 1) push(l++, e);
      if (r & 1) push(--r, e);
    }
  }
  void push(int32_t node, const Entry& e) {
    heap[node].push_back(e);
    std::push_heap(heap[node].begin(), heap[node].end(), worse);
  }
  template <typename IsCut>
  int32_t best(int32_t point, IsCut is_cut) {
    int32_t found = -1;
    Entry top{};
    for (int32_t node = point + size; node >= 1; node >>= 1) {
      auto& h = heap[node];
      while (!h.empty() && is_cut(h.front().gap)) { std::pop_heap(h.begin(), h.end(), worse); h.pop_back(); }
      if (!h.empty() && (found < 0 || worse(top, h.front()))) { top = h.front(); found = top.gap; }
    }
    return found;
  }
};

struct Planner {
  const ProgramView& pv;
  ss_device_config cfg;
  ss_search_options opt;
  std::vector<int64_t> t_start;   // no-stall start time of each task; t_start[nt] = total

  Planner(const ProgramView& p, const ss_device_config& c, const ss_search_options& o)
      : pv(p), cfg(c), opt(o) {
    t_start.assign(pv.n_tasks + 1, 0);
    for (int32_t t = 0; t < pv.n_tasks; ++t) t_start[t + 1] = t_start[t] + pv.duration[t];
  }

  int64_t fetch_ns(int32_t o) const {
    return transfer_ns(pv.bytes[o], cfg.fetch_concurrent_bps > 0 ? cfg.fetch_concurrent_bps
                                                                 : cfg.fetch_solo_bps,
                       cfg.fetch_latency_ns);
  }
  int64_t evict_ns(int32_t o) const {
    return transfer_ns(pv.bytes[o], cfg.evict_concurrent_bps > 0 ? cfg.evict_concurrent_bps
                                                                 : cfg.evict_solo_bps,
                       cfg.evict_latency_ns);
  }
  // number of tasks before `t` whose durations cover `ns` (the lead a transfer needs)
  int32_t lead_tasks(int32_t t, int64_t ns) const {
    int32_t lead = 0;
    int64_t acc = 0;
    while (t - 1 - lead >= 0 && acc < ns) { acc += pv.duration[t - 1 - lead]; ++lead; }
    return std::max(lead, 1);
  }
  // number of tasks after `t` an evict of `ns` stays resident
  int32_t tail_tasks(int32_t t, int64_t ns) const {
    int32_t tail = 0;
    int64_t acc = 0;
    while (t + 1 + tail < pv.n_tasks && acc < ns) { acc += pv.duration[t + 1 + tail]; ++tail; }
    return tail;
  }
  bool cuttable(int32_t o) const {
    return !pv.pinned_resident(o) && pv.bytes[o] >= opt.minimum_object_bytes_evict_eligible;
  }
  // Objects under the eviction threshold are never cut: long-lived and small, the worst shape for
  // the placer. Each gets a static home in a slice behind the main layout; the slice is taken out
  // of the capacity before reduction, so these objects are not charged per boundary.
  // (docs/architecture/fixed-placement.md:68-90 of the reference.)
  bool in_resident_slice(int32_t o) const {
    return !opt.no_resident_slice && !pv.pinned_resident(o) && !pv.object_uses[o].empty() &&
           pv.bytes[o] < opt.minimum_object_bytes_evict_eligible;
  }
  int64_t resident_slice_bytes() const {
    int64_t total = 0;
    const int64_t al = std::max<int64_t>(cfg.alignment, 1);
    for (int32_t o = 0; o < pv.n_objects; ++o) if (in_resident_slice(o)) total += align_up(pv.bytes[o], al);
    return total;
  }
  // per-boundary pressure requests added by the boundary-pressure repair (empty = none)
  std::vector<int64_t> extra_pressure;
  int32_t use_task(int32_t o, int32_t k) const { return pv.uses[pv.object_uses[o][k]].task; }
  int32_t use_mode(int32_t o, int32_t k) const { return pv.uses[pv.object_uses[o][k]].mode; }

  // ------------------------------------------------------------------ Reduce
  // Returns false if capacity cannot be met. `gaps` gets its cut flags set.
  // `tight` drops the prefetch leads and evict tails from the pressure estimate:
  // the schedule then relies on lanes waiting for room instead of on slack.
  bool reduce(int64_t capacity, int strategy, bool tight, std::vector<Gap>& gaps,
              std::string* trace, std::vector<int32_t>* order = nullptr) const {
    return opt.linear_reduce ? reduce_linear(capacity, strategy, tight, gaps, trace, order)
                             : reduce_indexed(capacity, strategy, tight, gaps, trace, order);
  }

  // The gaps of every object, the uncut pressure profile, and per gap the boundary range a cut
  // would relieve with its ranking key under `strategy` (all static for one reduction).
  struct GapInfo { int32_t lo, hi; double key[3]; };
  void prepare(int strategy, bool tight, std::vector<Gap>& gaps, std::vector<GapInfo>& info,
               std::vector<int64_t>& pressure) const {
    const int32_t nt = pv.n_tasks;
    pressure.assign(nt, 0);
    for (int32_t t = 0; t < nt; ++t) pressure[t] = pv.workspace[t] + (extra_pressure.empty() ? 0 : extra_pressure[t]);
    auto add = [&](int32_t lo, int32_t hi, int64_t b) {
      lo = std::max(lo, 0); hi = std::min(hi, nt - 1);
      for (int32_t t = lo; t <= hi; ++t) pressure[t] += b;
    };
    gaps.clear();
    for (int32_t o = 0; o < pv.n_objects; ++o) {
      const auto& us = pv.object_uses[o];
      if (us.empty() || in_resident_slice(o)) continue;
      const int32_t first = use_task(o, 0), last = use_task(o, static_cast<int32_t>(us.size()) - 1);
      const bool created = use_mode(o, 0) == SS_USE_CREATE;
      const int32_t lo = (created || tight) ? first : first - lead_tasks(first, fetch_ns(o));
      add(lo, last, pv.bytes[o]);
      for (int32_t k = 0; k + 1 < static_cast<int32_t>(us.size()); ++k) {
        Gap g{o, k, use_task(o, k), use_task(o, k + 1)};
        if (g.t_next - g.t_prev > 1 && cuttable(o)) gaps.push_back(g);
      }
    }
    info.resize(gaps.size());
    for (size_t gi = 0; gi < gaps.size(); ++gi) {
      const Gap& g = gaps[gi];
      const int32_t tail = tight ? 0 : tail_tasks(g.t_prev, evict_ns(g.object));
      const int32_t lead = tight ? 0 : lead_tasks(g.t_next, fetch_ns(g.object));
      GapInfo& f = info[gi];
      f.lo = g.t_prev + 1 + tail; f.hi = g.t_next - lead - 1;
      const int64_t span_ns = t_start[g.t_next] - t_start[g.t_prev + 1];
      const double exposed = std::max<double>(0.0, static_cast<double>(
                                 evict_ns(g.object) + fetch_ns(g.object) - span_ns));
      if (strategy == SS_STRATEGY_STALL) {
        f.key[0] = -exposed; f.key[1] = static_cast<double>(pv.bytes[g.object]);
        f.key[2] = static_cast<double>(span_ns);
      } else {   // traffic: longest gaps first, so the fewest bytes move per byte-second freed
        f.key[0] = static_cast<double>(span_ns); f.key[1] = static_cast<double>(pv.bytes[g.object]);
        f.key[2] = -exposed;
      }
    }
  }

  // Same decisions as reduce_linear, with the peak from a segment tree and the best gap covering
  // it from an index of heaps: O((gaps + cuts) log^2 tasks) instead of O(cuts x (tasks + gaps)).
  bool reduce_indexed(int64_t capacity, int strategy, bool tight, std::vector<Gap>& gaps,
                      std::string* trace, std::vector<int32_t>* order) const {
    const int32_t nt = pv.n_tasks;
    std::vector<GapInfo> info;
    std::vector<int64_t> pressure;
    prepare(strategy, tight, gaps, info, pressure);
    PressureTree tree;
    tree.build(pressure);
    CutIndex index;
    index.init(nt);
    for (size_t gi = 0; gi < gaps.size(); ++gi) {
      const GapInfo& f = info[gi];
      if (f.lo > f.hi) continue;               // a cut would relieve nothing once lead and tail are kept
      CutIndex::Entry e{{f.key[0], f.key[1], f.key[2]}, static_cast<int32_t>(gi)};
      index.insert(std::max(f.lo, 0), std::min(f.hi, nt - 1), e);
    }
    int cuts = 0;
    while (nt > 0 && tree.peak() > capacity) {
      const int32_t peak = tree.leftmost_peak();
      const int32_t best = index.best(peak, [&](int32_t gi) { return gaps[gi].cut; });
      if (best < 0) {
        if (trace) { std::ostringstream s; s << "reduce: infeasible at task " << peak << " pressure "
                     << tree.peak() << " capacity " << capacity << "\n"; *trace += s.str(); }
        return false;
      }
      gaps[best].cut = true;
      if (order) order->push_back(best);
      tree.add(std::max(info[best].lo, 0), std::min(info[best].hi, nt - 1), -pv.bytes[gaps[best].object]);
      ++cuts;
    }
    if (trace) { std::ostringstream s; s << "reduce: capacity " << capacity << " cuts " << cuts
                 << " of " << gaps.size() << " gaps (indexed)\n"; *trace += s.str(); }
    return true;
  }

  bool reduce_linear(int64_t capacity, int strategy, bool tight, std::vector<Gap>& gaps,
                     std::string* trace, std::vector<int32_t>* order) const {
    const int32_t nt = pv.n_tasks;
    std::vector<int64_t> pressure(nt, 0);
    for (int32_t t = 0; t < nt; ++t)
      pressure[t] = pv.workspace[t] + (extra_pressure.empty() ? 0 : extra_pressure[t]);
    auto add = [&](int32_t lo, int32_t hi, int64_t b) {
      lo = std::max(lo, 0); hi = std::min(hi, nt - 1);
      for (int32_t t = lo; t <= hi; ++t) pressure[t] += b;
    };
    gaps.clear();
    for (int32_t o = 0; o < pv.n_objects; ++o) {
      const auto& us = pv.object_uses[o];
      if (us.empty() || in_resident_slice(o)) continue;
      const int32_t first = use_task(o, 0), last = use_task(o, static_cast<int32_t>(us.size()) - 1);
      const bool created = use_mode(o, 0) == SS_USE_CREATE;
      const int32_t lo = (created || tight) ? first : first - lead_tasks(first, fetch_ns(o));
      add(lo, last, pv.bytes[o]);
      for (int32_t k = 0; k + 1 < static_cast<int32_t>(us.size()); ++k) {
        Gap g{o, k, use_task(o, k), use_task(o, k + 1)};
        if (g.t_next - g.t_prev > 1 && cuttable(o)) gaps.push_back(g);
      }
    }
    int cuts = 0;
    for (;;) {
      int32_t peak = 0;
      for (int32_t t = 1; t < nt; ++t) if (pressure[t] > pressure[peak]) peak = t;
      if (nt == 0 || pressure[peak] <= capacity) break;
      int best = -1;
      double best_key[3] = {0, 0, 0};
      int32_t best_lo = 0, best_hi = -1;
      for (int gi = 0; gi < static_cast<int>(gaps.size()); ++gi) {
        Gap& g = gaps[gi];
        if (g.cut || !(g.t_prev < peak && peak < g.t_next)) continue;
        const int32_t tail = tight ? 0 : tail_tasks(g.t_prev, evict_ns(g.object));
        const int32_t lead = tight ? 0 : lead_tasks(g.t_next, fetch_ns(g.object));
        const int32_t lo = g.t_prev + 1 + tail, hi = g.t_next - lead - 1;
        if (!(lo <= peak && peak <= hi)) continue;   // cutting would not relieve the peak
        const int64_t span_ns = t_start[g.t_next] - t_start[g.t_prev + 1];
        const double exposed = std::max<double>(0.0, static_cast<double>(
                                   evict_ns(g.object) + fetch_ns(g.object) - span_ns));
        double key[3];
        if (strategy == SS_STRATEGY_STALL) {
          key[0] = -exposed; key[1] = static_cast<double>(pv.bytes[g.object]);
          key[2] = static_cast<double>(span_ns);
        } else {   // traffic: longest gaps first, so the fewest bytes move per byte-second freed
          key[0] = static_cast<double>(span_ns); key[1] = static_cast<double>(pv.bytes[g.object]);
          key[2] = -exposed;
        }
        if (best < 0 || key[0] > best_key[0] ||
            (key[0] == best_key[0] && (key[1] > best_key[1] ||
                                       (key[1] == best_key[1] && key[2] > best_key[2])))) {
          best = gi; best_lo = lo; best_hi = hi;
          std::copy(key, key + 3, best_key);
        }
      }
      if (best < 0) {
        if (trace) { std::ostringstream s; s << "reduce: infeasible at task " << peak << " pressure "
                     << pressure[peak] << " capacity " << capacity << "\n"; *trace += s.str(); }
        return false;
      }
      gaps[best].cut = true;
      if (order) order->push_back(best);
      add(best_lo, best_hi, -pv.bytes[gaps[best].object]);
      ++cuts;
    }
    if (trace) { std::ostringstream s; s << "reduce: capacity " << capacity << " cuts " << cuts
                 << " of " << gaps.size() << " gaps\n"; *trace += s.str(); }
    return true;
  }

  // ------------------------------------------------------------------ Emit
  struct FetchReq { int32_t object, need_task; int64_t dur; int32_t trigger; };

  void emit(const std::vector<Gap>& gaps, int rule, int64_t capacity,
            std::vector<ss_action>& actions) const {
    const int32_t nt = pv.n_tasks;
    // cut lookup: (object, k) -> cut
    std::vector<std::vector<char>> cut(pv.n_objects);
    for (int32_t o = 0; o < pv.n_objects; ++o) cut[o].assign(pv.object_uses[o].size(), 0);
    for (const Gap& g : gaps) if (g.cut) cut[g.object][g.k] = 1;

    std::vector<FetchReq> fetches;
    std::vector<ss_action> ends;     // evict / release, trigger known
    // residency estimate for packed rules (task-granular)
    std::vector<int64_t> pressure(nt, 0);
    for (int32_t t = 0; t < nt; ++t)
      pressure[t] = pv.workspace[t] + (extra_pressure.empty() ? 0 : extra_pressure[t]);
    auto add = [&](int32_t lo, int32_t hi, int64_t b) {
      lo = std::max(lo, 0); hi = std::min(hi, nt - 1);
      for (int32_t t = lo; t <= hi; ++t) pressure[t] += b;
    };
    for (int32_t o = 0; o < pv.n_objects; ++o) {
      const auto& us = pv.object_uses[o];
      const int32_t n = static_cast<int32_t>(us.size());
      if (n == 0) continue;
      bool spill_valid = pv.persistent(o);   // is the spill copy current?
      int32_t k = 0;
      while (k < n) {
        int32_t j = k;
        bool dirty = false;
        const bool created = (k == 0 && use_mode(o, 0) == SS_USE_CREATE);
        if (created) { dirty = true; spill_valid = false; }
        for (;;) {
          if (use_mode(o, j) == SS_USE_MUTATE) dirty = true;
          if (j + 1 < n && !cut[o][j]) ++j; else break;
        }
        const int32_t seg_first = use_task(o, k), seg_last = use_task(o, j);
        if (!created) fetches.push_back({o, seg_first, fetch_ns(o), -2});
        const bool more = (j + 1 < n);
        ss_action e{};
        e.object = o; e.trigger_task = seg_last;
        if (dirty && (more || pv.persistent(o))) { e.kind = SS_ACT_EVICT; spill_valid = true; }
        else { e.kind = SS_ACT_RELEASE; (void)spill_valid; }
        ends.push_back(e);
        const int32_t tail = e.kind == SS_ACT_EVICT ? tail_tasks(seg_last, evict_ns(o)) : 0;
        if (!in_resident_slice(o)) add(seg_first, seg_last + tail, pv.bytes[o]);   // the slice is outside `capacity`
        k = j + 1;
      }
    }
    // ---- fetch triggers
    auto task_ending_by = [&](int64_t when) -> int32_t {   // largest t with end(t) <= when, or -1
      int32_t t = static_cast<int32_t>(std::upper_bound(t_start.begin() + 1, t_start.end(), when) -
                                       (t_start.begin() + 1)) - 1;
      return std::min(t, nt - 1);
    };
    if (rule == SS_FETCH_DEMAND) {
      for (auto& f : fetches) f.trigger = f.need_task - 1;
    } else if (rule == SS_FETCH_LATEST_SAFE || rule == SS_FETCH_PACKED_FIT) {
      std::vector<int32_t> idx(fetches.size());
      for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int32_t>(i);
      std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) {
        return fetches[a].need_task > fetches[b].need_task;
      });
      int64_t lane_free = std::numeric_limits<int64_t>::max();
      const double margin = rule == SS_FETCH_PACKED_FIT ? 1.25 : 1.0;
      for (int32_t i : idx) {
        FetchReq& f = fetches[i];
        const int64_t deadline = t_start[f.need_task];
        const int64_t finish = std::min(deadline, lane_free);
        const int64_t start = finish - static_cast<int64_t>(static_cast<double>(f.dur) * margin);
        lane_free = start;
        int32_t trig = start <= 0 ? -1 : task_ending_by(start);
        trig = std::min(trig, f.need_task - 1);
        f.trigger = trig;
      }
      // capacity clamp, in need order: a prefetch may not sit in memory during a task
      // whose planned pressure has no room for it (it would starve that task's own
      // reservations and stall the step for good)
      std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) {
        return fetches[a].need_task < fetches[b].need_task;
      });
      for (int32_t i : idx) {
        FetchReq& f = fetches[i];
        int32_t trig = f.trigger;
        const int64_t charged = in_resident_slice(f.object) ? 0 : pv.bytes[f.object];
        for (int32_t t = f.need_task - 1; t > trig; --t) {
          if (t >= 0 && pressure[t] + charged > capacity) { trig = t; break; }
        }
        f.trigger = trig;
        add(trig + 1, f.need_task - 1, charged);
      }
    } else {   // PACKED_FIFO: as early as the pressure estimate allows, in need order
      std::vector<int32_t> idx(fetches.size());
      for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int32_t>(i);
      std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) {
        return fetches[a].need_task < fetches[b].need_task;
      });
      int32_t floor_trigger = -1;
      for (int32_t i : idx) {
        FetchReq& f = fetches[i];
        int32_t trig = f.need_task - 1;
        const int32_t min_lead = lead_tasks(f.need_task, f.dur);
        const int32_t max_lead = 4 * min_lead + 2;
        while (trig - 1 >= floor_trigger && trig - 1 >= -1 && (f.need_task - trig) < max_lead) {
          const int32_t t = trig;   // moving the trigger before task t makes it resident during t
          if (t >= 0 && pressure[t] + (in_resident_slice(f.object) ? 0 : pv.bytes[f.object]) > capacity) break;
          --trig;
        }
        f.trigger = trig;
        floor_trigger = std::max(floor_trigger, trig);
        add(trig + 1, f.need_task - 1, in_resident_slice(f.object) ? 0 : pv.bytes[f.object]);
      }
    }
    // ---- assemble in issue order: by trigger; releases, evicts, then fetches by need
    actions.clear();
    actions.reserve(fetches.size() + ends.size());
    struct Keyed { int32_t trig, cls, need; ss_action a; };
    std::vector<Keyed> all;
    for (auto& e : ends) all.push_back({e.trigger_task, e.kind == SS_ACT_RELEASE ? 0 : 1, 0, e});
    for (auto& f : fetches) {
      ss_action a{}; a.kind = SS_ACT_FETCH; a.object = f.object; a.trigger_task = std::max(f.trigger, -1);
      all.push_back({a.trigger_task, 2, f.need_task, a});
    }
    std::stable_sort(all.begin(), all.end(), [](const Keyed& x, const Keyed& y) {
      if (x.trig != y.trig) return x.trig < y.trig;
      if (x.cls != y.cls) return x.cls < y.cls;
      return x.need < y.need;
    });
    for (auto& k : all) actions.push_back(k.a);
    // the fetch lane is FIFO over the whole step: keep fetches in need order globally
    // (a later-needed fetch must never sit in front of an earlier-needed one)
    std::vector<int32_t> fpos;
    for (int32_t i = 0; i < static_cast<int32_t>(actions.size()); ++i)
      if (actions[i].kind == SS_ACT_FETCH) fpos.push_back(i);
    std::vector<std::pair<int32_t, ss_action>> fl;   // (need, action)
    {
      size_t fi = 0;
      for (auto& k : all) if (k.cls == 2) { fl.push_back({k.need, k.a}); ++fi; }
    }
    std::stable_sort(fl.begin(), fl.end(), [](auto& x, auto& y) { return x.first < y.first; });
    // triggers must be non-decreasing along the lane order
    int32_t run = -1;
    for (auto& f : fl) { run = std::max(run, f.second.trigger_task); f.second.trigger_task = run; }
    // rebuild
    all.erase(std::remove_if(all.begin(), all.end(), [](const Keyed& k) { return k.cls == 2; }),
              all.end());
    int32_t ord = 0;
    for (auto& f : fl) all.push_back({f.second.trigger_task, 2, ord++, f.second});
    std::stable_sort(all.begin(), all.end(), [](const Keyed& x, const Keyed& y) {
      if (x.trig != y.trig) return x.trig < y.trig;
      if (x.cls != y.cls) return x.cls < y.cls;
      return x.need < y.need;
    });
    actions.clear();
    for (auto& k : all) actions.push_back(k.a);
  }

  // ------------------------------------------------------------------ Repair
  // Pull the fetch that made a task wait earlier; keep the change if it helps.
  void repair(std::vector<ss_action>& actions, SimOutput& sim, int& repairs,
              std::string* trace) const {
    for (int iter = 0; iter < opt.max_repairs; ++iter) {
      if (sim.result.status != SS_OK || sim.result.input_wait_ns <= 0) break;
      // the task that waited longest for an input
      int32_t worst = -1; int64_t worst_wait = 0;
      for (int32_t t = 0; t < pv.n_tasks; ++t) {
        const int64_t ready = t == 0 ? 0 : sim.task_end[t - 1];
        const int64_t w = sim.task_start[t] - ready;
        if (w > worst_wait) { worst_wait = w; worst = t; }
      }
      if (worst < 0) break;
      // its latest-arriving fetched input
      int32_t act = -1; int64_t latest = -1;
      for (int32_t i = pv.task_use_begin[worst]; i < pv.task_use_begin[worst + 1]; ++i) {
        const int32_t o = pv.uses[i].object;
        for (int32_t a = 0; a < static_cast<int32_t>(actions.size()); ++a) {
          if (actions[a].kind == SS_ACT_FETCH && actions[a].object == o &&
              actions[a].trigger_task < worst && sim.action_end[a] <= sim.task_start[worst] &&
              sim.action_end[a] > latest) { latest = sim.action_end[a]; act = a; }
        }
      }
      if (act < 0) break;
      // move every fetch at or before `act` in lane order whose trigger is not yet at the
      // floor one task earlier: the lane is FIFO, so the backlog in front matters as much
      std::vector<ss_action> trial = actions;
      const int32_t shift = std::max<int32_t>(1, lead_tasks(worst, worst_wait));
      bool changed = false;
      int32_t seen = 0;
      for (int32_t a = static_cast<int32_t>(trial.size()) - 1; a >= 0 && seen < 8; --a) {
        if (trial[a].kind != SS_ACT_FETCH || a > act) continue;
        ++seen;
        const int32_t nt2 = std::max(-1, trial[a].trigger_task - shift);
        if (nt2 != trial[a].trigger_task) { trial[a].trigger_task = nt2; changed = true; }
      }
      if (!changed) break;
      std::stable_sort(trial.begin(), trial.end(), [](const ss_action& x, const ss_action& y) {
        return x.trigger_task < y.trigger_task;
      });
      SimOutput s2;
      if (simulate(pv, cfg_with(sim_capacity), trial.data(), static_cast<int32_t>(trial.size()), s2) != SS_OK)
        break;
      if (s2.result.status == SS_OK && s2.result.makespan_ns < sim.result.makespan_ns) {
        actions.swap(trial);
        sim = std::move(s2);
        ++repairs;
      } else {
        break;
      }
    }
    if (trace) { std::ostringstream s; s << "repair: " << repairs << " accepted, makespan "
                 << sim.result.makespan_ns << "\n"; *trace += s.str(); }
  }

  mutable int64_t sim_capacity = 0;
  ss_device_config cfg_with(int64_t capacity) const {
    ss_device_config c = cfg; c.capacity_bytes = capacity; return c;
  }

  // ------------------------------------------------------------------ one candidate
  void evaluate(Candidate& c) const {
    std::string* tr = opt.trace ? &c.trace : nullptr;
    if (tr) { std::ostringstream s; s << "candidate strategy=" << c.strategy << " rule=" << c.rule << "\n"; *tr += s.str(); }
    const int64_t step = opt.capacity_refinement_step > 0 ? opt.capacity_refinement_step
                                                          : (256ll << 20);
    // the resident slice is reserved up front; reduction and emission plan the rest
    const int64_t slice = resident_slice_bytes();
    int64_t logical = cfg.capacity_bytes - slice;
    Planner local = *this;        // per-candidate copy: boundary requests and the simulated capacity
    int pressure_repairs = 0, last_stalled = -1;
    int64_t request = 0;
    for (int attempt = 0; attempt < 24 + opt.max_repairs && logical > 0; ++attempt) {
      std::vector<Gap> gaps;
      if (!local.reduce(logical, c.strategy, false, gaps, tr) &&
          !local.reduce(logical, c.strategy, true, gaps, tr)) {
        if (!local.extra_pressure.empty() && request > 0 && last_stalled >= 0) {
          // an escalated boundary request that cannot be reduced is taken back; tighten instead
          local.extra_pressure[last_stalled] -= request;
          request = 0; last_stalled = -1; pressure_repairs = opt.max_repairs;
          logical -= std::min<int64_t>(step, std::max<int64_t>(logical / 16, 1));
          continue;
        }
        c.status = SS_INFEASIBLE; return;
      }
      std::vector<ss_action> actions;
      local.emit(gaps, c.rule, logical, actions);
      SimOutput sim;
      // simulate against the logical capacity plus the slice: lanes wait for room, nothing overflows
      local.sim_capacity = logical + slice;
      if (simulate(pv, cfg_with(logical + slice), actions.data(), static_cast<int32_t>(actions.size()), sim) != SS_OK ||
          sim.result.status != SS_OK) {
        const int32_t stalled = sim.result.stalled_task;
        if (tr) { std::ostringstream o; o << "simulate: no progress (status " << sim.result.status
                  << ", task " << stalled << ", t=" << sim.result.makespan_ns << ")\n"; *tr += o.str(); }
        if (stalled >= 0 && stalled < pv.n_tasks && pressure_repairs < opt.max_repairs) {
          // boundary-pressure repair: ask the reducer for more room at the boundary that starved,
          // doubling the request when the same boundary fails again
          if (local.extra_pressure.empty()) local.extra_pressure.assign(pv.n_tasks, 0);
          request = (stalled == last_stalled && request > 0) ? 2 * request
                                                             : std::max<int64_t>(logical / 32, 1);
          request = std::min(request, logical);
          local.extra_pressure[stalled] += request;
          last_stalled = stalled;
          ++pressure_repairs;
          if (tr) { std::ostringstream o; o << "repair: boundary pressure +" << request << " at task "
                    << stalled << "\n"; *tr += o.str(); }
          continue;
        }
        logical -= std::min<int64_t>(step, std::max<int64_t>(logical / 16, 1));
        continue;
      }
      int repairs = 0;
      local.repair(actions, sim, repairs, tr);
      // place the simulated stays: slice objects take static homes behind the main layout
      const int32_t n = static_cast<int32_t>(sim.intervals.size());
      const int64_t al = std::max<int64_t>(cfg.alignment, 1);
      std::vector<int32_t> main_ix, slice_ix;
      for (int32_t i = 0; i < n; ++i)
        (in_resident_slice(sim.intervals[i].object) ? slice_ix : main_ix).push_back(i);
      const int32_t nm = static_cast<int32_t>(main_ix.size());
      std::vector<int64_t> b(nm), s(nm), e(nm), off(nm);
      for (int32_t j = 0; j < nm; ++j) {
        const auto& iv = sim.intervals[main_ix[j]];
        b[j] = align_up(iv.bytes, al); s[j] = iv.start_ns; e[j] = iv.end_ns;
      }
      int64_t span = 0;
      place_lifetimes(nm, b.data(), s.data(), e.data(), al, off.data(), &span);
      span = align_up(span, al);
      std::vector<int64_t> home(pv.n_objects, -1);
      int64_t slice_used = 0;
      for (int32_t i : slice_ix) {
        const int32_t o = sim.intervals[i].object;
        if (home[o] < 0) { home[o] = span + slice_used; slice_used += align_up(pv.bytes[o], al); }
      }
      const int64_t total_span = span + slice_used;
      // workspace sits above the layout: the tightest task decides
      int64_t max_ws = 0;
      for (int64_t w : pv.workspace) max_ws = std::max(max_ws, w);
      if (tr) { std::ostringstream o; o << "place: span " << span << " slice " << slice_used << " workspace "
                << max_ws << " capacity " << cfg.capacity_bytes << " makespan " << sim.result.makespan_ns
                << "\n"; *tr += o.str(); }
      if (total_span + max_ws <= cfg.capacity_bytes) {
        for (int32_t j = 0; j < nm; ++j) sim.intervals[main_ix[j]].offset = off[j];
        for (int32_t i : slice_ix) sim.intervals[i].offset = home[sim.intervals[i].object];
        c.actions.swap(actions);
        c.sim = std::move(sim);
        c.logical_capacity = logical + slice;
        c.span = total_span;
        c.repairs = repairs + pressure_repairs;
        c.status = SS_OK;
        return;
      }
      const int64_t over = total_span + max_ws - cfg.capacity_bytes;
      logical -= std::min(over, step);
    }
    c.status = SS_INFEASIBLE;
  }
};

}  // namespace
}  // namespace ssc

struct ss_search_result {
  ss_search_summary summary{};
  std::vector<ss_action> actions;
  std::vector<ss_interval> intervals;
  std::vector<int64_t> task_start, task_end, action_start, action_end;
  std::string trace;
};

extern "C" {

int ss_plan_reduce_emit(const ss_program* program, const ss_device_config* config,
                        const ss_search_options* options, int64_t capacity, int32_t strategy,
                        int32_t fetch_rule, int32_t tight, int32_t* cut_object, int32_t* cut_use,
                        int32_t max_cuts, int32_t* n_cuts, ss_action* actions, int32_t max_actions,
                        int32_t* n_actions) {
  if (!program || !config || !n_cuts || !n_actions) return SS_INVALID_ARGUMENT;
  ssc::ProgramView pv;
  if (int rc = ssc::unpack_program(program, pv)) return rc;
  ss_search_options opt{};
  if (options) opt = *options;
  if (opt.minimum_object_bytes_evict_eligible <= 0) opt.minimum_object_bytes_evict_eligible = 1 << 20;
  ssc::Planner planner(pv, *config, opt);
  std::vector<ssc::Gap> gaps;
  std::vector<int32_t> order;
  *n_cuts = *n_actions = 0;
  if (!planner.reduce(capacity, strategy, tight != 0, gaps, nullptr, &order)) return SS_INFEASIBLE;
  *n_cuts = static_cast<int32_t>(order.size());
  if (*n_cuts > max_cuts || (*n_cuts && (!cut_object || !cut_use))) return SS_OUT_OF_MEMORY;
  for (int32_t i = 0; i < *n_cuts; ++i) { cut_object[i] = gaps[order[i]].object; cut_use[i] = gaps[order[i]].k; }
  std::vector<ss_action> acts;
  planner.emit(gaps, fetch_rule, capacity, acts);
  *n_actions = static_cast<int32_t>(acts.size());
  if (*n_actions > max_actions || (*n_actions && !actions)) return SS_OUT_OF_MEMORY;
  for (int32_t i = 0; i < *n_actions; ++i) actions[i] = acts[i];
  return SS_OK;
}

int ss_plan_search(const ss_program* program, const ss_device_config* config,
                   const ss_search_options* options, ss_search_result** out) {
  if (!program || !config || !out) return SS_INVALID_ARGUMENT;
  ssc::ProgramView pv;
  if (int rc = ssc::unpack_program(program, pv)) return rc;
  ss_search_options opt{};
  if (options) opt = *options;
  if (opt.max_repairs <= 0) opt.max_repairs = 16;
  if (opt.minimum_object_bytes_evict_eligible <= 0) opt.minimum_object_bytes_evict_eligible = 1 << 20;
  const int smask = opt.strategy_mask ? opt.strategy_mask : 0x3;
  const int rmask = opt.fetch_rule_mask ? opt.fetch_rule_mask : 0xF;
  std::vector<ssc::Candidate> cands;
  for (int s = 0; s < 2; ++s)
    for (int r = 0; r < 4; ++r)
      if ((smask >> s & 1) && (rmask >> r & 1)) { ssc::Candidate c; c.strategy = s; c.rule = r; cands.push_back(std::move(c)); }
  ssc::Planner planner(pv, *config, opt);
  int workers = opt.workers > 0 ? opt.workers : ss_cpu_count();
  workers = std::max(1, std::min<int>(workers, static_cast<int>(cands.size())));
  std::atomic<size_t> next{0};
  auto work = [&]() {
    for (;;) {
      const size_t i = next.fetch_add(1);
      if (i >= cands.size()) return;
      planner.evaluate(cands[i]);
    }
  };
  if (workers == 1 || opt.deterministic) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int w = 0; w < workers; ++w) pool.emplace_back(work);
    for (auto& t : pool) t.join();
  }
  auto* res = new ss_search_result();
  int best = -1;
  for (size_t i = 0; i < cands.size(); ++i) {
    res->summary.candidates_evaluated++;
    if (opt.trace) res->trace += cands[i].trace;
    if (cands[i].status != SS_OK) continue;
    res->summary.candidates_feasible++;
    if (best < 0 || cands[i].sim.result.makespan_ns < cands[best].sim.result.makespan_ns)
      best = static_cast<int>(i);
  }
  if (best < 0) {
    res->summary.status = SS_INFEASIBLE;
    *out = res;
    return SS_OK;
  }
  ssc::Candidate& b = cands[best];
  res->summary.status = SS_OK;
  res->summary.best_strategy = b.strategy;
  res->summary.best_fetch_rule = b.rule;
  res->summary.repairs_applied = b.repairs;
  res->summary.logical_capacity = b.logical_capacity;
  res->summary.layout_span = b.span;
  res->summary.sim = b.sim.result;
  res->actions = std::move(b.actions);
  res->intervals = std::move(b.sim.intervals);
  res->task_start = std::move(b.sim.task_start);
  res->task_end = std::move(b.sim.task_end);
  res->action_start = std::move(b.sim.action_start);
  res->action_end = std::move(b.sim.action_end);
  res->summary.n_actions = static_cast<int32_t>(res->actions.size());
  res->summary.n_intervals = static_cast<int32_t>(res->intervals.size());
  *out = res;
  return SS_OK;
}

const ss_search_summary* ss_search_summary_of(const ss_search_result* r) { return &r->summary; }
const ss_action* ss_search_actions(const ss_search_result* r) { return r->actions.data(); }
const ss_interval* ss_search_intervals(const ss_search_result* r) { return r->intervals.data(); }
const int64_t* ss_search_task_start(const ss_search_result* r) { return r->task_start.data(); }
const int64_t* ss_search_task_end(const ss_search_result* r) { return r->task_end.data(); }
const int64_t* ss_search_action_start(const ss_search_result* r) { return r->action_start.data(); }
const int64_t* ss_search_action_end(const ss_search_result* r) { return r->action_end.data(); }
const char* ss_search_trace(const ss_search_result* r) { return r->trace.c_str(); }
void ss_search_result_destroy(ss_search_result* r) { delete r; }

}  // extern "C"
