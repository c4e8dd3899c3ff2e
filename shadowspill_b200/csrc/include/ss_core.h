/* C ABI of the native core: simulator, planner (pressure reduction, fetch
 * emission, repair, fixed-offset placement) and the execution runtime (pools,
 * lanes, worker thread, failure latch, trace ring) over a pluggable backend.
 *
 * Everything crosses the boundary as flat arrays of fixed-width integers, so the
 * Python side needs only ctypes. The library links libc, libstdc++ and pthreads;
 * device backends are separate shared objects opened with dlopen, as in the
 * reference's layering (packages/engine/csrc/README.md:86-98).
 */
#ifndef SS_CORE_H
#define SS_CORE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
typedef enum ss_status {
  SS_OK = 0,
  SS_INVALID_ARGUMENT = 1,
  SS_OUT_OF_MEMORY = 2,
  SS_NO_PROGRESS = 3,       /* a reservation can never be satisfied */
  SS_BACKEND_FAILURE = 4,   /* the device backend returned an error */
  SS_CLOSED = 5,
  SS_FAILED = 6,            /* the runtime failure latch is set */
  SS_TIMEOUT = 7,
  SS_INFEASIBLE = 8,        /* no schedule fits the capacity */
  SS_INTERNAL = 9,
  SS_IO_ERROR = 10          /* the file-backed spill pool could not be read or written */
} ss_status;

const char* ss_status_string(int status);
int64_t ss_monotonic_ns(void);
int ss_cpu_count(void);
uint32_t ss_abi_version(void);
size_t ss_struct_size(const char* name);   /* ABI canary: sizeof by struct name */

/* ------------------------------------------------------------------ program */
enum { SS_USE_READ = 0, SS_USE_CREATE = 1, SS_USE_MUTATE = 2 };
enum {
  SS_OBJ_PERSISTENT = 1,  /* home is the spill pool; must be back there at step end */
  SS_OBJ_PINNED_RESIDENT = 2  /* never cut: fetched at step start, held to the end */
};

typedef struct ss_program {
  int32_t n_tasks;
  const int64_t* task_duration_ns;
  const int64_t* task_workspace_bytes;
  int32_t n_objects;
  const int64_t* object_bytes;
  const int32_t* object_flags;
  int32_t n_uses;               /* sorted by task, then object */
  const int32_t* use_task;
  const int32_t* use_object;
  const int32_t* use_mode;
} ss_program;

typedef struct ss_device_config {
  int64_t capacity_bytes;
  double fetch_solo_bps;        /* spill -> device */
  double fetch_concurrent_bps;  /* ... while an evict is in flight */
  double evict_solo_bps;        /* device -> spill */
  double evict_concurrent_bps;
  int64_t fetch_latency_ns;
  int64_t evict_latency_ns;
  int64_t alignment;            /* placement alignment in bytes */
} ss_device_config;

/* ------------------------------------------------------------------ schedule */
enum { SS_ACT_FETCH = 0, SS_ACT_EVICT = 1, SS_ACT_RELEASE = 2 };

typedef struct ss_action {
  int32_t kind;
  int32_t object;
  int32_t trigger_task;   /* issued when this task completes; -1 = step start */
  int32_t reserved;
} ss_action;

/* One stay of an object in device memory. */
typedef struct ss_interval {
  int32_t object;
  int32_t begin_action;   /* index of the fetch action, or -1 when a task creates it */
  int32_t begin_task;     /* creating task, or the fetch's trigger task */
  int32_t end_action;     /* index of the evict/release action */
  int64_t bytes;
  int64_t start_ns;       /* simulated reservation time */
  int64_t end_ns;         /* simulated free time */
  int64_t offset;         /* fixed device offset (placement); -1 if unplaced */
} ss_interval;

/* ------------------------------------------------------------------ simulator */
typedef struct ss_sim_result {
  int32_t status;
  int32_t stalled_task;          /* first task that could not start (NO_PROGRESS), else -1 */
  int64_t makespan_ns;
  int64_t compute_ns;            /* sum of task durations */
  int64_t input_wait_ns;         /* compute idle waiting for fetches */
  int64_t capacity_wait_ns;      /* compute or lanes idle waiting for memory */
  int64_t peak_bytes;
  int64_t fetch_bytes;
  int64_t evict_bytes;
  int64_t fetch_busy_ns;
  int64_t evict_busy_ns;
} ss_sim_result;

/* task_start/task_end: n_tasks entries; action_start/action_end: n_actions entries
 * (any may be NULL). intervals: capacity max_intervals; *n_intervals receives the count. */
int ss_simulate(const ss_program* program, const ss_device_config* config,
                const ss_action* actions, int32_t n_actions, ss_sim_result* result,
                int64_t* task_start, int64_t* task_end, int64_t* action_start,
                int64_t* action_end, ss_interval* intervals, int32_t max_intervals,
                int32_t* n_intervals);

/* Validates a schedule without timing it: every read finds its object resident,
 * persistent objects end in spill, nothing is fetched twice. Returns SS_OK or
 * SS_INVALID_ARGUMENT with *bad_action / *bad_task set (either may be -1). */
int ss_check_schedule(const ss_program* program, const ss_action* actions, int32_t n_actions,
                      int32_t* bad_action, int32_t* bad_task);

int64_t ss_transfer_duration_ns(int64_t bytes, double bytes_per_second, int64_t latency_ns);

/* ------------------------------------------------------------------ placement */
/* Fixed-offset placement: largest first, lowest aligned gap clear of every
 * time-overlapping placed lease. offsets[i] receives the offset; *span the total extent. */
int ss_place_lifetimes(int32_t n, const int64_t* bytes, const int64_t* start_ns,
                       const int64_t* end_ns, int64_t alignment, int64_t* offsets, int64_t* span);

/* For each lease, the earlier leases whose address range it reuses and that it
 * must therefore wait for (most recent occupant of every byte). pred_index has
 * capacity max_preds; pred_begin has n+1 entries (CSR). */
int ss_recover_layout_reuse(int32_t n, const int64_t* bytes, const int64_t* start_ns,
                            const int64_t* end_ns, const int64_t* offsets, int32_t* pred_begin,
                            int32_t* pred_index, int32_t max_preds);

/* ------------------------------------------------------------------ planner */
enum { SS_FETCH_DEMAND = 0, SS_FETCH_LATEST_SAFE = 1, SS_FETCH_PACKED_FIFO = 2,
       SS_FETCH_PACKED_FIT = 3 };
enum { SS_STRATEGY_STALL = 0, SS_STRATEGY_TRAFFIC = 1 };

typedef struct ss_search_options {
  int32_t workers;               /* 0 = all CPUs */
  int32_t strategy_mask;         /* bit per SS_STRATEGY_*; 0 = all */
  int32_t fetch_rule_mask;       /* bit per SS_FETCH_*; 0 = all */
  int32_t max_repairs;
  int64_t minimum_object_bytes_evict_eligible;
  int64_t capacity_refinement_step;   /* bytes given back when the layout overruns */
  int32_t deterministic;
  int32_t trace;                 /* record per-candidate trace lines */
  int32_t linear_reduce;         /* 1 = the plain O(cuts x gaps) reducer (the indexed one's reference) */
  int32_t no_resident_slice;     /* 1 = place small never-cut objects among the other leases */
} ss_search_options;

typedef struct ss_search_summary {
  int32_t status;
  int32_t best_strategy;
  int32_t best_fetch_rule;
  int32_t candidates_evaluated;
  int32_t candidates_feasible;
  int32_t repairs_applied;
  int32_t n_actions;
  int32_t n_intervals;
  int64_t logical_capacity;      /* capacity the winning schedule was reduced to */
  int64_t layout_span;           /* extent of the fixed layout */
  ss_sim_result sim;
} ss_search_summary;

typedef struct ss_search_result ss_search_result;   /* opaque */

int ss_plan_search(const ss_program* program, const ss_device_config* config,
                   const ss_search_options* options, ss_search_result** out);
/* One Reduce + Emit pass at a given capacity, without simulation, repair or placement: the cut gaps
 * as (object, index of the use the gap follows) pairs in the order they were cut, and the emitted
 * actions. For differential tests against independent implementations. SS_INFEASIBLE when the
 * capacity cannot be met; SS_OUT_OF_MEMORY when an output array is too short. */
int ss_plan_reduce_emit(const ss_program* program, const ss_device_config* config,
                        const ss_search_options* options, int64_t capacity, int32_t strategy,
                        int32_t fetch_rule, int32_t tight, int32_t* cut_object, int32_t* cut_use,
                        int32_t max_cuts, int32_t* n_cuts, ss_action* actions, int32_t max_actions,
                        int32_t* n_actions);
const ss_search_summary* ss_search_summary_of(const ss_search_result* r);
const ss_action* ss_search_actions(const ss_search_result* r);
const ss_interval* ss_search_intervals(const ss_search_result* r);
const int64_t* ss_search_task_start(const ss_search_result* r);
const int64_t* ss_search_task_end(const ss_search_result* r);
const int64_t* ss_search_action_start(const ss_search_result* r);
const int64_t* ss_search_action_end(const ss_search_result* r);
const char* ss_search_trace(const ss_search_result* r);
void ss_search_result_destroy(ss_search_result* r);

/* ------------------------------------------------------------------ backend table */
typedef struct ss_backend {
  void* self;
  const char* name;
  int (*device_alloc)(void* self, size_t bytes, void** out);
  int (*device_free)(void* self, void* ptr);
  int (*host_alloc)(void* self, size_t bytes, int numa_node, void** out);   /* pinned */
  int (*host_free)(void* self, void* ptr, size_t bytes);
  int (*stream_create)(void* self, void** out);
  int (*stream_destroy)(void* self, void* stream);
  int (*event_create)(void* self, int timing, void** out);
  int (*event_destroy)(void* self, void* event);
  int (*event_record)(void* self, void* event, void* stream);
  int (*event_query)(void* self, void* event);           /* SS_OK done, SS_TIMEOUT pending */
  int (*event_synchronize)(void* self, void* event);
  int (*event_elapsed_ns)(void* self, void* start, void* end, int64_t* out);
  int (*stream_wait_event)(void* self, void* stream, void* event);
  int (*stream_synchronize)(void* self, void* stream);
  int (*copy_async)(void* self, void* dst, const void* src, size_t bytes, int kind, void* stream);
  int (*memset_async)(void* self, void* dst, int value, size_t bytes, void* stream);
  int (*device_memory_info)(void* self, size_t* free_bytes, size_t* total_bytes);
  int (*range_push)(void* self, const char* name);       /* profiler annotations; may be NULL */
  int (*range_pop)(void* self);
  void (*destroy)(void* self);
} ss_backend;

enum { SS_COPY_H2D = 0, SS_COPY_D2H = 1, SS_COPY_D2D = 2, SS_COPY_H2H = 3 };
enum { SS_OP_DEVICE_ALLOC = 0, SS_OP_HOST_ALLOC, SS_OP_STREAM_CREATE, SS_OP_EVENT_CREATE,
       SS_OP_EVENT_RECORD, SS_OP_STREAM_WAIT, SS_OP_COPY, SS_OP_MEMSET, SS_OP_SYNC,
       SS_OP_COUNT };

/* Mock backend: host memory as device memory, real ordered stream threads,
 * optional per-byte delay, and injection of a failure into the n-th operation
 * of a kind (1-based; 0 disables). */
ss_backend* ss_mock_backend_create(double bytes_per_second, int64_t latency_ns);
int ss_mock_fail_operation(ss_backend* backend, int op_kind, int64_t nth);
int64_t ss_mock_operation_count(ss_backend* backend, int op_kind);
/* Enqueue host "compute" of a given duration on a mock stream (tests). */
int ss_mock_enqueue_compute(ss_backend* backend, void* stream, int64_t duration_ns);

/* Opens lib path and calls its `ss_backend_open(int device)` entry. */
ss_backend* ss_backend_dlopen(const char* path, int device, char* error, size_t error_len);

/* ------------------------------------------------------------------ runtime */
typedef struct ss_runtime ss_runtime;

typedef struct ss_runtime_config {
  int64_t device_bytes;        /* device pool arena */
  int64_t spill_bytes;         /* pinned host pool arena */
  int32_t numa_node;           /* -1 = no binding */
  int32_t trace_capacity;      /* events in the trace ring; 0 = tracing off */
  int64_t worker_poll_ns;
  int32_t max_objects;
  int32_t event_pool;          /* dependency events reserved at creation */
  void* external_device_base;  /* caller-owned device pool (e.g. symmetric memory); NULL = allocate */
  /* File-backed spill pool (optional third pool, on a local drive). Objects whose home is in
   * it move through staged lanes: bounded rings of pinned host memory, `file_queue_depth`
   * chunks of `file_chunk_bytes` per direction, filled and drained by disk threads. */
  int64_t file_bytes;          /* 0 = no file pool */
  const char* file_directory;  /* existing directory for the unlinked scratch file */
  const char* file_image;      /* optional named file that is the whole pool and is kept */
  int32_t file_create_image;   /* 0 open file_image read-write; 1 create it (must not exist); 2 adopt it:
                                  read-only first bytes of the pool, the rest a scratch file in file_directory */
  int32_t file_queue_depth;    /* slots per direction; 0 = 16 */
  int64_t file_chunk_bytes;    /* multiple of 4096; 0 = 2 MiB */
  int32_t file_io_threads;     /* disk threads per direction; 0 = 4 */
  int32_t reserved0;
  /* "host:port" of a memory daemon: the pool's file_bytes are then held by that daemon
   * instead of a local file (same staged lanes, chunks travel over TCP). */
  const char* remote_address;
} ss_runtime_config;

typedef struct ss_failure {
  int32_t status;
  int32_t reason;              /* ss_failure_reason */
  int32_t task;
  int32_t object;
  int32_t action;
  int32_t pool;                /* 0 device, 1 spill, 2 file */
  char message[192];
} ss_failure;

enum { SS_FAIL_NONE = 0, SS_FAIL_BACKEND_COPY, SS_FAIL_BACKEND_EVENT, SS_FAIL_BACKEND_ALLOC,
       SS_FAIL_CAPACITY, SS_FAIL_PLAN, SS_FAIL_OBJECT_STATE, SS_FAIL_EXTERNAL };

enum { SS_TRACE_TASK_BEGIN = 0, SS_TRACE_TASK_END, SS_TRACE_FETCH_ISSUE, SS_TRACE_FETCH_DONE,
       SS_TRACE_EVICT_ISSUE, SS_TRACE_EVICT_DONE, SS_TRACE_RELEASE, SS_TRACE_REUSE_WAIT,
       SS_TRACE_INPUT_WAIT, SS_TRACE_STEP_BEGIN, SS_TRACE_STEP_END, SS_TRACE_FAILURE,
       SS_TRACE_WORKER_IDLE, SS_TRACE_USER };

typedef struct ss_trace_event {
  int32_t kind;
  int32_t a;                   /* task / action / object id depending on kind */
  int64_t host_ns;             /* monotonic host clock */
  int64_t bytes;
} ss_trace_event;

typedef struct ss_runtime_stats {
  int64_t steps;
  int64_t tasks;
  int64_t fetches, fetch_bytes;
  int64_t evicts, evict_bytes;
  int64_t releases;
  int64_t reuse_waits;
  int64_t events_created;      /* stays constant in steady state */
  int64_t host_allocations;    /* stays constant in steady state */
  int64_t worker_wakeups;
  int64_t staged_read_chunks, staged_read_bytes;     /* file / remote pool -> pinned ring */
  int64_t staged_write_chunks, staged_write_bytes;   /* pinned ring -> file / remote pool */
} ss_runtime_stats;

int ss_runtime_create(ss_backend* backend, const ss_runtime_config* config, ss_runtime** out);
int ss_runtime_close(ss_runtime* rt);        /* drain, then release everything */
void ss_runtime_abandon(ss_runtime* rt);     /* process exit: no drain, no sync */
void ss_runtime_destroy(ss_runtime* rt);
void* ss_runtime_device_base(ss_runtime* rt);
void* ss_runtime_spill_base(ss_runtime* rt);
int ss_runtime_failure(ss_runtime* rt, ss_failure* out);         /* SS_OK if latched */
int ss_runtime_latch_failure(ss_runtime* rt, int reason, int status, const char* message);
int ss_runtime_stats_read(ss_runtime* rt, ss_runtime_stats* out);
int ss_trace_begin(ss_runtime* rt);
int ss_trace_end(ss_runtime* rt);
int32_t ss_trace_read(ss_runtime* rt, ss_trace_event* out, int32_t capacity);
/* Device-clock start and end of every transfer of the plan's last step, relative to the
 * step's first event; -1 where an action moved nothing. Only on runtimes created with
 * trace_capacity > 0 (their events carry timestamps). Returns the action count or -1. */
int32_t ss_plan_transfer_times(ss_runtime* rt, int32_t plan_id, int64_t* begin_ns, int64_t* end_ns,
                               int32_t capacity);

/* Plan admission: objects get spill homes, intervals fixed device offsets.
 * spill_offset[o] < 0 means the object never touches the spill pool. */
typedef struct ss_plan_desc {
  int32_t n_tasks;
  int32_t n_objects;
  const int64_t* object_bytes;
  const int64_t* spill_offset;
  int32_t n_actions;
  const ss_action* actions;           /* sorted by trigger_task, stable */
  int32_t n_intervals;
  const ss_interval* intervals;       /* offsets assigned */
  const int32_t* reuse_pred_begin;    /* CSR over intervals (n_intervals+1) */
  const int32_t* reuse_pred_index;
  int32_t n_uses;
  const int32_t* use_task;
  const int32_t* use_object;
  const int32_t* use_mode;
  const int64_t* file_offset;         /* home in the file pool per object, -1 = not there; may be
                                         NULL. An object has at most one home. */
} ss_plan_desc;

int ss_plan_admit(ss_runtime* rt, const ss_plan_desc* desc, int32_t* plan_id);
int ss_plan_close(ss_runtime* rt, int32_t plan_id);

/* Step protocol, called by the dispatcher thread. `compute_stream` is the
 * backend stream handle the caller enqueues the task's kernels on. */
int ss_step_begin(ss_runtime* rt, int32_t plan_id, void* compute_stream);
/* Makes compute_stream wait for the task's inputs and for the previous occupants
 * of every range the task creates; device pointers of the task's objects are
 * written to ptrs (one per use of the task, in use order). */
int ss_before_task(ss_runtime* rt, int32_t plan_id, int32_t task, void** ptrs, int32_t max_ptrs);
/* Records the task fence on compute_stream and publishes the actions it triggers. */
int ss_after_task(ss_runtime* rt, int32_t plan_id, int32_t task);
/* The same boundaries for a task that runs on another stream than the step's compute stream
 * (a collective on a communication stream): waits are enqueued on, and the fence is recorded on,
 * `stream`. Null means the compute stream. */
int ss_before_task_on(ss_runtime* rt, int32_t plan_id, int32_t task, void** ptrs, int32_t max_ptrs,
                      void* stream);
int ss_after_task_on(ss_runtime* rt, int32_t plan_id, int32_t task, void* stream);
/* Waits until every action of the step has completed; returns the failure latch state. */
int ss_step_end(ss_runtime* rt, int32_t plan_id);
/* Ends a step that the caller could not finish (a task raised): latches a caller failure, waits
 * for the copies in flight, and marks the plan inactive so that it can be closed. The runtime is
 * terminal afterwards, like after any other latched failure. */
int ss_step_abandon(ss_runtime* rt, int32_t plan_id, const char* why);
int ss_runtime_wait_idle(ss_runtime* rt);

/* Direct object I/O on the spill home (initialisation, checkpoints). */
int ss_spill_write(ss_runtime* rt, int64_t spill_offset, const void* src, int64_t bytes);
int ss_spill_read(ss_runtime* rt, int64_t spill_offset, void* dst, int64_t bytes);

/* The same for objects whose home is the file pool. */
int ss_file_write(ss_runtime* rt, int64_t file_offset, const void* src, int64_t bytes);
int ss_file_read(ss_runtime* rt, int64_t file_offset, void* dst, int64_t bytes);
/* direct: 1 if the pool file accepted O_DIRECT (0 for a remote pool). ring_bytes: pinned
 * staging per direction. */
int ss_runtime_file_info(ss_runtime* rt, int32_t* direct, int64_t* ring_bytes);

/* Route calibration: times copies of `bytes` alone and with the opposite
 * direction in flight. Rates in bytes/second. */
typedef struct ss_transfer_profile {
  double fetch_solo_bps, fetch_concurrent_bps, evict_solo_bps, evict_concurrent_bps;
  int64_t fetch_latency_ns, evict_latency_ns;
} ss_transfer_profile;
int ss_calibrate_transfers(ss_runtime* rt, int64_t bytes, int32_t repeats,
                           ss_transfer_profile* out);
/* The same through the staged lanes of the file pool (device <-> file). Call with no step
 * in flight; it overwrites the first 2*bytes of the device pool and of the file. */
int ss_calibrate_file_transfers(ss_runtime* rt, int64_t bytes, int32_t repeats,
                                ss_transfer_profile* out);

/* ------------------------------------------------------------------ BLAKE3 */
void* ss_blake3_new(void);
void ss_blake3_update(void* hasher, const void* data, size_t len);
void ss_blake3_finalize(void* hasher, uint8_t* out32);   /* may be called mid-stream */
void ss_blake3_free(void* hasher);

#ifdef __cplusplus
}
#endif
#endif /* SS_CORE_H */
