// CUDA device backend: the flat operation table of ss_core.h over the CUDA
// runtime API. Device pool memory comes from cudaMalloc, the spill pool from
// cudaHostAlloc (pinned, portable), lanes are non-blocking streams and copies
// are cudaMemcpyAsync, which the copy engines execute next to running kernels.
// Built as its own shared object and opened with dlopen by the core, which
// therefore never links CUDA itself.
//
// Role model: packages/engine/csrc/backends/cuda/src/backend_cuda.c (driver-API
// table) and profiler_nvtx.c.
#include "ss_core.h"

#include <cuda_runtime.h>

#include <sched.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

namespace {

struct Cuda {
  int device;
};

int rc_of(cudaError_t e) {
  if (e == cudaSuccess) return SS_OK;
  if (e == cudaErrorMemoryAllocation) return SS_OUT_OF_MEMORY;
  return SS_BACKEND_FAILURE;
}
int bind(void* self) { return rc_of(cudaSetDevice(static_cast<Cuda*>(self)->device)); }

int device_alloc(void* self, size_t bytes, void** out) {
  if (int rc = bind(self)) return rc;
  return rc_of(cudaMalloc(out, bytes));
}
int device_free(void* self, void* p) { bind(self); return rc_of(cudaFree(p)); }
// NUMA node of a GPU from sysfs (-1 when unknown).
int numa_node_of_device(int device) {
  char bus[32] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof bus, device) != cudaSuccess) return -1;
  for (char* c = bus; *c; ++c) *c = static_cast<char>(std::tolower(*c));
  const std::string path = std::string("/sys/bus/pci/devices/") + bus + "/numa_node";
  FILE* f = std::fopen(path.c_str(), "r");
  if (!f) return -1;
  int node = -1;
  if (std::fscanf(f, "%d", &node) != 1) node = -1;
  std::fclose(f);
  return node;
}

// CPUs of a NUMA node ("0-31,64-95") into a mask; false when the list cannot be read.
bool cpus_of_node(int node, cpu_set_t* set) {
  char path[96];
  std::snprintf(path, sizeof path, "/sys/devices/system/node/node%d/cpulist", node);
  FILE* f = std::fopen(path, "r");
  if (!f) return false;
  char buf[4096] = {0};
  const bool got = std::fgets(buf, sizeof buf, f) != nullptr;
  std::fclose(f);
  if (!got) return false;
  CPU_ZERO(set);
  int n = 0;
  for (char* p = buf; *p;) {
    char* end;
    long lo = std::strtol(p, &end, 10);
    if (end == p) break;
    long hi = lo;
    if (*end == '-') { p = end + 1; hi = std::strtol(p, &end, 10); }
    for (long c = lo; c <= hi && c < CPU_SETSIZE; ++c) { CPU_SET(static_cast<int>(c), set); ++n; }
    p = (*end == ',') ? end + 1 : end;
    if (*end != ',' ) break;
  }
  return n > 0;
}

// Pinned host memory lands on the node of the CPU that allocates it: run the allocation on
// the GPU's own node (numa_node < 0: look it up), then put the thread's affinity back. With
// eight ranks on a two-socket host this keeps every rank's spill traffic off the inter-socket link.
int host_alloc(void* self, size_t bytes, int numa_node, void** out) {
  if (int rc = bind(self)) return rc;
  if (numa_node < 0) numa_node = numa_node_of_device(static_cast<Cuda*>(self)->device);
  cpu_set_t old_set, node_set;
  bool moved = false;
  if (numa_node >= 0 && cpus_of_node(numa_node, &node_set) &&
      sched_getaffinity(0, sizeof old_set, &old_set) == 0) {
    cpu_set_t both;
    CPU_AND(&both, &node_set, &old_set);          // stay inside the cpuset we were given
    if (CPU_COUNT(&both) > 0) moved = sched_setaffinity(0, sizeof both, &both) == 0;
  }
  const cudaError_t e = cudaHostAlloc(out, bytes, cudaHostAllocPortable);
  if (moved) sched_setaffinity(0, sizeof old_set, &old_set);
  return rc_of(e);
}
int host_free(void* self, void* p, size_t) { bind(self); return rc_of(cudaFreeHost(p)); }
int stream_create(void* self, void** out) {
  if (int rc = bind(self)) return rc;
  cudaStream_t s;
  cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  *out = s;
  return rc_of(e);
}
int stream_destroy(void* self, void* s) {
  bind(self);
  return rc_of(cudaStreamDestroy(static_cast<cudaStream_t>(s)));
}
int event_create(void* self, int timing, void** out) {
  if (int rc = bind(self)) return rc;
  cudaEvent_t e;
  cudaError_t r = cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming);
  *out = e;
  return rc_of(r);
}
int event_destroy(void* self, void* e) {
  bind(self);
  return rc_of(cudaEventDestroy(static_cast<cudaEvent_t>(e)));
}
int event_record(void* self, void* e, void* s) {
  bind(self);
  return rc_of(cudaEventRecord(static_cast<cudaEvent_t>(e), static_cast<cudaStream_t>(s)));
}
int event_query(void* self, void* e) {
  bind(self);
  cudaError_t r = cudaEventQuery(static_cast<cudaEvent_t>(e));
  if (r == cudaErrorNotReady) {
    (void)cudaGetLastError();   // "not ready" is recorded as this thread's last error: clear it, or
                                // the next launch check on this thread would report it
    return SS_TIMEOUT;
  }
  return rc_of(r);
}
int event_synchronize(void* self, void* e) {
  bind(self);
  return rc_of(cudaEventSynchronize(static_cast<cudaEvent_t>(e)));
}
int event_elapsed_ns(void* self, void* a, void* b, int64_t* out) {
  bind(self);
  float ms = 0.f;
  cudaError_t r = cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(a), static_cast<cudaEvent_t>(b));
  *out = static_cast<int64_t>(ms * 1e6);
  return rc_of(r);
}
int stream_wait_event(void* self, void* s, void* e) {
  bind(self);
  return rc_of(cudaStreamWaitEvent(static_cast<cudaStream_t>(s), static_cast<cudaEvent_t>(e), 0));
}
int stream_synchronize(void* self, void* s) {
  bind(self);
  return rc_of(cudaStreamSynchronize(static_cast<cudaStream_t>(s)));
}
int copy_async(void* self, void* dst, const void* src, size_t bytes, int kind, void* s) {
  bind(self);
  cudaMemcpyKind k = kind == SS_COPY_H2D   ? cudaMemcpyHostToDevice
                     : kind == SS_COPY_D2H ? cudaMemcpyDeviceToHost
                     : kind == SS_COPY_D2D ? cudaMemcpyDeviceToDevice
                                           : cudaMemcpyHostToHost;
  return rc_of(cudaMemcpyAsync(dst, src, bytes, k, static_cast<cudaStream_t>(s)));
}
int memset_async(void* self, void* dst, int value, size_t bytes, void* s) {
  bind(self);
  return rc_of(cudaMemsetAsync(dst, value, bytes, static_cast<cudaStream_t>(s)));
}
int device_memory_info(void* self, size_t* f, size_t* t) {
  bind(self);
  return rc_of(cudaMemGetInfo(f, t));
}
void destroy(void* self) { delete static_cast<Cuda*>(self); }

}  // namespace

extern "C" ss_backend* ss_backend_open(int device, char* error, size_t error_len) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device < 0 || device >= count) {
    if (error && error_len)
      std::snprintf(error, error_len, "cuda device %d unavailable: %s", device,
                    e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
    return nullptr;
  }
  auto* b = new ss_backend();
  std::memset(b, 0, sizeof *b);
  b->self = new Cuda{device};
  b->name = "cuda";
  b->device_alloc = device_alloc; b->device_free = device_free;
  b->host_alloc = host_alloc; b->host_free = host_free;
  b->stream_create = stream_create; b->stream_destroy = stream_destroy;
  b->event_create = event_create; b->event_destroy = event_destroy;
  b->event_record = event_record; b->event_query = event_query;
  b->event_synchronize = event_synchronize; b->event_elapsed_ns = event_elapsed_ns;
  b->stream_wait_event = stream_wait_event; b->stream_synchronize = stream_synchronize;
  b->copy_async = copy_async; b->memset_async = memset_async;
  b->device_memory_info = device_memory_info;
  b->destroy = destroy;
  return b;
}
