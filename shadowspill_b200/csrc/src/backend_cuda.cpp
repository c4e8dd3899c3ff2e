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

#include <cstdio>
#include <cstring>

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
int host_alloc(void* self, size_t bytes, int, void** out) {
  if (int rc = bind(self)) return rc;
  return rc_of(cudaHostAlloc(out, bytes, cudaHostAllocPortable));
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
  if (r == cudaErrorNotReady) return SS_TIMEOUT;
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
