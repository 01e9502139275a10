// C-ABI runtime: devices, streams, events, buffers, kernel modules.
// Stands in for the CUDA backend of the reference's host HAL
// (crates/tile_hal/src/cuda.rs: CudaDevice :293-417, CudaStream :134-166,
// CudaBuffer :170-218, CudaLauncher :222-289), which binds 17 driver-API
// symbols through dlopen, copies synchronously and can drive one device only.
// Here every handle remembers its device, each call makes that device current,
// copies are stream-ordered, and events give device-side timing.
#include <dlfcn.h>

#include <cstring>

#include "common.hpp"

namespace tsm100 {

std::string& last_error_ref() {
  static thread_local std::string err;
  return err;
}

int32_t fail(int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  last_error_ref() = buf;
  return code;
}

int32_t check_cuda(cudaError_t e, int32_t code, const char* what) {
  if (e == cudaSuccess) return TSM100_OK;
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInitializationError)
    code = TSM100_ERR_NO_DEVICE;
  cudaGetLastError();  // clear the sticky slot for non-fatal errors
  return fail(code, "%s failed: %s (%d)", what, cudaGetErrorString(e), static_cast<int>(e));
}

int32_t use_device(tsm100_device_t dev) {
  if (!dev) return fail(TSM100_ERR_INVALID, "null device handle");
  TSM_CUDA(cudaSetDevice(dev->ordinal), TSM100_ERR_RUNTIME);
  return TSM100_OK;
}

int32_t read_status(tsm100_device_t dev, cudaStream_t stream, uint32_t* value) {
  uint32_t v = 0;
  TSM_CUDA(cudaMemcpyAsync(&v, dev->status, sizeof v, cudaMemcpyDeviceToHost, stream), TSM100_ERR_RUNTIME);
  TSM_CUDA(cudaStreamSynchronize(stream), TSM100_ERR_STREAM);
  if (v != 0) TSM_CUDA(cudaMemsetAsync(dev->status, 0, sizeof v, stream), TSM100_ERR_RUNTIME);
  *value = v;
  return TSM100_OK;
}

}  // namespace tsm100

using namespace tsm100;

struct tsm100_module_s {
  tsm100_device_t dev = nullptr;
  void* handle = nullptr;
  std::string path;
};

extern "C" {

int32_t tsm100_version(void) { return TSM100_VERSION; }

size_t tsm100_last_error(char* buf, size_t cap) {
  const std::string& e = last_error_ref();
  if (buf && cap) {
    const size_t n = e.size() < cap - 1 ? e.size() : cap - 1;
    std::memcpy(buf, e.data(), n);
    buf[n] = '\0';
  }
  return e.size();
}

int32_t tsm100_device_count(int32_t* count) {
  if (!count) return fail(TSM100_ERR_INVALID, "null count pointer");
  int n = 0;
  TSM_CUDA(cudaGetDeviceCount(&n), TSM100_ERR_NO_DEVICE);
  *count = n;
  return TSM100_OK;
}

int32_t tsm100_device_open(int32_t ordinal, tsm100_device_t* out) {
  if (!out) return fail(TSM100_ERR_INVALID, "null output handle");
  *out = nullptr;
  int n = 0;
  TSM_CUDA(cudaGetDeviceCount(&n), TSM100_ERR_NO_DEVICE);
  if (ordinal < 0 || ordinal >= n) return fail(TSM100_ERR_INVALID, "device ordinal %d out of range [0, %d)", ordinal, n);
  TSM_CUDA(cudaSetDevice(ordinal), TSM100_ERR_RUNTIME);
  cudaDeviceProp prop;
  TSM_CUDA(cudaGetDeviceProperties(&prop, ordinal), TSM100_ERR_RUNTIME);
  if (prop.major != 10)
    return fail(TSM100_ERR_NO_DEVICE, "device %d (%s) is sm_%d%d; this library carries sm_100a code only", ordinal,
                prop.name, prop.major, prop.minor);
  tsm100_device_t d = new tsm100_device_s();
  d->ordinal = ordinal;
  d->sm_count = prop.multiProcessorCount;
  d->name = prop.name;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&d->status), sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(d->status, 0, sizeof(uint32_t));
  if (e != cudaSuccess) {
    delete d;
    return check_cuda(e, TSM100_ERR_MEMORY, "status word allocation");
  }
  *out = d;
  return TSM100_OK;
}

int32_t tsm100_device_close(tsm100_device_t dev) {
  if (!dev) return TSM100_OK;
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  HostPipe& p = dev->pipe;
  for (int i = 0; i < HostPipe::kSlots; ++i) {
    if (p.done[i]) cudaEventDestroy(p.done[i]);
    if (p.stream[i]) cudaStreamDestroy(p.stream[i]);
  }
  if (p.dev_buf) cudaFree(p.dev_buf);
  if (p.pin_buf) cudaFreeHost(p.pin_buf);
  if (dev->status) cudaFree(dev->status);
  delete dev;
  return TSM100_OK;
}

int32_t tsm100_device_ordinal(tsm100_device_t dev, int32_t* ordinal) {
  if (!dev || !ordinal) return fail(TSM100_ERR_INVALID, "null argument");
  *ordinal = dev->ordinal;
  return TSM100_OK;
}

int32_t tsm100_device_name(tsm100_device_t dev, char* buf, size_t cap) {
  if (!dev || !buf || !cap) return fail(TSM100_ERR_INVALID, "null argument");
  snprintf(buf, cap, "%s", dev->name.c_str());
  return TSM100_OK;
}

int32_t tsm100_device_sm_count(tsm100_device_t dev, int32_t* sms) {
  if (!dev || !sms) return fail(TSM100_ERR_INVALID, "null argument");
  *sms = dev->sm_count;
  return TSM100_OK;
}

int32_t tsm100_mem_info(tsm100_device_t dev, size_t* free_bytes, size_t* total_bytes) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  size_t f = 0, t = 0;
  TSM_CUDA(cudaMemGetInfo(&f, &t), TSM100_ERR_RUNTIME);
  if (free_bytes) *free_bytes = f;
  if (total_bytes) *total_bytes = t;
  return TSM100_OK;
}

int32_t tsm100_device_status(tsm100_device_t dev, void* stream, uint32_t* status) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!status) return fail(TSM100_ERR_INVALID, "null status pointer");
  return read_status(dev, static_cast<cudaStream_t>(stream), status);
}

// ---- streams / events ------------------------------------------------------
int32_t tsm100_stream_create(tsm100_device_t dev, void** stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!stream) return fail(TSM100_ERR_INVALID, "null stream pointer");
  cudaStream_t s;
  TSM_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), TSM100_ERR_STREAM);
  *stream = s;
  return TSM100_OK;
}

int32_t tsm100_stream_destroy(tsm100_device_t dev, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!stream) return TSM100_OK;
  TSM_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)), TSM100_ERR_STREAM);
  return TSM100_OK;
}

// Also reports a kernel whose bounded wait ran out since the last synchronise.
int32_t tsm100_stream_synchronize(tsm100_device_t dev, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  uint32_t v = 0;
  st = read_status(dev, static_cast<cudaStream_t>(stream), &v);
  if (st != TSM100_OK) return st;
  if (v != 0) return fail(TSM100_ERR_TIMEOUT, "a kernel gave up a bounded device-side wait (status 0x%x)", v);
  return TSM100_OK;
}

int32_t tsm100_stream_query(tsm100_device_t dev, void* stream, int32_t* done) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!done) return fail(TSM100_ERR_INVALID, "null done pointer");
  cudaError_t e = cudaStreamQuery(static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) { *done = 1; return TSM100_OK; }
  if (e == cudaErrorNotReady) { *done = 0; return TSM100_OK; }
  return check_cuda(e, TSM100_ERR_STREAM, "cudaStreamQuery");
}

int32_t tsm100_event_create(tsm100_device_t dev, void** event) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!event) return fail(TSM100_ERR_INVALID, "null event pointer");
  cudaEvent_t e;
  TSM_CUDA(cudaEventCreate(&e), TSM100_ERR_STREAM);
  *event = e;
  return TSM100_OK;
}

int32_t tsm100_event_record(tsm100_device_t dev, void* event, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  TSM_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)), TSM100_ERR_STREAM);
  return TSM100_OK;
}

int32_t tsm100_event_synchronize(tsm100_device_t dev, void* event) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  TSM_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)), TSM100_ERR_STREAM);
  return TSM100_OK;
}

int32_t tsm100_event_elapsed_ms(tsm100_device_t dev, void* start, void* stop, float* ms) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!ms) return fail(TSM100_ERR_INVALID, "null ms pointer");
  TSM_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)), TSM100_ERR_STREAM);
  return TSM100_OK;
}

int32_t tsm100_event_destroy(tsm100_device_t dev, void* event) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!event) return TSM100_OK;
  TSM_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)), TSM100_ERR_STREAM);
  return TSM100_OK;
}

// ---- buffers ---------------------------------------------------------------
int32_t tsm100_alloc(tsm100_device_t dev, size_t bytes, void** dptr) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!dptr) return fail(TSM100_ERR_INVALID, "null dptr pointer");
  *dptr = nullptr;
  if (bytes == 0) return TSM100_OK;  // an empty buffer is a null pointer, like a zero-length Vec
  TSM_CUDA(cudaMalloc(dptr, bytes), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_free(tsm100_device_t dev, void* dptr) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!dptr) return TSM100_OK;
  TSM_CUDA(cudaFree(dptr), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_host_alloc(size_t bytes, void** hptr) {
  if (!hptr) return fail(TSM100_ERR_INVALID, "null hptr pointer");
  *hptr = nullptr;
  if (bytes == 0) return TSM100_OK;
  TSM_CUDA(cudaHostAlloc(hptr, bytes, cudaHostAllocPortable), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_host_free(void* hptr) {
  if (!hptr) return TSM100_OK;
  TSM_CUDA(cudaFreeHost(hptr), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_memcpy_h2d(tsm100_device_t dev, void* dst, const void* host, size_t bytes, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (bytes == 0) return TSM100_OK;
  if (!dst || !host) return fail(TSM100_ERR_INVALID, "null copy pointer");
  TSM_CUDA(cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_memcpy_d2h(tsm100_device_t dev, void* host, const void* src, size_t bytes, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (bytes == 0) return TSM100_OK;
  if (!src || !host) return fail(TSM100_ERR_INVALID, "null copy pointer");
  TSM_CUDA(cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

int32_t tsm100_memset(tsm100_device_t dev, void* dst, int32_t byte, size_t bytes, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (bytes == 0) return TSM100_OK;
  if (!dst) return fail(TSM100_ERR_INVALID, "null memset pointer");
  TSM_CUDA(cudaMemsetAsync(dst, byte, bytes, static_cast<cudaStream_t>(stream)), TSM100_ERR_MEMORY);
  return TSM100_OK;
}

// ---- kernel modules ----------------------------------------------------------
// A module is a shared library built from tsm100_emit() output.  For every
// entry kernel <name> it exports
//   int32_t <name>_launch(void** args, uint32_t nargs, uint32_t blocks, void* stream,
//                         uint32_t* status_word, char* err, size_t err_cap);
typedef int32_t (*ModuleLaunchFn)(void**, uint32_t, uint32_t, void*, uint32_t*, char*, size_t);

int32_t tsm100_module_load(tsm100_device_t dev, const char* path, tsm100_module_t* out) {
  if (!dev || !path || !out) return fail(TSM100_ERR_INVALID, "null argument");
  *out = nullptr;
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return fail(TSM100_ERR_LAUNCH, "cannot load kernel module %s: %s", path, dlerror());
  tsm100_module_t m = new tsm100_module_s();
  m->dev = dev;
  m->handle = h;
  m->path = path;
  *out = m;
  return TSM100_OK;
}

int32_t tsm100_module_unload(tsm100_module_t mod) {
  if (!mod) return TSM100_OK;
  if (mod->handle) dlclose(mod->handle);
  delete mod;
  return TSM100_OK;
}

int32_t tsm100_launch(tsm100_module_t mod, const char* name, uint32_t blocks, void** args, uint32_t nargs,
                      void* stream) {
  if (!mod || !name) return fail(TSM100_ERR_INVALID, "null argument");
  int32_t st = use_device(mod->dev);
  if (st != TSM100_OK) return st;
  const std::string sym = std::string(name) + "_launch";
  void* fn = dlsym(mod->handle, sym.c_str());
  if (!fn) return fail(TSM100_ERR_LAUNCH, "kernel %s not found in module %s", name, mod->path.c_str());
  char err[384] = {0};
  st = reinterpret_cast<ModuleLaunchFn>(fn)(args, nargs, blocks, stream, mod->dev->status, err, sizeof err);
  if (st != TSM100_OK) return fail(st, "%s: %s", name, err);
  return TSM100_OK;
}

int32_t tsm100_shard_range(int64_t units, int32_t world, int32_t rank, int64_t* first, int64_t* count) {
  if (!first || !count) return fail(TSM100_ERR_INVALID, "null output pointer");
  if (units < 0 || world <= 0 || rank < 0 || rank >= world)
    return fail(TSM100_ERR_INVALID, "bad shard request: units=%lld world=%d rank=%d", static_cast<long long>(units), world, rank);
  const int64_t base = units / world, extra = units % world;
  *count = base + (rank < extra ? 1 : 0);
  *first = base * rank + (rank < extra ? rank : extra);
  return TSM100_OK;
}

}  // extern "C"
