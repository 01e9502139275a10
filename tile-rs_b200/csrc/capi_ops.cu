// C-ABI operators: tsm100_softmax / tsm100_gemm / tsm100_attention on device
// memory, and their *_host forms that take ordinary host pointers and overlap
// upload, kernel and download in chunks (the alloc_from_slice -> launch ->
// copy_to_host sequence of a tile_hal host program,
// crates/tile_hal/src/cuda.rs:348-371, :245-288, :190-199).
#include <algorithm>

#include "common.hpp"
#include "ops.cuh"
#include "selftest.cuh"

using namespace tsm100;

namespace {

int32_t finish(int32_t st, const std::string& err) {
  if (st != TSM100_OK) last_error_ref() = err;
  return st;
}

// Streams, events and a grow-only device workspace for the *_host operators.
int32_t ensure_pipe(tsm100_device_t dev, size_t dev_bytes) {
  HostPipe& p = dev->pipe;
  if (!p.ready) {
    for (int i = 0; i < HostPipe::kSlots; ++i) {
      TSM_CUDA(cudaStreamCreateWithFlags(&p.stream[i], cudaStreamNonBlocking), TSM100_ERR_STREAM);
      TSM_CUDA(cudaEventCreateWithFlags(&p.done[i], cudaEventDisableTiming), TSM100_ERR_STREAM);
    }
    p.ready = true;
  }
  if (dev_bytes > p.dev_bytes) {
    if (p.dev_buf) {
      TSM_CUDA(cudaDeviceSynchronize(), TSM100_ERR_RUNTIME);
      TSM_CUDA(cudaFree(p.dev_buf), TSM100_ERR_MEMORY);
      p.dev_buf = nullptr;
      p.dev_bytes = 0;
    }
    TSM_CUDA(cudaMalloc(&p.dev_buf, dev_bytes), TSM100_ERR_MEMORY);
    p.dev_bytes = dev_bytes;
  }
  return TSM100_OK;
}

int32_t sync_pipe(tsm100_device_t dev) {
  HostPipe& p = dev->pipe;
  for (int i = 0; i < HostPipe::kSlots; ++i) TSM_CUDA(cudaStreamSynchronize(p.stream[i]), TSM100_ERR_STREAM);
  uint32_t v = 0;
  int32_t st = read_status(dev, p.stream[0], &v);
  if (st != TSM100_OK) return st;
  if (v != 0) return fail(TSM100_ERR_TIMEOUT, "a kernel gave up a bounded device-side wait (status 0x%x)", v);
  return TSM100_OK;
}

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// `rows` rows of `width` bytes between buffers with row pitches dpitch / spitch: one plain copy when both are packed.
int32_t copy_rows(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, int64_t rows, cudaMemcpyKind kind,
                  cudaStream_t s) {
  if (rows <= 0 || width == 0) return TSM100_OK;
  if (dpitch == width && spitch == width) {
    TSM_CUDA(cudaMemcpyAsync(dst, src, width * static_cast<size_t>(rows), kind, s), TSM100_ERR_MEMORY);
  } else {
    TSM_CUDA(cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, static_cast<size_t>(rows), kind, s), TSM100_ERR_MEMORY);
  }
  return TSM100_OK;
}

}  // namespace

extern "C" {

int32_t tsm100_softmax(tsm100_device_t dev, const tsm100_softmax_desc* desc, const void* x, void* y, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::softmax(&err, desc, x, y, stream), err);
}

int32_t tsm100_rms_norm(tsm100_device_t dev, const tsm100_rms_norm_desc* desc, const void* x, void* y, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::rms_norm(&err, desc, x, y, stream), err);
}

int32_t tsm100_reduce(tsm100_device_t dev, const tsm100_reduce_desc* desc, const void* x, void* y, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::reduce(&err, desc, x, y, stream), err);
}

int32_t tsm100_silu_mul(tsm100_device_t dev, const tsm100_silu_mul_desc* desc, const void* gate, const void* up, void* y,
                        void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::silu_mul(&err, desc, gate, up, y, stream), err);
}

int32_t tsm100_rope(tsm100_device_t dev, const tsm100_rope_desc* desc, void* x, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::rope(&err, desc, x, stream), err);
}

int32_t tsm100_kv_cache_update(tsm100_device_t dev, const tsm100_kv_cache_update_desc* desc, const void* src, void* cache,
                               void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::kv_cache_update(&err, desc, src, cache, stream), err);
}

int32_t tsm100_attention_decode(tsm100_device_t dev, const tsm100_attention_decode_desc* desc, const void* q,
                                const void* k_cache, const void* v_cache, void* o, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::attention_decode(&err, desc, q, k_cache, v_cache, o, stream), err);
}

int32_t tsm100_gemm(tsm100_device_t dev, const tsm100_gemm_desc* desc, const void* a, const void* b, void* c,
                    void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::gemm(&err, desc, a, b, c, dev->status, stream), err);
}

int32_t tsm100_attention(tsm100_device_t dev, const tsm100_attention_desc* desc, const void* q, const void* k,
                         const void* v, void* o, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::attention(&err, desc, q, k, v, o, dev->status, stream), err);
}

int32_t tsm100_attention_prefill(tsm100_device_t dev, const tsm100_attention_prefill_desc* desc, const void* q,
                                 const void* k_cache, const void* v_cache, void* o, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  std::string err;
  return finish(ops::attention_prefill(&err, desc, q, k_cache, v_cache, o, dev->status, stream), err);
}

int32_t tsm100_selftest_wait_timeout(tsm100_device_t dev, uint32_t limit_us, uint32_t* observed_host, void* stream) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (limit_us == 0 || limit_us > 1000000u) return fail(TSM100_ERR_INVALID, "selftest_wait_timeout: limit must be 1 .. 1000000 us");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* observed = nullptr;
  TSM_CUDA(cudaMalloc(reinterpret_cast<void**>(&observed), 2 * sizeof(uint32_t)), TSM100_ERR_MEMORY);
  cudaError_t e = cudaMemsetAsync(observed, 0, 2 * sizeof(uint32_t), s);
  if (e == cudaSuccess) {
    selftest::wait_timeout_kernel<<<1, 64, 0, s>>>(dev->status, static_cast<unsigned long long>(limit_us) * 1000ull, observed);
    e = cudaGetLastError();
  }
  uint32_t host[2] = {0, 0};
  if (e == cudaSuccess) e = cudaMemcpyAsync(host, observed, sizeof host, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(observed);
  if (e != cudaSuccess) return check_cuda(e, TSM100_ERR_LAUNCH, "selftest_wait_timeout");
  if (observed_host) {
    observed_host[0] = host[0];
    observed_host[1] = host[1];
  }
  return TSM100_OK;
}

// ---------------------------------------------------------------------------
// host-memory operators
// ---------------------------------------------------------------------------
int32_t tsm100_softmax_host(tsm100_device_t dev, const tsm100_softmax_desc* desc, const void* x, void* y) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!desc || !ops::dtype_valid(desc->dtype) || desc->rows < 0 || desc->cols < 0)
    return fail(TSM100_ERR_INVALID, "softmax_host: bad descriptor");
  if (desc->rows == 0 || desc->cols == 0) return TSM100_OK;
  if (!x || !y) return fail(TSM100_ERR_INVALID, "softmax_host: null buffer");
  std::lock_guard<std::mutex> lock(dev->mu);
  const size_t row_bytes = static_cast<size_t>(desc->cols) * ops::dtype_size(desc->dtype);
  constexpr size_t kChunkTarget = 32u << 20;
  const int64_t rows_per_chunk = std::max<int64_t>(1, std::min<int64_t>(desc->rows, kChunkTarget / std::max<size_t>(row_bytes, 1)));
  const size_t chunk_bytes = round_up(static_cast<size_t>(rows_per_chunk) * row_bytes, 256);
  st = ensure_pipe(dev, chunk_bytes * 2 * HostPipe::kSlots);
  if (st != TSM100_OK) return st;
  HostPipe& p = dev->pipe;
  std::string err;
  int64_t row = 0;
  for (int i = 0; row < desc->rows; ++i, row += rows_per_chunk) {
    const int slot = i % HostPipe::kSlots;
    cudaStream_t s = p.stream[slot];
    char* din = static_cast<char*>(p.dev_buf) + static_cast<size_t>(slot) * 2 * chunk_bytes;
    char* dout = din + chunk_bytes;
    tsm100_softmax_desc d = *desc;
    d.rows = std::min<int64_t>(rows_per_chunk, desc->rows - row);
    const size_t bytes = static_cast<size_t>(d.rows) * row_bytes;
    const size_t off = static_cast<size_t>(row) * row_bytes;
    TSM_CUDA(cudaMemcpyAsync(din, static_cast<const char*>(x) + off, bytes, cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
    st = ops::softmax(&err, &d, din, dout, s);
    if (st != TSM100_OK) return finish(st, err);
    TSM_CUDA(cudaMemcpyAsync(static_cast<char*>(y) + off, dout, bytes, cudaMemcpyDeviceToHost, s), TSM100_ERR_MEMORY);
  }
  return sync_pipe(dev);
}

int32_t tsm100_gemm_host(tsm100_device_t dev, const tsm100_gemm_desc* desc, const void* a, const void* b, void* c) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!desc || !ops::dtype_valid(desc->dtype) || !ops::dtype_valid(desc->out_dtype) || desc->m < 0 || desc->n < 0 ||
      desc->k < 0 || desc->batch < 0)
    return fail(TSM100_ERR_INVALID, "gemm_host: bad descriptor");
  const ops::GemmPitch ld = ops::gemm_pitch(desc);  // pitches of the HOST matrices; the device copies are packed
  const int64_t b_rows = desc->b_transposed ? desc->n : desc->k, b_cols = desc->b_transposed ? desc->k : desc->n;
  if (ld.lda < desc->k || ld.ldb < b_cols || ld.ldc < desc->n)
    return fail(TSM100_ERR_INVALID, "gemm_host: a row pitch (lda, ldb, ldc) is shorter than its row");
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return TSM100_OK;
  if (!a || !b || !c) return fail(TSM100_ERR_INVALID, "gemm_host: null buffer");
  std::lock_guard<std::mutex> lock(dev->mu);
  const size_t es = ops::dtype_size(desc->dtype), os = ops::dtype_size(desc->out_dtype);
  const size_t a_row = static_cast<size_t>(desc->k) * es, b_row = static_cast<size_t>(b_cols) * es,
               c_row = static_cast<size_t>(desc->n) * os;
  const size_t b_bytes = round_up(static_cast<size_t>(b_rows) * b_row, 256);
  tsm100_gemm_desc packed = *desc;
  packed.lda = packed.ldb = packed.ldc = 0;
  std::string err;
  if (desc->batch == 1) {
    // B stays resident; A and C stream through in row blocks.
    int64_t rows_per_chunk = std::max<int64_t>(128, (16ll << 20) / std::max<int64_t>(1, static_cast<int64_t>(a_row)));
    rows_per_chunk = std::min<int64_t>(desc->m, (rows_per_chunk + 127) / 128 * 128);
    const size_t a_chunk = round_up(static_cast<size_t>(rows_per_chunk) * a_row, 256);
    const size_t c_chunk = round_up(static_cast<size_t>(rows_per_chunk) * c_row, 256);
    st = ensure_pipe(dev, b_bytes + (a_chunk + c_chunk) * HostPipe::kSlots);
    if (st != TSM100_OK) return st;
    HostPipe& p = dev->pipe;
    char* db = static_cast<char*>(p.dev_buf);
    st = copy_rows(db, b_row, b, static_cast<size_t>(ld.ldb) * es, b_row, b_rows, cudaMemcpyHostToDevice, p.stream[0]);
    if (st != TSM100_OK) return st;
    TSM_CUDA(cudaEventRecord(p.done[0], p.stream[0]), TSM100_ERR_STREAM);
    int64_t row = 0;
    for (int i = 0; row < desc->m; ++i, row += rows_per_chunk) {
      const int slot = i % HostPipe::kSlots;
      cudaStream_t s = p.stream[slot];
      char* da = db + b_bytes + static_cast<size_t>(slot) * (a_chunk + c_chunk);
      char* dc = da + a_chunk;
      tsm100_gemm_desc d = packed;
      d.m = std::min<int64_t>(rows_per_chunk, desc->m - row);
      st = copy_rows(da, a_row, static_cast<const char*>(a) + static_cast<size_t>(row) * ld.lda * es,
                     static_cast<size_t>(ld.lda) * es, a_row, d.m, cudaMemcpyHostToDevice, s);
      if (st != TSM100_OK) return st;
      TSM_CUDA(cudaStreamWaitEvent(s, p.done[0], 0), TSM100_ERR_STREAM);
      st = ops::gemm(&err, &d, da, db, dc, dev->status, s);
      if (st != TSM100_OK) return finish(st, err);
      st = copy_rows(static_cast<char*>(c) + static_cast<size_t>(row) * ld.ldc * os, static_cast<size_t>(ld.ldc) * os, dc, c_row,
                     c_row, d.m, cudaMemcpyDeviceToHost, s);
      if (st != TSM100_OK) return st;
    }
    return sync_pipe(dev);
  }
  // batched: one problem per slot
  const size_t a_bytes = round_up(static_cast<size_t>(desc->m) * a_row, 256);
  const size_t c_bytes = round_up(static_cast<size_t>(desc->m) * c_row, 256);
  const size_t unit = a_bytes + b_bytes + c_bytes;
  st = ensure_pipe(dev, unit * HostPipe::kSlots);
  if (st != TSM100_OK) return st;
  HostPipe& p = dev->pipe;
  const size_t a_host = static_cast<size_t>(desc->m) * ld.lda * es, b_host = static_cast<size_t>(b_rows) * ld.ldb * es,
               c_host = static_cast<size_t>(desc->m) * ld.ldc * os;
  packed.batch = 1;
  for (int i = 0; i < desc->batch; ++i) {
    const int slot = i % HostPipe::kSlots;
    cudaStream_t s = p.stream[slot];
    char* da = static_cast<char*>(p.dev_buf) + static_cast<size_t>(slot) * unit;
    char* db = da + a_bytes;
    char* dc = db + b_bytes;
    st = copy_rows(da, a_row, static_cast<const char*>(a) + i * a_host, static_cast<size_t>(ld.lda) * es, a_row, desc->m,
                   cudaMemcpyHostToDevice, s);
    if (st == TSM100_OK)
      st = copy_rows(db, b_row, static_cast<const char*>(b) + i * b_host, static_cast<size_t>(ld.ldb) * es, b_row, b_rows,
                     cudaMemcpyHostToDevice, s);
    if (st != TSM100_OK) return st;
    st = ops::gemm(&err, &packed, da, db, dc, dev->status, s);
    if (st != TSM100_OK) return finish(st, err);
    st = copy_rows(static_cast<char*>(c) + i * c_host, static_cast<size_t>(ld.ldc) * os, dc, c_row, c_row, desc->m,
                   cudaMemcpyDeviceToHost, s);
    if (st != TSM100_OK) return st;
  }
  return sync_pipe(dev);
}

int32_t tsm100_attention_host(tsm100_device_t dev, const tsm100_attention_desc* desc, const void* q, const void* k,
                              const void* v, void* o) {
  int32_t st = use_device(dev);
  if (st != TSM100_OK) return st;
  if (!desc || !ops::dtype_valid(desc->dtype) || desc->batch < 0 || desc->heads_q < 0 || desc->heads_kv < 0 ||
      desc->seq < 0 || desc->head_dim < 0)
    return fail(TSM100_ERR_INVALID, "attention_host: bad descriptor");
  if (desc->batch == 0 || desc->heads_q == 0 || desc->seq == 0 || desc->head_dim == 0) return TSM100_OK;
  if (desc->heads_kv <= 0 || desc->heads_q % desc->heads_kv != 0)
    return fail(TSM100_ERR_INVALID, "attention_host: heads_q must be a positive multiple of heads_kv");
  if (!q || !k || !v || !o) return fail(TSM100_ERR_INVALID, "attention_host: null buffer");
  std::lock_guard<std::mutex> lock(dev->mu);
  const size_t es = ops::dtype_size(desc->dtype);
  const int group = desc->heads_q / desc->heads_kv;
  const int64_t units = static_cast<int64_t>(desc->batch) * desc->heads_kv;  // (batch, kv head) groups
  const size_t head_bytes = static_cast<size_t>(desc->seq) * desc->head_dim * es;
  const size_t unit_q = head_bytes * group;
  // enough units per chunk to move >= 16 MiB of Q and to fill the SMs
  int64_t upc = std::max<int64_t>(1, (16ll << 20) / static_cast<int64_t>(unit_q));
  upc = std::min<int64_t>(upc, units);
  const size_t cq = round_up(unit_q * upc, 256), ckv = round_up(head_bytes * upc, 256);
  const size_t per_slot = 2 * cq + 2 * ckv;
  st = ensure_pipe(dev, per_slot * HostPipe::kSlots);
  if (st != TSM100_OK) return st;
  HostPipe& p = dev->pipe;
  std::string err;
  int64_t u0 = 0;
  for (int i = 0; u0 < units; ++i, u0 += upc) {
    const int slot = i % HostPipe::kSlots;
    cudaStream_t s = p.stream[slot];
    const int64_t nu = std::min<int64_t>(upc, units - u0);
    char* dq = static_cast<char*>(p.dev_buf) + static_cast<size_t>(slot) * per_slot;
    char* dk = dq + cq;
    char* dv = dk + ckv;
    char* dout = dv + ckv;
    TSM_CUDA(cudaMemcpyAsync(dq, static_cast<const char*>(q) + u0 * unit_q, nu * unit_q, cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
    TSM_CUDA(cudaMemcpyAsync(dk, static_cast<const char*>(k) + u0 * head_bytes, nu * head_bytes, cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
    TSM_CUDA(cudaMemcpyAsync(dv, static_cast<const char*>(v) + u0 * head_bytes, nu * head_bytes, cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
    tsm100_attention_desc d = *desc;
    d.batch = static_cast<int32_t>(nu);
    d.heads_q = group;
    d.heads_kv = 1;
    st = ops::attention(&err, &d, dq, dk, dv, dout, dev->status, s);
    if (st != TSM100_OK) return finish(st, err);
    TSM_CUDA(cudaMemcpyAsync(static_cast<char*>(o) + u0 * unit_q, dout, nu * unit_q, cudaMemcpyDeviceToHost, s), TSM100_ERR_MEMORY);
  }
  return sync_pipe(dev);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Tensor-core GEMM for callers that must not allocate device memory.
//
// Every other entry point needs a tsm100_device_t, and opening one calls
// cudaMalloc for the word the kernel reports a timed-out wait in.  Some callers
// cannot allocate at all: code that runs while a stream is being captured into a
// CUDA graph (cudaMalloc is refused there), hosts that freeze their device heap
// after start-up, and latency-critical loops that cannot take the implicit
// device synchronisation of cudaMalloc / cudaFree.  For them the scratch word
// lives in the file-scope array below, which every GPU that loads this library
// holds (256 bytes) until the process exits.
//
// In host code `g_static_scratch` is only a stand-in for the symbol, not a device
// address; the address is asked for once per device with cudaGetSymbolAddress
// while that device is current, and that pointer is what the kernel receives.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxStaticDevices] = {};

// Device address of g_static_scratch on the current device (looked up on first use).
int32_t static_scratch_address(void** out) {
  int dev = -1;
  TSM_CUDA(cudaGetDevice(&dev), TSM100_ERR_NO_DEVICE);
  if (dev < 0 || dev >= kMaxStaticDevices) return fail(TSM100_ERR_INVALID, "device ordinal %d is beyond the %d this entry point tracks", dev, kMaxStaticDevices);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    TSM_CUDA(cudaGetSymbolAddress(&p, g_static_scratch), TSM100_ERR_RUNTIME);
    if (!p) return fail(TSM100_ERR_RUNTIME, "cudaGetSymbolAddress returned a null address for the static scratch");
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return TSM100_OK;
}

// Scratch the tensor-core GEMM needs for a problem: one status word, whatever the shape.
size_t gemm_tc_scratch_bytes(const tsm100_gemm_desc*) { return sizeof(uint32_t); }

// The shapes the tensor-core kernel takes (the same conditions under which tsm100_gemm picks it).
bool gemm_tc_takes(const tsm100_gemm_desc* d, const void* a, const void* b, const void* c) {
  const ops::GemmPitch ld = ops::gemm_pitch(d);
  return d->dtype != TSM100_F32 && ops::aligned16(a) && ops::aligned16(b) && ops::aligned16(c) && d->k % 8 == 0 &&
         (d->b_transposed || d->n % 8 == 0) && (d->n * ops::dtype_size(d->out_dtype)) % 16 == 0 &&
         ld.lda % 8 == 0 && ld.ldb % 8 == 0 && (ld.ldc * ops::dtype_size(d->out_dtype)) % 16 == 0 &&
         (static_cast<int64_t>((d->m + 127) / 128) * ((d->n + 255) / 256) * d->batch < 0x7fffffff);
}

}  // namespace

extern "C" int32_t tsm100_gemm_static_scratch(const tsm100_gemm_desc* desc, const void* a, const void* b, void* c,
                                              void* stream, uint32_t* status_host) {
  if (!desc || !a || !b || !c) return fail(TSM100_ERR_INVALID, "gemm_static_scratch: null argument");
  if (!ops::dtype_valid(desc->dtype) || !ops::dtype_valid(desc->out_dtype) || desc->m <= 0 || desc->n <= 0 ||
      desc->k <= 0 || desc->batch <= 0)
    return fail(TSM100_ERR_INVALID, "gemm_static_scratch: bad descriptor (every dimension must be positive)");
  if (!gemm_tc_takes(desc, a, b, c))
    return fail(TSM100_ERR_INVALID,
                "gemm_static_scratch: only the tensor-core kernel is offered without allocation: 16-bit inputs, 16-byte "
                "aligned pointers, K (and N for row-major B) a multiple of 8; use tsm100_gemm for this problem");
  const size_t need = gemm_tc_scratch_bytes(desc);
  if (need > kStaticScratchBytes)
    return fail(TSM100_ERR_INVALID, "gemm_static_scratch: this problem needs %zu bytes of scratch, the static array holds %zu",
                need, kStaticScratchBytes);
  void* scratch = nullptr;
  int32_t st = static_scratch_address(&scratch);
  if (st != TSM100_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the last call left: the status word must start at zero.
  TSM_CUDA(cudaMemsetAsync(scratch, 0, need, s), TSM100_ERR_RUNTIME);
  std::string err;
  st = ops::gemm(&err, desc, a, b, c, static_cast<uint32_t*>(scratch), stream);
  if (st != TSM100_OK) return finish(st, err);
  if (status_host)
    TSM_CUDA(cudaMemcpyAsync(status_host, scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost, s), TSM100_ERR_RUNTIME);
  return TSM100_OK;
}
