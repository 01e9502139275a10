// Multi-GPU launcher: one problem described once, split over a list of devices.
//
// The reference's HAL drives one GPU per process (crates/tile_hal/src/cuda.rs:321-327
// creates one context and never re-selects it; crates/tile_hal/src/backend.rs:95-112
// hands out devices one at a time).  The hot path has no exchange step, so a problem
// splits into independent shards: softmax rows, GEMM batches (or N-column blocks of one
// large GEMM), attention (batch, KV head) groups - the per-block tiles of #[tile_kernel]
// (crates/tile_std_macros/src/lib.rs:237-254).  tsm100_multi_run gives every listed
// device its shard on a host thread of its own: upload from the caller's host buffers,
// `launches` kernel launches on the resident shard (timed with CUDA events), download
// into the caller's output buffer.  Devices never read each other's memory and no
// collective is involved; the calling thread only watches the clock.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "common.hpp"

using namespace tsm100;

namespace {

inline size_t dtype_bytes(int32_t dtype) { return dtype == TSM100_F32 ? 4 : 2; }
inline size_t round256(size_t v) { return (v + 255) / 256 * 256; }
constexpr int64_t kColumnGranule = 256;  // one N tile of the CTA-pair GEMM

void set_message(tsm100_multi_report* r, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void set_message(tsm100_multi_report* r, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(r->message, sizeof r->message, fmt, ap);
  va_end(ap);
}

// How many units the job has and what they are.
int32_t job_units(const tsm100_multi_job* job, int64_t* units, int64_t* granule) {
  *granule = 1;
  if (!job || !job->desc) return fail(TSM100_ERR_INVALID, "multi: null job or descriptor");
  switch (job->op) {
    case TSM100_OP_SOFTMAX: {
      const auto* d = static_cast<const tsm100_softmax_desc*>(job->desc);
      if (d->rows < 0 || d->cols < 0) return fail(TSM100_ERR_INVALID, "multi: negative softmax shape");
      *units = d->rows;
      return TSM100_OK;
    }
    case TSM100_OP_GEMM: {
      const auto* d = static_cast<const tsm100_gemm_desc*>(job->desc);
      if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0) return fail(TSM100_ERR_INVALID, "multi: negative GEMM shape");
      if (d->batch == 1) {  // one large problem: N-column blocks, whole N tiles
        *granule = kColumnGranule;
        *units = d->n;
      } else {
        if (d->lda || d->ldb || d->ldc) return fail(TSM100_ERR_INVALID, "multi: a batched GEMM is split by problems and must be packed (lda = ldb = ldc = 0)");
        *units = d->batch;
      }
      return TSM100_OK;
    }
    case TSM100_OP_ATTENTION: {
      const auto* d = static_cast<const tsm100_attention_desc*>(job->desc);
      if (d->batch < 0 || d->heads_q < 0 || d->heads_kv <= 0 || d->heads_q % d->heads_kv != 0 || d->seq < 0 || d->head_dim < 0)
        return fail(TSM100_ERR_INVALID, "multi: bad attention shape (heads_q must be a multiple of heads_kv > 0)");
      *units = static_cast<int64_t>(d->batch) * d->heads_kv;
      return TSM100_OK;
    }
    default:
      return fail(TSM100_ERR_INVALID, "multi: unknown op %d", job->op);
  }
}

// ---------------------------------------------------------------------------
// per-device resources, kept between runs (a grow-only workspace: cudaMalloc of a few GiB
// costs milliseconds, which would otherwise sit inside every end-to-end time)
// ---------------------------------------------------------------------------
struct DeviceSlot {
  std::mutex mu;  // one run at a time per device
  tsm100_device_t dev = nullptr;
  void* stream = nullptr;
  void* ev[4] = {nullptr, nullptr, nullptr, nullptr};
  void* buf = nullptr;
  size_t cap = 0;
};
constexpr int kMaxDevices = 64;
DeviceSlot g_slots[kMaxDevices];

int32_t slot_prepare(DeviceSlot& s, int32_t ordinal, size_t bytes) {
  int32_t st;
  if (!s.dev) {
    if ((st = tsm100_device_open(ordinal, &s.dev)) != TSM100_OK) return st;
    if ((st = tsm100_stream_create(s.dev, &s.stream)) != TSM100_OK) return st;
    for (auto& e : s.ev)
      if ((st = tsm100_event_create(s.dev, &e)) != TSM100_OK) return st;
  }
  if (bytes > s.cap) {
    if (s.buf) {
      if ((st = tsm100_free(s.dev, s.buf)) != TSM100_OK) return st;
      s.buf = nullptr;
      s.cap = 0;
    }
    if ((st = tsm100_alloc(s.dev, bytes, &s.buf)) != TSM100_OK) return st;
    s.cap = bytes;
  }
  return TSM100_OK;
}

void slot_release(DeviceSlot& s) {
  if (!s.dev) return;
  if (s.buf) tsm100_free(s.dev, s.buf);
  for (auto& e : s.ev)
    if (e) tsm100_event_destroy(s.dev, e);
  if (s.stream) tsm100_stream_destroy(s.dev, s.stream);
  tsm100_device_close(s.dev);
  s.dev = nullptr;
  s.stream = nullptr;
  for (auto& e : s.ev) e = nullptr;
  s.buf = nullptr;
  s.cap = 0;
}

// Rows between the caller's (pitched) host matrix and the device's packed copy.
int32_t rows_h2d(char* dst, const char* src, size_t spitch, size_t width, int64_t rows, cudaStream_t s) {
  if (rows <= 0 || width == 0) return TSM100_OK;
  if (spitch == width) {
    TSM_CUDA(cudaMemcpyAsync(dst, src, width * static_cast<size_t>(rows), cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
  } else {
    TSM_CUDA(cudaMemcpy2DAsync(dst, width, src, spitch, width, static_cast<size_t>(rows), cudaMemcpyHostToDevice, s), TSM100_ERR_MEMORY);
  }
  return TSM100_OK;
}
int32_t rows_d2h(char* dst, size_t dpitch, const char* src, size_t width, int64_t rows, cudaStream_t s) {
  if (rows <= 0 || width == 0) return TSM100_OK;
  if (dpitch == width) {
    TSM_CUDA(cudaMemcpyAsync(dst, src, width * static_cast<size_t>(rows), cudaMemcpyDeviceToHost, s), TSM100_ERR_MEMORY);
  } else {
    TSM_CUDA(cudaMemcpy2DAsync(dst, dpitch, src, width, width, static_cast<size_t>(rows), cudaMemcpyDeviceToHost, s), TSM100_ERR_MEMORY);
  }
  return TSM100_OK;
}

// The built-in worker: this device's shard on this device.
int32_t cuda_worker(void*, const tsm100_multi_job* job, int32_t ordinal, int64_t first, int64_t count,
                    tsm100_multi_report* rep) {
  if (count == 0) return TSM100_OK;  // more devices than units: nothing to do here
  if (ordinal < 0 || ordinal >= kMaxDevices) return fail(TSM100_ERR_INVALID, "device ordinal %d is beyond the %d the launcher tracks", ordinal, kMaxDevices);
  if (!job->out || !job->in[0]) return fail(TSM100_ERR_INVALID, "multi: null host buffer");
  DeviceSlot& slot = g_slots[ordinal];
  std::lock_guard<std::mutex> lock(slot.mu);
  const int launches = job->launches < 1 ? 1 : job->launches;
  int32_t st;

  // --- sizes of the shard's device buffers -------------------------------------------------
  size_t in_bytes[3] = {0, 0, 0}, out_bytes = 0;
  tsm100_softmax_desc sd{};
  tsm100_gemm_desc gd{};
  tsm100_attention_desc ad{};
  bool column_split = false;
  if (job->op == TSM100_OP_SOFTMAX) {
    sd = *static_cast<const tsm100_softmax_desc*>(job->desc);
    in_bytes[0] = out_bytes = static_cast<size_t>(count) * sd.cols * dtype_bytes(sd.dtype);
    sd.rows = count;
  } else if (job->op == TSM100_OP_GEMM) {
    gd = *static_cast<const tsm100_gemm_desc*>(job->desc);
    if (!job->in[1]) return fail(TSM100_ERR_INVALID, "multi: null host buffer");
    const size_t es = dtype_bytes(gd.dtype), os = dtype_bytes(gd.out_dtype);
    column_split = gd.batch == 1;
    if (column_split) {
      in_bytes[0] = static_cast<size_t>(gd.m) * gd.k * es;
      in_bytes[1] = static_cast<size_t>(gd.k) * count * es;
      out_bytes = static_cast<size_t>(gd.m) * count * os;
    } else {
      in_bytes[0] = static_cast<size_t>(count) * gd.m * gd.k * es;
      in_bytes[1] = static_cast<size_t>(count) * gd.k * gd.n * es;
      out_bytes = static_cast<size_t>(count) * gd.m * gd.n * os;
    }
  } else {
    ad = *static_cast<const tsm100_attention_desc*>(job->desc);
    if (!job->in[1] || !job->in[2]) return fail(TSM100_ERR_INVALID, "multi: null host buffer");
    const int group = ad.heads_q / ad.heads_kv;
    const size_t head = static_cast<size_t>(ad.seq) * ad.head_dim * dtype_bytes(ad.dtype);
    in_bytes[0] = out_bytes = head * group * count;
    in_bytes[1] = in_bytes[2] = head * count;
  }
  const size_t total = round256(in_bytes[0]) + round256(in_bytes[1]) + round256(in_bytes[2]) + round256(out_bytes);
  if ((st = slot_prepare(slot, ordinal, total)) != TSM100_OK) return st;
  char* din[3];
  din[0] = static_cast<char*>(slot.buf);
  din[1] = din[0] + round256(in_bytes[0]);
  din[2] = din[1] + round256(in_bytes[1]);
  char* dout = din[2] + round256(in_bytes[2]);
  cudaStream_t s = static_cast<cudaStream_t>(slot.stream);
  const char* h0 = static_cast<const char*>(job->in[0]);
  const char* h1 = static_cast<const char*>(job->in[1]);
  const char* h2 = static_cast<const char*>(job->in[2]);
  char* hout = static_cast<char*>(job->out);

  // --- upload ---------------------------------------------------------------------------------
  if ((st = tsm100_event_record(slot.dev, slot.ev[0], slot.stream)) != TSM100_OK) return st;
  if (job->op == TSM100_OP_SOFTMAX) {
    st = rows_h2d(din[0], h0 + static_cast<size_t>(first) * sd.cols * dtype_bytes(sd.dtype), in_bytes[0], in_bytes[0], 1, s);
  } else if (job->op == TSM100_OP_GEMM) {
    const size_t es = dtype_bytes(gd.dtype);
    if (column_split) {
      const size_t lda = static_cast<size_t>(gd.lda ? gd.lda : gd.k) * es;
      st = rows_h2d(din[0], h0, lda, static_cast<size_t>(gd.k) * es, gd.m, s);
      if (st == TSM100_OK) {
        if (gd.b_transposed) {  // B stored [N, K]: the column block of C is a row block of it
          const size_t ldb = static_cast<size_t>(gd.ldb ? gd.ldb : gd.k) * es;
          st = rows_h2d(din[1], h1 + static_cast<size_t>(first) * ldb, ldb, static_cast<size_t>(gd.k) * es, count, s);
        } else {                // B stored [K, N]: columns [first, first + count) of every row
          const size_t ldb = static_cast<size_t>(gd.ldb ? gd.ldb : gd.n) * es;
          st = rows_h2d(din[1], h1 + static_cast<size_t>(first) * es, ldb, static_cast<size_t>(count) * es, gd.k, s);
        }
      }
    } else {
      st = rows_h2d(din[0], h0 + static_cast<size_t>(first) * gd.m * gd.k * es, in_bytes[0], in_bytes[0], 1, s);
      if (st == TSM100_OK) st = rows_h2d(din[1], h1 + static_cast<size_t>(first) * gd.k * gd.n * es, in_bytes[1], in_bytes[1], 1, s);
    }
  } else {
    const int group = ad.heads_q / ad.heads_kv;
    const size_t head = static_cast<size_t>(ad.seq) * ad.head_dim * dtype_bytes(ad.dtype);
    st = rows_h2d(din[0], h0 + static_cast<size_t>(first) * group * head, in_bytes[0], in_bytes[0], 1, s);
    if (st == TSM100_OK) st = rows_h2d(din[1], h1 + static_cast<size_t>(first) * head, in_bytes[1], in_bytes[1], 1, s);
    if (st == TSM100_OK) st = rows_h2d(din[2], h2 + static_cast<size_t>(first) * head, in_bytes[2], in_bytes[2], 1, s);
  }
  if (st != TSM100_OK) return st;
  if ((st = tsm100_event_record(slot.dev, slot.ev[1], slot.stream)) != TSM100_OK) return st;

  // --- compute: `launches` launches on the resident shard ----------------------------------
  for (int l = 0; l < launches; ++l) {
    if (job->op == TSM100_OP_SOFTMAX) {
      st = tsm100_softmax(slot.dev, &sd, din[0], dout, slot.stream);
    } else if (job->op == TSM100_OP_GEMM) {
      tsm100_gemm_desc d = gd;
      d.lda = d.ldb = d.ldc = 0;  // the device copies are packed
      if (column_split) d.n = count;
      else d.batch = static_cast<int32_t>(count);
      st = tsm100_gemm(slot.dev, &d, din[0], din[1], dout, slot.stream);
    } else {
      tsm100_attention_desc d = ad;
      d.batch = static_cast<int32_t>(count);
      d.heads_q = ad.heads_q / ad.heads_kv;
      d.heads_kv = 1;
      st = tsm100_attention(slot.dev, &d, din[0], din[1], din[2], dout, slot.stream);
    }
    if (st != TSM100_OK) return st;
  }
  if ((st = tsm100_event_record(slot.dev, slot.ev[2], slot.stream)) != TSM100_OK) return st;

  // --- download ---------------------------------------------------------------------------------
  if (job->op == TSM100_OP_SOFTMAX) {
    st = rows_d2h(hout + static_cast<size_t>(first) * sd.cols * dtype_bytes(sd.dtype), out_bytes, dout, out_bytes, 1, s);
  } else if (job->op == TSM100_OP_GEMM) {
    const size_t os = dtype_bytes(gd.out_dtype);
    if (column_split) {
      const size_t ldc = static_cast<size_t>(gd.ldc ? gd.ldc : gd.n) * os;
      st = rows_d2h(hout + static_cast<size_t>(first) * os, ldc, dout, static_cast<size_t>(count) * os, gd.m, s);
    } else {
      st = rows_d2h(hout + static_cast<size_t>(first) * gd.m * gd.n * os, out_bytes, dout, out_bytes, 1, s);
    }
  } else {
    const int group = ad.heads_q / ad.heads_kv;
    const size_t head = static_cast<size_t>(ad.seq) * ad.head_dim * dtype_bytes(ad.dtype);
    st = rows_d2h(hout + static_cast<size_t>(first) * group * head, out_bytes, dout, out_bytes, 1, s);
  }
  if (st != TSM100_OK) return st;
  if ((st = tsm100_event_record(slot.dev, slot.ev[3], slot.stream)) != TSM100_OK) return st;

  // --- wait (the kernels' own waits are bounded, so this ends) and collect ------------------
  uint32_t word = 0;
  if ((st = tsm100_device_status(slot.dev, slot.stream, &word)) != TSM100_OK) return st;
  rep->device_status = word;
  float ms = 0.f;
  if (tsm100_event_elapsed_ms(slot.dev, slot.ev[0], slot.ev[1], &ms) == TSM100_OK) rep->upload_ms = ms;
  if (tsm100_event_elapsed_ms(slot.dev, slot.ev[1], slot.ev[2], &ms) == TSM100_OK) rep->kernel_ms = ms / launches;
  if (tsm100_event_elapsed_ms(slot.dev, slot.ev[2], slot.ev[3], &ms) == TSM100_OK) rep->download_ms = ms;
  if (word != 0) return fail(TSM100_ERR_TIMEOUT, "a kernel gave up a bounded device-side wait (status 0x%x)", word);
  return TSM100_OK;
}

struct WorkerState {
  std::thread thread;
  std::atomic<bool> done{false};
  bool timed_out = false;
  tsm100_multi_report local{};
  std::string error;
};

}  // namespace

extern "C" {

int32_t tsm100_multi_plan(const tsm100_multi_job* job, int32_t n, int32_t index, int64_t* first, int64_t* count) {
  if (!first || !count) return fail(TSM100_ERR_INVALID, "multi_plan: null output pointer");
  int64_t units = 0, granule = 1;
  int32_t st = job_units(job, &units, &granule);
  if (st != TSM100_OK) return st;
  if (n <= 0 || index < 0 || index >= n) return fail(TSM100_ERR_INVALID, "multi_plan: bad device index %d of %d", index, n);
  // whole granules are dealt out like tsm100_shard_range deals units; the last block may be ragged
  const int64_t blocks = (units + granule - 1) / granule;
  int64_t bf = 0, bc = 0;
  st = tsm100_shard_range(blocks, n, index, &bf, &bc);
  if (st != TSM100_OK) return st;
  const int64_t lo = std::min(units, bf * granule), hi = std::min(units, (bf + bc) * granule);
  *first = lo;
  *count = hi - lo;
  return TSM100_OK;
}

int32_t tsm100_multi_run_with(const tsm100_multi_job* job, const int32_t* ordinals, int32_t n, tsm100_multi_report* reports,
                              tsm100_multi_worker_fn worker, void* user) {
  if (!job || !ordinals || !reports || n <= 0) return fail(TSM100_ERR_INVALID, "multi_run: null argument or empty device list");
  if (!worker) worker = cuda_worker;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < i; ++j)
      if (ordinals[i] == ordinals[j]) return fail(TSM100_ERR_INVALID, "multi_run: device %d is listed twice", ordinals[i]);
  std::vector<int64_t> first(n), count(n);
  for (int i = 0; i < n; ++i) {
    int32_t st = tsm100_multi_plan(job, n, i, &first[i], &count[i]);
    if (st != TSM100_OK) return st;
  }
  std::vector<WorkerState> ws(n);
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < n; ++i) {
    WorkerState& w = ws[i];
    w.local.ordinal = ordinals[i];
    w.local.first = first[i];
    w.local.count = count[i];
    w.thread = std::thread([&, i] {
      WorkerState& me = ws[i];
      last_error_ref().clear();
      const auto w0 = std::chrono::steady_clock::now();
      me.local.status = worker(user, job, ordinals[i], first[i], count[i], &me.local);
      me.local.total_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - w0).count();
      if (me.local.status != TSM100_OK) me.error = me.local.message[0] ? me.local.message : last_error_ref();
      me.done.store(true, std::memory_order_release);
    });
  }
  // the calling thread only watches the clock: a device past its limit is named at once, and joined when it has drained
  if (job->timeout_ms > 0) {
    int pending = n;
    while (pending > 0) {
      pending = 0;
      const float elapsed = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
      for (int i = 0; i < n; ++i) {
        if (ws[i].done.load(std::memory_order_acquire)) continue;
        ++pending;
        if (elapsed > static_cast<float>(job->timeout_ms)) ws[i].timed_out = true;
      }
      if (pending) std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
  }
  for (auto& w : ws) w.thread.join();
  int32_t result = TSM100_OK;
  std::string result_msg;
  for (int i = 0; i < n; ++i) {
    WorkerState& w = ws[i];
    reports[i] = w.local;
    if (w.timed_out) {
      reports[i].status = TSM100_ERR_TIMEOUT;
      set_message(&reports[i], "device %d did not finish within %d ms (it took %.1f ms)", ordinals[i], job->timeout_ms,
                  w.local.total_ms);
    } else if (w.local.status != TSM100_OK) {
      set_message(&reports[i], "device %d: %s", ordinals[i], w.error.c_str());
    }
    if (reports[i].status != TSM100_OK && result == TSM100_OK) {
      result = reports[i].status;
      result_msg = reports[i].message;
    }
  }
  if (result != TSM100_OK) return fail(result, "%s", result_msg.c_str());
  return TSM100_OK;
}

int32_t tsm100_multi_run(const tsm100_multi_job* job, const int32_t* ordinals, int32_t n, tsm100_multi_report* reports) {
  return tsm100_multi_run_with(job, ordinals, n, reports, nullptr, nullptr);
}

int32_t tsm100_multi_release(void) {
  for (auto& s : g_slots) {
    std::lock_guard<std::mutex> lock(s.mu);
    slot_release(s);
  }
  return TSM100_OK;
}

}  // extern "C"
