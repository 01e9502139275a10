// Host-side plumbing shared by the C-ABI translation units: per-thread error
// text, the device handle, CUDA error mapping.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tile_sm100.h"

namespace tsm100 {

std::string& last_error_ref();

// Records a formatted message for tsm100_last_error() and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Maps a CUDA runtime status to a C-ABI status, recording "<what> failed: ...".
int32_t check_cuda(cudaError_t e, int32_t code, const char* what);

#define TSM_CUDA(expr, code)                                  \
  do {                                                        \
    int32_t _st = ::tsm100::check_cuda((expr), (code), #expr); \
    if (_st != TSM100_OK) return _st;                         \
  } while (0)

// Staging resources for the *_host operators, created on first use and kept.
struct HostPipe {
  static constexpr int kSlots = 3;
  cudaStream_t stream[kSlots] = {nullptr, nullptr, nullptr};
  cudaEvent_t done[kSlots] = {nullptr, nullptr, nullptr};
  void* dev_buf = nullptr;     // grow-only device workspace
  size_t dev_bytes = 0;
  void* pin_buf = nullptr;     // grow-only page-locked bounce buffer (for pageable callers)
  size_t pin_bytes = 0;
  bool ready = false;
};

}  // namespace tsm100

struct tsm100_device_s {
  int32_t ordinal = 0;
  int32_t sm_count = 0;
  std::string name;
  uint32_t* status = nullptr;  // device word written by kernels whose bounded waits ran out
  std::mutex mu;               // guards `pipe`
  tsm100::HostPipe pipe;
};

namespace tsm100 {

// Makes dev's CUDA device current for the calling thread.
int32_t use_device(tsm100_device_t dev);

// Reads and clears the device status word (synchronises `stream`).
int32_t read_status(tsm100_device_t dev, cudaStream_t stream, uint32_t* value);

}  // namespace tsm100
