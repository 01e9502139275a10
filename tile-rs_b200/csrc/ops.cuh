// Host-side launch logic for the three operators: argument validation, kernel
// selection, tensor-map construction, launch.  Header-only so that both the
// library (capi_ops.cu) and the translation units the cuda_sm100 target emits
// instantiate the same kernels with the same dispatch.
//
// Every function returns a TSM100_* status and, on failure, writes a message
// to *err.  Nothing here synchronises; the one operator that needs device scratch (the
// tcgen05 f32 GEMM: the hi / lo planes of its operands) takes it from, and returns it to,
// the device's stream-ordered memory pool on the caller's stream.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <type_traits>

#include "../../include/tile_sm100.h"
#include "attention_decode.cuh"
#include "attention_simt.cuh"
#include "attention_tc.cuh"
#include "attention_tf32x3.cuh"
#include "ewise.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "gemm_tc2.cuh"
#include "gemm_tf32_tc.cuh"
#include "gemm_tf32x3.cuh"
#include "rowops.cuh"
#include "softmax.cuh"

namespace tsm100 {
namespace ops {

inline int32_t op_fail(std::string* err, int32_t code, const std::string& msg) {
  if (err) *err = msg;
  return code;
}

inline int32_t cuda_ok(std::string* err, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TSM100_OK;
  const int32_t code = (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? TSM100_ERR_NO_DEVICE
                                                                                      : TSM100_ERR_LAUNCH;
  return op_fail(err, code, std::string(what) + " failed: " + cudaGetErrorString(e));
}

inline size_t dtype_size(int32_t dtype) { return dtype == TSM100_F32 ? 4 : 2; }
inline bool dtype_valid(int32_t dtype) { return dtype == TSM100_F32 || dtype == TSM100_F16 || dtype == TSM100_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// per-(kernel, device) facts: asked of the CUDA runtime once, then remembered
// ---------------------------------------------------------------------------
// cudaFuncSetAttribute and the occupancy queries cost a few microseconds each, which is as long as
// a small launch itself; their answers depend on the kernel and the device only.
struct KernelFacts {
  std::mutex mu;
  std::map<std::tuple<const void*, int, int>, int> value;  // (kernel, device, what) -> answer
};
inline KernelFacts& kernel_facts() {
  static KernelFacts f;
  return f;
}
enum { kFactSmemSet = 1, kFactNonPortableSet = 2, kFactBlocksPerSm = 3, kFactClusters = 4 };

// `compute` returns (ok, answer); an answer is remembered only when ok.
template <typename F>
inline bool kernel_fact(const void* kern, int what, int* answer, F compute) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  KernelFacts& f = kernel_facts();
  const auto key = std::make_tuple(kern, dev, what);
  {
    std::lock_guard<std::mutex> lock(f.mu);
    auto it = f.value.find(key);
    if (it != f.value.end()) {
      *answer = it->second;
      return true;
    }
  }
  if (!compute(answer)) return false;
  std::lock_guard<std::mutex> lock(f.mu);
  f.value[key] = *answer;
  return true;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize, set once per kernel and device.
template <typename K>
inline cudaError_t set_dyn_smem_once(K kern, int bytes) {
  cudaError_t e = cudaSuccess;
  int unused = 0;
  kernel_fact(reinterpret_cast<const void*>(kern), kFactSmemSet, &unused, [&](int* out) {
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern), cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    *out = bytes;
    return e == cudaSuccess;
  });
  return e;
}
template <typename K>
inline cudaError_t allow_wide_clusters_once(K kern) {
  cudaError_t e = cudaSuccess;
  int unused = 0;
  kernel_fact(reinterpret_cast<const void*>(kern), kFactNonPortableSet, &unused, [&](int* out) {
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern), cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    *out = 1;
    return e == cudaSuccess;
  });
  return e;
}
// Resident CTAs per SM of a kernel launched with `threads` threads and no dynamic shared memory (at least 1).
template <typename K>
inline int blocks_per_sm(K kern, int threads) {
  int per_sm = 1;
  kernel_fact(reinterpret_cast<const void*>(kern), kFactBlocksPerSm + (threads << 8), &per_sm, [&](int* out) {
    int n = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, 0) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      return false;
    }
    *out = n;
    return true;
  });
  return per_sm < 1 ? 1 : per_sm;
}

// ---------------------------------------------------------------------------
// tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int32_t encode_fn(std::string* err, EncodeTiledFn* out) {
  static EncodeTiledFn cached = nullptr;
  if (!cached) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return op_fail(err, TSM100_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return TSM100_OK;
}

// A map is a pure function of its arguments, and a repeated launch (same pointers, same shape) asks for the same
// ones again: each thread keeps the last few it encoded.
struct TmapKey {
  const void* base;
  uint64_t dim[3], stride[2];
  uint32_t box[2];
  int32_t dtype;
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used = false;
};

// dims (x contiguous, y, z), strides in elements of `elem_bytes`, box (box_x, box_y, 1), 128-byte swizzle,
// out-of-range elements read as zero.
inline int32_t make_tmap_3d(std::string* err, CUtensorMap* out, const void* base, uint64_t dim_x, uint64_t dim_y,
                            uint64_t dim_z, uint64_t stride_y, uint64_t stride_z, uint32_t box_x, uint32_t box_y,
                            CUtensorMapDataType dtype, uint32_t elem_bytes) {
  constexpr int kSlots = 16;
  static thread_local TmapSlot cache[kSlots];
  static thread_local int next = 0;
  TmapKey key;
  std::memset(&key, 0, sizeof key);
  key.base = base;
  key.dim[0] = dim_x, key.dim[1] = dim_y, key.dim[2] = dim_z;
  key.stride[0] = stride_y, key.stride[1] = stride_z;
  key.box[0] = box_x, key.box[1] = box_y;
  key.dtype = static_cast<int32_t>(dtype);
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].used && std::memcmp(&cache[i].key, &key, sizeof key) == 0) {
      *out = cache[i].map;
      return TSM100_OK;
    }
  EncodeTiledFn fn;
  int32_t st = encode_fn(err, &fn);
  if (st != TSM100_OK) return st;
  cuuint64_t dims[3] = {dim_x, dim_y, dim_z};
  cuuint64_t strides[2] = {stride_y * elem_bytes, stride_z * elem_bytes};  // bytes; dimension 0 is contiguous
  cuuint32_t box[3] = {box_x, box_y, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((strides[0] & 15u) || (strides[1] & 15u) || !aligned16(base))
    return op_fail(err, TSM100_ERR_INVALID, "tensor map needs a 16-byte aligned base and 16-byte-multiple strides");
  CUresult r = fn(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed: CUresult %d", static_cast<int>(r));
    return op_fail(err, TSM100_ERR_LAUNCH, buf);
  }
  TmapSlot& slot = cache[next];
  next = (next + 1) % kSlots;
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return TSM100_OK;
}

// 16-bit elements (bf16 or f16).
inline int32_t make_tmap_16bit_3d(std::string* err, CUtensorMap* out, const void* base, uint64_t dim_x,
                                  uint64_t dim_y, uint64_t dim_z, uint64_t stride_y, uint64_t stride_z,
                                  uint32_t box_x, uint32_t box_y, bool is_bf16) {
  return make_tmap_3d(err, out, base, dim_x, dim_y, dim_z, stride_y, stride_z, box_x, box_y,
                      is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2);
}

inline int32_t sm_count(std::string* err, int* sms) {
  static int cached[64] = {0};
  int dev = 0;
  int32_t st = cuda_ok(err, cudaGetDevice(&dev), "cudaGetDevice");
  if (st != TSM100_OK) return st;
  if (dev < 64 && cached[dev]) {
    *sms = cached[dev];
    return TSM100_OK;
  }
  int n = 0;
  st = cuda_ok(err, cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
  if (st != TSM100_OK) return st;
  if (dev < 64) cached[dev] = n;
  *sms = n;
  return TSM100_OK;
}

// ---------------------------------------------------------------------------
// softmax
// ---------------------------------------------------------------------------
template <typename T, int CHUNKS>
inline cudaError_t launch_softmax_warp(const T* x, T* y, int64_t rows, int32_t cols, cudaStream_t s) {
  constexpr int WARPS = 4;
  const int64_t grid = (rows + WARPS - 1) / WARPS;
  softmax::softmax_rows_warp<T, CHUNKS, WARPS><<<static_cast<unsigned>(grid), WARPS * 32, 0, s>>>(x, y, rows, cols);
  return cudaGetLastError();
}

template <typename T>
inline int32_t softmax_typed(std::string* err, const T* x, T* y, int64_t rows, int64_t cols, cudaStream_t s) {
  constexpr int PV = softmax::Elem<T>::kPerVec;
  const bool vec_ok = (cols % PV == 0) && aligned16(x) && aligned16(y);
  const int64_t nvec = cols / PV;
  cudaError_t e;
  if (vec_ok && nvec <= 32 * 8 && rows <= 4ll * 0x7fffffff) {  // one warp per row
    const int32_t c = static_cast<int32_t>(cols);
    if (nvec <= 32 * 1) e = launch_softmax_warp<T, 1>(x, y, rows, c, s);
    else if (nvec <= 32 * 2) e = launch_softmax_warp<T, 2>(x, y, rows, c, s);
    else if (nvec <= 32 * 4) e = launch_softmax_warp<T, 4>(x, y, rows, c, s);
    else e = launch_softmax_warp<T, 8>(x, y, rows, c, s);
    return cuda_ok(err, e, "softmax_rows_warp launch");
  }
  if (vec_ok && nvec <= 256 * 8) {  // 128 or 256 threads per row, 32 values each
    int sms_cta = 0;
    int32_t st_cta = sm_count(err, &sms_cta);
    if (st_cta != TSM100_OK) return st_cta;
    const int32_t c = static_cast<int32_t>(cols);
    // persistent CTAs: exactly as many as are resident at once, each striding over the rows
    auto launch = [&](auto kern, int threads) {
      const int per_sm = blocks_per_sm(kern, threads);
      const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, static_cast<int64_t>(sms_cta) * per_sm));
      kern<<<grid, threads, 0, s>>>(x, y, rows, c);
    };
    if (nvec <= 128 * 4) launch(softmax::softmax_rows_cta<T, 4, 128>, 128);
    else if (nvec <= 128 * 8) launch(softmax::softmax_rows_cta<T, 8, 128>, 128);
    else launch(softmax::softmax_rows_cta<T, 8, 256>, 256);
    return cuda_ok(err, cudaGetLastError(), "softmax_rows_cta launch");
  }
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  constexpr int64_t kMaxBlockCols = 56 * 1024;  // 224 KiB of f32 in shared memory
  if (vec_ok && cols <= kMaxBlockCols) {
    constexpr int THREADS = 512;
    const size_t smem = static_cast<size_t>(cols) * sizeof(float);
    auto kern = softmax::softmax_rows_block<T, THREADS>;
    e = set_dyn_smem_once(kern, static_cast<int>(kMaxBlockCols * sizeof(float)));  // the most this path ever asks for
    if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(softmax_rows_block)");
    const int per_sm = static_cast<int>(std::max<size_t>(1, std::min<size_t>(4, (220 * 1024) / (smem + 1024))));
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, static_cast<int64_t>(sms) * per_sm));
    kern<<<grid, THREADS, smem, s>>>(x, y, rows, static_cast<int32_t>(cols));
    return cuda_ok(err, cudaGetLastError(), "softmax_rows_block launch");
  }
  constexpr int THREADS = 512;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, static_cast<int64_t>(sms) * 4));
  softmax::softmax_rows_stream<T, THREADS><<<grid, THREADS, 0, s>>>(x, y, rows, cols);
  return cuda_ok(err, cudaGetLastError(), "softmax_rows_stream launch");
}

inline int32_t softmax(std::string* err, const tsm100_softmax_desc* d, const void* x, void* y, void* stream) {
  if (!d || !x || !y) return op_fail(err, TSM100_ERR_INVALID, "softmax: null argument");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "softmax: unknown dtype");
  if (d->rows < 0 || d->cols < 0) return op_fail(err, TSM100_ERR_INVALID, "softmax: negative shape");
  if (d->rows == 0 || d->cols == 0) return TSM100_OK;  // empty tile: nothing to do
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (d->dtype) {
    case TSM100_F32:
      return softmax_typed<float>(err, static_cast<const float*>(x), static_cast<float*>(y), d->rows, d->cols, s);
    case TSM100_BF16:
      return softmax_typed<__nv_bfloat16>(err, static_cast<const __nv_bfloat16*>(x),
                                          static_cast<__nv_bfloat16*>(y), d->rows, d->cols, s);
    default:
      return softmax_typed<__half>(err, static_cast<const __half*>(x), static_cast<__half*>(y), d->rows, d->cols, s);
  }
}

// ---------------------------------------------------------------------------
// rms_norm / row reductions / SiLU * Mul
// ---------------------------------------------------------------------------
template <typename T, int OP>
inline int32_t row_op_typed(std::string* err, const T* x, T* y, int64_t rows, int64_t cols, float eps, cudaStream_t s) {
  namespace ro = rowops;
  constexpr int PV = softmax::Elem<T>::kPerVec;
  const bool vec_ok = (cols % PV == 0) && aligned16(x) && (OP != ro::kRmsNorm || aligned16(y));
  const int64_t nvec = cols / PV;
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  // persistent CTAs: exactly as many as are resident at once, each striding over the rows
  auto launch = [&](auto kern, int threads, int rows_per_cta) {
    const int per_sm = blocks_per_sm(kern, threads);
    const int64_t want = (rows + rows_per_cta - 1) / rows_per_cta;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(want, static_cast<int64_t>(sms) * per_sm));
    kern<<<grid, threads, 0, s>>>(x, y, rows, static_cast<int32_t>(cols), eps);
  };
  if (vec_ok && nvec <= 32 * 8) {  // one warp per row, four rows per CTA
    if (nvec <= 32 * 1) launch(ro::row_op_kernel<T, OP, 1, 32, 128>, 128, 4);
    else if (nvec <= 32 * 2) launch(ro::row_op_kernel<T, OP, 2, 32, 128>, 128, 4);
    else if (nvec <= 32 * 4) launch(ro::row_op_kernel<T, OP, 4, 32, 128>, 128, 4);
    else launch(ro::row_op_kernel<T, OP, 8, 32, 128>, 128, 4);
    return cuda_ok(err, cudaGetLastError(), "row_op_kernel (warp per row) launch");
  }
  if (vec_ok && nvec <= 256 * 8) {  // 128 or 256 threads per row, 32 values each
    if (nvec <= 128 * 4) launch(ro::row_op_kernel<T, OP, 4, 128, 128>, 128, 1);
    else if (nvec <= 128 * 8) launch(ro::row_op_kernel<T, OP, 8, 128, 128>, 128, 1);
    else launch(ro::row_op_kernel<T, OP, 8, 256, 256>, 256, 1);
    return cuda_ok(err, cudaGetLastError(), "row_op_kernel (CTA per row) launch");
  }
  constexpr int THREADS = 512;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, static_cast<int64_t>(sms) * 4));
  ro::row_op_stream_kernel<T, OP, THREADS><<<grid, THREADS, 0, s>>>(x, y, rows, cols, eps);
  return cuda_ok(err, cudaGetLastError(), "row_op_stream_kernel launch");
}

template <int OP>
inline int32_t row_op(std::string* err, int32_t dtype, int64_t rows, int64_t cols, float eps, const void* x, void* y,
                      void* stream, const char* what) {
  if (!dtype_valid(dtype)) return op_fail(err, TSM100_ERR_INVALID, std::string(what) + ": unknown dtype");
  if (rows < 0 || cols < 0) return op_fail(err, TSM100_ERR_INVALID, std::string(what) + ": negative shape");
  // an empty tile has no input bytes: its pointer may be anything, a reduction still writes its fill value
  if (!y || (!x && rows > 0 && cols > 0)) return op_fail(err, TSM100_ERR_INVALID, std::string(what) + ": null argument");
  if (rows == 0) return TSM100_OK;
  if (cols == 0 && OP == rowops::kRmsNorm) return TSM100_OK;  // empty tile: nothing to write
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TSM100_F32:
      return row_op_typed<float, OP>(err, static_cast<const float*>(x), static_cast<float*>(y), rows, cols, eps, s);
    case TSM100_BF16:
      return row_op_typed<__nv_bfloat16, OP>(err, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y),
                                              rows, cols, eps, s);
    default:
      return row_op_typed<__half, OP>(err, static_cast<const __half*>(x), static_cast<__half*>(y), rows, cols, eps, s);
  }
}

inline int32_t rms_norm(std::string* err, const tsm100_rms_norm_desc* d, const void* x, void* y, void* stream) {
  if (!d) return op_fail(err, TSM100_ERR_INVALID, "rms_norm: null descriptor");
  return row_op<rowops::kRmsNorm>(err, d->dtype, d->rows, d->cols, d->eps, x, y, stream, "rms_norm");
}

inline int32_t reduce(std::string* err, const tsm100_reduce_desc* d, const void* x, void* y, void* stream) {
  if (!d) return op_fail(err, TSM100_ERR_INVALID, "reduce: null descriptor");
  if (d->kind == TSM100_REDUCE_SUM)
    return row_op<rowops::kReduceSum>(err, d->dtype, d->rows, d->cols, 0.f, x, y, stream, "reduce");
  if (d->kind == TSM100_REDUCE_MAX)
    return row_op<rowops::kReduceMax>(err, d->dtype, d->rows, d->cols, 0.f, x, y, stream, "reduce");
  return op_fail(err, TSM100_ERR_INVALID, "reduce: unknown kind");
}

template <typename T>
inline int32_t silu_mul_typed(std::string* err, const T* gate, const T* up, T* y, int64_t n, cudaStream_t s) {
  namespace ro = rowops;
  constexpr int PV = softmax::Elem<T>::kPerVec;
  // 16-bit data: twice the elements per byte, so twice the threads keep the same bytes in flight (measured: 5.87 -> 6.16 TB/s)
  constexpr int THREADS = sizeof(T) == 2 ? 512 : 256, UNROLL = 4;
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  const bool vec_ok = (n % PV == 0) && aligned16(gate) && aligned16(y) && (!up || aligned16(up));
  if (vec_ok) {
    const int64_t nvec = n / PV;
    const int64_t want = (nvec + THREADS * UNROLL - 1) / (THREADS * UNROLL);
    const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sms) * 8)));
    if (up) ro::silu_mul_kernel<T, true, UNROLL, THREADS><<<grid, THREADS, 0, s>>>(gate, up, y, nvec);
    else ro::silu_mul_kernel<T, false, UNROLL, THREADS><<<grid, THREADS, 0, s>>>(gate, up, y, nvec);
    return cuda_ok(err, cudaGetLastError(), "silu_mul_kernel launch");
  }
  const int64_t want = (n + THREADS - 1) / THREADS;
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sms) * 8)));
  if (up) ro::silu_mul_scalar_kernel<T, true, THREADS><<<grid, THREADS, 0, s>>>(gate, up, y, n);
  else ro::silu_mul_scalar_kernel<T, false, THREADS><<<grid, THREADS, 0, s>>>(gate, up, y, n);
  return cuda_ok(err, cudaGetLastError(), "silu_mul_scalar_kernel launch");
}

inline int32_t silu_mul(std::string* err, const tsm100_silu_mul_desc* d, const void* gate, const void* up, void* y,
                        void* stream) {
  if (!d || !gate || !y) return op_fail(err, TSM100_ERR_INVALID, "silu_mul: null argument");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "silu_mul: unknown dtype");
  if (d->rows < 0 || d->cols < 0) return op_fail(err, TSM100_ERR_INVALID, "silu_mul: negative shape");
  if (d->rows == 0 || d->cols == 0) return TSM100_OK;
  const int64_t n = d->rows * d->cols;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (d->dtype) {
    case TSM100_F32:
      return silu_mul_typed<float>(err, static_cast<const float*>(gate), static_cast<const float*>(up), static_cast<float*>(y), n, s);
    case TSM100_BF16:
      return silu_mul_typed<__nv_bfloat16>(err, static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                                           static_cast<__nv_bfloat16*>(y), n, s);
    default:
      return silu_mul_typed<__half>(err, static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                    static_cast<__half*>(y), n, s);
  }
}

// ---------------------------------------------------------------------------
// RoPE and KV-cache update
// ---------------------------------------------------------------------------
inline int32_t rope(std::string* err, const tsm100_rope_desc* d, void* x, void* stream) {
  if (!d) return op_fail(err, TSM100_ERR_INVALID, "rope: null descriptor");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "rope: unknown dtype");
  if (d->batch < 0 || d->seq_len < 0 || d->heads < 0 || d->head_dim < 0 || d->start_pos < 0 || d->head_dim % 2 != 0)
    return op_fail(err, TSM100_ERR_INVALID, "rope: bad shape (head_dim must be even, nothing negative)");
  if (!(d->theta > 0.f)) return op_fail(err, TSM100_ERR_INVALID, "rope: theta must be positive");
  const int64_t tokens = static_cast<int64_t>(d->batch) * d->seq_len;
  if (tokens == 0 || d->heads == 0 || d->head_dim == 0) return TSM100_OK;
  if (!x) return op_fail(err, TSM100_ERR_INVALID, "rope: null buffer");
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int pv = d->dtype == TSM100_F32 ? 4 : 8;  // elements per 16 bytes
  const bool vec = d->head_dim % pv == 0 && aligned16(x);
  const int64_t n = tokens * (vec ? d->head_dim / pv : d->head_dim / 2);
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, static_cast<int64_t>(sms) * 8)));
  auto launch = [&](auto* xt) {
    using T = std::remove_pointer_t<decltype(xt)>;
    if (vec) rowops::rope_vec_kernel<T><<<grid, 256, 0, s>>>(xt, tokens, d->seq_len, d->heads, d->head_dim, d->start_pos, d->theta);
    else rowops::rope_kernel<T><<<grid, 256, 0, s>>>(xt, tokens, d->seq_len, d->heads, d->head_dim, d->start_pos, d->theta);
  };
  if (d->dtype == TSM100_F32) launch(static_cast<float*>(x));
  else if (d->dtype == TSM100_BF16) launch(static_cast<__nv_bfloat16*>(x));
  else launch(static_cast<__half*>(x));
  return cuda_ok(err, cudaGetLastError(), "rope_kernel launch");
}

template <typename T>
inline cudaError_t kv_cache_update_typed(const tsm100_kv_cache_update_desc* d, const void* src, void* cache, int sms, cudaStream_t s) {
  constexpr int PV = softmax::Elem<T>::kPerVec;
  const bool vec = d->head_dim % PV == 0 && aligned16(src) && aligned16(cache);
  const int64_t n = static_cast<int64_t>(d->batch) * d->seq_len * d->heads * (vec ? d->head_dim / PV : d->head_dim);
  const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, static_cast<int64_t>(sms) * 8)));
  const bool small = n + static_cast<int64_t>(grid) * 256 < 0xffffffffll;  // the loop index cannot wrap
  auto launch = [&](auto vec_tag, auto index_tag) {
    constexpr int V = decltype(vec_tag)::value;
    using I = decltype(index_tag);
    rowops::kv_cache_update_kernel<T, V, I><<<grid, 256, 0, s>>>(static_cast<const T*>(src), static_cast<T*>(cache), d->batch,
                                                                 d->seq_len, d->heads, d->head_dim, d->start_pos, d->max_seq);
  };
  if (vec && small) launch(std::integral_constant<int, PV>{}, uint32_t{});
  else if (vec) launch(std::integral_constant<int, PV>{}, int64_t{});
  else if (small) launch(std::integral_constant<int, 1>{}, uint32_t{});
  else launch(std::integral_constant<int, 1>{}, int64_t{});
  return cudaGetLastError();
}

inline int32_t kv_cache_update(std::string* err, const tsm100_kv_cache_update_desc* d, const void* src, void* cache, void* stream) {
  if (!d) return op_fail(err, TSM100_ERR_INVALID, "kv_cache_update: null descriptor");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "kv_cache_update: unknown dtype");
  if (d->batch < 0 || d->seq_len < 0 || d->heads < 0 || d->head_dim < 0 || d->start_pos < 0 ||
      static_cast<int64_t>(d->start_pos) + d->seq_len > d->max_seq)
    return op_fail(err, TSM100_ERR_INVALID, "kv_cache_update: bad shape (need start_pos + seq_len <= max_seq, nothing negative)");
  if (static_cast<int64_t>(d->batch) * d->seq_len * d->heads * d->head_dim == 0) return TSM100_OK;
  if (!src || !cache) return op_fail(err, TSM100_ERR_INVALID, "kv_cache_update: null buffer");
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = d->dtype == TSM100_F32    ? kv_cache_update_typed<float>(d, src, cache, sms, s)
                  : d->dtype == TSM100_BF16 ? kv_cache_update_typed<__nv_bfloat16>(d, src, cache, sms, s)
                                            : kv_cache_update_typed<__half>(d, src, cache, sms, s);
  return cuda_ok(err, e, "kv_cache_update_kernel launch");
}

// ---------------------------------------------------------------------------
// GEMM
// ---------------------------------------------------------------------------
// Row pitches of A, B and C in elements: the descriptor's value, or the row length when it is 0.
struct GemmPitch {
  int64_t lda, ldb, ldc;
};
inline GemmPitch gemm_pitch(const tsm100_gemm_desc* d) {
  return {d->lda ? d->lda : d->k, d->ldb ? d->ldb : (d->b_transposed ? d->k : d->n), d->ldc ? d->ldc : d->n};
}
template <typename InT, typename OutT>
inline int32_t gemm_simt_launch(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                                cudaStream_t s) {
  const GemmPitch ld = gemm_pitch(d);
  gemm_simt::Params p{static_cast<int32_t>(d->m), static_cast<int32_t>(d->n), static_cast<int32_t>(d->k), d->batch,
                      d->b_transposed, ld.lda, ld.ldb, ld.ldc};
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  const int64_t big_tiles = ((d->m + 63) / 64) * ((d->n + 63) / 64) * d->batch;
  if (big_tiles >= 2ll * sms) {
    dim3 grid(static_cast<unsigned>((d->n + 63) / 64), static_cast<unsigned>((d->m + 63) / 64),
              static_cast<unsigned>(d->batch));
    gemm_simt::gemm_simt_kernel<InT, OutT, 64, 64, 16, 4, 4><<<grid, 256, 0, s>>>(
        static_cast<const InT*>(a), static_cast<const InT*>(b), static_cast<OutT*>(c), p);
  } else {
    dim3 grid(static_cast<unsigned>((d->n + 31) / 32), static_cast<unsigned>((d->m + 31) / 32),
              static_cast<unsigned>(d->batch));
    gemm_simt::gemm_simt_kernel<InT, OutT, 32, 32, 16, 4, 4><<<grid, 64, 0, s>>>(
        static_cast<const InT*>(a), static_cast<const InT*>(b), static_cast<OutT*>(c), p);
  }
  return cuda_ok(err, cudaGetLastError(), "gemm_simt launch");
}

// f32 inputs on tensor cores (three TF32 products per product, see gemm_tf32x3.cuh)
inline int32_t gemm_tf32x3_launch(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                                  cudaStream_t s) {
  namespace g = gemm_tf32x3;
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  const int64_t tiles = ((d->m + g::kBM - 1) / g::kBM) * ((d->n + g::kBN - 1) / g::kBN) * d->batch;
  if (tiles * g::kMaxSplit > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "gemm: too many tiles for one launch");
  // fewer tiles than SMs: a cluster splits K while all CTAs still fit the GPU at once (two per SM) and every CTA
  // keeps at least four 32-deep slices
  int splits = 1;
  while (splits < g::kMaxSplit && tiles * splits * 2 <= 2 * sms && d->k / (2 * splits) >= 4 * g::kBK) splits *= 2;
  g::Params p;
  p.m = static_cast<int32_t>(d->m);
  p.n = static_cast<int32_t>(d->n);
  p.k = static_cast<int32_t>(d->k);
  p.batch = d->batch;
  p.k_per_cta = static_cast<int32_t>(((d->k + splits - 1) / splits + g::kBK - 1) / g::kBK * g::kBK);
  const GemmPitch ld = gemm_pitch(d);
  p.lda = ld.lda, p.ldb = ld.ldb, p.ldc = ld.ldc;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(g::kThreads);
  const int stages = splits > 1 ? g::kStagesSplit : g::kStages;
  cfg.dynamicSmemBytes = static_cast<size_t>(stages) * g::kStageBytes;
  cfg.stream = s;
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * splits));
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t e = set_dyn_smem_once(kern, g::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c), p);
  };
  cudaError_t e;
  if (d->b_transposed)
    e = splits > 1 ? launch(g::gemm_tf32x3_kernel<true, g::kStagesSplit>) : launch(g::gemm_tf32x3_kernel<true, g::kStages>);
  else
    e = splits > 1 ? launch(g::gemm_tf32x3_kernel<false, g::kStagesSplit>) : launch(g::gemm_tf32x3_kernel<false, g::kStages>);
  return cuda_ok(err, e, "gemm_tf32x3_kernel launch");
}

// The device's default memory pool keeps what is freed into it (no trimming at synchronisation points), so
// that after the first call cudaMallocAsync / cudaFreeAsync are bookkeeping on the stream.  Once per device.
inline cudaError_t keep_pool_memory_once() {
  cudaError_t e = cudaSuccess;
  int unused = 0;
  kernel_fact(nullptr, 5, &unused, [&](int* out) {
    int dev = 0;
    cudaMemPool_t pool;
    e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetDefaultMemPool(&pool, dev);
    uint64_t keep = ~0ull;
    if (e == cudaSuccess) e = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    *out = 1;
    return e == cudaSuccess;
  });
  return e;
}

// f32 inputs on the tcgen05 tensor cores: split pass (hi / lo planes, B's planes K-major), then the
// contraction with chunked accumulation (gemm_tf32_tc.cuh).  The planes live in stream-ordered scratch.
inline int32_t gemm_tf32_tc_launch(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                                   uint32_t* status, cudaStream_t s) {
  namespace g = gemm_tf32_tc;
  const uint64_t M = d->m, N = d->n, K = d->k, B = d->batch;
  const GemmPitch ld = gemm_pitch(d);
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  cudaError_t e = keep_pool_memory_once();
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaMemPoolSetAttribute");
  const size_t a_plane = static_cast<size_t>(B) * M * K, b_plane = static_cast<size_t>(B) * N * K;  // elements
  float* ws = nullptr;
  e = cudaMallocAsync(reinterpret_cast<void**>(&ws), 2 * (a_plane + b_plane) * sizeof(float), s);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return op_fail(err, TSM100_ERR_MEMORY, std::string("gemm: scratch for the operand planes: ") + cudaGetErrorString(e));
  }
  float *a_hi = ws, *a_lo = ws + a_plane, *b_hi = ws + 2 * a_plane, *b_lo = b_hi + b_plane;
  const float* af = static_cast<const float*>(a);
  const float* bf = static_cast<const float*>(b);
  auto grid1d = [&](uint64_t items) {
    return static_cast<unsigned>(std::max<uint64_t>(1, std::min<uint64_t>((items + 255) / 256, static_cast<uint64_t>(sms) * 16)));
  };
  g::split_rows_kernel<<<dim3(grid1d(M * K / 4), static_cast<unsigned>(B)), 256, 0, s>>>(
      af, ld.lda, static_cast<int64_t>(M) * ld.lda, a_hi, a_lo, static_cast<int64_t>(M), static_cast<int32_t>(K));
  if (d->b_transposed) {
    g::split_rows_kernel<<<dim3(grid1d(N * K / 4), static_cast<unsigned>(B)), 256, 0, s>>>(
        bf, ld.ldb, static_cast<int64_t>(N) * ld.ldb, b_hi, b_lo, static_cast<int64_t>(N), static_cast<int32_t>(K));
  } else {
    g::split_transpose_kernel<<<dim3(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>((K + 31) / 32), static_cast<unsigned>(B)), 256, 0, s>>>(
        bf, ld.ldb, static_cast<int64_t>(K) * ld.ldb, b_hi, b_lo, static_cast<int32_t>(K), static_cast<int32_t>(N));
  }
  st = cuda_ok(err, cudaGetLastError(), "gemm operand split launch");
  CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
  const CUtensorMapDataType f32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  // Problems with more than one 128-row and 128-column block run on CTA pairs (256 x 256 tiles, each CTA staging
  // 128 rows of A and 128 columns of B); the rest on single CTAs (128 x 256 tiles).
  const bool pairs = M > 128 && N > 128;
  const uint32_t box_b = pairs ? g::pair::kCtaN : g::kBN;
  if (st == TSM100_OK) st = make_tmap_3d(err, &ta_hi, a_hi, K, M, B, K, M * K, g::kBK, g::kBM, f32, 4);
  if (st == TSM100_OK) st = make_tmap_3d(err, &ta_lo, a_lo, K, M, B, K, M * K, g::kBK, g::kBM, f32, 4);
  if (st == TSM100_OK) st = make_tmap_3d(err, &tb_hi, b_hi, K, N, B, K, N * K, g::kBK, box_b, f32, 4);
  if (st == TSM100_OK) st = make_tmap_3d(err, &tb_lo, b_lo, K, N, B, K, N * K, g::kBK, box_b, f32, 4);
  if (st == TSM100_OK) {
    g::Params p;
    p.m = static_cast<int32_t>(M);
    p.n = static_cast<int32_t>(N);
    p.k = static_cast<int32_t>(K);
    p.batch = d->batch;
    p.m_blocks = static_cast<int32_t>((M + (pairs ? g::pair::kPairM : g::kBM) - 1) / (pairs ? g::pair::kPairM : g::kBM));
    p.n_blocks = static_cast<int32_t>((N + g::kBN - 1) / g::kBN);
    p.c_batch_stride = static_cast<int64_t>(M) * ld.ldc;
    p.ldc = ld.ldc;
    p.status = status;
    const int64_t tiles = static_cast<int64_t>(p.m_blocks) * p.n_blocks * p.batch;
    if (pairs) {
      auto kern = g::pair::gemm_tf32_tc2_kernel;
      e = set_dyn_smem_once(kern, g::pair::kSmemBytes);
      if (e == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.blockDim = dim3(g::kThreads);
        cfg.dynamicSmemBytes = g::pair::kSmemBytes;
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
        int max_clusters = sms / 2;
        kernel_fact(reinterpret_cast<const void*>(kern), kFactClusters, &max_clusters, [&](int* out) {
          int n = 0;
          if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
            (void)cudaGetLastError();
            return false;
          }
          *out = n;
          return true;
        });
        const int64_t npairs = std::min<int64_t>(tiles, std::min<int64_t>(max_clusters, sms / 2));
        cfg.gridDim = dim3(static_cast<unsigned>(2 * npairs));
        e = cudaLaunchKernelEx(&cfg, kern, ta_hi, ta_lo, tb_hi, tb_lo, static_cast<float*>(c), p);
      }
      st = cuda_ok(err, e, "gemm_tf32_tc2_kernel launch");
    } else {
      auto kern = g::gemm_tf32_tc_kernel;
      e = set_dyn_smem_once(kern, g::kSmemBytes);
      if (e == cudaSuccess) {
        const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, sms));
        kern<<<grid, g::kThreads, g::kSmemBytes, s>>>(ta_hi, ta_lo, tb_hi, tb_lo, static_cast<float*>(c), p);
        e = cudaGetLastError();
      }
      st = cuda_ok(err, e, "gemm_tf32_tc_kernel launch");
    }
  }
  e = cudaFreeAsync(ws, s);  // stream-ordered: after the kernel that reads the planes
  if (st == TSM100_OK && e != cudaSuccess) st = cuda_ok(err, e, "cudaFreeAsync");
  return st;
}

template <typename OutT, bool kBT, bool kBf16>
inline int32_t gemm_tc_launch(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                              uint32_t* status, cudaStream_t s) {
  namespace g = gemm_tc;
  CUtensorMap ta, tb;
  const uint64_t M = d->m, N = d->n, K = d->k, B = d->batch;
  const GemmPitch ld = gemm_pitch(d);
  const uint64_t lda = ld.lda, ldb = ld.ldb;
  int32_t st = make_tmap_16bit_3d(err, &ta, a, K, M, B, lda, M * lda, g::kBK, g::kBM, kBf16);
  if (st != TSM100_OK) return st;
  if (kBT)
    st = make_tmap_16bit_3d(err, &tb, b, K, N, B, ldb, N * ldb, g::kBK, g::kBN, kBf16);
  else
    st = make_tmap_16bit_3d(err, &tb, b, N, K, B, ldb, K * ldb, 64, g::kBK, kBf16);
  if (st != TSM100_OK) return st;
  g::Params p;
  p.m = static_cast<int32_t>(M);
  p.n = static_cast<int32_t>(N);
  p.k = static_cast<int32_t>(K);
  p.batch = d->batch;
  p.m_blocks = static_cast<int32_t>((M + g::kBM - 1) / g::kBM);
  p.n_blocks = static_cast<int32_t>((N + g::kBN - 1) / g::kBN);
  p.c_batch_stride = static_cast<int64_t>(M) * ld.ldc;
  p.ldc = ld.ldc;
  p.status = status;
  int sms = 0;
  st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  const int64_t tiles = static_cast<int64_t>(p.m_blocks) * p.n_blocks * p.batch;
  auto kern = g::gemm_tc_kernel<OutT, kBT, kBf16>;
  cudaError_t e = set_dyn_smem_once(kern, g::kSmemBytes);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(gemm_tc_kernel)");
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, sms));
  kern<<<grid, g::kThreads, g::kSmemBytes, s>>>(ta, tb, static_cast<OutT*>(c), p);
  return cuda_ok(err, cudaGetLastError(), "gemm_tc_kernel launch");
}

// CTA-pair kernel (256 x 256 tile per two SMs), launched as clusters of two.
template <typename OutT, bool kBT, bool kBf16>
inline int32_t gemm_tc2_launch(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                               uint32_t* status, cudaStream_t s) {
  namespace g = gemm_tc2;
  CUtensorMap ta, tb;
  const uint64_t M = d->m, N = d->n, K = d->k, B = d->batch;
  const GemmPitch ld = gemm_pitch(d);
  const uint64_t lda = ld.lda, ldb = ld.ldb;
  int32_t st = make_tmap_16bit_3d(err, &ta, a, K, M, B, lda, M * lda, g::kBK, g::kCtaM, kBf16);
  if (st != TSM100_OK) return st;
  if (kBT)
    st = make_tmap_16bit_3d(err, &tb, b, K, N, B, ldb, N * ldb, g::kBK, g::kCtaN, kBf16);
  else
    st = make_tmap_16bit_3d(err, &tb, b, N, K, B, ldb, K * ldb, 64, g::kBK, kBf16);
  if (st != TSM100_OK) return st;
  gemm_tc::Params p;
  p.m = static_cast<int32_t>(M);
  p.n = static_cast<int32_t>(N);
  p.k = static_cast<int32_t>(K);
  p.batch = d->batch;
  p.m_blocks = static_cast<int32_t>((M + g::kPairM - 1) / g::kPairM);
  p.n_blocks = static_cast<int32_t>((N + g::kBN - 1) / g::kBN);
  p.c_batch_stride = static_cast<int64_t>(M) * ld.ldc;
  p.ldc = ld.ldc;
  p.status = status;
  auto kern = g::gemm_tc2_kernel<OutT, kBT, kBf16>;
  cudaError_t e = set_dyn_smem_once(kern, g::kSmemBytes);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(gemm_tc2_kernel)");
  int sms = 0;
  st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(g::kThreads);
  cfg.dynamicSmemBytes = g::kSmemBytes;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
  int max_clusters = sms / 2;  // how many pairs the GPU holds at once: asked once per kernel and device
  kernel_fact(reinterpret_cast<const void*>(kern), kFactClusters, &max_clusters, [&](int* out) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      return false;
    }
    *out = n;
    return true;
  });
  const int64_t tiles = static_cast<int64_t>(p.m_blocks) * p.n_blocks * p.batch;
  const int64_t pairs = std::min<int64_t>(tiles, std::min<int64_t>(max_clusters, sms / 2));
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  e = cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<OutT*>(c), p);
  return cuda_ok(err, e, "gemm_tc2_kernel launch");
}

// `status` is a device word the tensor-core kernel writes if one of its bounded
// waits runs out; it must be zero when the launch starts.
inline int32_t gemm(std::string* err, const tsm100_gemm_desc* d, const void* a, const void* b, void* c,
                    uint32_t* status, void* stream) {
  if (!d || !a || !b || !c) return op_fail(err, TSM100_ERR_INVALID, "gemm: null argument");
  if (!dtype_valid(d->dtype) || !dtype_valid(d->out_dtype)) return op_fail(err, TSM100_ERR_INVALID, "gemm: unknown dtype");
  if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0) return op_fail(err, TSM100_ERR_INVALID, "gemm: negative shape");
  if (d->m > 0x7fffffff || d->n > 0x7fffffff || d->k > 0x7fffffff)
    return op_fail(err, TSM100_ERR_INVALID, "gemm: dimension exceeds 2^31-1");
  if (d->dtype == TSM100_F32 && d->out_dtype != TSM100_F32)
    return op_fail(err, TSM100_ERR_INVALID, "gemm: f32 inputs produce f32 output");
  if (d->dtype != TSM100_F32 && d->out_dtype != TSM100_F32 && d->out_dtype != d->dtype)
    return op_fail(err, TSM100_ERR_INVALID, "gemm: 16-bit inputs produce the same 16-bit type or f32");
  const GemmPitch ld = gemm_pitch(d);
  if (ld.lda < d->k || ld.ldb < (d->b_transposed ? d->k : d->n) || ld.ldc < d->n)
    return op_fail(err, TSM100_ERR_INVALID, "gemm: a row pitch (lda, ldb, ldc) is shorter than its row");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d->m == 0 || d->n == 0 || d->batch == 0) return TSM100_OK;
  if (d->k == 0) {  // empty contraction: C = 0 (linalg.fill)
    const size_t os = dtype_size(d->out_dtype);
    return cuda_ok(err, cudaMemset2DAsync(c, static_cast<size_t>(ld.ldc) * os, 0, static_cast<size_t>(d->n) * os,
                                          static_cast<size_t>(d->batch) * d->m, s), "cudaMemset2DAsync");
  }
  if (d->dtype == TSM100_F32) {
    // rows that start on 16-byte boundaries: tensor cores; anything else: the FP32 pipe
    const bool vec_ok = aligned16(a) && aligned16(b) && aligned16(c) && d->k % 4 == 0 && (d->b_transposed || d->n % 4 == 0) &&
                        d->n % 2 == 0 && ld.lda % 4 == 0 && ld.ldb % 4 == 0 && ld.ldc % 2 == 0;
    if (vec_ok) {
      // enough 128 x 256 tiles to occupy the GPU: the persistent tcgen05 kernels (operand planes from a split pass)
      const int64_t tiles = ((d->m + 127) / 128) * ((d->n + 255) / 256) * d->batch;
      if (status != nullptr && tiles >= 64 && tiles < 0x7fffffff && d->k >= 256) return gemm_tf32_tc_launch(err, d, a, b, c, status, s);
      // fewer tiles (the 512^3 configuration has 8): the warp-level kernel, whose 64 x 64 tiles and cluster split-K
      // spread a small problem over the SMs
      return gemm_tf32x3_launch(err, d, a, b, c, s);
    }
    return gemm_simt_launch<float, float>(err, d, a, b, c, s);
  }

  const bool bf16 = d->dtype == TSM100_BF16;
  const bool out_f32 = d->out_dtype == TSM100_F32;
  // TMA needs 16-byte-multiple row pitches; the epilogue stores 16-byte vectors.
  const bool tma_ok = status != nullptr && aligned16(a) && aligned16(b) && aligned16(c) && (d->k % 8 == 0) &&
                      (d->b_transposed || d->n % 8 == 0) && (d->n * dtype_size(d->out_dtype)) % 16 == 0 &&
                      ld.lda % 8 == 0 && ld.ldb % 8 == 0 && (ld.ldc * dtype_size(d->out_dtype)) % 16 == 0 &&
                      (static_cast<int64_t>((d->m + 127) / 128) * ((d->n + 255) / 256) * d->batch < 0x7fffffff);
  if (tma_ok) {
    const bool pair = d->m > 128 && d->n > 128;  // large enough for 256 x 256 tiles on CTA pairs
#define TSM_GEMM_TC(OUT, BT, BF)                                                     \
  return pair ? gemm_tc2_launch<OUT, BT, BF>(err, d, a, b, c, status, s) \
              : gemm_tc_launch<OUT, BT, BF>(err, d, a, b, c, status, s)
    if (bf16) {
      if (out_f32) { if (d->b_transposed) TSM_GEMM_TC(float, true, true); else TSM_GEMM_TC(float, false, true); }
      else { if (d->b_transposed) TSM_GEMM_TC(__nv_bfloat16, true, true); else TSM_GEMM_TC(__nv_bfloat16, false, true); }
    } else {
      if (out_f32) { if (d->b_transposed) TSM_GEMM_TC(float, true, false); else TSM_GEMM_TC(float, false, false); }
      else { if (d->b_transposed) TSM_GEMM_TC(__half, true, false); else TSM_GEMM_TC(__half, false, false); }
    }
#undef TSM_GEMM_TC
  }
  if (bf16) {
    if (out_f32) return gemm_simt_launch<__nv_bfloat16, float>(err, d, a, b, c, s);
    return gemm_simt_launch<__nv_bfloat16, __nv_bfloat16>(err, d, a, b, c, s);
  }
  if (out_f32) return gemm_simt_launch<__half, float>(err, d, a, b, c, s);
  return gemm_simt_launch<__half, __half>(err, d, a, b, c, s);
}

// ---------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------
// Head dims 32, 64, 96 (and 128 for f32) with 16-byte aligned rows: the warp-level tensor-core kernel (f32: three
// TF32 products per product; 16-bit data, whose values are TF32 numbers already: one for Q K^T, two for P V).
template <typename T>
inline bool attention_tf32x3_ok(const attn_simt::Params& p, const void* q, const void* k, const void* v, const void* o) {
  constexpr int64_t vec = 16 / static_cast<int64_t>(sizeof(T));
  const bool dim_ok = p.head_dim == 32 || p.head_dim == 64 || p.head_dim == 96 || (sizeof(T) == 4 && p.head_dim == 128);
  return dim_ok && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && p.q_row_stride % vec == 0 &&
         p.q_head_stride % vec == 0 && p.kv_head_stride % vec == 0 && p.o_row_stride % vec == 0 && p.o_head_stride % vec == 0;
}
template <typename T, int D>
inline int32_t attention_tf32x3_launch_d(std::string* err, const attn_simt::Params& p, const T* q, const T* k,
                                         const T* v, T* o, cudaStream_t s) {
  namespace at = attn_tf32;
  const int64_t grid = static_cast<int64_t>((p.seq + at::kBM - 1) / at::kBM) * p.batch * p.heads_q;
  if (grid > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "attention: too many query blocks for one launch");
  auto kern = at::attention_tf32x3_kernel<T, D>;
  constexpr int smem = at::smem_bytes<T, D>();
  cudaError_t e = set_dyn_smem_once(kern, smem);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_tf32x3_kernel)");
  kern<<<static_cast<unsigned>(grid), at::kThreads, smem, s>>>(q, k, v, o, p);
  return cuda_ok(err, cudaGetLastError(), "attention_tf32x3_kernel launch");
}
template <typename T>
inline int32_t attention_tf32x3_launch(std::string* err, const attn_simt::Params& p, const void* q, const void* k,
                                       const void* v, void* o, cudaStream_t s) {
  const T* qf = static_cast<const T*>(q);
  const T* kf = static_cast<const T*>(k);
  const T* vf = static_cast<const T*>(v);
  T* of = static_cast<T*>(o);
  if constexpr (sizeof(T) == 4)
    if (p.head_dim == 128) return attention_tf32x3_launch_d<T, 128>(err, p, qf, kf, vf, of, s);
  switch (p.head_dim) {
    case 96: return attention_tf32x3_launch_d<T, 96>(err, p, qf, kf, vf, of, s);
    case 64: return attention_tf32x3_launch_d<T, 64>(err, p, qf, kf, vf, of, s);
    default: return attention_tf32x3_launch_d<T, 32>(err, p, qf, kf, vf, of, s);
  }
}

template <typename T>
inline int32_t attention_simt_launch(std::string* err, const tsm100_attention_desc* d, const void* q, const void* k,
                                     const void* v, void* o, cudaStream_t s) {
  const int64_t sd = static_cast<int64_t>(d->seq) * d->head_dim;
  attn_simt::Params p{d->seq, d->head_dim, d->heads_q, d->heads_kv, d->batch, d->causal,
                      static_cast<float>(1.0 / std::sqrt(static_cast<double>(d->head_dim))),
                      d->seq, 0, d->head_dim, sd, sd, d->head_dim, sd};
  if (attention_tf32x3_ok<T>(p, q, k, v, o)) return attention_tf32x3_launch<T>(err, p, q, k, v, o, s);
  const int64_t rows = static_cast<int64_t>(d->batch) * d->heads_q * d->seq;
  const int64_t grid = (rows + attn_simt::kWarps - 1) / attn_simt::kWarps;
  if (grid > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "attention: too many query rows for one launch");
  attn_simt::attention_simt_kernel<T><<<static_cast<unsigned>(grid), attn_simt::kWarps * 32, 0, s>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(o), p);
  return cuda_ok(err, cudaGetLastError(), "attention_simt launch");
}

// ---------------------------------------------------------------------------
// prefill attention: seq_len new tokens against a KV cache that already holds them and start_pos earlier ones
// ---------------------------------------------------------------------------
template <typename T>
inline int32_t attention_prefill_simt_launch(std::string* err, const tsm100_attention_prefill_desc* d, const void* q,
                                             const void* k, const void* v, void* o, cudaStream_t s) {
  const int64_t hd = static_cast<int64_t>(d->heads_q) * d->head_dim;
  attn_simt::Params p{d->seq_len, d->head_dim, d->heads_q, d->heads_kv, 1, 1,
                      static_cast<float>(1.0 / std::sqrt(static_cast<double>(d->head_dim))),
                      d->start_pos + d->seq_len, d->start_pos, hd, d->head_dim,
                      static_cast<int64_t>(d->max_seq) * d->head_dim, hd, d->head_dim};
  if (attention_tf32x3_ok<T>(p, q, k, v, o)) return attention_tf32x3_launch<T>(err, p, q, k, v, o, s);
  const int64_t rows = static_cast<int64_t>(d->heads_q) * d->seq_len;
  const int64_t grid = (rows + attn_simt::kWarps - 1) / attn_simt::kWarps;
  if (grid > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: too many query rows for one launch");
  attn_simt::attention_simt_kernel<T><<<static_cast<unsigned>(grid), attn_simt::kWarps * 32, 0, s>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(o), p);
  return cuda_ok(err, cudaGetLastError(), "attention_simt (prefill) launch");
}

// KV heads per band of the causal launch order: as many as keep K and V of the band (16-bit, head_dim 128) within
// 32 MiB, a quarter of the L2, so that the blocks in flight - a few weight levels of one band, at a band's end
// together with the start of the next - read K and V from DRAM once.
inline int32_t attention_kv_band(uint64_t kv_len, int64_t kv_heads) {
  const uint64_t per_head = std::max<uint64_t>(1, kv_len * attn::kD * 2 * 2);
  const int64_t band = static_cast<int64_t>((32ull << 20) / per_head);
  return static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(band, std::max<int64_t>(kv_heads, 1))));
}

template <bool kBf16>
inline int32_t attention_prefill_tc_launch(std::string* err, const tsm100_attention_prefill_desc* d, const void* q, const void* k,
                                           const void* v, void* o, uint32_t* status, cudaStream_t s) {
  namespace at = attn;
  CUtensorMap tq, tk, tv;
  const uint64_t D = at::kD, hq = d->heads_q, hkv = d->heads_kv, kv_len = static_cast<uint64_t>(d->start_pos) + d->seq_len;
  // token-major Q: row pitch heads_q * D, head pitch D; caches: row pitch D, head pitch max_seq * D, kv_len rows visible
  int32_t st = make_tmap_16bit_3d(err, &tq, q, D, d->seq_len, hq, hq * D, D, 64, at::kBQ, kBf16);
  if (st == TSM100_OK) st = make_tmap_16bit_3d(err, &tk, k, D, kv_len, hkv, D, static_cast<uint64_t>(d->max_seq) * D, 64, at::kBKV, kBf16);
  if (st == TSM100_OK) st = make_tmap_16bit_3d(err, &tv, v, D, kv_len, hkv, D, static_cast<uint64_t>(d->max_seq) * D, 64, at::kBKV, kBf16);
  if (st != TSM100_OK) return st;
  at::Params p;
  p.seq = d->seq_len;
  p.heads_q = d->heads_q;
  p.heads_kv = d->heads_kv;
  p.batch = 1;
  p.causal = 1;
  p.q_blocks = (d->seq_len + 2 * at::kBQ - 1) / (2 * at::kBQ);
  p.kv_band = attention_kv_band(kv_len, d->heads_kv);
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(D))) * 1.4426950408889634);
  p.status = status;
  p.seq_kv = static_cast<int32_t>(kv_len);
  p.q_offset = d->start_pos;
  p.o_row_stride = static_cast<int64_t>(hq * D);
  p.o_head_stride = static_cast<int64_t>(D);
  const int64_t grid = static_cast<int64_t>(p.q_blocks) * d->heads_q;
  if (grid > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: too many tiles for one launch");
  auto kern = at::attention_fwd_kernel<kBf16, true>;
  cudaError_t e = set_dyn_smem_once(kern, at::kSmemBytes);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_fwd_kernel, cache)");
  kern<<<static_cast<unsigned>(grid), at::kThreads, at::kSmemBytes, s>>>(tq, tk, tv, static_cast<uint16_t*>(o), p);
  return cuda_ok(err, cudaGetLastError(), "attention_fwd_kernel (prefill) launch");
}

inline int32_t attention_prefill(std::string* err, const tsm100_attention_prefill_desc* d, const void* q, const void* k,
                                 const void* v, void* o, uint32_t* status, void* stream) {
  if (!d || !q || !k || !v || !o) return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: null argument");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: unknown dtype");
  if (d->heads_q <= 0 || d->heads_kv <= 0 || d->seq_len < 0 || d->start_pos < 0 || d->head_dim <= 0 ||
      static_cast<int64_t>(d->start_pos) + d->seq_len > d->max_seq)
    return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: bad shape (need heads > 0 and start_pos + seq_len <= max_seq)");
  if (d->heads_q % d->heads_kv != 0)
    return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: heads_q must be a multiple of heads_kv");
  if (d->head_dim > attn_simt::kMaxD) return op_fail(err, TSM100_ERR_INVALID, "attention_prefill: head_dim > 256 unsupported");
  if (d->seq_len == 0) return TSM100_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc_ok = d->dtype != TSM100_F32 && d->head_dim == attn::kD && status != nullptr && aligned16(q) && aligned16(k) &&
                     aligned16(v) && aligned16(o);
  if (tc_ok) {
    if (d->dtype == TSM100_BF16) return attention_prefill_tc_launch<true>(err, d, q, k, v, o, status, s);
    return attention_prefill_tc_launch<false>(err, d, q, k, v, o, status, s);
  }
  if (d->dtype == TSM100_F32) return attention_prefill_simt_launch<float>(err, d, q, k, v, o, s);
  if (d->dtype == TSM100_BF16) return attention_prefill_simt_launch<__nv_bfloat16>(err, d, q, k, v, o, s);
  return attention_prefill_simt_launch<__half>(err, d, q, k, v, o, s);
}

// ---------------------------------------------------------------------------
// decode attention (one query token against a KV cache)
// ---------------------------------------------------------------------------
template <typename T, int G, int D>
inline int32_t attention_decode_launch(std::string* err, const tsm100_attention_decode_desc* d, const T* q, const T* k,
                                       const T* v, T* o, int head_base, int heads_here, int splits, cudaStream_t s) {
  namespace ad = attn_decode;
  ad::Params p;
  p.batch = d->batch;
  p.heads_q = d->heads_q;
  p.heads_kv = d->heads_kv;
  p.seq_len = d->seq_len;
  p.max_seq = d->max_seq;
  p.group = d->heads_q / d->heads_kv;
  p.head_base = head_base;
  p.heads_here = heads_here;
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(D))) * 1.4426950408889634);
  auto kern = ad::attention_decode_kernel<T, G, D>;
  constexpr int smem = ad::smem_floats<T, G, D>() * static_cast<int>(sizeof(float));
  cudaError_t e = set_dyn_smem_once(kern, smem);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_decode_kernel)");
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(ad::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.gridDim = dim3(static_cast<unsigned>(static_cast<int64_t>(d->batch) * d->heads_kv * splits));
  e = cudaLaunchKernelEx(&cfg, kern, q, k, v, o, p);
  return cuda_ok(err, e, "attention_decode_kernel launch");
}

// The tensor-core decode kernel for an element type: mma.sync on 16-bit caches, three TF32 products on f32 caches.
template <typename T, int D, int STAGES, int WARPS>
struct DecodeTc {
  static auto kernel() {
    if constexpr (sizeof(T) == 4) return attn_decode::tf32::attention_decode_tf32_kernel<D, STAGES, WARPS>;
    else return attn_decode::mma::attention_decode_mma_kernel<T, D, STAGES, WARPS>;
  }
  static constexpr int smem() {
    if constexpr (sizeof(T) == 4) return attn_decode::tf32::smem_bytes<D, STAGES, WARPS>();
    else return attn_decode::mma::smem_bytes<D, STAGES, WARPS>();
  }
};

template <typename T, int D, int STAGES, int WARPS>
inline int32_t attention_decode_mma_launch(std::string* err, const tsm100_attention_decode_desc* d, const T* q, const T* k,
                                           const T* v, T* o, int head_base, int heads_here, int splits, cudaStream_t s) {
  namespace ad = attn_decode;
  ad::Params p;
  p.batch = d->batch;
  p.heads_q = d->heads_q;
  p.heads_kv = d->heads_kv;
  p.seq_len = d->seq_len;
  p.max_seq = d->max_seq;
  p.group = d->heads_q / d->heads_kv;
  p.head_base = head_base;
  p.heads_here = heads_here;
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(D))) * 1.4426950408889634);
  auto kern = DecodeTc<T, D, STAGES, WARPS>::kernel();
  constexpr int smem = DecodeTc<T, D, STAGES, WARPS>::smem();
  cudaError_t e = set_dyn_smem_once(kern, smem);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_decode_mma_kernel)");
  if (splits > ad::kMaxSplits) {
    e = allow_wide_clusters_once(kern);
    if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_decode_mma_kernel, wide clusters)");
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.gridDim = dim3(static_cast<unsigned>(static_cast<int64_t>(d->batch) * d->heads_kv * splits));
  e = cudaLaunchKernelEx(&cfg, kern, q, k, v, o, p);
  return cuda_ok(err, e, "attention_decode_mma_kernel launch");
}

// How many clusters of `size` CTAs of the eight-warp decode kernel the GPU holds at once (asked once per
// kernel, size and device; 0 if such clusters cannot be placed at all).
template <typename T, int D>
inline int decode_lone_clusters(int size) {
  namespace ad = attn_decode;
  static int cached[64][2] = {};  // [device][size == 16]: 0 unknown, else count + 1
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int& slot = cached[dev][size > ad::kMaxSplits ? 1 : 0];
  if (size != ad::kMaxSplits && size != ad::kMaxSplitsWide) return 0;
  if (slot == 0) {
    auto kern = DecodeTc<T, D, 3, 8>::kernel();
    constexpr int smem = DecodeTc<T, D, 3, 8>::smem();
    int clusters = 0;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(size);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.blockDim = dim3(8 * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.gridDim = dim3(static_cast<unsigned>(size));
    const bool ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                    cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
                    cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) == cudaSuccess;
    if (!ok) (void)cudaGetLastError();  // the answer is "none", not an error of the caller's launch
    slot = (ok ? clusters : 0) + 1;
  }
  return slot - 1;
}

// f32 caches: from this many query heads per cache on, the tensor-core kernel (three TF32 products) is faster than
// the FP32-pipe kernel, whose instruction count grows with the heads while the cache row is read once either way
constexpr int kDecodeF32TensorCoreGroup = 5;

template <typename T, int D>
inline int32_t attention_decode_typed(std::string* err, const tsm100_attention_decode_desc* d, const void* q, const void* k,
                                      const void* v, void* o, cudaStream_t s) {
  int sms = 0;
  int32_t st = sm_count(err, &sms);
  if (st != TSM100_OK) return st;
  const int64_t units = static_cast<int64_t>(d->batch) * d->heads_kv;
  // split the positions of one (batch, KV head) over a cluster until the GPU is covered about twice, keeping
  // at least 256 positions per CTA
  int splits = 1;
  while (splits < attn_decode::kMaxSplits && units * splits < 2ll * sms && d->seq_len / (2 * splits) >= 256) splits *= 2;
  const int group = d->heads_q / d->heads_kv;
  const T* qp = static_cast<const T*>(q);
  const T* kp = static_cast<const T*>(k);
  const T* vp = static_cast<const T*>(v);
  T* op = static_cast<T*>(o);
  if (sizeof(T) == 2 || group >= kDecodeF32TensorCoreGroup) {
    // 16-bit storage, or f32 with several query heads per cache: tensor cores, up to 16 query heads of a group per
    // pass; 4 warps per CTA, so the GPU is covered about four times before the ranges get shorter than 256 positions
    splits = 1;
    while (splits < attn_decode::kMaxSplits && units * splits < 4ll * sms && d->seq_len / (2 * splits) >= 256) splits *= 2;
    // a handful of sequences: clusters of 16 if the GPU holds all of them at once (one CTA per SM; a B200
    // holds 7), so that most SMs take part
    if (splits == attn_decode::kMaxSplits && d->seq_len / (2 * attn_decode::kMaxSplitsWide) >= 256 &&
        units <= decode_lone_clusters<T, D>(attn_decode::kMaxSplitsWide))
      splits = attn_decode::kMaxSplitsWide;
    // every CTA alone on its SM from start to end: eight warps and a deeper ring, so that it hides its own latencies
    const bool lone = units * splits <= sms && (splits < attn_decode::kMaxSplits || units <= decode_lone_clusters<T, D>(splits));
    for (int base = 0; base < group && st == TSM100_OK; base += 16)
      st = lone ? attention_decode_mma_launch<T, D, 3, 8>(err, d, qp, kp, vp, op, base, std::min(16, group - base), splits, s)
                : attention_decode_mma_launch<T, D, 2, 4>(err, d, qp, kp, vp, op, base, std::min(16, group - base), splits, s);
    return st;
  }
  // groups wider than 8 query heads run in passes of 8 (the cache is then re-read, from L2 when it fits)
  for (int base = 0; base < group && st == TSM100_OK; base += 8) {
    const int here = std::min(8, group - base);
    if (here == 1) st = attention_decode_launch<T, 1, D>(err, d, qp, kp, vp, op, base, here, splits, s);
    else if (here == 2) st = attention_decode_launch<T, 2, D>(err, d, qp, kp, vp, op, base, here, splits, s);
    else if (here <= 4) st = attention_decode_launch<T, 4, D>(err, d, qp, kp, vp, op, base, here, splits, s);
    else st = attention_decode_launch<T, 8, D>(err, d, qp, kp, vp, op, base, here, splits, s);
  }
  return st;
}

inline int32_t attention_decode(std::string* err, const tsm100_attention_decode_desc* d, const void* q, const void* k,
                                const void* v, void* o, void* stream) {
  if (!d || !q || !k || !v || !o) return op_fail(err, TSM100_ERR_INVALID, "attention_decode: null argument");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "attention_decode: unknown dtype");
  if (d->batch < 0 || d->heads_q <= 0 || d->heads_kv <= 0 || d->seq_len < 0 || d->max_seq < d->seq_len)
    return op_fail(err, TSM100_ERR_INVALID, "attention_decode: bad shape (need heads > 0 and 0 <= seq_len <= max_seq)");
  if (d->heads_q % d->heads_kv != 0)
    return op_fail(err, TSM100_ERR_INVALID, "attention_decode: heads_q must be a multiple of heads_kv");
  if (d->head_dim != 64 && d->head_dim != 128)
    return op_fail(err, TSM100_ERR_INVALID, "attention_decode: head_dim must be 64 or 128");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return op_fail(err, TSM100_ERR_INVALID, "attention_decode: buffers must be 16-byte aligned");
  if (d->batch == 0) return TSM100_OK;
  if (static_cast<int64_t>(d->batch) * d->heads_kv * attn_decode::kMaxSplitsWide > 0x7fffffff)
    return op_fail(err, TSM100_ERR_INVALID, "attention_decode: too many (batch, KV head) units for one launch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool d128 = d->head_dim == 128;
  switch (d->dtype) {
    case TSM100_F32:
      return d128 ? attention_decode_typed<float, 128>(err, d, q, k, v, o, s) : attention_decode_typed<float, 64>(err, d, q, k, v, o, s);
    case TSM100_BF16:
      return d128 ? attention_decode_typed<__nv_bfloat16, 128>(err, d, q, k, v, o, s)
                  : attention_decode_typed<__nv_bfloat16, 64>(err, d, q, k, v, o, s);
    default:
      return d128 ? attention_decode_typed<__half, 128>(err, d, q, k, v, o, s) : attention_decode_typed<__half, 64>(err, d, q, k, v, o, s);
  }
}

template <bool kBf16>
inline int32_t attention_tc_launch(std::string* err, const tsm100_attention_desc* d, const void* q, const void* k,
                                   const void* v, void* o, uint32_t* status, cudaStream_t s) {
  namespace at = attn;
  CUtensorMap tq, tk, tv;
  const uint64_t S = d->seq, D = at::kD;
  const uint64_t nq = static_cast<uint64_t>(d->batch) * d->heads_q, nkv = static_cast<uint64_t>(d->batch) * d->heads_kv;
  int32_t st = make_tmap_16bit_3d(err, &tq, q, D, S, nq, D, S * D, 64, at::kBQ, kBf16);
  if (st == TSM100_OK) st = make_tmap_16bit_3d(err, &tk, k, D, S, nkv, D, S * D, 64, at::kBKV, kBf16);
  if (st == TSM100_OK) st = make_tmap_16bit_3d(err, &tv, v, D, S, nkv, D, S * D, 64, at::kBKV, kBf16);
  if (st != TSM100_OK) return st;
  at::Params p;
  p.seq = d->seq;
  p.heads_q = d->heads_q;
  p.heads_kv = d->heads_kv;
  p.batch = d->batch;
  p.causal = d->causal ? 1 : 0;
  p.q_blocks = (d->seq + 2 * at::kBQ - 1) / (2 * at::kBQ);
  p.kv_band = attention_kv_band(S, static_cast<int64_t>(nkv));
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(D))) * 1.4426950408889634);
  p.status = status;
  p.seq_kv = d->seq;
  p.q_offset = 0;
  p.o_row_stride = p.o_head_stride = 0;
  const int64_t grid = static_cast<int64_t>(p.q_blocks) * nq;
  if (grid > 0x7fffffff) return op_fail(err, TSM100_ERR_INVALID, "attention: too many tiles for one launch");
  auto kern = at::attention_fwd_kernel<kBf16>;
  cudaError_t e = set_dyn_smem_once(kern, at::kSmemBytes);
  if (e != cudaSuccess) return cuda_ok(err, e, "cudaFuncSetAttribute(attention_fwd_kernel)");
  kern<<<static_cast<unsigned>(grid), at::kThreads, at::kSmemBytes, s>>>(tq, tk, tv, static_cast<uint16_t*>(o), p);
  return cuda_ok(err, cudaGetLastError(), "attention_fwd_kernel launch");
}

inline int32_t attention(std::string* err, const tsm100_attention_desc* d, const void* q, const void* k,
                         const void* v, void* o, uint32_t* status, void* stream) {
  if (!d || !q || !k || !v || !o) return op_fail(err, TSM100_ERR_INVALID, "attention: null argument");
  if (!dtype_valid(d->dtype)) return op_fail(err, TSM100_ERR_INVALID, "attention: unknown dtype");
  if (d->batch < 0 || d->heads_q < 0 || d->heads_kv < 0 || d->seq < 0 || d->head_dim < 0)
    return op_fail(err, TSM100_ERR_INVALID, "attention: negative shape");
  if (d->batch == 0 || d->heads_q == 0 || d->seq == 0 || d->head_dim == 0) return TSM100_OK;
  if (d->heads_kv <= 0 || d->heads_q % d->heads_kv != 0)
    return op_fail(err, TSM100_ERR_INVALID, "attention: heads_q must be a positive multiple of heads_kv");
  if (d->head_dim > attn_simt::kMaxD) return op_fail(err, TSM100_ERR_INVALID, "attention: head_dim > 256 unsupported");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc_ok = d->dtype != TSM100_F32 && d->head_dim == attn::kD && status != nullptr && aligned16(q) &&
                     aligned16(k) && aligned16(v) && aligned16(o);
  if (tc_ok) {
    if (d->dtype == TSM100_BF16) return attention_tc_launch<true>(err, d, q, k, v, o, status, s);
    return attention_tc_launch<false>(err, d, q, k, v, o, status, s);
  }
  if (d->dtype == TSM100_F32) return attention_simt_launch<float>(err, d, q, k, v, o, s);
  if (d->dtype == TSM100_BF16) return attention_simt_launch<__nv_bfloat16>(err, d, q, k, v, o, s);
  return attention_simt_launch<__half>(err, d, q, k, v, o, s);
}

}  // namespace ops
}  // namespace tsm100
