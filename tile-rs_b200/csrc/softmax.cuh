// Row softmax for sm_100a: y[r, :] = exp(x[r, :] - max) / sum(exp(x[r, :] - max)).
//
// Semantics follow __tile_softmax_f32 / _f16 (crates/tile_std/src/tile.rs:189-190,
// :2162-2163) as the linalg bridge defines them, `linalg.softmax dimension(1)`
// (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1305-1343).  The reference's
// own CUDA lowering is one thread per element with two block reductions through
// shared memory and requires cols == blockDim <= 1024
// (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1242-1336); nothing of it is kept.
//
// The operator is bound by HBM: 2 * sizeof(T) algorithmic bytes per element.
// Four kernels, picked by the host from the row width:
//   * softmax_rows_warp  : one warp per row, the whole row held in registers,
//     128-bit coalesced streaming loads, shuffle reductions, one global read and
//     one global write per element.  Rows of up to 256 16-byte vectors.
//   * softmax_rows_cta   : 128 or 256 threads per row, 32 values per thread in
//     registers, warp shuffles plus one shared-memory exchange per reduction;
//     persistent CTAs stride over the rows.  Rows of up to 2048 vectors (the
//     4096-wide configuration runs here with eight resident CTAs per SM).
//   * softmax_rows_block : one CTA per row, the row staged once in shared memory
//     as f32 (up to 56 Ki elements); still one read + one write.
//   * softmax_rows_stream: any width or alignment; online max/sum in a first
//     pass, normalisation in a second (two reads + one write).
// bf16 / f16 rows are widened to f32 on load; all arithmetic is f32; the store
// narrows with round-to-nearest-even.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tsm100 {
namespace softmax {

struct alignas(16) Vec16 {
  uint32_t w[4];
};

template <typename T>
struct Elem;  // conversion between storage type and f32

template <>
struct Elem<float> {
  static constexpr int kPerVec = 4;
  __device__ static __forceinline__ void unpack(const Vec16& v, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(v.w[i]);
  }
  __device__ static __forceinline__ Vec16 pack(const float* f) {
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) v.w[i] = __float_as_uint(f[i]);
    return v;
  }
  __device__ static __forceinline__ float load1(const float* p) { return *p; }
  __device__ static __forceinline__ void store1(float* p, float f) { *p = f; }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ void unpack(const Vec16& v, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(v.w[i] << 16);
      f[2 * i + 1] = __uint_as_float(v.w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ Vec16 pack(const float* f) {
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      v.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return v;
  }
  __device__ static __forceinline__ __nv_bfloat16 zero() { return __float2bfloat16_rn(0.f); }
  __device__ static __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static __forceinline__ void store1(__nv_bfloat16* p, float f) { *p = __float2bfloat16_rn(f); }
};

template <>
struct Elem<__half> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ void unpack(const Vec16& v, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&v.w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ Vec16 pack(const float* f) {
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      v.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return v;
  }
  __device__ static __forceinline__ __half zero() { return __float2half_rn(0.f); }
  __device__ static __forceinline__ float load1(const __half* p) { return __half2float(*p); }
  __device__ static __forceinline__ void store1(__half* p, float f) { *p = __float2half_rn(f); }
};

// 128-bit streaming accesses: rows are touched exactly once, so they are
// marked evict-first and kept out of L1.
__device__ __forceinline__ Vec16 ld_stream(const Vec16* p) {
  Vec16 v;
  asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(Vec16* p, const Vec16& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]),
               "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// One warp per row; lane l owns 16-byte vectors l, l+32, l+64, ... (CHUNKS of
// them).  cols must be a multiple of Elem<T>::kPerVec and x, y 16-byte aligned
// with a 16-byte-multiple row pitch (the host checks).
// ---------------------------------------------------------------------------
template <typename T, int CHUNKS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
softmax_rows_warp(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t cols) {
  constexpr int PV = Elem<T>::kPerVec;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = cols / PV;
  const Vec16* xr = reinterpret_cast<const Vec16*>(x + row * cols);
  Vec16* yr = reinterpret_cast<Vec16*>(y + row * cols);

  float v[CHUNKS][PV];
  Vec16 raw[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = c * 32 + lane;
    if (i < nvec) raw[c] = ld_stream(xr + i);
  }
  float m = -INFINITY;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = c * 32 + lane;
    if (i < nvec) {
      Elem<T>::unpack(raw[c], v[c]);
#pragma unroll
      for (int e = 0; e < PV; ++e) m = fmaxf(m, v[c][e]);
    } else {
#pragma unroll
      for (int e = 0; e < PV; ++e) v[c][e] = -INFINITY;
    }
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
    for (int e = 0; e < PV; ++e) {
      // exp(-inf - m) = 0 for the padding; a row of all -inf yields NaN like the oracle.
      const float t = expf(v[c][e] - m);
      v[c][e] = t;
      s += t;
    }
  }
  s = warp_sum(s);
  const float inv = 1.0f / s;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = c * 32 + lane;
    if (i < nvec) {
#pragma unroll
      for (int e = 0; e < PV; ++e) v[c][e] *= inv;
      st_stream(yr + i, Elem<T>::pack(v[c]));
    }
  }
}

// exp(x - m) as 2^(x*log2e - m*log2e): one FMA and one MUFU op.  For |x - m| up to
// ~100 the rounding of the FMA argument costs less than 4e-6 relative, inside the
// 1e-5 bound of the f32 configuration; results below 2^-126 flush to zero.
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float exp_shifted(float x, float m_log2e) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(x, kLog2e, -m_log2e)));
  return y;
}

// ---------------------------------------------------------------------------
// THREADS threads per row, VPT 16-byte vectors per thread (vector k*THREADS + tid).
// Same alignment contract as the warp kernel; cols <= THREADS * VPT * kPerVec.
// ---------------------------------------------------------------------------
template <typename T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_rows_cta(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t cols) {
  constexpr int PV = Elem<T>::kPerVec;
  constexpr int NW = THREADS / 32;
  __shared__ float red_max[NW];
  __shared__ float red_sum[NW];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = cols / PV;
  // Software pipeline: the loads of the next row are in flight while this row is
  // reduced and stored, which doubles the bytes each SM keeps outstanding.
  Vec16 raw[VPT];
  if (static_cast<int64_t>(blockIdx.x) < rows) {
    const Vec16* x0 = reinterpret_cast<const Vec16*>(x + static_cast<int64_t>(blockIdx.x) * cols);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = k * THREADS + tid;
      if (i < nvec) raw[k] = ld_stream(x0 + i);
    }
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16* yr = reinterpret_cast<Vec16*>(y + row * cols);
    Vec16 nxt[VPT];
    const int64_t next_row = row + gridDim.x;
    if (next_row < rows) {
      const Vec16* xn = reinterpret_cast<const Vec16*>(x + next_row * cols);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = k * THREADS + tid;
        if (i < nvec) nxt[k] = ld_stream(xn + i);
      }
    }
    float v[VPT][PV];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = k * THREADS + tid;
      if (i < nvec) {
        Elem<T>::unpack(raw[k], v[k]);
#pragma unroll
        for (int e = 0; e < PV; ++e) m = fmaxf(m, v[k][e]);
      } else {
#pragma unroll
        for (int e = 0; e < PV; ++e) v[k][e] = -INFINITY;
      }
    }
    m = warp_max(m);
    if (lane == 0) red_max[warp] = m;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < NW; ++w) m = fmaxf(m, red_max[w]);
    const float ml = m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
#pragma unroll
      for (int e = 0; e < PV; ++e) {
        const float t = exp_shifted(v[k][e], ml);  // padding: 2^(-inf) = 0
        v[k][e] = t;
        s += t;
      }
    }
    s = warp_sum(s);
    if (lane == 0) red_sum[warp] = s;
    __syncthreads();
    s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += red_sum[w];
    const float inv = 1.0f / s;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = k * THREADS + tid;
      if (i < nvec) {
#pragma unroll
        for (int e = 0; e < PV; ++e) v[k][e] *= inv;
        st_stream(yr + i, Elem<T>::pack(v[k]));
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) raw[k] = nxt[k];
    // red_max is rewritten only after this row's second barrier and red_sum only
    // after the next row's first one, so neither is overwritten while still read.
  }
}

// ---------------------------------------------------------------------------
// One CTA per row, row staged in dynamic shared memory as f32 (cols * 4 bytes).
// Same alignment contract as the warp kernel.
// ---------------------------------------------------------------------------
template <int THREADS>
__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();  // red[] may still be read from a previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? red[lane] : (is_max ? -INFINITY : 0.f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_rows_block(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t cols) {
  constexpr int PV = Elem<T>::kPerVec;
  extern __shared__ __align__(16) float row_f32[];
  __shared__ float red[32];
  const int nvec = cols / PV;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const Vec16* xr = reinterpret_cast<const Vec16*>(x + row * cols);
    Vec16* yr = reinterpret_cast<Vec16*>(y + row * cols);
    float m = -INFINITY;
    for (int i = threadIdx.x; i < nvec; i += THREADS) {
      float f[PV];
      Elem<T>::unpack(ld_stream(xr + i), f);
#pragma unroll
      for (int e = 0; e < PV; ++e) {
        m = fmaxf(m, f[e]);
        row_f32[i * PV + e] = f[e];
      }
    }
    m = block_reduce<THREADS>(m, red, true);
    float s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += THREADS) {
#pragma unroll
      for (int e = 0; e < PV; ++e) {
        const float t = expf(row_f32[i * PV + e] - m);
        row_f32[i * PV + e] = t;
        s += t;
      }
    }
    s = block_reduce<THREADS>(s, red, false);
    const float inv = 1.0f / s;
    for (int i = threadIdx.x; i < nvec; i += THREADS) {
      float f[PV];
#pragma unroll
      for (int e = 0; e < PV; ++e) f[e] = row_f32[i * PV + e] * inv;
      st_stream(yr + i, Elem<T>::pack(f));
    }
    __syncthreads();  // row_f32 is reused by the next row
  }
}

// ---------------------------------------------------------------------------
// Any width, any alignment: scalar accesses, online (max, sum) in pass one.
// ---------------------------------------------------------------------------
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_rows_stream(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    T* yr = y + row * cols;
    float m = -INFINITY, s = 0.f;
    for (int64_t i = threadIdx.x; i < cols; i += THREADS) {
      const float f = Elem<T>::load1(xr + i);
      if (f > m) {
        s = s * expf(m - f);  // m = -inf on the first element: s is 0, expf(-inf) = 0
        m = f;
      }
      s += expf(f - m);
    }
    const float gm = block_reduce<THREADS>(m, red, true);
    // a thread that saw no element has m = -inf and s = 0: contributes 0
    s = (m == -INFINITY) ? 0.f : s * expf(m - gm);
    s = block_reduce<THREADS>(s, red, false);
    const float inv = 1.0f / s;
    for (int64_t i = threadIdx.x; i < cols; i += THREADS)
      Elem<T>::store1(yr + i, expf(Elem<T>::load1(xr + i) - gm) * inv);
  }
}

}  // namespace softmax
}  // namespace tsm100
