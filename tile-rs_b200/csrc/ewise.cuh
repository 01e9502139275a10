// Building blocks of the element-wise kernels the `cuda_sm100` target generates for
// chains of tile_std's element-wise intrinsics between tile loads and one tile store
// (add / sub / mul / div / max / min, exp / log / neg / tanh / abs / sqrt / rsqrt /
// sigmoid / silu / relu, scale, clamp, fill, casts).  The reference's NVIDIA emitter
// lowers such a chain one scalar per thread with every intermediate tile named in the
// generated source (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:647-800); here the
// whole chain is one pass over memory with 16-byte accesses and f32 arithmetic.
//
// Semantics per operator follow the linalg bridge
// (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:422-470: linalg.add/sub/mul/div/max/min,
// linalg.exp/log/negf/tanh/abs/sqrt; :756-790: rsqrt, sigmoid = 1/(1+exp(-x)),
// silu = x/(1+exp(-x)), relu = max(x, 0); :805-905: scale = x * c; :907-982:
// clamp = min(max(x, lo), hi)).
#pragma once

#include "softmax.cuh"

namespace tsm100 {
namespace ewise {

using softmax::Elem;
using softmax::Vec16;

// Eight consecutive elements starting at element 8 * i: one 16-byte vector of a 16-bit
// type, two of f32.  The pointer must be 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, int64_t i, float (&f)[8]) {
  const Vec16* v = reinterpret_cast<const Vec16*>(p);
  if (sizeof(T) == 4) {
    Elem<T>::unpack(softmax::ld_stream(v + 2 * i), f);
    Elem<T>::unpack(softmax::ld_stream(v + 2 * i + 1), f + 4);
  } else {
    Elem<T>::unpack(softmax::ld_stream(v + i), f);
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* __restrict__ p, int64_t i, const float (&f)[8]) {
  Vec16* v = reinterpret_cast<Vec16*>(p);
  if (sizeof(T) == 4) {
    softmax::st_stream(v + 2 * i, Elem<T>::pack(f));
    softmax::st_stream(v + 2 * i + 1, Elem<T>::pack(f + 4));
  } else {
    softmax::st_stream(v + i, Elem<T>::pack(f));
  }
}
template <typename T>
__device__ __forceinline__ float load1(const T* p, int64_t i) { return Elem<T>::load1(p + i); }
template <typename T>
__device__ __forceinline__ void store1(T* p, int64_t i, float f) { Elem<T>::store1(p + i, f); }

__device__ __forceinline__ float op_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float op_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float op_relu(float x) { return fmaxf(x, 0.0f); }
__device__ __forceinline__ float op_rsqrt(float x) { return 1.0f / sqrtf(x); }
__device__ __forceinline__ float op_clamp(float x, float lo, float hi) { return fminf(fmaxf(x, lo), hi); }

}  // namespace ewise
}  // namespace tsm100
