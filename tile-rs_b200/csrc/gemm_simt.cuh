// FP32-pipe GEMM: C[b][M,N] = A[b][M,K] * B[b], f32 accumulation with FMA.
//
// This is the kernel behind __tile_matmul_f32 (crates/tile_std/src/tile.rs:192-193;
// linalg.fill 0 + linalg.matmul, crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1345-1393)
// and __tile_matmul_transposed_f32 (tile.rs:2017-2031) when the rows of the operands
// do not start on 16-byte boundaries (aligned f32 problems run on tensor cores with three
// TF32 products per product, gemm_tf32x3.cuh), and the any-shape path for 16-bit inputs
// whose leading dimensions are not 16-byte multiples (TMA cannot address those).
//
// Tiling: BM x BN output tile per CTA, BK-deep shared-memory panels, TM x TN
// register micro-tile per thread, every access bounds-checked.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tsm100 {
namespace gemm_simt {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

struct Params {
  int32_t m, n, k, batch;
  int32_t b_transposed;
  int64_t lda, ldb, ldc;  // row pitches in elements (>= the row length); problems of a batch are rows * pitch apart
};

template <typename InT, typename OutT, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const InT* __restrict__ a, const InT* __restrict__ b, OutT* __restrict__ c, const Params p) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float sa[BK][BM + 1];  // A panel, transposed so the k loop reads rows
  __shared__ float sb[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  const InT* ab = a + bz * static_cast<int64_t>(p.m) * p.lda;
  const InT* bb = b + bz * static_cast<int64_t>(p.b_transposed ? p.n : p.k) * p.ldb;
  OutT* cb = c + bz * static_cast<int64_t>(p.m) * p.ldc;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < p.k; k0 += BK) {
    // A panel: BM x BK, consecutive threads along k (contiguous in memory)
    for (int e = tid; e < BM * BK; e += THREADS) {
      const int r = e / BK, kk = e % BK;
      const int gr = m0 + r, gk = k0 + kk;
      sa[kk][r] = (gr < p.m && gk < p.k) ? to_f32(ab[static_cast<int64_t>(gr) * p.lda + gk]) : 0.f;
    }
    if (!p.b_transposed) {
      for (int e = tid; e < BK * BN; e += THREADS) {
        const int kk = e / BN, cidx = e % BN;
        const int gk = k0 + kk, gc = n0 + cidx;
        sb[kk][cidx] = (gk < p.k && gc < p.n) ? to_f32(bb[static_cast<int64_t>(gk) * p.ldb + gc]) : 0.f;
      }
    } else {
      for (int e = tid; e < BK * BN; e += THREADS) {
        const int cidx = e / BK, kk = e % BK;
        const int gk = k0 + kk, gc = n0 + cidx;
        sb[kk][cidx] = (gk < p.k && gc < p.n) ? to_f32(bb[static_cast<int64_t>(gc) * p.ldb + gk]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float ra[TM], rb[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) ra[i] = sa[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) rb[j] = sb[kk][tx + j * (BN / TN)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ra[i], rb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gr = m0 + ty * TM + i;
    if (gr >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gc = n0 + tx + j * (BN / TN);
      if (gc < p.n) cb[static_cast<int64_t>(gr) * p.ldc + gc] = from_f32<OutT>(acc[i][j]);
    }
  }
}

}  // namespace gemm_simt
}  // namespace tsm100
