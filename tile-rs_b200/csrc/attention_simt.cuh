// FP32-pipe fused attention forward: the path for f32 tensors
// (__tile_attention_f32 on real f32 data, crates/tile_std/src/tile.rs:218-224)
// and for head dimensions the tensor-core kernel does not cover.  Same
// semantics as attention_tc.cuh: softmax(Q K^T / sqrt(d)) V with an optional
// causal mask (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1781-1902,
// :1191-1244) and grouped KV heads (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1657-1673).
//
// One warp per query row, flash style: 32 keys per step (one per lane for the
// q.k dot products), online max/sum, then every lane accumulates its slice of
// head_dim over those 32 values.  All arithmetic f32.  head_dim <= 256.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_simt.cuh"

namespace tsm100 {
namespace attn_simt {

// Strides in elements.  Plain attention: Q, O [batch*heads_q][seq][d], K, V [batch*heads_kv][seq][d], q_offset 0.
// Prefill against a KV cache: Q, O token-major [seq][heads_q][d], K, V [heads_kv][max_seq][d] of which seq_kv
// positions are filled, query row i sits at position q_offset + i.
struct Params {
  int32_t seq, head_dim;       // query rows per head
  int32_t heads_q, heads_kv, batch;
  int32_t causal;
  float scale;
  int32_t seq_kv, q_offset;
  int64_t q_row_stride, q_head_stride, kv_head_stride, o_row_stride, o_head_stride;
};

constexpr int kWarps = 4;
constexpr int kMaxD = 256;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      T* __restrict__ o, const Params p) {
  using gemm_simt::from_f32;
  using gemm_simt::to_f32;
  __shared__ float sq[kWarps][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_id = static_cast<int64_t>(blockIdx.x) * kWarps + warp;  // over batch*heads_q*seq
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.seq;
  if (row_id >= total) return;
  const int i = static_cast<int>(row_id % p.seq);
  const int64_t bh = row_id / p.seq;
  const int b = static_cast<int>(bh / p.heads_q), h = static_cast<int>(bh % p.heads_q);
  const int64_t kvh = static_cast<int64_t>(b) * p.heads_kv + h / (p.heads_q / p.heads_kv);
  const int d = p.head_dim;
  const T* qi = q + bh * p.q_head_stride + i * p.q_row_stride;
  const T* kb = k + kvh * p.kv_head_stride;
  const T* vb = v + kvh * p.kv_head_stride;

  for (int c = lane; c < d; c += 32) sq[warp][c] = to_f32(qi[c]);
  __syncwarp();

  float acc[kMaxD / 32];
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) acc[t] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int lim = p.causal ? min(p.seq_kv, i + p.q_offset + 1) : p.seq_kv;
  for (int j0 = 0; j0 < lim; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < lim) {
      const T* kj = kb + static_cast<int64_t>(j) * d;
      float a = 0.f;
      for (int c = 0; c < d; ++c) a = fmaf(sq[warp][c], to_f32(kj[c]), a);
      s = a * p.scale;
    }
    float mx = s;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m, mx);
    const float alpha = expf(m - m_new);  // m = -inf on the first step: alpha = 0, acc is 0 anyway
    const float pj = (j < lim) ? expf(s - m_new) : 0.f;
    float ps = pj;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
    l = l * alpha + ps;
    m = m_new;
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) acc[t] *= alpha;
    const int nk = min(32, lim - j0);
    for (int t2 = 0; t2 < nk; ++t2) {
      const float pt = __shfl_sync(0xffffffffu, pj, t2);
      const T* vj = vb + static_cast<int64_t>(j0 + t2) * d;
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) {
        const int c = lane + 32 * t;
        if (c < d) acc[t] = fmaf(pt, to_f32(vj[c]), acc[t]);
      }
    }
  }
  const float inv = 1.0f / l;
  T* oi = o + bh * p.o_head_stride + i * p.o_row_stride;
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) {
    const int c = lane + 32 * t;
    if (c < d) oi[c] = from_f32<T>(acc[t] * inv);
  }
}

}  // namespace attn_simt
}  // namespace tsm100
