// Fused attention forward for f32 tensors on tensor cores with f32-grade accuracy.
//
// __tile_attention_f32 (crates/tile_std/src/tile.rs:218-224) is an f32 operator: the linalg
// bridge lowers it to transpose, matmul, scale by 1/sqrt(D), row softmax, matmul, all in f32
// (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1781-1902), with __tile_causal_mask_f32
// (mlir_to_linalg.rs:1191-1244) between scale and softmax, and the grouped-query form maps
// kv_head = h / (heads_q / heads_kv) (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1657-1673).
// Agreement with an f32 CPU evaluation to 1e-5 rules out plain TF32 products (11 significant
// bits), so every operand is split in registers into hi (its top 11 significant bits) and
// lo = x - hi, and a product is hi*hi + hi*lo + lo*hi on mma.sync.m16n8k8.tf32 with f32
// accumulation - the scheme of gemm_tf32x3.cuh, here for both S = Q K^T and O += P V.
//
// Flash style: a CTA of 8 warps owns 128 query rows of one head (16 per warp); K and V go
// through a two-stage cp.async ring in 64-key tiles (rows padded by 16 bytes so that the
// B-fragment loads hit 32 banks); the score tile lives in the accumulator fragments, online
// max / sum per row, and the accumulator layout of S is used directly as the A operand of
// P V (the k index of that product is a permutation of the keys, applied to the V loads).
// 16-bit tensors with head sizes the tcgen05 kernel does not cover (32, 64, 96) use the same kernel:
// a bf16 or f16 value is a TF32 number already (8 / 11 significant bits), its lo part is zero, so
// Q K^T is ONE product and P V two (P is f32), still with f32-grade accuracy before the final rounding.
// Same strided layouts as attention_simt.cuh: plain [batch*heads][seq][d] tensors, or
// token-major Q / O against a KV cache with a position offset (prefill).
#pragma once

#include "attention_decode.cuh"  // cp.async helpers
#include "attention_simt.cuh"    // Params
#include "ptx.cuh"

namespace tsm100 {
namespace attn_tf32 {

using attn_simt::Params;

constexpr int kBM = 128;       // query rows per CTA
constexpr int kBN = 64;        // keys per step
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 2;

template <typename T, int D>
constexpr int pitch_bytes() { return D * static_cast<int>(sizeof(T)) + 16; }  // rows 4 banks apart for D = 32, 64, 96, 128
template <typename T, int D>
constexpr int tile_bytes() { return kBN * pitch_bytes<T, D>(); }
template <typename T, int D>
constexpr int smem_bytes() { return kStages * 2 * tile_bytes<T, D>(); }  // K and V tiles

__device__ __forceinline__ void split(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;          // what the tensor core reads of x
  lo = __float_as_uint(x - __uint_as_float(hi));  // exact; the tensor core reads its top 11 bits
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// d += a * b, small terms first.  f32 B: three products.  A 16-bit B value (bf16: 8 significant bits, f16: 11)
// is a TF32 number already, its lo part is zero: two products, or one when A is 16-bit data as well.
template <bool kExactA, bool kExactB>
__device__ __forceinline__ void mma_split(float (&d)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4], float b0, float b1) {
  if (kExactB) {
    if (!kExactA) mma_tf32(d, al, __float_as_uint(b0), __float_as_uint(b1));
    mma_tf32(d, ah, __float_as_uint(b0), __float_as_uint(b1));
  } else {
    uint32_t b0h, b0l, b1h, b1l;
    split(b0, b0h, b0l);
    split(b1, b1h, b1l);
    mma_tf32(d, al, b0h, b1h);
    mma_tf32(d, ah, b0l, b1l);
    mma_tf32(d, ah, b0h, b1h);
  }
}

// The same for N independent accumulators that share A: the products are issued term by term across the group,
// so that an MMA never waits for the one just before it (which writes the same accumulator).
template <bool kExactA, bool kExactB, int N>
__device__ __forceinline__ void mma_split_group(float (*d)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                                const float (&b0)[N], const float (&b1)[N]) {
  if (kExactB) {
    if (!kExactA) {
#pragma unroll
      for (int n = 0; n < N; ++n) mma_tf32(d[n], al, __float_as_uint(b0[n]), __float_as_uint(b1[n]));
    }
#pragma unroll
    for (int n = 0; n < N; ++n) mma_tf32(d[n], ah, __float_as_uint(b0[n]), __float_as_uint(b1[n]));
  } else {
    uint32_t b0h[N], b0l[N], b1h[N], b1l[N];
#pragma unroll
    for (int n = 0; n < N; ++n) {
      split(b0[n], b0h[n], b0l[n]);
      split(b1[n], b1h[n], b1l[n]);
    }
#pragma unroll
    for (int n = 0; n < N; ++n) mma_tf32(d[n], al, b0h[n], b1h[n]);  // small terms first
#pragma unroll
    for (int n = 0; n < N; ++n) mma_tf32(d[n], ah, b0l[n], b1l[n]);
#pragma unroll
    for (int n = 0; n < N; ++n) mma_tf32(d[n], ah, b0h[n], b1h[n]);
  }
}

// 16-bit data with head_dim <= 64 needs few enough registers for two CTAs per SM (16 warps hide each other's latencies)
template <typename T, int D>
__global__ void __launch_bounds__(kThreads, (sizeof(T) == 2 && D <= 64) ? 2 : 1)
attention_tf32x3_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        T* __restrict__ o, const Params p) {
  namespace cp = attn_decode::mma;
  using gemm_simt::from_f32;
  using gemm_simt::to_f32;
  constexpr bool kExact = sizeof(T) == 2;  // 16-bit data: every input value is a TF32 number
  constexpr int PW = pitch_bytes<T, D>() / static_cast<int>(sizeof(T));  // row pitch in elements
  constexpr int KSTEPS = D / 8;   // k-steps of Q K^T; 8-wide output tiles of P V
  constexpr int VEC = 16 / static_cast<int>(sizeof(T));
  constexpr int CHUNKS = D / VEC;  // 16-byte pieces per row
  extern __shared__ __align__(16) uint8_t smem_f[];
  const uint32_t smem_base = ptx::smem_u32(smem_f);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gr = lane >> 2, tq = lane & 3;

  // block -> (head, query block): the query blocks of a head are adjacent (K and V stay in L2), heaviest first when causal
  const int q_blocks = (p.seq + kBM - 1) / kBM;
  const int qb_raw = static_cast<int>(blockIdx.x % q_blocks);
  const int64_t bh = blockIdx.x / q_blocks;
  const int q0 = (p.causal ? q_blocks - 1 - qb_raw : qb_raw) * kBM;
  const int b = static_cast<int>(bh / p.heads_q), h = static_cast<int>(bh % p.heads_q);
  const int64_t kvh = static_cast<int64_t>(b) * p.heads_kv + h / (p.heads_q / p.heads_kv);
  const T* kb = k + kvh * p.kv_head_stride;
  const T* vb = v + kvh * p.kv_head_stride;
  const int n_all = (p.seq_kv + kBN - 1) / kBN;
  const int n_tiles = p.causal ? min(n_all, (q0 + kBM - 1 + p.q_offset) / kBN + 1) : n_all;

  auto prefetch = [&](int tile, int stage) {
    const uint32_t ks = smem_base + stage * 2 * tile_bytes<T, D>(), vs = ks + tile_bytes<T, D>();
    for (int i = tid; i < kBN * CHUNKS; i += kThreads) {
      const int r = i / CHUNKS, c4 = (i % CHUNKS) * VEC;
      const int key = tile * kBN + r;
      const bool ok = key < p.seq_kv;  // rows past the end are zero-filled: 0 * V must stay finite
      const int64_t off = ok ? static_cast<int64_t>(key) * D + c4 : 0;
      cp::cp_async_16(ks + (r * PW + c4) * static_cast<int>(sizeof(T)), kb + off, ok);
      cp::cp_async_16(vs + (r * PW + c4) * static_cast<int>(sizeof(T)), vb + off, ok);
    }
  };
  if (n_tiles > 0) prefetch(0, 0);
  cp::cp_async_commit();

  // A fragments of Q: a0 (row gr, k tq), a1 (row gr+8, k tq), a2 (row gr, k tq+4), a3 (row gr+8, k tq+4)
  const int r0 = q0 + warp * 16 + gr, r1 = r0 + 8;
  float qa[KSTEPS][4];
  {
    const T* q_r0 = q + bh * p.q_head_stride + static_cast<int64_t>(r0) * p.q_row_stride;
    const T* q_r1 = q + bh * p.q_head_stride + static_cast<int64_t>(r1) * p.q_row_stride;
    const bool ok0 = r0 < p.seq, ok1 = r1 < p.seq;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = ok0 ? to_f32(q_r0[kk * 8 + tq]) : 0.f;
      qa[kk][1] = ok1 ? to_f32(q_r1[kk * 8 + tq]) : 0.f;
      qa[kk][2] = ok0 ? to_f32(q_r0[kk * 8 + tq + 4]) : 0.f;
      qa[kk][3] = ok1 ? to_f32(q_r1[kk * 8 + tq + 4]) : 0.f;
    }
  }
  // last visible key of the two rows
  const int lim0 = p.causal ? min(r0 + p.q_offset, p.seq_kv - 1) : p.seq_kv - 1;
  const int lim1 = p.causal ? min(r1 + p.q_offset, p.seq_kv - 1) : p.seq_kv - 1;
  const float sl2 = p.scale * 1.4426950408889634f;

  float oacc[KSTEPS][4];
#pragma unroll
  for (int i = 0; i < KSTEPS; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    if (t + 1 < n_tiles) prefetch(t + 1, (t + 1) & 1);
    cp::cp_async_commit();
    cp::cp_async_wait<1>();  // tile t has landed (this thread's copies) ...
    __syncthreads();         // ... and everybody's
    const T* ks = reinterpret_cast<const T*>(smem_f + (t & 1) * 2 * tile_bytes<T, D>());
    const T* vs = reinterpret_cast<const T*>(smem_f + (t & 1) * 2 * tile_bytes<T, D>() + tile_bytes<T, D>());

    // S = Q K^T for 16 rows x 64 keys: b0 (k tq, key gr), b1 (k tq+4, key gr) of every 8-key group
    float s[kBN / 8][4];
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (kExact) ah[e] = __float_as_uint(qa[kk][e]), al[e] = 0u;
        else split(qa[kk][e], ah[e], al[e]);
      }
      float kv0[kBN / 8], kv1[kBN / 8];
#pragma unroll
      for (int n = 0; n < kBN / 8; ++n) {
        const T* kr = ks + (n * 8 + gr) * PW + kk * 8 + tq;
        kv0[n] = to_f32(kr[0]);
        kv1[n] = to_f32(kr[4]);
      }
      mma_split_group<kExact, kExact, kBN / 8>(s, ah, al, kv0, kv1);
    }
    // scale to log2 units, mask, row maxima (c0, c1: row gr, keys 2tq, 2tq+1; c2, c3: row gr+8)
    const int key0 = t * kBN + 2 * tq;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) {
      const int kx = key0 + n * 8;
      s[n][0] = kx <= lim0 ? s[n][0] * sl2 : -INFINITY;
      s[n][1] = kx + 1 <= lim0 ? s[n][1] * sl2 : -INFINITY;
      s[n][2] = kx <= lim1 ? s[n][2] * sl2 : -INFINITY;
      s[n][3] = kx + 1 <= lim1 ? s[n][3] * sl2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float ref0 = n0 == -INFINITY ? 0.f : n0, ref1 = n1 == -INFINITY ? 0.f : n1;  // a row with nothing visible yet
    const float a0 = ptx::ex2_approx(m0 - ref0), a1 = ptx::ex2_approx(m1 - ref1);      // 2^(-inf) = 0
    m0 = n0;
    m1 = n1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) {
      s[n][0] = ptx::ex2_approx(s[n][0] - ref0);
      s[n][1] = ptx::ex2_approx(s[n][1] - ref0);
      s[n][2] = ptx::ex2_approx(s[n][2] - ref1);
      s[n][3] = ptx::ex2_approx(s[n][3] - ref1);
      sum0 += s[n][0] + s[n][1];
      sum1 += s[n][2] + s[n][3];
    }
    l0 = fmaf(l0, a0, sum0);
    l1 = fmaf(l1, a1, sum1);
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      oacc[i][0] *= a0;
      oacc[i][1] *= a0;
      oacc[i][2] *= a1;
      oacc[i][3] *= a1;
    }
    // O += P V.  The accumulator fragment of S is the A fragment of this product with k index tq -> key 2tq and
    // k index tq+4 -> key 2tq+1 of the 8-key group; the V rows are read in that order.
#pragma unroll
    for (int n = 0; n < kBN / 8; ++n) {
      uint32_t ah[4], al[4];
      split(s[n][0], ah[0], al[0]);
      split(s[n][2], ah[1], al[1]);
      split(s[n][1], ah[2], al[2]);
      split(s[n][3], ah[3], al[3]);
      const T* vr = vs + (n * 8 + 2 * tq) * PW + gr;
      constexpr int G = KSTEPS % 8 == 0 ? 8 : 4;  // output tiles per group of independent accumulators
#pragma unroll
      for (int i0 = 0; i0 < KSTEPS; i0 += G) {
        float vv0[G], vv1[G];
#pragma unroll
        for (int i = 0; i < G; ++i) {
          vv0[i] = to_f32(vr[(i0 + i) * 8]);
          vv1[i] = to_f32(vr[PW + (i0 + i) * 8]);
        }
        mma_split_group<false, kExact, G>(oacc + i0, ah, al, vv0, vv1);
      }
    }
    __syncthreads();  // the stage is refilled at the top of the next iteration
  }
  cp::cp_async_wait<0>();

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
  T* o_r0 = o + bh * p.o_head_stride + static_cast<int64_t>(r0) * p.o_row_stride + 2 * tq;
  T* o_r1 = o + bh * p.o_head_stride + static_cast<int64_t>(r1) * p.o_row_stride + 2 * tq;
#pragma unroll
  for (int i = 0; i < KSTEPS; ++i) {
    if (r0 < p.seq) {
      o_r0[i * 8] = from_f32<T>(oacc[i][0] * inv0);
      o_r0[i * 8 + 1] = from_f32<T>(oacc[i][1] * inv0);
    }
    if (r1 < p.seq) {
      o_r1[i * 8] = from_f32<T>(oacc[i][2] * inv1);
      o_r1[i * 8 + 1] = from_f32<T>(oacc[i][3] * inv1);
    }
  }
}

}  // namespace attn_tf32
}  // namespace tsm100
