// f32 GEMM on tensor cores with f32-grade accuracy: C[b][M,N] = A[b][M,K] * B[b].
//
// __tile_matmul_f32 / __tile_matmul_transposed_f32 (crates/tile_std/src/tile.rs:192-193,
// :2017-2031; linalg.fill 0 + linalg.matmul, crates/rustc_codegen_tile/src/mlir_to_linalg.rs:
// 1345-1393) must agree with an f32 CPU contraction to 1e-5, which one TF32 product (11
// significant bits) cannot give.  Every operand is therefore split in registers into
// hi = its top 11 significant bits and lo = x - hi (exact), and a product is the sum of three
// tensor-core products  hi*hi + hi*lo + lo*hi  accumulated in f32; the dropped lo*lo term and
// the truncation of lo are below 2^-21 of |a||b|, the size of f32 rounding itself.
//
// 64 x 64 output tile per CTA, 4 warps of 32 x 32 (2 x 4 mma.sync.m16n8k8.tf32 tiles), 32-deep
// K slices through a three- or four-stage cp.async ring; rows padded so that fragment loads are
// conflict-free.  A CTA cluster may split K (the 512^3 configuration has only 64 output tiles
// for 148 SMs): every CTA of a cluster accumulates its share of K and the partial tiles are
// added through distributed shared memory in rank order (every CTA its share of the tile), so the result
// does not depend on timing.
// Needs 16-byte aligned rows: K % 4 == 0, and N % 4 == 0 for row-major B.
#pragma once

#include "attention_decode.cuh"  // cp.async helpers
#include "ptx.cuh"

namespace tsm100 {
namespace gemm_tf32x3 {

constexpr int kBM = 64, kBN = 64, kBK = 32;
constexpr int kStages = 3;       // large problems (several CTAs per SM)
constexpr int kStagesSplit = 4;  // K split over a cluster: few slices per CTA, all of them in flight at once
constexpr int kThreads = 128;
constexpr int kPitchA = kBK + 4;   // floats: rows 4 banks apart -> A fragment loads hit 32 banks
constexpr int kPitchB = kBN + 8;   // row-major B [K][N]: rows 8 banks apart
constexpr int kPitchBT = kBK + 4;  // B stored [N][K]: same pattern as A
constexpr int kABytes = kBM * kPitchA * 4;
constexpr int kBBytes = (kBK * kPitchB > kBN * kPitchBT ? kBK * kPitchB : kBN * kPitchBT) * 4;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmemBytes = kStagesSplit * kStageBytes;   // the most a launch asks for; the 64 x 64 f32 tile for the cluster sum (16 KiB) overlays the ring
constexpr int kMaxSplit = 4;

struct Params {
  int32_t m, n, k, batch;
  int32_t k_per_cta;  // K range of one CTA of a cluster, a multiple of kBK
  int64_t lda, ldb, ldc;  // row pitches in elements (multiples of 4, 4 and 2); problems of a batch are rows * pitch apart
};

__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  // hi = x rounded to the nearest TF32 number (ties away from zero), not truncated: a truncated hi leaves a lo
  // of x's own sign, whose truncation inside the tensor core then errs the same way for every term, and the
  // error grows with K instead of sqrt(K) (3e-5 of the largest element at K = 4096)
  hi = (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));  // exact, either sign; the tensor core reads its top 11 bits
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kBTransposed, int STAGES = kStages>
__global__ void __launch_bounds__(kThreads)
gemm_tf32x3_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, const Params p) {
  namespace cp = attn_decode::mma;
  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t rank = ptx::cluster_ctarank(), splits = ptx::cluster_nctarank();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;  // this warp's 32 x 32 corner of the tile
  const int n_blocks = (p.n + kBN - 1) / kBN, m_blocks = (p.m + kBM - 1) / kBM;
  const int tile = blockIdx.x / splits;
  const int bz = tile / (n_blocks * m_blocks);
  const int m0 = ((tile / n_blocks) % m_blocks) * kBM, n0 = (tile % n_blocks) * kBN;
  const int k_begin = static_cast<int>(rank) * p.k_per_cta;
  const int k_end = min(p.k, k_begin + p.k_per_cta);
  const int n_slices = k_end > k_begin ? (k_end - k_begin + kBK - 1) / kBK : 0;
  const float* ab = a + static_cast<int64_t>(bz) * p.m * p.lda;
  const float* bb = b + static_cast<int64_t>(bz) * (kBTransposed ? p.n : p.k) * p.ldb;

  auto prefetch = [&](int slice, int stage) {
    const int k0 = k_begin + slice * kBK;
    const uint32_t as = smem_base + stage * kStageBytes, bs = as + kABytes;
    // A: 64 rows x 32 floats = 512 16-byte pieces
    for (int i = tid; i < kBM * (kBK / 4); i += kThreads) {
      const int r = i / (kBK / 4), c4 = (i % (kBK / 4)) * 4;
      const bool ok = m0 + r < p.m && k0 + c4 < k_end;  // K % 4 == 0: a piece is inside or outside as a whole
      cp::cp_async_16(as + (r * kPitchA + c4) * 4, ab + (ok ? static_cast<int64_t>(m0 + r) * p.lda + k0 + c4 : 0), ok);
    }
    if (kBTransposed) {  // B stored [N][K]
      for (int i = tid; i < kBN * (kBK / 4); i += kThreads) {
        const int r = i / (kBK / 4), c4 = (i % (kBK / 4)) * 4;
        const bool ok = n0 + r < p.n && k0 + c4 < k_end;
        cp::cp_async_16(bs + (r * kPitchBT + c4) * 4, bb + (ok ? static_cast<int64_t>(n0 + r) * p.ldb + k0 + c4 : 0), ok);
      }
    } else {             // B stored [K][N]
      for (int i = tid; i < kBK * (kBN / 4); i += kThreads) {
        const int r = i / (kBN / 4), c4 = (i % (kBN / 4)) * 4;
        const bool ok = k0 + r < k_end && n0 + c4 < p.n;  // N % 4 == 0
        cp::cp_async_16(bs + (r * kPitchB + c4) * 4, bb + (ok ? static_cast<int64_t>(k0 + r) * p.ldb + n0 + c4 : 0), ok);
      }
    }
  };

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_slices) prefetch(s, s);
    cp::cp_async_commit();
  }
  for (int s = 0; s < n_slices; ++s) {
    cp::cp_async_wait<STAGES - 2>();  // slice s has landed (for this thread's copies)
    __syncthreads();                  // ... for everybody's; and the stage refilled below is no longer read
    if (s + STAGES - 1 < n_slices) prefetch(s + STAGES - 1, (s + STAGES - 1) % STAGES);
    cp::cp_async_commit();
    const float* as = reinterpret_cast<const float*>(smem + (s % STAGES) * kStageBytes);
    const float* bs = reinterpret_cast<const float*>(smem + (s % STAGES) * kStageBytes + kABytes);
#pragma unroll
    for (int kk = 0; kk < kBK / 8; ++kk) {
      uint32_t ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {  // a0 (row g, k t), a1 (row g+8, k t), a2 (row g, k t+4), a3 (row g+8, k t+4)
        const float* r0 = as + (wm + i * 16 + g) * kPitchA + kk * 8;
        const float* r1 = r0 + 8 * kPitchA;
        split_tf32(r0[t], ah[i][0], al[i][0]);
        split_tf32(r1[t], ah[i][1], al[i][1]);
        split_tf32(r0[t + 4], ah[i][2], al[i][2]);
        split_tf32(r1[t + 4], ah[i][3], al[i][3]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // b0 (k t, n g), b1 (k t+4, n g)
        float v0, v1;
        if (kBTransposed) {
          const float* r = bs + (wn + j * 8 + g) * kPitchBT + kk * 8;
          v0 = r[t];
          v1 = r[t + 4];
        } else {
          const float* r = bs + (kk * 8 + t) * kPitchB + wn + j * 8 + g;
          v0 = r[0];
          v1 = r[4 * kPitchB];
        }
        split_tf32(v0, bh[j][0], bl[j][0]);
        split_tf32(v1, bh[j][1], bl[j][1]);
      }
      // small terms first; term by term across the eight accumulators, so that an MMA never waits for the one
      // just before it (which would write the same accumulator)
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], al[i], bh[j][0], bh[j][1]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ah[i], bl[j][0], bl[j][1]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ah[i], bh[j][0], bh[j][1]);
    }
  }
  cp::cp_async_wait<0>();

  if (splits > 1) {
    // every CTA parks its partial tile in its own shared memory; rank 0 adds them in rank order
    __syncthreads();  // the ring is no longer read
    float* tile_s = reinterpret_cast<float*>(smem);  // [64][64]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = wm + i * 16 + g, cc = wn + j * 8 + 2 * t;
        tile_s[r * kBN + cc] = acc[i][j][0];
        tile_s[r * kBN + cc + 1] = acc[i][j][1];
        tile_s[(r + 8) * kBN + cc] = acc[i][j][2];
        tile_s[(r + 8) * kBN + cc + 1] = acc[i][j][3];
      }
    ptx::cluster_sync_all();
    {
      // every CTA adds its share of the tile (pairs of columns; N is even), all its remote loads in flight
      // together, ranks in rank order: a single CTA walking the whole tile spent more time here than in the MMAs
      float* cb = c + static_cast<int64_t>(bz) * p.m * p.ldc;
      const int per = kBM * kBN / 2 / static_cast<int>(splits);  // column pairs per rank
      for (int i = static_cast<int>(rank) * per + tid; i < (static_cast<int>(rank) + 1) * per; i += kThreads) {
        const int r = (2 * i) / kBN, cc = (2 * i) % kBN;
        if (m0 + r >= p.m || n0 + cc >= p.n) continue;
        float2 part[kMaxSplit];
#pragma unroll
        for (int q = 0; q < kMaxSplit; ++q)
          part[q] = q < static_cast<int>(splits) ? ptx::ld_shared_cluster_f32x2(ptx::mapa_shared(smem_base + i * 8, static_cast<uint32_t>(q)))
                                                  : make_float2(0.f, 0.f);
        float2 v = part[0];
#pragma unroll
        for (int q = 1; q < kMaxSplit; ++q)
          if (q < static_cast<int>(splits)) {
            v.x += part[q].x;
            v.y += part[q].y;
          }
        *reinterpret_cast<float2*>(cb + static_cast<int64_t>(m0 + r) * p.ldc + n0 + cc) = v;
      }
    }
    ptx::cluster_sync_all();  // nobody leaves while its shared memory may still be read
    return;
  }
  float* cb = c + static_cast<int64_t>(bz) * p.m * p.ldc;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + wm + i * 16 + g, cc = n0 + wn + j * 8 + 2 * t;  // N % 4 == 0 and cc even: cc + 1 < n when cc < n
      if (cc < p.n) {
        if (r < p.m) *reinterpret_cast<float2*>(cb + static_cast<int64_t>(r) * p.ldc + cc) = make_float2(acc[i][j][0], acc[i][j][1]);
        if (r + 8 < p.m) *reinterpret_cast<float2*>(cb + static_cast<int64_t>(r + 8) * p.ldc + cc) = make_float2(acc[i][j][2], acc[i][j][3]);
      }
    }
}

}  // namespace gemm_tf32x3
}  // namespace tsm100
