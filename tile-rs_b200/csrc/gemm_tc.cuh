// 16-bit GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   C[b][M,N] = A[b][M,K] * B[b]        A, C row-major; f32 accumulation
//   B row-major [K,N]  (__tile_matmul_f16, crates/tile_std/src/tile.rs:1982-1986)
//   or  B stored [N,K] (__tile_matmul_transposed_f16, tile.rs:2017-2031)
//
// Semantics: linalg.fill 0 + linalg.matmul
// (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1345-1393) on 16-bit inputs
// widened exactly, f32 accumulate, one round-to-nearest-even narrowing.  The
// reference's NVIDIA emitter has no implementation of this contraction
// (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1373-1397 emits a TODO comment).
//
// Design (one CTA per SM, persistent over output tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128 x 64 A tile and
//               a 64 x 256 B tile (128-byte swizzle) into a kStages-deep ring,
//               signalled through mbarriers.  No multicast: each CTA loads its own.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16)
//               straight from shared memory into a 128 x 256 f32 accumulator in
//               tensor memory; two accumulators (512 columns) alternate so the
//               next tile's main loop overlaps this tile's epilogue.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM
//               lanes), narrow, 16-byte global stores.
// B in its row-major [K,N] form is consumed as an MN-major operand, so no
// transpose pass over B is ever made.
//
// Roofline: tensor pipe.  Algorithmic work 2*M*N*K flop per problem.
#pragma once

#include "ptx.cuh"

namespace tsm100 {
namespace gemm_tc {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;                      // 64 x 16-bit = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kABytes = kBM * kBK * 2;       // 16 KiB
constexpr int kBBytes = kBN * kBK * 2;       // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;               // two 256-column accumulators
constexpr int kGroupM = 16;                  // m-blocks per rasterisation band (L2 reuse)

struct alignas(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + sizeof(Barriers) + 1024;  // + alignment slack

struct Params {
  int32_t m, n, k, batch;
  int32_t m_blocks, n_blocks;
  int64_t c_batch_stride;  // elements
  int64_t ldc;             // row pitch of C in elements
  uint32_t* status;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& b, int& mb, int& nb) {
  const int per_batch = p.m_blocks * p.n_blocks;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  const int band_tiles = kGroupM * p.n_blocks;
  const int band = t / band_tiles;
  const int first_m = band * kGroupM;
  const int rows_in_band = min(kGroupM, p.m_blocks - first_m);
  t -= band * band_tiles;
  mb = first_m + t % rows_in_band;
  nb = t / rows_in_band;
}

template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const uint32_t (&acc)[32], int valid);

template <>
__device__ __forceinline__ void store_row_chunk<float>(float* dst, const uint32_t (&acc)[32], int valid) {
  if (valid >= 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = __uint_as_float(acc[i]);
  }
}

template <>
__device__ __forceinline__ void store_row_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&acc)[32],
                                                              int valid) {
  if (valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v;
      v.x = ptx::pack_bf16x2(__uint_as_float(acc[8 * i + 0]), __uint_as_float(acc[8 * i + 1]));
      v.y = ptx::pack_bf16x2(__uint_as_float(acc[8 * i + 2]), __uint_as_float(acc[8 * i + 3]));
      v.z = ptx::pack_bf16x2(__uint_as_float(acc[8 * i + 4]), __uint_as_float(acc[8 * i + 5]));
      v.w = ptx::pack_bf16x2(__uint_as_float(acc[8 * i + 6]), __uint_as_float(acc[8 * i + 7]));
      reinterpret_cast<uint4*>(dst)[i] = v;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(acc[i]));
  }
}

template <>
__device__ __forceinline__ void store_row_chunk<__half>(__half* dst, const uint32_t (&acc)[32], int valid) {
  if (valid >= 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 h = __floats2half2_rn(__uint_as_float(acc[8 * i + 2 * j]), __uint_as_float(acc[8 * i + 2 * j + 1]));
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = __float2half_rn(__uint_as_float(acc[i]));
  }
}

// kBTransposed: B is stored [N,K] (K-major operand); otherwise [K,N] (MN-major).
// kIsBf16: inputs are bf16 (else IEEE f16).
template <typename OutT, bool kBTransposed, bool kIsBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               OutT* __restrict__ c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.batch * p.m_blocks * p.n_blocks;
  const int num_kb = (p.k + kBK - 1) / kBK;
  volatile uint32_t* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&bars->acc_full[a], 1);
      ptx::mbar_init(&bars->acc_empty[a], 4);  // one arrival per epilogue warp
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, mb, nb;
        tile_coords(p, tile, b, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 1)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&bars->full[stage], kStageBytes);
          ptx::tma_load_3d(smem_a + stage * kABytes, &tmap_a, &bars->full[stage], kb * kBK, mb * kBM, b);
          if (kBTransposed) {
            ptx::tma_load_3d(smem_b + stage * kBBytes, &tmap_b, &bars->full[stage], kb * kBK, nb * kBN, b);
          } else {
#pragma unroll
            for (int j = 0; j < kBN / 64; ++j)
              ptx::tma_load_3d(smem_b + stage * kBBytes + j * (64 * kBK * 2), &tmap_b, &bars->full[stage],
                               nb * kBN + j * 64, kb * kBK, b);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(kBM, kBN, false, !kBTransposed, kIsBf16);
      // A: K-major, 8-row groups 1024 B apart.  B: see ptx.cuh for the two forms.
      constexpr uint64_t a_base = ptx::make_smem_desc_base(16, 1024);
      constexpr uint64_t b_base =
          kBTransposed ? ptx::make_smem_desc_base(16, 1024) : ptx::make_smem_desc_base(64 * kBK * 2, 1024);
      constexpr uint32_t a_kstep = kUmmaK * 2;                          // 32 B inside the swizzle row
      constexpr uint32_t b_kstep = kBTransposed ? kUmmaK * 2 : (kUmmaK / 8) * 1024;  // or two 8-row groups
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!ptx::mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2)) break;
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_relaxed(&bars->full[stage], phase, abort_flag, p.status, 3)) {  // relaxed: the data goes straight to the async proxy
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_addr = ptx::smem_u32(smem_a + stage * kABytes);
          const uint32_t b_addr = ptx::smem_u32(smem_b + stage * kBBytes);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            ptx::tcgen05_mma_f16_ss(d_tmem, ptx::smem_desc(a_base, a_addr + kk * a_kstep),
                                    ptx::smem_desc(b_base, b_addr + kk * b_kstep), idesc,
                                    (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::tcgen05_commit(&bars->empty[stage]);  // stage reusable once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::tcgen05_commit(&bars->acc_full[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      int b, mb, nb;
      tile_coords(p, tile, b, mb, nb);
      // tcgen05.ld is warp-collective: leave the loop only as a whole warp.
      const bool ready = ptx::mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 4);
      if (!__all_sync(0xffffffffu, ready)) break;
      ptx::tcgen05_fence_after_thread_sync();
      const int row = mb * kBM + quad * 32 + lane;
      OutT* crow = c + static_cast<int64_t>(b) * p.c_batch_stride + static_cast<int64_t>(row) * p.ldc;
#pragma unroll 1
      for (int cc = 0; cc < kBN / 32; ++cc) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBN + cc * 32, v);
        ptx::tmem_ld_wait();
        const int col = nb * kBN + cc * 32;
        if (row < p.m && col < p.n) store_row_chunk<OutT>(crow + col, v, p.n - col);
      }
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[acc]);
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (*abort_flag != 0u) {
    // A wait gave up: give copies and MMAs already in flight time to land before
    // shared and tensor memory are released.
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) {
    }
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace gemm_tc
}  // namespace tsm100
