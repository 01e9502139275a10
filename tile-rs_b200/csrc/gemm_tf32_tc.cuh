// f32 GEMM on the 5th-generation tensor cores (tcgen05, kind::tf32) with f32-grade results.
//
//   C[b][M,N] = A[b][M,K] * B[b]       all f32, row-major; B [K,N] or stored [N,K]
//   __tile_matmul_f32 / __tile_matmul_transposed_f32 (crates/tile_std/src/tile.rs:192-193, :2017-2031);
//   semantics linalg.fill 0 + linalg.matmul (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1345-1393).
//
// One TF32 product keeps 11 significant bits, which cannot meet a 1e-5 bar; three can.  Every operand x is
// split once, by a streaming pass, into hi = tf32(x) (round to nearest) and lo = tf32(x - hi); a product is
// then  lo*hi + hi*lo + hi*hi  on the tensor cores, f32 accumulation in tensor memory; what is dropped (lo*lo,
// the rounding of lo) is below 2^-21 of |a||b|.  The same pass writes B's planes K-major ([N][K]), so the
// contraction kernel sees K-major operands only, whatever layout B came in.
//
// The tensor core rounds its f32 accumulator toward zero at every instruction, so a long K accumulated in one go
// drifts by about 2^-25.6 per instruction, all in one direction (3e-5 of the result at K = 4096).  The K loop is
// therefore cut into chunks of kChunkKb k-blocks: each chunk is accumulated from zero in one of two tensor-memory
// accumulators and then added, round-to-nearest, to running sums that the eight epilogue warps keep in registers
// (128 x 256 tile / 256 threads = 128 sums per thread) while the tensor core works on the next chunk.
//
// Per CTA (one per SM, persistent over 128 x 256 output tiles): warp 0 TMA producer (four planes per 32-deep
// k-block, 96 KiB per stage, two stages, no multicast), warp 1 tensor-memory allocation and MMA issue (12
// instructions of 128 x 256 x 8 per k-block), warps 2..9 chunk drain and output.
// Roofline: tensor pipe at the TF32 rate / 3.  Algorithmic work 2*M*N*K flop per problem.
#pragma once

#include "ptx.cuh"

namespace tsm100 {
namespace gemm_tf32_tc {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 32;                  // 32 x f32 = one 128-byte swizzle row
constexpr int kStages = 2;
constexpr int kUmmaK = 8;                // 32 bytes of K per instruction
constexpr int kChunkKb = 4;              // k-blocks per accumulation chunk: K = 128 per chunk
constexpr int kThreads = 320;            // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int kAPlane = kBM * kBK * 4;   // 16 KiB
constexpr int kBPlane = kBN * kBK * 4;   // 32 KiB
constexpr int kStageBytes = 2 * kAPlane + 2 * kBPlane;  // 96 KiB: A_hi, A_lo, B_hi, B_lo
constexpr int kTmemCols = 512;           // two 256-column accumulators
constexpr int kGroupM = 16;              // m-blocks per rasterisation band (L2 reuse)

struct alignas(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + sizeof(Barriers) + 1024;

struct Params {
  int32_t m, n, k, batch;
  int32_t m_blocks, n_blocks;
  int64_t c_batch_stride;  // elements
  int64_t ldc;             // row pitch of C in elements
  uint32_t* status;
};

// x rounded to the nearest TF32 number (10 explicit mantissa bits; ties away from zero)
__device__ __forceinline__ float tf32_rn(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// ---------------------------------------------------------------------------
// the split pass
// ---------------------------------------------------------------------------
// src [rows][cols] with row pitch ld -> hi, lo [rows][cols] packed.  cols % 4 == 0; one thread per four values.
// blockIdx.y = problem of the batch.
__global__ void __launch_bounds__(256)
split_rows_kernel(const float* __restrict__ src, int64_t ld, int64_t src_batch_stride, float* __restrict__ hi,
                  float* __restrict__ lo, int64_t rows, int32_t cols) {
  const int64_t vec_per_row = cols >> 2;
  const int64_t total = rows * vec_per_row;
  const float* s = src + blockIdx.y * src_batch_stride;
  float* h = hi + blockIdx.y * rows * cols;
  float* l = lo + blockIdx.y * rows * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c4 = (i - r * vec_per_row) << 2;
    const float4 x = *reinterpret_cast<const float4*>(s + r * ld + c4);
    float4 a, b;
    a.x = tf32_rn(x.x), a.y = tf32_rn(x.y), a.z = tf32_rn(x.z), a.w = tf32_rn(x.w);
    b.x = tf32_rn(x.x - a.x), b.y = tf32_rn(x.y - a.y), b.z = tf32_rn(x.z - a.z), b.w = tf32_rn(x.w - a.w);
    *reinterpret_cast<float4*>(h + r * cols + c4) = a;
    *reinterpret_cast<float4*>(l + r * cols + c4) = b;
  }
}

// src [K][N] with row pitch ld -> hi, lo [N][K] packed (transposed), 32 x 32 tiles through shared memory.
// grid (ceil(N/32), ceil(K/32), batch), 256 threads (32 x 8).
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ src, int64_t ld, int64_t src_batch_stride, float* __restrict__ hi,
                       float* __restrict__ lo, int32_t k, int32_t n) {
  __shared__ float tile[32][33];
  const float* s = src + blockIdx.z * src_batch_stride;
  float* h = hi + static_cast<int64_t>(blockIdx.z) * n * k;
  float* l = lo + static_cast<int64_t>(blockIdx.z) * n * k;
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int kk = k0 + ty + 8 * j, nn = n0 + tx;
    tile[ty + 8 * j][tx] = (kk < k && nn < n) ? s[static_cast<int64_t>(kk) * ld + nn] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int nn = n0 + ty + 8 * j, kk = k0 + tx;
    if (nn < n && kk < k) {
      const float x = tile[tx][ty + 8 * j];
      const float a = tf32_rn(x);
      h[static_cast<int64_t>(nn) * k + kk] = a;
      l[static_cast<int64_t>(nn) * k + kk] = tf32_rn(x - a);
    }
  }
}

// ---------------------------------------------------------------------------
// the contraction
// ---------------------------------------------------------------------------
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

// 32-bit instruction descriptor for kind::tf32 with f32 accumulation, both operands K-major.
//   [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format (2 = tf32)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_tf32(uint32_t m, uint32_t n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void tcgen05_mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_tc_kernel(const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo,
                    const __grid_constant__ CUtensorMap tmap_b_hi, const __grid_constant__ CUtensorMap tmap_b_lo,
                    float* __restrict__ c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.batch * p.m_blocks * p.n_blocks;
  const int num_kb = (p.k + kBK - 1) / kBK;
  const int num_chunks = (num_kb + kChunkKb - 1) / kChunkKb;
  volatile uint32_t* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&bars->acc_full[a], 1);
      ptx::mbar_init(&bars->acc_empty[a], 8);  // one arrival per epilogue warp
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
      ptx::prefetch_tensormap(&tmap_a_hi);
      ptx::prefetch_tensormap(&tmap_a_lo);
      ptx::prefetch_tensormap(&tmap_b_hi);
      ptx::prefetch_tensormap(&tmap_b_lo);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, mb, nb;
        tile_coords(p, tile, b, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 41)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + stage * kStageBytes;
          ptx::mbar_arrive_expect_tx(&bars->full[stage], kStageBytes);
          ptx::tma_load_3d(st, &tmap_a_hi, &bars->full[stage], kb * kBK, mb * kBM, b);
          ptx::tma_load_3d(st + kAPlane, &tmap_a_lo, &bars->full[stage], kb * kBK, mb * kBM, b);
          ptx::tma_load_3d(st + 2 * kAPlane, &tmap_b_hi, &bars->full[stage], kb * kBK, nb * kBN, b);
          ptx::tma_load_3d(st + 2 * kAPlane + kBPlane, &tmap_b_lo, &bars->full[stage], kb * kBK, nb * kBN, b);
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
      constexpr uint32_t idesc = make_idesc_tf32(kBM, kBN);
      constexpr uint64_t kmajor = ptx::make_smem_desc_base(16, 1024);  // 8-row groups 1024 B apart
      constexpr uint32_t kstep = kUmmaK * 4;                            // 32 B inside the swizzle row
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t chunk_count = 0;  // chunks issued by this CTA so far: picks the accumulator and its barrier phase
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int ch = 0; ch < num_chunks && ok; ++ch, ++chunk_count) {
          const uint32_t acc = chunk_count & 1u;
          const uint32_t acc_phase = (chunk_count >> 1) & 1u;
          if (!ptx::mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 42)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t d_tmem = tmem_base + acc * kBN;
          const int kb_end = min(num_kb, (ch + 1) * kChunkKb);
          for (int kb = ch * kChunkKb; kb < kb_end; ++kb) {
            if (!ptx::mbar_wait_relaxed(&bars->full[stage], phase, abort_flag, p.status, 43)) {
              ok = false;
              break;
            }
            ptx::tcgen05_fence_after_thread_sync();
            const uint32_t a_hi = ptx::smem_u32(smem + stage * kStageBytes);
            const uint32_t a_lo = a_hi + kAPlane;
            const uint32_t b_hi = a_hi + 2 * kAPlane;
            const uint32_t b_lo = b_hi + kBPlane;
            const bool first_kb = kb == ch * kChunkKb;
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
              const uint32_t off = kk * kstep;
              // the two small products first, then the large one
              tcgen05_mma_tf32_ss(d_tmem, ptx::smem_desc(kmajor, a_lo + off), ptx::smem_desc(kmajor, b_hi + off), idesc,
                                  (first_kb && kk == 0) ? 0u : 1u);
              tcgen05_mma_tf32_ss(d_tmem, ptx::smem_desc(kmajor, a_hi + off), ptx::smem_desc(kmajor, b_lo + off), idesc, 1u);
              tcgen05_mma_tf32_ss(d_tmem, ptx::smem_desc(kmajor, a_hi + off), ptx::smem_desc(kmajor, b_hi + off), idesc, 1u);
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
    }
  } else {
    // ------------------------------ chunk drain and output ----------------------
    const int quad = warp & 3;            // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int half = (warp - 2) >> 2;     // which 128 columns of the 256-column accumulator
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + half * 128;
    uint32_t chunk_count = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      int b, mb, nb;
      tile_coords(p, tile, b, mb, nb);
      float sum[4][32];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) sum[cc][i] = 0.f;
      for (int ch = 0; ch < num_chunks; ++ch, ++chunk_count) {
        const uint32_t acc = chunk_count & 1u;
        const uint32_t acc_phase = (chunk_count >> 1) & 1u;
        // tcgen05.ld is warp-collective: leave the loop only as a whole warp
        const bool ready = ptx::mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 44);
        if (!__all_sync(0xffffffffu, ready)) {
          alive = false;
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(lane_addr + acc * kBN + cc * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sum[cc][i] += __uint_as_float(v[i]);  // round-to-nearest add of the chunk
        }
        ptx::tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[acc]);
      }
      if (!alive) break;
      const int row = mb * kBM + quad * 32 + lane;
      if (row < p.m) {
        float* crow = c + static_cast<int64_t>(b) * p.c_batch_stride + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int col = nb * kBN + half * 128 + cc * 32;
          if (col + 32 <= p.n) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(crow + col)[i] = make_float4(sum[cc][4 * i], sum[cc][4 * i + 1], sum[cc][4 * i + 2], sum[cc][4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.n) crow[col + i] = sum[cc][i];
          }
        }
      }
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

// ---------------------------------------------------------------------------
// the contraction on CTA pairs (tcgen05 cta_group::2): a 256 x 256 output tile per pair of SMs
// ---------------------------------------------------------------------------
// With hi and lo planes a single CTA's stage is 96 KiB: two stages fit, and the loads of a stage have one
// stage of MMA time to arrive (measured: tensor pipe 75 % busy).  In a pair each CTA stages its own 128 rows of
// A and its own 128 columns of B (64 KiB per k-block, three stages), the hardware feeds both halves of B to both
// SMs, and the leader's thread issues for both.  No TMA multicast: every CTA loads exactly the bytes it keeps,
// completion bytes counted on the leader's mbarrier.  Chunked accumulation as above; each CTA's eight epilogue
// warps keep the running sums of its own 128 x 256 half.
namespace pair {
constexpr int kPairM = 256;
constexpr int kCtaM = 128;
constexpr int kCtaN = 128;             // columns of B staged by each CTA
constexpr int kStages = 3;
constexpr int kPlane = kCtaM * kBK * 4;            // 16 KiB: every plane a CTA stages
constexpr int kStageBytes = 4 * kPlane;            // A_hi, A_lo, B_hi, B_lo
constexpr int kGroupM = 8;             // pair tiles per band

struct alignas(8) Barriers {
  uint64_t full[kStages];      // used in the leader: both CTAs' bytes of a stage have landed
  uint64_t empty[kStages];     // in each CTA: the MMAs reading the stage have retired
  uint64_t acc_full[2];        // in each CTA: chunk accumulator complete
  uint64_t acc_empty[2];       // used in the leader: 16 epilogue warps of the pair have drained it
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + sizeof(Barriers) + 1024;

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

__device__ __forceinline__ void tcgen05_mma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// m_blocks / n_blocks of Params count 256 x 256 pair tiles here.
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo,
                     const __grid_constant__ CUtensorMap tmap_b_hi, const __grid_constant__ CUtensorMap tmap_b_lo,
                     float* __restrict__ c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.batch * p.m_blocks * p.n_blocks;
  const int num_kb = (p.k + kBK - 1) / kBK;
  const int num_chunks = (num_kb + kChunkKb - 1) / kChunkKb;
  volatile uint32_t* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&bars->acc_full[a], 1);
      ptx::mbar_init(&bars->acc_empty[a], 16);  // 8 epilogue warps in each CTA of the pair
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish_alloc_permit_pair();
  }
  ptx::tcgen05_fence_before_thread_sync();
  ptx::cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a_hi);
      ptx::prefetch_tensormap(&tmap_a_lo);
      ptx::prefetch_tensormap(&tmap_b_hi);
      ptx::prefetch_tensormap(&tmap_b_lo);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        int b, mb, nb;
        pair::tile_coords(p, tile, b, mb, nb);
        const int row0 = mb * kPairM + static_cast<int>(rank) * kCtaM;
        const int col0 = nb * kBN + static_cast<int>(rank) * kCtaN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 45)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = ptx::mapa_shared(ptx::smem_u32(&bars->full[stage]), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(&bars->full[stage], 2 * kStageBytes);
          uint8_t* st = smem + stage * kStageBytes;
          ptx::tma_load_3d_pair(st, &tmap_a_hi, full_leader, kb * kBK, row0, b);
          ptx::tma_load_3d_pair(st + kPlane, &tmap_a_lo, full_leader, kb * kBK, row0, b);
          ptx::tma_load_3d_pair(st + 2 * kPlane, &tmap_b_hi, full_leader, kb * kBK, col0, b);
          ptx::tma_load_3d_pair(st + 3 * kPlane, &tmap_b_lo, full_leader, kb * kBK, col0, b);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_tf32(kPairM, kBN);
      constexpr uint64_t kmajor = ptx::make_smem_desc_base(16, 1024);
      constexpr uint32_t kstep = kUmmaK * 4;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t chunk_count = 0;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        for (int ch = 0; ch < num_chunks && ok; ++ch, ++chunk_count) {
          const uint32_t acc = chunk_count & 1u;
          const uint32_t acc_phase = (chunk_count >> 1) & 1u;
          if (!ptx::mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 46)) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t d_tmem = tmem_base + acc * kBN;
          const int kb_end = min(num_kb, (ch + 1) * kChunkKb);
          for (int kb = ch * kChunkKb; kb < kb_end; ++kb) {
            if (!ptx::mbar_wait_relaxed(&bars->full[stage], phase, abort_flag, p.status, 47)) {
              ok = false;
              break;
            }
            ptx::tcgen05_fence_after_thread_sync();
            const uint32_t a_hi = ptx::smem_u32(smem + stage * kStageBytes);
            const uint32_t a_lo = a_hi + kPlane, b_hi = a_hi + 2 * kPlane, b_lo = a_hi + 3 * kPlane;
            const bool first_kb = kb == ch * kChunkKb;
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
              const uint32_t off = kk * kstep;
              tcgen05_mma_tf32_ss_pair(d_tmem, ptx::smem_desc(kmajor, a_lo + off), ptx::smem_desc(kmajor, b_hi + off), idesc,
                                       (first_kb && kk == 0) ? 0u : 1u);
              tcgen05_mma_tf32_ss_pair(d_tmem, ptx::smem_desc(kmajor, a_hi + off), ptx::smem_desc(kmajor, b_lo + off), idesc, 1u);
              tcgen05_mma_tf32_ss_pair(d_tmem, ptx::smem_desc(kmajor, a_hi + off), ptx::smem_desc(kmajor, b_hi + off), idesc, 1u);
            }
            ptx::tcgen05_commit_pair(&bars->empty[stage], 3);  // frees the stage in both CTAs
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) ptx::tcgen05_commit_pair(&bars->acc_full[acc], 3);
        }
      }
    }
  } else {
    // ------------------------------ chunk drain and output (both CTAs) ----------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + half * 128;
    uint32_t chunk_count = 0;
    bool alive = true;
    for (int tile = pair_id; tile < num_tiles && alive; tile += num_pairs) {
      int b, mb, nb;
      pair::tile_coords(p, tile, b, mb, nb);
      float sum[4][32];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) sum[cc][i] = 0.f;
      for (int ch = 0; ch < num_chunks; ++ch, ++chunk_count) {
        const uint32_t acc = chunk_count & 1u;
        const uint32_t acc_phase = (chunk_count >> 1) & 1u;
        const bool ready = ptx::mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 48);
        if (!__all_sync(0xffffffffu, ready)) {
          alive = false;
          break;
        }
        ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(lane_addr + acc * kBN + cc * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sum[cc][i] += __uint_as_float(v[i]);
        }
        ptx::tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&bars->acc_empty[acc]), 0));
      }
      if (!alive) break;
      const int row = mb * kPairM + static_cast<int>(rank) * kCtaM + quad * 32 + lane;
      if (row < p.m) {
        float* crow = c + static_cast<int64_t>(b) * p.c_batch_stride + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int col = nb * kBN + half * 128 + cc * 32;
          if (col + 32 <= p.n) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(crow + col)[i] = make_float4(sum[cc][4 * i], sum[cc][4 * i + 1], sum[cc][4 * i + 2], sum[cc][4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.n) crow[col + i] = sum[cc][i];
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (*abort_flag != 0u) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) {
    }
  }
  ptx::tcgen05_fence_before_thread_sync();
  // Neither CTA may leave while the other can still read its shared memory (the leader's MMAs) or signal its barriers.
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}
}  // namespace pair

}  // namespace gemm_tf32_tc
}  // namespace tsm100
