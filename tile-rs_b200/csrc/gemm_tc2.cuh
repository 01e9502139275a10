// 16-bit GEMM on CTA pairs: tcgen05.mma.cta_group::2, a 256 x 256 output tile per
// pair of SMs.  Same contract as gemm_tc.cuh (C[b] = A[b] * B[b], f32 accumulate,
// B row-major [K,N] or stored [N,K]); this is the kernel large problems run on.
//
// Why pairs: with one CTA per 128 x 256 tile the tensor core reads 96 B/clk of
// operands from shared memory while TMA writes another 96 B/clk into it, and the
// pipe idles ~18 % of the time.  In a pair each CTA stages only its own 128 rows of
// A and its own 128 columns of B (32 KiB per 64-deep K step instead of 48 KiB);
// the hardware feeds both halves of B to both SMs.  No TMA multicast is involved:
// every CTA loads exactly the bytes it keeps.
//
// Per CTA: warp 0 TMA producer (its halves; completion bytes are counted on the
// LEADER's mbarrier), warp 1 allocates tensor memory and, in the leader CTA only,
// issues the MMAs (M = 256 over the pair, N = 256, K = 16) and multicasts the
// "stage free" / "accumulator ready" commits to both CTAs; warps 2..5 drain this
// CTA's 128 x 256 accumulator half (two accumulators alternate) and report "drained"
// to the leader.  Six 32 KiB stages.
#pragma once

#include "gemm_tc.cuh"

namespace tsm100 {
namespace gemm_tc2 {

constexpr int kPairM = 256;   // rows per pair tile
constexpr int kCtaM = 128;    // rows per CTA
constexpr int kBN = 256;      // columns per pair tile
constexpr int kCtaN = 128;    // columns of B staged by each CTA
constexpr int kBK = 64;
constexpr int kStages = 6;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kABytes = kCtaM * kBK * 2;  // 16 KiB
constexpr int kBBytes = kCtaN * kBK * 2;  // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;  // pair tiles per band: a wave of 74 tiles is 16 x 4.6 tiles; the band's rows of A are re-used from the L2 by the next wave (see the producer)

struct alignas(8) Barriers {
  uint64_t full[kStages];      // used in the leader: both CTAs' bytes of a stage have landed
  uint64_t empty[kStages];     // in each CTA: the MMAs reading the stage have retired
  uint64_t acc_full[2];        // in each CTA: accumulator complete
  uint64_t acc_empty[2];       // used in the leader: 8 epilogue warps of the pair have drained it
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kSmemBytes = kStages * kStageBytes + sizeof(Barriers) + 1024;

using gemm_tc::Params;  // m_blocks / n_blocks count 256 x 256 pair tiles here

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

template <typename OutT, bool kBTransposed, bool kIsBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                OutT* __restrict__ c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
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
      ptx::mbar_init(&bars->acc_empty[a], 8);
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
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int b, mb, nb;
        gemm_tc2::tile_coords(p, tile, b, mb, nb);
        const int row0 = mb * kPairM + static_cast<int>(rank) * kCtaM;
        const int col0 = nb * kBN + static_cast<int>(rank) * kCtaN;
        // Every other wave of tiles walks K backwards.  All pairs sweep K in step, so the band's rows of A a wave
        // touched last are its last K slices; the next wave, which needs the same rows, starts with those and finds
        // them in the L2 still (walking forwards again it would start with the slices touched longest ago).  The
        // wave is counted inside the tile's own problem, so equal problems of a batch are summed in the same order
        // and give the same bits wherever they stand in the batch.
        const bool backward = (((tile % (p.m_blocks * p.n_blocks)) / num_pairs) & 1) != 0;
        for (int kq = 0; kq < num_kb; ++kq) {
          const int kb = backward ? num_kb - 1 - kq : kq;
          if (!ptx::mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 31)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = ptx::mapa_shared(ptx::smem_u32(&bars->full[stage]), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(&bars->full[stage], 2 * kStageBytes);
          ptx::tma_load_3d_pair(smem_a + stage * kABytes, &tmap_a, full_leader, kb * kBK, row0, b);
          if (kBTransposed) {
            ptx::tma_load_3d_pair(smem_b + stage * kBBytes, &tmap_b, full_leader, kb * kBK, col0, b);
          } else {
#pragma unroll
            for (int j = 0; j < kCtaN / 64; ++j)
              ptx::tma_load_3d_pair(smem_b + stage * kBBytes + j * (64 * kBK * 2), &tmap_b, full_leader,
                                    col0 + j * 64, kb * kBK, b);
          }
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
      constexpr uint32_t idesc = ptx::make_idesc_f16(kPairM, kBN, false, !kBTransposed, kIsBf16);
      constexpr uint64_t a_base = ptx::make_smem_desc_base(16, 1024);
      constexpr uint64_t b_base =
          kBTransposed ? ptx::make_smem_desc_base(16, 1024) : ptx::make_smem_desc_base(64 * kBK * 2, 1024);
      constexpr uint32_t a_kstep = kUmmaK * 2;
      constexpr uint32_t b_kstep = kBTransposed ? kUmmaK * 2 : (kUmmaK / 8) * 1024;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!ptx::mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 32)) break;
        ptx::tcgen05_fence_after_thread_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_relaxed(&bars->full[stage], phase, abort_flag, p.status, 33)) {  // relaxed: the data goes straight to the async proxy
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const uint32_t a_addr = ptx::smem_u32(smem_a + stage * kABytes);
          const uint32_t b_addr = ptx::smem_u32(smem_b + stage * kBBytes);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            ptx::tcgen05_mma_f16_ss_pair(d_tmem, ptx::smem_desc(a_base, a_addr + kk * a_kstep),
                                         ptx::smem_desc(b_base, b_addr + kk * b_kstep), idesc,
                                         (kb | kk) != 0 ? 1u : 0u);
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
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quad = warp & 3;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      int b, mb, nb;
      gemm_tc2::tile_coords(p, tile, b, mb, nb);
      const bool ready = ptx::mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 34);
      if (!__all_sync(0xffffffffu, ready)) break;
      ptx::tcgen05_fence_after_thread_sync();
      const int row = mb * kPairM + static_cast<int>(rank) * kCtaM + quad * 32 + lane;
      OutT* crow = c + static_cast<int64_t>(b) * p.c_batch_stride + static_cast<int64_t>(row) * p.ldc;
#pragma unroll 1
      for (int cc = 0; cc < kBN / 32; ++cc) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBN + cc * 32, v);
        ptx::tmem_ld_wait();
        const int col = nb * kBN + cc * 32;
        if (row < p.m && col < p.n) gemm_tc::store_row_chunk<OutT>(crow + col, v, p.n - col);
      }
      ptx::tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&bars->acc_empty[acc]), 0));
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (*abort_flag != 0u) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) {
    }
  }
  ptx::tcgen05_fence_before_thread_sync();
  // Neither CTA may leave while the other can still read its shared memory (the
  // leader's MMAs) or signal its barriers (commits, remote arrivals).
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace gemm_tc2
}  // namespace tsm100
