// Fused attention forward for sm_100a: O = softmax(Q K^T / sqrt(d)) V, flash
// style (the S x S score tile is never written to memory).
//
// Semantics: __tile_attention_f32 (crates/tile_std/src/tile.rs:218-224) as the
// linalg bridge decomposes it — transpose(K), matmul, scale by 1/sqrt(D), row
// softmax, matmul (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1781-1902);
// `causal` applies __tile_causal_mask_f32 (mlir_to_linalg.rs:1191-1244: column >
// row -> -inf) between the scale and the softmax; heads_q > heads_kv is the
// grouped-query form of __tile_attention_gqa_* with kv_head = h / (heads_q /
// heads_kv) (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:1657-1673).  The
// reference has no fused NVIDIA lowering: __tile_attention_f32 is unhandled
// (mlir_to_gpu.rs:1976-1979) and the GQA form recomputes every q.k dot product
// three times per output element (mlir_to_gpu.rs:1624-1711).
//
// Layout: Q,O [batch*heads_q][seq][128], K,V [batch*heads_kv][seq][128], 16-bit.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles A and B.
//   warp 8      TMA producer: Q once, then K_0,K_1,V_0,K_2,V_1,... (128 x 128 tiles,
//               128-byte swizzle) through a 3-deep ring.  No multicast.
//   warp 9      issues every S_g = Q_g K_j^T, warp 10 every O_g += P_g V_j (one thread
//               each), all operands from shared memory (V consumed as an MN-major
//               operand straight from its row-major form).  S and O live in tensor
//               memory (4 x 128 columns).
//   warps 0..3  softmax of tile A, warps 4..7 of tile B: one thread per query
//               row (TMEM lane), so row max and row sum need no shuffles.  A thread
//               reads its whole 128-wide score row into registers and at once hands
//               S_g back to the tensor core ("s_free"), so that the NEXT step's
//               Q_g K^T runs while this step's exponentials are computed; the 16-bit
//               probabilities go to a shared-memory tile (written in the swizzled
//               K-major layout the P V product reads).  A tile's steps are therefore
//               not a serial chain QK -> softmax -> PV -> QK any more: its softmax
//               runs back to back and the tensor core always has the other tile's
//               or the next step's product to do.  The running max is only raised
//               when it grows by more than 2^8 (the accumulator in TMEM is then
//               rescaled).
// Launch order keeps CTAs that share K/V (the query blocks of a head, the heads of
// a KV group) adjacent so that K/V tiles are served from L2.
// Roofline: tensor pipe; 4*seq^2*d flop per head (half of it when causal).
#pragma once

#include "ptx.cuh"

namespace tsm100 {
namespace attn {

constexpr int kD = 128;          // head_dim
constexpr int kBQ = 128;         // query rows per tile (two tiles per CTA)
constexpr int kBKV = 128;        // key/value rows per step
constexpr int kThreads = 384;         // warps 0..3 softmax A, 4..7 softmax B, 8 TMA, 9 QK MMAs, 10 PV MMAs, 11 idle
constexpr int kRegsSoftmax = 224;      // register budget after setmaxnreg (launch: 168 per thread)
constexpr int kRegsOther = 56;
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: any 128 x 128 16-bit tile
constexpr int kHalfBytes = kTileBytes / 2; // one 128-row x 64-column swizzled half
constexpr int kRing = 3;
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr int kPolyPairs = 2;  // of every 8 pairs of exponentials, how many avoid MUFU

struct alignas(8) Barriers {
  uint64_t q_full;
  uint64_t kv_full[kRing];
  uint64_t kv_empty[kRing];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t p_ready[2];
  uint64_t pv_done[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t pv_steps;   // how many KV steps the P V issuer has issued completely (only grows)
};

// Q_A, Q_B, P_A, P_B, ring
constexpr int kSmemBytes = (4 + kRing) * kTileBytes + sizeof(Barriers) + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget of one CTA");

struct Params {
  int32_t seq;
  int32_t heads_q, heads_kv, batch;
  int32_t causal;
  int32_t q_blocks;        // ceil(seq / 256)
  int32_t kv_band;         // causal launch order: KV heads per band (>= 1), see the block index mapping in the kernel
  float scale_log2;        // (1/sqrt(d)) * log2(e)
  uint32_t* status;
  // prefill against a KV cache (kCache kernels only): query row i sits at position q_offset + i of seq_kv
  // filled positions; O is token-major, row and head strides in elements
  int32_t seq_kv, q_offset;
  int64_t o_row_stride, o_head_stride;
};

template <bool kIsBf16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  if (kIsBf16) return ptx::pack_bf16x2(lo, hi);
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <bool kIsBf16>
__device__ __forceinline__ float unpack16_lo(uint32_t w) {
  if (kIsBf16) return __uint_as_float(w << 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
}
template <bool kIsBf16>
__device__ __forceinline__ float unpack16_hi(uint32_t w) {
  if (kIsBf16) return __uint_as_float(w & 0xffff0000u);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

// kCache = false: plain attention, Q, O [batch*heads_q][seq][128], K, V [batch*heads_kv][seq][128] (the tensor
// maps say so).  kCache = true: causal prefill against a KV cache - the tensor maps describe token-major Q and the
// filled part of the caches, query rows are offset by q_offset, O is written with the strides of Params.
template <bool kIsBf16, bool kCache = false>
__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, uint16_t* __restrict__ o, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;                         // 2 tiles
  uint8_t* smem_p = smem + 2 * kTileBytes;        // 2 tiles: the probabilities of tile A and of tile B
  uint8_t* smem_kv = smem + 4 * kTileBytes;       // ring
  Barriers* bars = reinterpret_cast<Barriers*>(smem + (4 + kRing) * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars->abort_flag;

  // blockIdx -> (head, query block).  Heads of a KV group vary fastest.  Non-causal: then the query blocks of that
  // group, then the (batch, KV head) groups.  Causal: a query block's work grows with its position, so within a band
  // of kv_band KV heads (whose K and V fit the L2 together) all heads' heaviest blocks come first, then the next
  // lighter ones, ...: longest-first over 16+ times more blocks than one head has, which is what keeps the SMs evenly
  // loaded when a launch has only a few blocks per SM (a shard of the heads on one of several GPUs).
  const int group = p.heads_q / p.heads_kv;
  const int hg = blockIdx.x % group;
  const int t_rest = blockIdx.x / group;
  int qb_raw, kvh;                           // kvh: flattened (batch, KV head)
  if (p.causal) {
    const int total_kv = static_cast<int>(gridDim.x) / (group * p.q_blocks);
    const int per_band = p.kv_band * p.q_blocks;
    const int band = t_rest / per_band, rem = t_rest - band * per_band;
    const int heads_here = min(p.kv_band, total_kv - band * p.kv_band);  // the last band may be smaller
    qb_raw = rem / heads_here;
    kvh = band * p.kv_band + rem - qb_raw * heads_here;
  } else {
    qb_raw = t_rest % p.q_blocks;
    kvh = t_rest / p.q_blocks;
  }
  const int bh = kvh * group + hg;           // flattened (batch, query head)
  const int qb = p.causal ? (p.q_blocks - 1 - qb_raw) : qb_raw;
  const int q0 = qb * 2 * kBQ;
  const int seq_kv = kCache ? p.seq_kv : p.seq;
  const int q_off = kCache ? p.q_offset : 0;
  const int n_kv_all = (seq_kv + kBKV - 1) / kBKV;
  // number of KV steps each tile needs (causal: up to and including the step of its last row's own position)
  const int n_a = p.causal ? min(n_kv_all, (q0 + kBQ - 1 + q_off) / kBKV + 1) : n_kv_all;
  const int n_b = p.causal ? min(n_kv_all, (q0 + 2 * kBQ - 1 + q_off) / kBKV + 1) : n_kv_all;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      ptx::mbar_init(&bars->kv_full[s], 1);
      ptx::mbar_init(&bars->kv_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      ptx::mbar_init(&bars->s_full[g], 1);
      ptx::mbar_init(&bars->s_free[g], 128);
      ptx::mbar_init(&bars->p_ready[g], 128);
      ptx::mbar_init(&bars->pv_done[g], 1);
    }
    bars->abort_flag = 0;
    bars->pv_steps = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 9) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s = tmem_base;        // S_A at +0, S_B at +128
  const uint32_t tmem_o = tmem_base + 256;  // O_A at +256, O_B at +384

  // The non-softmax warpgroup (warps 8..11) gives most of its registers to the softmax
  // warpgroups; each role branch starts with its own setmaxnreg so that the register
  // budget is unambiguous inside it.
  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    ptx::setmaxnreg_dec<kRegsOther>();
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_q);
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_v);
      ptx::mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          ptx::tma_load_3d(smem_q + g * kTileBytes + c * kHalfBytes, &tmap_q, &bars->q_full, c * 64,
                           q0 + g * kBQ, bh);
      // ring order = the order the tensor core first needs the tiles in: K_0, K_1, V_0, K_2, V_1, ..., K_{n-1}, V_{n-2}, V_{n-1}
      const int total = 2 * n_b;
      for (int idx = 0; idx < total; ++idx) {
        const int slot = idx % kRing;
        const uint32_t phase = (idx / kRing) & 1u;
        if (!ptx::mbar_wait(&bars->kv_empty[slot], phase ^ 1u, abort_flag, p.status, 11)) break;
        ptx::mbar_arrive_expect_tx(&bars->kv_full[slot], kTileBytes);
        // idx 0 -> K_0; then pairs (K_{i+1}, V_i) for i = 0 .. n-2; last -> V_{n-1}
        const bool is_v = idx == total - 1 || (idx >= 2 && (idx & 1) == 0);
        const int step = idx == 0 ? 0 : idx == total - 1 ? n_b - 1 : is_v ? (idx >> 1) - 1 : (idx + 1) >> 1;
        const CUtensorMap* tm = is_v ? &tmap_v : &tmap_k;
        const int row0 = step * kBKV;
#pragma unroll
        for (int c = 0; c < 2; ++c)
          ptx::tma_load_3d(smem_kv + slot * kTileBytes + c * kHalfBytes, tm, &bars->kv_full[slot], c * 64,
                           row0, kvh);
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------ MMA issuers --------------------------------
    // Two issuing warps: warp 9 issues every S_g = Q_g K^T, warp 10 every O_g += P_g V.  One thread cannot
    // feed the tensor core alone here: issuing a 128 x 128 x 16 product costs it about as long as the tensor core
    // needs to execute one (measured ~70 cycles against 64), and every barrier test between batches another
    // 150-200; with both kinds on one thread its loop took 3800 cycles per step for 2048 cycles of tensor work.
    ptx::setmaxnreg_dec<kRegsOther>();
    {  // the whole warp runs the loop (uniform control flow, uniform operands); one elected lane issues
      constexpr uint32_t idesc_qk = ptx::make_idesc_f16(kBQ, kBKV, false, false, kIsBf16);
      constexpr uint32_t idesc_pv = ptx::make_idesc_f16(kBQ, kD, false, true, kIsBf16);
      constexpr uint64_t kmajor = ptx::make_smem_desc_base(16, 1024);
      constexpr uint64_t v_mnmajor = ptx::make_smem_desc_base(kHalfBytes, 1024);

      // Waits that only hand TMA-written shared memory or tensor memory on to the tensor core are relaxed
      // (same async proxy; tensor memory sits behind the tcgen05 fence): an acquiring wait costs the issuing
      // thread about twice as long.  The probabilities are written by ordinary stores, so that wait acquires.
      auto wait_kv = [&](int idx) -> bool {
        const bool r = ptx::mbar_wait_relaxed(&bars->kv_full[idx % kRing], (idx / kRing) & 1u, abort_flag, p.status, 13);
        return __all_sync(0xffffffffu, r);  // the warp stays converged, also when a wait gives up
      };
      // Everything per MMA is reduced to one add on the low word of each descriptor (the start-address
      // field; the high words are constants).
      constexpr uint32_t k_hi = static_cast<uint32_t>(kmajor >> 32), v_hi = static_cast<uint32_t>(v_mnmajor >> 32);
      constexpr uint32_t k_lo_base = static_cast<uint32_t>(kmajor), v_lo_base = static_cast<uint32_t>(v_mnmajor);
      auto desc64 = [](uint32_t hi, uint32_t lo) -> uint64_t { return (static_cast<uint64_t>(hi) << 32) | lo; };
      // ring positions of the tiles (see the producer): K_0, K_1, V_0, K_2, V_1, ..., K_{n-1}, V_{n-2}, V_{n-1}
      auto k_pos = [&](int j) { return j == 0 ? 0 : 2 * j - 1; };
      auto v_pos = [&](int j) { return j == n_b - 1 ? 2 * n_b - 1 : 2 * j + 2; };

      if (warp == 9) {
        // ---- S_g = Q_g K^T, one step ahead of the softmax: both operands K-major, head_dim in two 64-wide halves
        const uint32_t q_lo = k_lo_base | (ptx::smem_u32(smem_q) >> 4);       // + g * (kTileBytes >> 4)
        const uint32_t ring_k_lo = k_lo_base | (ptx::smem_u32(smem_kv) >> 4);  // + slot * (kTileBytes >> 4)
        auto issue_qk = [&](int g, int idx) {
          const uint32_t a_lo = q_lo + g * (kTileBytes >> 4);
          const uint32_t b_lo = ring_k_lo + (idx % kRing) * (kTileBytes >> 4);
          const uint32_t d = tmem_s + g * 128;
          if (ptx::elect_one_sync()) {
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) {
              constexpr int kHalf16 = kHalfBytes >> 4;
              const uint32_t off = (kk >> 2) * kHalf16 + (kk & 3) * 2;  // in 16-byte units
              ptx::tcgen05_mma_f16_ss(d, desc64(k_hi, a_lo + off), desc64(k_hi, b_lo + off), idesc_qk, kk != 0 ? 1u : 0u);
            }
            ptx::tcgen05_commit(&bars->s_full[g]);
          }
          __syncwarp();
        };
        auto wait_s_free = [&](int g, int j) -> bool {  // every softmax thread of tile g holds the scores of step j in registers
          const bool r = ptx::mbar_wait_relaxed(&bars->s_free[g], j & 1u, abort_flag, p.status, 22 + g);
          ptx::tcgen05_fence_after_thread_sync();
          return __all_sync(0xffffffffu, r);
        };
        bool ok = __all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&bars->q_full, 0, abort_flag, p.status, 12));
        ptx::tcgen05_fence_after_thread_sync();
        // Step j of tile g is issued once K_j has landed and the softmax of step j - 1 has read S_g - but not
        // before the P V products of step j - 2 are in the tensor core's queue: those are waited for within the
        // softmax of step j - 1 (they free P_g), while S_g of step j is not needed before that softmax ends.
        // Both tiles finish their softmax at about the same time; without this rule the Q K^T products slip
        // in front of the P V products and every softmax step waits ~600 cycles for its P tile.
        volatile uint32_t* pv_steps = &bars->pv_steps;
        for (int j = 0; j < n_b && ok; ++j) {
          if (j >= 2 && !(ok = __all_sync(0xffffffffu, ptx::wait_counter_ge(pv_steps, static_cast<uint32_t>(j - 1), abort_flag, p.status, 26)))) break;
          if (!(ok = wait_kv(k_pos(j)))) break;
          if (j < n_a) {
            if (j > 0 && !(ok = wait_s_free(0, j - 1))) break;
            issue_qk(0, k_pos(j));
          }
          if (j > 0 && !(ok = wait_s_free(1, j - 1))) break;
          issue_qk(1, k_pos(j));  // last reader of K_j
          if (ptx::elect_one_sync()) ptx::tcgen05_commit(&bars->kv_empty[k_pos(j) % kRing]);
        }
      } else {
        // ---- O_g (+)= P_g V : P K-major from its shared-memory tile (keys in two 64-wide halves), V MN-major
        const uint32_t p_lo = k_lo_base | (ptx::smem_u32(smem_p) >> 4);       // + g * (kTileBytes >> 4)
        const uint32_t ring_v_lo = v_lo_base | (ptx::smem_u32(smem_kv) >> 4);
        auto issue_pv = [&](int g, int idx, bool accumulate) {
          const uint32_t a_lo = p_lo + g * (kTileBytes >> 4);
          const uint32_t b_lo = ring_v_lo + (idx % kRing) * (kTileBytes >> 4);
          const uint32_t d = tmem_o + g * 128;
          if (ptx::elect_one_sync()) {
#pragma unroll
            for (int kk = 0; kk < kBKV / 16; ++kk) {
              constexpr int kHalf16 = kHalfBytes >> 4;
              const uint32_t a_off = (kk >> 2) * kHalf16 + (kk & 3) * 2;
              ptx::tcgen05_mma_f16_ss(d, desc64(k_hi, a_lo + a_off), desc64(v_hi, b_lo + kk * (2048 >> 4)), idesc_pv,
                                      (accumulate || kk != 0) ? 1u : 0u);
            }
            ptx::tcgen05_commit(&bars->pv_done[g]);
          }
          __syncwarp();
        };
        auto wait_p = [&](int g, int j) -> bool {  // the probabilities of step j are in shared memory (ordinary stores, fenced by the writers)
          const bool r = ptx::mbar_wait(&bars->p_ready[g], j & 1u, abort_flag, p.status, 14 + g);
          ptx::tcgen05_fence_after_thread_sync();
          return __all_sync(0xffffffffu, r);
        };
        bool ok = true;
        for (int j = 0; j < n_b && ok; ++j) {
          if (!(ok = wait_kv(v_pos(j)))) break;
          if (j < n_a) {
            if (!(ok = wait_p(0, j))) break;
            issue_pv(0, v_pos(j), j > 0);
          }
          if (!(ok = wait_p(1, j))) break;
          issue_pv(1, v_pos(j), j > 0);  // last reader of V_j
          if (ptx::elect_one_sync()) {
            ptx::tcgen05_commit(&bars->kv_empty[v_pos(j) % kRing]);
            *const_cast<volatile uint32_t*>(&bars->pv_steps) = static_cast<uint32_t>(j + 1);
          }
        }
      }
    }
  } else if (warp == 11) {
    ptx::setmaxnreg_dec<kRegsOther>();
  } else {
    // ------------------------------ softmax / output ---------------------------
    ptx::setmaxnreg_inc<kRegsSoftmax>();
    const int g = warp >> 2;          // 0: tile A, 1: tile B
    const int quad = warp & 3;              // TMEM lanes this warp may touch
    const int r = quad * 32 + lane;         // row inside the tile == TMEM lane
    const int n_g = g == 0 ? n_a : n_b;
    const int qrow = q0 + g * kBQ + r;
    const int limit = p.causal ? min(qrow + q_off, seq_kv - 1) : (seq_kv - 1);  // last visible column
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_s + g * 128 + lane_base;
    const uint32_t to = tmem_o + g * 128 + lane_base;
    const float sl2 = p.scale_log2;
    const uint32_t p_row = ptx::smem_u32(smem_p) + g * kTileBytes + r * 128;  // this row in the first 64-key half of P_g

    float m_used = -INFINITY;  // running max in raw score units
    float l = 0.f;
    bool alive = true;
    for (int j = 0; j < n_g; ++j) {
      bool ready = ptx::mbar_wait(&bars->s_full[g], j & 1u, abort_flag, p.status, 16 + g);
      if (!__all_sync(0xffffffffu, ready)) {
        alive = false;
        break;
      }
      ptx::tcgen05_fence_after_thread_sync();
      const int col0 = j * kBKV;
      const bool masked = col0 + kBKV - 1 > limit;

      // the whole score row of this step, read once
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32b_x32(ts + c * 32, v[c]);
      ptx::tmem_ld_wait();
      // the scores are in registers: S_g goes back to the tensor core for the next step's Q K^T
      ptx::tcgen05_fence_before_thread_sync();
      ptx::mbar_arrive(&bars->s_free[g]);

      float mx = -INFINITY;
      if (masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col0 + c * 32 + i > limit) v[c][i] = 0xff800000u;  // -inf
            mx = fmaxf(mx, __uint_as_float(v[c][i]));
          }
      } else {
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2)  // three-input max: 64 instructions for 128 values
            mx4[(i >> 1) & 3] = ptx::fmax3(mx4[(i >> 1) & 3], __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      const float m_new = fmaxf(m_used, mx);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = (m_new - m_used) * sl2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O_g is rescaled in place, once the previous step's P V has retired (the next one is not issued
          // before this step's probabilities are handed over)
          ready = ptx::mbar_wait(&bars->pv_done[g], (j - 1) & 1u, abort_flag, p.status, 18 + g);
          if (!__all_sync(0xffffffffu, ready)) {
            alive = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const float alpha = need ? ptx::ex2_approx((m_used - m_new) * sl2) : 1.0f;
          if (need) m_used = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            ptx::tmem_ld_32x32b_x32(to + c * 32, ov);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            ptx::tmem_st_32x32b_x32(to + c * 32, ov);
          }
          ptx::tmem_st_wait();
          ptx::tcgen05_fence_before_thread_sync();  // the rescaled O is ordered before the p_ready arrival below
        }
      }

      // probabilities: exp2, round to 16 bit, written to the shared-memory tile P_g in the layout the tensor
      // core reads a K-major operand in: two 64-key halves of 128 rows x 128 bytes, 16-byte chunk c of row r at
      // chunk position c ^ (r & 7) (the 128-byte swizzle).  A warp's 32 rows x 16 bytes cover all banks evenly.
      // Of every 8 pairs, kPolyPairs go through the FMA-pipe polynomial and the rest through
      // MUFU ex2, so that neither pipe alone bounds the exponentials.  The row sum adds the
      // f32 probabilities before they are rounded (packed adds, two per instruction).
      const float ms = m_used * sl2;
      const ptx::f32x2_t sl2x2 = ptx::pack_f32x2(sl2, sl2);
      const ptx::f32x2_t nmsx2 = ptx::pack_f32x2(-ms, -ms);
      ptx::f32x2_t lsum[2] = {0ull, 0ull};  // (+0.0f, +0.0f)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = h2 * 2 + (i >> 4);
          const int e0 = (i & 15) * 2;
          const ptx::f32x2_t t2 = ptx::fma_f32x2(
              ptx::pack_f32x2(__uint_as_float(v[c][e0]), __uint_as_float(v[c][e0 + 1])), sl2x2, nmsx2);
          float p0, p1;
          if ((i & 7) < kPolyPairs) {
            ptx::exp2_poly_x2(t2, p0, p1);
          } else {
            float t0, t1;
            ptx::unpack_f32x2(t2, t0, t1);
            p0 = ptx::ex2_approx(t0);  // 2^(-inf) = 0
            p1 = ptx::ex2_approx(t1);
          }
          pk[i] = pack16x2<kIsBf16>(p0, p1);
          lsum[i & 1] = ptx::add_f32x2(lsum[i & 1], ptx::pack_f32x2(p0, p1));
        }
        if (h2 == 0 && j > 0) {  // P_g is free once the previous step's P V has read it (usually long ago)
          ready = ptx::mbar_wait(&bars->pv_done[g], (j - 1) & 1u, abort_flag, p.status, 24 + g);
          if (!__all_sync(0xffffffffu, ready)) {
            alive = false;
            break;
          }
        }
        const uint32_t prow = p_row + h2 * kHalfBytes;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          ptx::st_shared_v4(prow + ((c ^ (r & 7)) << 4), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      if (!alive) break;
      float l4[4];
      ptx::unpack_f32x2(lsum[0], l4[0], l4[1]);
      ptx::unpack_f32x2(lsum[1], l4[2], l4[3]);
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      ptx::fence_proxy_async_smem();  // the tensor core reads P through the async proxy
      ptx::mbar_arrive(&bars->p_ready[g]);
    }

    if (alive && n_g > 0) {
      bool ready = ptx::mbar_wait(&bars->pv_done[g], (n_g - 1) & 1u, abort_flag, p.status, 20 + g);
      if (__all_sync(0xffffffffu, ready)) {
        ptx::tcgen05_fence_after_thread_sync();
        const float inv = 1.0f / l;
        uint16_t* orow = kCache ? o + bh * p.o_head_stride + qrow * p.o_row_stride
                                : o + (static_cast<int64_t>(bh) * p.seq + qrow) * kD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          ptx::tmem_ld_32x32b_x32(to + c * 32, ov);
          ptx::tmem_ld_wait();
          if (qrow < p.seq) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              uint4 w;
              w.x = pack16x2<kIsBf16>(__uint_as_float(ov[8 * t + 0]) * inv, __uint_as_float(ov[8 * t + 1]) * inv);
              w.y = pack16x2<kIsBf16>(__uint_as_float(ov[8 * t + 2]) * inv, __uint_as_float(ov[8 * t + 3]) * inv);
              w.z = pack16x2<kIsBf16>(__uint_as_float(ov[8 * t + 4]) * inv, __uint_as_float(ov[8 * t + 5]) * inv);
              w.w = pack16x2<kIsBf16>(__uint_as_float(ov[8 * t + 6]) * inv, __uint_as_float(ov[8 * t + 7]) * inv);
              reinterpret_cast<uint4*>(orow + c * 32)[t] = w;
            }
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
  __syncthreads();
  if (warp == 9) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace attn
}  // namespace tsm100
