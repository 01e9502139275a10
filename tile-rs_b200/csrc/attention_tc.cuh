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
// Persistent: one CTA per SM walks a static list of 256-row query blocks.  A block is
// two 128-row tiles A and B that take turns on the tensor core while the other is in
// its softmax; the K/V ring, the barrier phases and tensor memory run on from one
// block to the next, so the next block's Q/K/V arrive and its first score tile is
// computed while the softmax warps still write the previous block's output.
//   warp 8      TMA producer: Q once, then K_0,V_0,K_1,V_1,... (128 x 128 tiles,
//               128-byte swizzle) through a 5-deep ring.  No multicast.
//   warp 9      MMA issuer (one thread): S_g = Q_g K_j^T (both operands from shared
//               memory) and O_g += P_g V_j with P read from TENSOR MEMORY and V
//               consumed as an MN-major operand straight from its row-major form.
//               S and O live in tensor memory (4 x 128 columns).
//   warps 0..3  softmax of tile A, warps 4..7 of tile B: one thread per query
//               row (TMEM lane), so row max and row sum need no shuffles.  A thread
//               reads its whole 128-wide score row once, and writes the 16-bit
//               probabilities back over the first 64 columns of the same row, where
//               the PV product picks them up.  The running max is only raised when
//               it grows by more than 2^8 (the accumulator in TMEM is then rescaled).
// The item order keeps CTAs that share K/V (the query blocks of a head, the heads of
// a KV group) adjacent so that K/V tiles are served from L2.
// Roofline: tensor pipe; 4*seq^2*d flop per head (half of it when causal).
#pragma once

#include "ptx.cuh"

namespace tsm100 {
namespace attn {

constexpr int kD = 128;          // head_dim
constexpr int kBQ = 128;         // query rows per tile (two tiles per CTA)
constexpr int kBKV = 128;        // key/value rows per K/V tile in shared memory
constexpr int kHalfKV = 64;      // key/value rows per half-step (one score buffer)
constexpr int kSoftmaxWarps = 16;     // per tile 8: two threads per query row, 32 of a half-step's 64 keys each
constexpr int kWarpTma = 16, kWarpMmaA = 17, kWarpMmaB = 18;
constexpr int kThreads = 640;         // warps 0..7 softmax A, 8..15 softmax B, 16 TMA, 17/18 MMA issuers, 19 idle
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KiB: any 128 x 128 16-bit tile
constexpr int kHalfBytes = kTileBytes / 2; // one 128-row x 64-column swizzled half
constexpr int kRing = 5;
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef TSM100_POLY_PAIRS
#define TSM100_POLY_PAIRS 2
#endif
constexpr int kPolyPairs = TSM100_POLY_PAIRS;  // of every 8 pairs of exponentials, how many avoid MUFU

struct alignas(8) Barriers {
  uint64_t q_full;
  uint64_t q_empty[2];         // per tile: its issuer has no MMA reading Q in flight
  uint64_t kv_full[kRing];
  uint64_t kv_empty[2][kRing];  // per tile: its issuer has no MMA reading the slot in flight
  uint64_t s_full[2][2];   // [tile][score buffer]
  uint64_t p_ready[2][2];
  uint64_t pv_done[2][2];  // [tile][half-step parity]: the PV product of that half-step has retired
  uint32_t tmem_base;
  uint32_t abort_flag;
  int16_t row_max[2][2][2][kBQ];  // [half-step parity][tile][column half][row]: that half's maximum, whole log2 units
};

// Q_A, Q_B, ring
// No slack for aligning the base: the kernel checks that the dynamic shared memory window
// starts on a 1024-byte boundary (the 128-byte swizzle needs it) and reports kStatusSmemLayout if not.
constexpr int kSmemBytes = (2 + kRing) * kTileBytes + sizeof(Barriers);
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

struct Params {
  int32_t seq;
  int32_t heads_q, heads_kv, batch;
  int32_t causal;
  int32_t q_blocks;        // ceil(seq / 256)
  int32_t slots;           // work items per head: q_blocks, or ceil(q_blocks / 2) pairs when causal
  int32_t work_items;      // batch * heads_q * slots
  float scale_log2;        // (1/sqrt(d)) * log2(e)
  uint32_t* status;
};

#ifdef TSM100_TRACE
// Development aid (never compiled into the library): per-step clock stamps of CTA 0.
__device__ long long g_attn_trace[5 * 64 * 8];
#define TSM_TRACE(role, j, slot)                                                                  \
  do {                                                                                            \
    if (blockIdx.x == 0 && (j) < 40) g_attn_trace[((role) * 64 + (j)) * 8 + (slot)] = clock64(); \
  } while (0)
// per query block (rows 40..63 of each role): coarse stamps at the block boundaries
#define TSM_TRACE_BLOCK(role, blk, slot)                                                                       \
  do {                                                                                                         \
    if (blockIdx.x == 0 && (blk) < 24) g_attn_trace[((role) * 64 + 40 + (blk)) * 8 + (slot)] = clock64(); \
  } while (0)
#else
#define TSM_TRACE(role, j, slot) \
  do {                           \
  } while (0)
#define TSM_TRACE_BLOCK(role, blk, slot) \
  do {                                   \
  } while (0)
#endif

// One 256-row query block of one head.
struct Work {
  int bh;        // flattened (batch, query head)
  int kvh;       // flattened (batch, KV head)
  int q0;        // first query row
  int n_a, n_b;  // KV steps of tile A / tile B (causal: up to and including the diagonal step)
};

// The CTAs share a static list of work items: item w -> (head, slot) with the heads of a KV
// group varying fastest, then the slots of that group, then the (batch, KV head) groups, so
// that CTAs running at the same time read the same K/V from L2.  A CTA takes items
// blockIdx.x, blockIdx.x + gridDim.x, ...  Non-causal: a slot is one query block.  Causal:
// a slot is the PAIR of query blocks (q_blocks-1-s, s), whose KV steps add up to the same
// number for every s, so the static assignment is balanced without a work counter.
__device__ __forceinline__ bool decode_work(const Params& p, int w, int sub, Work& wk) {
  const int group = p.heads_q / p.heads_kv;
  const int hg = w % group;
  const int rest = w / group;
  const int slot = rest % p.slots;
  wk.kvh = rest / p.slots;
  wk.bh = wk.kvh * group + hg;
  int qb = slot;
  if (p.causal) {
    const int heavy = p.q_blocks - 1 - slot;
    if (sub == 0) {
      qb = heavy;
    } else if (heavy == slot) {
      return false;  // odd number of query blocks: the middle one has no partner
    }
  }
  wk.q0 = qb * 2 * kBQ;
  const int n_kv_all = (p.seq + kBKV - 1) / kBKV;
  wk.n_a = p.causal ? min(n_kv_all, wk.q0 / kBKV + 1) : n_kv_all;
  wk.n_b = p.causal ? min(n_kv_all, wk.q0 / kBKV + 2) : n_kv_all;
  return true;
}

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

template <bool kIsBf16>
__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, uint16_t* __restrict__ o, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0u) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0) atomicCAS(p.status, ptx::kStatusOk, ptx::kStatusSmemLayout);
    return;
  }
  uint8_t* smem_q = smem;                         // 2 tiles
  uint8_t* smem_kv = smem + 2 * kTileBytes;       // ring
  Barriers* bars = reinterpret_cast<Barriers*>(smem + (2 + kRing) * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int n_sub = p.causal ? 2 : 1;  // query blocks per work item

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    ptx::mbar_init(&bars->q_empty[0], 1);
    ptx::mbar_init(&bars->q_empty[1], 1);
    for (int s = 0; s < kRing; ++s) {
      ptx::mbar_init(&bars->kv_full[s], 1);
      ptx::mbar_init(&bars->kv_empty[0][s], 1);
      ptx::mbar_init(&bars->kv_empty[1][s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      for (int b = 0; b < 2; ++b) {
        ptx::mbar_init(&bars->s_full[g][b], 1);
        ptx::mbar_init(&bars->p_ready[g][b], 256);
        ptx::mbar_init(&bars->pv_done[g][b], 1);
      }
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kWarpMmaA) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // S_A buffers at +0 / +64, S_B buffers at +128 / +192 (64 columns = one half-step each);
  // the packed probabilities of a half-step overlay the first 32 columns of its score buffer
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 256;  // O_A at +256, O_B at +384

  // The non-softmax warpgroup (warps 8..11) gives most of its registers to the softmax
  // warpgroups; each role branch starts with its own setmaxnreg so that the register
  // budget is unambiguous inside it.
  if (warp == kWarpTma) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_q);
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_v);
      uint32_t ring_pos = 0;  // K/V tiles loaded so far (the ring runs on across query blocks)
      uint32_t blocks = 0;    // query blocks started so far
      bool ok = true;
      for (int w = blockIdx.x; w < p.work_items && ok; w += gridDim.x) {
        for (int sub = 0; sub < n_sub && ok; ++sub) {
          Work wk;
          if (!decode_work(p, w, sub, wk)) continue;
          // Q of the previous block is free once its last QK product has retired
          if (!ptx::mbar_wait(&bars->q_empty[0], (blocks & 1u) ^ 1u, abort_flag, p.status, 10) ||
              !ptx::mbar_wait(&bars->q_empty[1], (blocks & 1u) ^ 1u, abort_flag, p.status, 10)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
#pragma unroll
          for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int c = 0; c < 2; ++c)
              ptx::tma_load_3d(smem_q + g * kTileBytes + c * kHalfBytes, &tmap_q, &bars->q_full, c * 64,
                               wk.q0 + g * kBQ, wk.bh);
          const int total = 2 * wk.n_b;  // K_0, V_0, K_1, V_1, ...
          for (int idx = 0; idx < total; ++idx) {
            const uint32_t pos = ring_pos + idx;
            const uint32_t slot = pos % kRing;
            const uint32_t phase = (pos / kRing) & 1u;
            TSM_TRACE(3, idx, 0);
            if (!ptx::mbar_wait(&bars->kv_empty[0][slot], phase ^ 1u, abort_flag, p.status, 11) ||
                !ptx::mbar_wait(&bars->kv_empty[1][slot], phase ^ 1u, abort_flag, p.status, 11)) {
              ok = false;
              break;
            }
            TSM_TRACE(3, idx, 1);
            ptx::mbar_arrive_expect_tx(&bars->kv_full[slot], kTileBytes);
            const CUtensorMap* tm = (idx & 1) ? &tmap_v : &tmap_k;
            const int row0 = (idx >> 1) * kBKV;
#pragma unroll
            for (int c = 0; c < 2; ++c)
              ptx::tma_load_3d(smem_kv + slot * kTileBytes + c * kHalfBytes, tm, &bars->kv_full[slot], c * 64,
                               row0, wk.kvh);
            TSM_TRACE(3, idx, 2);
          }
          ring_pos += total;
          ++blocks;
        }
      }
    }
  } else if (warp == kWarpMmaA || warp == kWarpMmaB) {
    // ------------------------------ MMA issuers -------------------------------
    // One warp per tile (warp 9: A, warp 10: B).  Issuing an MMA costs a thread about 40
    // cycles and every barrier test 70 to 300, which for 64-key half-steps is more than
    // one thread can do in the time the tensor core needs for both tiles.  The whole warp
    // runs the loop (uniform control flow, uniform operands); one elected lane issues.
    const int g = warp - kWarpMmaA;
    {
      constexpr uint32_t idesc_qk = ptx::make_idesc_f16(kBQ, kHalfKV, false, false, kIsBf16);
      constexpr uint32_t idesc_pv = ptx::make_idesc_f16(kBQ, kD, false, true, kIsBf16);
      constexpr uint64_t kmajor = ptx::make_smem_desc_base(16, 1024);
      constexpr uint64_t v_mnmajor = ptx::make_smem_desc_base(kHalfBytes, 1024);
      bool ok = true;
      uint32_t ring_base = 0;  // ring position of this query block's K_0
      uint32_t blocks = 0;     // query blocks started so far
      uint32_t done = 0;       // half-steps this tile has been through (barrier phases run on)

      // The issuing thread's waits are relaxed: it only hands TMA-written shared memory to
      // the tensor core (same async proxy), and tensor memory behind the tcgen05 fence; an
      // acquiring wait costs this thread (and so the tensor pipe) about twice as long.
      int kv_seen = 0;  // K/V tiles of this block (K_0, V_0, K_1, ...) known to have landed
      auto need_kv = [&](int idx) -> bool {
        bool r = true;
#ifdef TSM100_DEBUG_NO_KV_WAIT
        if (idx > 0) return true;  // development aid (results may be wrong): what do these waits cost the issuer?
#endif
        while (kv_seen <= idx && r) {  // tiles land in ring order
          const uint32_t pos = ring_base + kv_seen;
          r = ptx::mbar_wait_relaxed(&bars->kv_full[pos % kRing], (pos / kRing) & 1u, abort_flag, p.status, 13);
          r = __all_sync(0xffffffffu, r);  // the warp stays converged, also when a wait gives up
          ++kv_seen;
        }
        return r;
      };
      // Everything per MMA is one add on the low word of a descriptor (the start-address
      // field, in 16-byte units); the high words are constants.
      constexpr uint32_t k_hi = static_cast<uint32_t>(kmajor >> 32), v_hi = static_cast<uint32_t>(v_mnmajor >> 32);
      constexpr uint32_t k_lo_base = static_cast<uint32_t>(kmajor), v_lo_base = static_cast<uint32_t>(v_mnmajor);
      const uint32_t q_lo = (k_lo_base | (ptx::smem_u32(smem_q) >> 4)) + g * (kTileBytes >> 4);
      const uint32_t ring_k_lo = k_lo_base | (ptx::smem_u32(smem_kv) >> 4);  // + slot * (kTileBytes >> 4)
      const uint32_t ring_v_lo = v_lo_base | (ptx::smem_u32(smem_kv) >> 4);
      const uint32_t s_tmem = tmem_s + g * 128, o_tmem = tmem_o + g * 128;
      auto desc64 = [](uint32_t hi, uint32_t lo) -> uint64_t { return (static_cast<uint64_t>(hi) << 32) | lo; };
      // Half-step i covers key rows [64 i, 64 i + 64): half (i & 1) of K/V tile i / 2, score
      // buffer (i & 1) of the tile.
      // S[i & 1] = Q K^T : both operands K-major in shared memory, 8 MMAs of 128 x 64 x 16
      auto issue_qk = [&](int i) {
        const uint32_t b_lo = ring_k_lo + ((ring_base + 2 * (i >> 1)) % kRing) * (kTileBytes >> 4) +
                              (i & 1) * ((kHalfKV * 128) >> 4);  // 64 rows of 128 swizzled bytes
        const uint32_t d = s_tmem + (i & 1) * kHalfKV;
        if (ptx::elect_one_sync()) {
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            constexpr int kHalf16 = kHalfBytes >> 4;
            const uint32_t off = (kk >> 2) * kHalf16 + (kk & 3) * 2;  // in 16-byte units
            ptx::tcgen05_mma_f16_ss(d, desc64(k_hi, q_lo + off), desc64(k_hi, b_lo + off), idesc_qk, kk != 0 ? 1u : 0u);
          }
          ptx::tcgen05_commit(&bars->s_full[g][i & 1]);
        }
        __syncwarp();
      };
      // O (+)= P[i & 1] V : P from tensor memory (16 keys = 8 columns per MMA), V MN-major
      auto issue_pv = [&](int i) {
        const uint32_t b_lo = ring_v_lo + ((ring_base + 2 * (i >> 1) + 1) % kRing) * (kTileBytes >> 4) +
                              (i & 1) * ((kHalfKV / 16) * (2048 >> 4));
        const uint32_t a = s_tmem + (i & 1) * kHalfKV;
        if (ptx::elect_one_sync()) {
          ptx::tcgen05_mma_f16_ts(o_tmem, a, desc64(v_hi, b_lo), idesc_pv, i > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < kHalfKV / 16; ++kk)
            ptx::tcgen05_mma_f16_ts(o_tmem, a + kk * 8, desc64(v_hi, b_lo + kk * (2048 >> 4)), idesc_pv, 1u);
          ptx::tcgen05_commit(&bars->pv_done[g][i & 1]);
        }
        __syncwarp();
      };
      auto wait_p = [&](int i) -> bool {
        const uint32_t use = (done + i) >> 1;  // how often this buffer has been used before
        const bool r = ptx::mbar_wait_relaxed(&bars->p_ready[g][i & 1], use & 1u, abort_flag, p.status, 14 + g);
        ptx::tcgen05_fence_after_thread_sync();
        return __all_sync(0xffffffffu, r);
      };
      // This tile's share of "slot free" (the barrier counts both tiles): arrives once
      // everything this thread has issued so far has retired.
      auto free_slot = [&](int idx) {
        if (ptx::elect_one_sync()) ptx::tcgen05_commit(&bars->kv_empty[g][(ring_base + idx) % kRing]);
      };

      for (int w = blockIdx.x; w < p.work_items && ok; w += gridDim.x) {
        for (int sub = 0; sub < n_sub && ok; ++sub) {
          Work wk;
          if (!decode_work(p, w, sub, wk)) continue;
          const int n_g = 2 * (g == 0 ? wk.n_a : wk.n_b);  // half-steps of this tile
          const int nb = 2 * wk.n_b;                       // half-steps the K/V stream is loaded for
          kv_seen = 0;
          TSM_TRACE_BLOCK(1 + g * 3, blocks, 0);
          ok = __all_sync(0xffffffffu, ptx::mbar_wait_relaxed(&bars->q_full, blocks & 1u, abort_flag, p.status, 12));
          if (!ok) break;
          ptx::tcgen05_fence_after_thread_sync();
          TSM_TRACE_BLOCK(1 + g * 3, blocks, 1);
          // The tile has two score buffers, so QK(i+1) is issued BEFORE the wait for the
          // probabilities of half-step i: the tensor core fills the other buffer while the
          // softmax warps work, and they never wait for a score tile in steady state.
          // QK(i+2) overwrites the buffer P(i) is read from; it follows PV(i) in this thread's
          // in-order stream.  The first PV of a block overwrites O only after the softmax
          // warps, which drained O before they produced that P, have said so.
          if (!(ok = need_kv(0))) break;
          issue_qk(0);
          for (int i = 0; i < n_g && ok; ++i) {
            const int k_next = 2 * ((i + 1) >> 1), v_idx = 2 * (i >> 1) + 1;
            TSM_TRACE(1 + g * 3, i, 0);
            if (i + 1 < n_g) {
              if (!(ok = need_kv(k_next))) break;
              TSM_TRACE(1 + g * 3, i, 1);
              issue_qk(i + 1);
              if ((i + 1) & 1) free_slot(k_next);  // second half of K_j: this tile is done with it
            }
            if (i + 1 == n_g - 1) {
              if (ptx::elect_one_sync()) ptx::tcgen05_commit(&bars->q_empty[g]);  // this tile's last use of Q
            }
            TSM_TRACE(1 + g * 3, i, 2);
            if (!(ok = need_kv(v_idx))) break;
            TSM_TRACE(1 + g * 3, i, 3);
            if (!(ok = wait_p(i))) break;
            TSM_TRACE(1 + g * 3, i, 4);
            issue_pv(i);
            if (i & 1) free_slot(v_idx);  // second half of V_j
            TSM_TRACE(1 + g * 3, i, 5);
          }
          if (!ok) break;
          // causal: tile A stops one K/V pair before tile B; it still owes the ring its share
          // of "slot free" for those tiles (after they have landed, so that the arrival
          // counts for the right phase of the slot)
          for (int idx = n_g; idx < nb && ok; ++idx) {
            if (!(ok = need_kv(idx))) break;
            free_slot(idx);
          }
          if (!ok) break;
          TSM_TRACE_BLOCK(1 + g * 3, blocks, 3);
          ring_base += nb;  // 2 tiles per 128-row step = one per half-step
          done += n_g;
          ++blocks;
        }
      }
    }
  } else if (warp < kSoftmaxWarps) {
    // ------------------------------ softmax / output ---------------------------
    // Two threads per query row: thread (row, h) owns keys [32 h, 32 h + 32) of every
    // half-step and output columns [64 h, 64 h + 64).  Four such warps share a scheduler,
    // which hides the latencies of tensor-memory loads, barriers and the exp pipeline.
    const int g = warp >> 3;          // 0: tile A, 1: tile B
    const int h = (warp >> 2) & 1;    // column half
    const int quad = warp & 3;        // TMEM lanes this warp may touch
    const int r = quad * 32 + lane;   // row inside the tile == TMEM lane
    const uint32_t pair_bar = 1 + g * 4 + quad;  // named barrier of the two warps that share these rows
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_s + g * 128 + lane_base;
    const uint32_t to = tmem_o + g * 128 + lane_base + h * 64;
    const float sl2 = p.scale_log2;
    const bool tracer = (threadIdx.x & 255) == 0;
    // row_max[parity][g][h][r]; the other parity's entry is kBQ * 4 further on
    int16_t* my_max = &bars->row_max[0][g][h][r];
    const int16_t* other_max = &bars->row_max[0][g][h ^ 1][r];
    bool alive = true;
    uint32_t done = 0;   // half-steps this tile has been through (barrier phases run on across query blocks)
    int blk = 0;         // query blocks so far (trace builds only)

    for (int w = blockIdx.x; w < p.work_items && alive; w += gridDim.x) {
    for (int sub = 0; sub < n_sub && alive; ++sub) {
    Work wk;
    if (!decode_work(p, w, sub, wk)) continue;
    const int n_g = 2 * (g == 0 ? wk.n_a : wk.n_b);  // half-steps of 64 keys
    const int bh = wk.bh;
    const int qrow = wk.q0 + g * kBQ + r;
    const int limit = p.causal ? min(qrow, p.seq - 1) : (p.seq - 1);  // last visible column
    // The running maximum is kept in whole log2 units (rounded up), so that the two threads
    // of a row agree on it exactly after exchanging 16-bit values; being up to one unit above
    // the true maximum only scales P and l by the same factor.
    float ms = -INFINITY;
    float l = 0.f;  // this thread's share of the row sum
    if (tracer) TSM_TRACE_BLOCK(g * 2, blk, 0);
    for (int i = 0; i < n_g; ++i) {
      const int buf = i & 1;
      const uint32_t tsb = ts + buf * kHalfKV;
      if (tracer) TSM_TRACE(g * 2, i, 0);
      bool ready = ptx::mbar_wait(&bars->s_full[g][buf], ((done + i) >> 1) & 1u, abort_flag, p.status, 16 + g);
      if (!__all_sync(0xffffffffu, ready)) {
        alive = false;
        break;
      }
      ptx::tcgen05_fence_after_thread_sync();
      if (tracer) TSM_TRACE(g * 2, i, 1);
      if (tracer && i == 0) TSM_TRACE_BLOCK(g * 2, blk, 1);
      const int col0 = i * kHalfKV + h * 32;
      const bool masked = col0 + 31 > limit;

      // this thread's 32 scores of the half-step, read once
      uint32_t v[32];
      ptx::tmem_ld_32x32b_x32(tsb + h * 32, v);
      ptx::tmem_ld_wait();
      if (tracer) TSM_TRACE(g * 2, i, 2);

      float mx = -INFINITY;
      if (masked) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (col0 + e > limit) v[e] = 0xff800000u;  // -inf
          mx = fmaxf(mx, __uint_as_float(v[e]));
        }
      } else {
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 32; e += 2)  // three-input max: 16 instructions for 32 values
          mx4[(e >> 1) & 3] = ptx::fmax3(mx4[(e >> 1) & 3], __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      // exchange with the thread that owns the other 32 keys of this row (also orders its
      // tensor-memory reads of this buffer before this thread's P stores below)
      const int mine = max(-32768, min(32767, __float2int_ru(mx * sl2)));  // -inf -> -32768
      // (two sets of slots alternate: the value of half-step i is read before its reader
      // arrives at the pair barrier of half-step i+1, the slot is rewritten after that barrier)
      my_max[buf * (4 * kBQ)] = static_cast<int16_t>(mine);
      ptx::named_bar_sync(pair_bar, 64);
      const int both = max(mine, static_cast<int>(other_max[buf * (4 * kBQ)]));
      const float m_new = fmaxf(ms, both == -32768 ? -INFINITY : static_cast<float>(both));
      if (tracer) TSM_TRACE(g * 2, i, 3);
      if (i == 0) {
        ms = m_new;
      } else {
        const bool need = m_new - ms > kRescaleThreshold;  // identical in both threads of the row
        if (__any_sync(0xffffffffu, need)) {
          // O_g is rescaled in place once the PV product of the previous half-step has retired
          // (the one of this half-step cannot start before this thread reports its probabilities).
          // Two barriers alternate so that a parity wait can never be a whole phase ahead: the
          // previous user of this barrier, PV(i-3), retired before S(i-1) was complete.
          ready = ptx::mbar_wait(&bars->pv_done[g][(i - 1) & 1], ((done + i - 1) >> 1) & 1u, abort_flag, p.status, 18 + g);
          if (!__all_sync(0xffffffffu, ready)) {
            alive = false;
            break;
          }
          ptx::tcgen05_fence_after_thread_sync();
          const float alpha = need ? ptx::ex2_approx(ms - m_new) : 1.0f;
          if (need) ms = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {  // this thread's 64 output columns
            uint32_t ov[32];
            ptx::tmem_ld_32x32b_x32(to + c * 32, ov);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            ptx::tmem_st_32x32b_x32(to + c * 32, ov);
          }
          ptx::tmem_st_wait();
        }
      }

      // probabilities: exp2, round to 16 bit, two per 32-bit TMEM column; the 32 packed
      // columns of a half-step overlay the first 32 columns of its score buffer (this thread:
      // 16 of them).  Of every 8 pairs, kPolyPairs go through the FMA-pipe polynomial and the
      // rest through MUFU ex2, so that neither pipe alone bounds the exponentials.  The row
      // sum adds the f32 probabilities before they are rounded (packed adds).
      const ptx::f32x2_t sl2x2 = ptx::pack_f32x2(sl2, sl2);
      const ptx::f32x2_t nmsx2 = ptx::pack_f32x2(-ms, -ms);
      ptx::f32x2_t lsum[2] = {0ull, 0ull};  // (+0.0f, +0.0f)
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const ptx::f32x2_t t2 = ptx::fma_f32x2(
            ptx::pack_f32x2(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1])), sl2x2, nmsx2);
        float p0, p1;
        if ((e & 7) < kPolyPairs) {
          ptx::exp2_poly_x2(t2, p0, p1);
        } else {
          float t0, t1;
          ptx::unpack_f32x2(t2, t0, t1);
          p0 = ptx::ex2_approx(t0);  // 2^(-inf) = 0
          p1 = ptx::ex2_approx(t1);
        }
        pk[e] = pack16x2<kIsBf16>(p0, p1);
        lsum[e & 1] = ptx::add_f32x2(lsum[e & 1], ptx::pack_f32x2(p0, p1));
      }
      ptx::tmem_st_32x32b_x16(tsb + h * 16, pk);
      float l4[4];
      ptx::unpack_f32x2(lsum[0], l4[0], l4[1]);
      ptx::unpack_f32x2(lsum[1], l4[2], l4[3]);
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      if (tracer) TSM_TRACE(g * 2, i, 4);
      ptx::tmem_st_wait();
      ptx::tcgen05_fence_before_thread_sync();  // P stores (and O rescale) ordered before the arrive
      ptx::mbar_arrive(&bars->p_ready[g][buf]);
      if (tracer) TSM_TRACE(g * 2, i, 5);
      if (tracer && i == n_g - 1) TSM_TRACE_BLOCK(g * 2, blk, 2);
    }

    if (alive) {
      // the commit behind the last PV product covers every earlier MMA of that issuer
      bool ready = ptx::mbar_wait(&bars->pv_done[g][(n_g - 1) & 1], ((done + n_g - 1) >> 1) & 1u, abort_flag, p.status, 20 + g);
      if (!__all_sync(0xffffffffu, ready)) {
        alive = false;
      } else {
        ptx::tcgen05_fence_after_thread_sync();
        if (tracer) TSM_TRACE_BLOCK(g * 2, blk, 3);
        // this thread's 64 output columns; then the two row-sum shares change hands through
        // the first column of each thread's (already read) part of O
        uint32_t ov[2][32];
        ptx::tmem_ld_32x32b_x32(to, ov[0]);
        ptx::tmem_ld_32x32b_x32(to + 32, ov[1]);
        ptx::tmem_ld_wait();
        ptx::tmem_st_32x32b_x1(to, __float_as_uint(l));
        ptx::tmem_st_wait();
        ptx::tcgen05_fence_before_thread_sync();
        ptx::named_bar_sync(pair_bar, 64);
        ptx::tcgen05_fence_after_thread_sync();
        const float l_other = __uint_as_float(ptx::tmem_ld_32x32b_x1(to + 64 - 2 * h * 64));
        ptx::tmem_ld_wait();
        const float inv = 1.0f / (l + l_other);
        if (qrow < p.seq) {
          uint16_t* orow = o + (static_cast<int64_t>(bh) * p.seq + qrow) * kD + h * 64;
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              uint4 w4;
              w4.x = pack16x2<kIsBf16>(__uint_as_float(ov[c][8 * t + 0]) * inv, __uint_as_float(ov[c][8 * t + 1]) * inv);
              w4.y = pack16x2<kIsBf16>(__uint_as_float(ov[c][8 * t + 2]) * inv, __uint_as_float(ov[c][8 * t + 3]) * inv);
              w4.z = pack16x2<kIsBf16>(__uint_as_float(ov[c][8 * t + 4]) * inv, __uint_as_float(ov[c][8 * t + 5]) * inv);
              w4.w = pack16x2<kIsBf16>(__uint_as_float(ov[c][8 * t + 6]) * inv, __uint_as_float(ov[c][8 * t + 7]) * inv);
              reinterpret_cast<uint4*>(orow + c * 32)[t] = w4;
            }
        }
      }
    }
    if (tracer) TSM_TRACE_BLOCK(g * 2, blk, 4);
    ++blk;
    done += n_g;
    }  // query blocks of a work item
    }  // work items
  }

  // ------------------------------ teardown ------------------------------------
  if (*abort_flag != 0u) {
    const unsigned long long t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) {
    }
  }
  ptx::tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == kWarpMmaA) {
    ptx::tcgen05_fence_after_thread_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace attn
}  // namespace tsm100
