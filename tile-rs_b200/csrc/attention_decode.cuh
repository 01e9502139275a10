// Single-token attention against a KV cache (the decode step of a transformer):
//   o[h,:] = softmax_p( q[h,:] . K[g,p,:] / sqrt(d) ) V[g,p,:],  p < seq_len,  g = h / (heads_q / heads_kv)
// __tile_attention_decode_f32 (crates/tile_std/src/tile.rs:2120-2124; wrapper :3004-3018):
// q and o are [heads_q][d], the caches [heads_kv][max_seq][d].  The intrinsic is opaque in
// the linalg bridge (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:502-505); its arithmetic
// is the Metal lowering's five phases - scores with scale rsqrt(d), max, exp and sum,
// normalise, weighted V sum (crates/rustc_codegen_tile/src/mlir_to_msl.rs:10747-10812), where
// seq_len, max_seq and the head counts are run-time constants of the kernel.  A leading
// batch dimension repeats the problem (caches [batch][heads_kv][max_seq][d]).
//
// The work is reading the cache once: 2 * heads_kv * seq_len * d elements per batch entry.
// A cluster of `splits` CTAs owns one (batch, KV head): every CTA takes a contiguous range
// of positions and all query heads of the group, so K and V are read from HBM exactly once
// however many query heads share them; the partial results (running max, sum, weighted V)
// are merged through distributed shared memory - no workspace, no second kernel.
// Inside a CTA 16 (or 8) lanes share one cache row, a warp works on two (or four) positions
// at a time with the next ones in flight, 8 warps stride over the range.
// Roofline: HBM.
#pragma once

#include <type_traits>

#include "ptx.cuh"
#include "softmax.cuh"

namespace tsm100 {
namespace attn_decode {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// Lanes that share one cache row: 16, or 8 where 16 would leave a lane less than one 16-byte
// vector (16-bit storage with head_dim 64).  A warp works on 32 / lanes positions at a time.
template <typename T, int D>
constexpr int lanes_per_pos() { return (D / 16) % softmax::Elem<T>::kPerVec == 0 ? 16 : 8; }
template <typename T, int D>
constexpr int slots() { return kWarps * (32 / lanes_per_pos<T, D>()); }  // (warp, lane group) pairs, each with its own running state
constexpr int kMaxSplits = 8;     // portable cluster size
constexpr int kMaxSplitsWide = 16;  // non-portable size, used for a handful of sequences when the GPU can place such clusters

// Merge of the per-CTA records of a cluster into the output, through distributed shared memory.
// `mine` is this CTA's record [ROWS][D + 2] (O, running max, sum), at the same shared-memory offset in
// every CTA; `scratch` (>= (3 * kMaxSplitsWide + 1) * ROWS floats, no longer in use) receives the
// per-(row, rank) weights.  Every CTA merges its share of the ROWS x D outputs, all its remote loads in
// flight together; ranks are added in rank order, so the result does not depend on timing.  The caller
// brackets the call with cluster barriers.  seq_len == 0: no position contributes; 0 / 0 = NaN, as the
// five phases of the reference give.
template <typename T, int ROWS, int D, int THREADS>
__device__ __forceinline__ void cluster_merge(const float* mine, float* scratch, uint32_t rank, uint32_t splits,
                                              int rows_valid, T* __restrict__ o_rows) {
  constexpr int REC = D + 2;
  float* m_all = scratch;                              // [ROWS][kMaxSplitsWide] running maxima of the ranks
  float* w_all = scratch + ROWS * kMaxSplitsWide;      // ... their weights 2^(m_r - M)
  float* l_all = scratch + 2 * ROWS * kMaxSplitsWide;  // ... their sums
  float* l_row = scratch + 3 * ROWS * kMaxSplitsWide;  // [ROWS] merged sums
  const int tid = threadIdx.x;
  const uint32_t mine_addr = ptx::smem_u32(mine);
  const int ns = static_cast<int>(splits);
  for (int i = tid; i < ROWS * ns; i += THREADS) {
    const int hh = i / ns, r = i % ns;
    const uint32_t base = ptx::mapa_shared(mine_addr + (hh * REC + D) * 4, static_cast<uint32_t>(r));
    m_all[hh * kMaxSplitsWide + r] = ptx::ld_shared_cluster_f32(base);
    l_all[hh * kMaxSplitsWide + r] = ptx::ld_shared_cluster_f32(base + 4);
  }
  __syncthreads();
  for (int hh = tid; hh < ROWS; hh += THREADS) {
    float mm = -INFINITY;
    for (int r = 0; r < ns; ++r) mm = fmaxf(mm, m_all[hh * kMaxSplitsWide + r]);
    float ll = 0.f;
    for (int r = 0; r < ns; ++r) {
      const float mr = m_all[hh * kMaxSplitsWide + r];
      const float wgt = mr == -INFINITY ? 0.f : ptx::ex2_approx(mr - mm);  // a rank without positions carries no weight
      w_all[hh * kMaxSplitsWide + r] = wgt;
      ll = fmaf(l_all[hh * kMaxSplitsWide + r], wgt, ll);
    }
    l_row[hh] = ll;
  }
  __syncthreads();
  const int per = (ROWS * D + ns - 1) / ns;
  const int i_end = min(ROWS * D, (static_cast<int>(rank) + 1) * per);
  for (int i = static_cast<int>(rank) * per + tid; i < i_end; i += THREADS) {
    const int hh = i / D, dd = i % D;
    if (hh >= rows_valid) continue;
    float part_o[kMaxSplitsWide];
#pragma unroll
    for (int r = 0; r < kMaxSplitsWide; ++r)
      part_o[r] = r < ns ? ptx::ld_shared_cluster_f32(ptx::mapa_shared(mine_addr + (hh * REC + dd) * 4, static_cast<uint32_t>(r))) : 0.f;
    float oo = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxSplitsWide; ++r)
      if (r < ns) oo = fmaf(part_o[r], w_all[hh * kMaxSplitsWide + r], oo);
    softmax::Elem<T>::store1(o_rows + hh * D + dd, oo / l_row[hh]);
  }
}

struct Params {
  int32_t batch, heads_q, heads_kv;
  int32_t seq_len, max_seq;
  int32_t group;        // heads_q / heads_kv
  int32_t head_base;    // first query head of the group handled by this launch (groups wider than G run in passes)
  int32_t heads_here;   // query heads of the group handled by this launch (<= G)
  float scale_log2;     // rsqrt(d) * log2(e)
};

template <typename T, int DPL>
__device__ __forceinline__ void load_row(const T* __restrict__ row, int sub, float (&f)[DPL]) {
  // lane `sub` of a row's lanes owns elements [sub * DPL, sub * DPL + DPL) of the row
  constexpr int PV = softmax::Elem<T>::kPerVec;
  const softmax::Vec16* v = reinterpret_cast<const softmax::Vec16*>(row + sub * DPL);
#pragma unroll
  for (int k = 0; k < DPL / PV; ++k) softmax::Elem<T>::unpack(softmax::ld_stream(v + k), f + k * PV);
}

// shared memory: q [G][D] floats, then per slot and per head a record of D + 2 floats
// (o[D], m, l), then this CTA's merged record per head (same layout) for the cluster merge.
template <typename T, int G, int D>
constexpr int smem_floats() { return G * D + (slots<T, D>() + 1) * G * (D + 2); }

template <typename T, int G, int D>
__global__ void __launch_bounds__(kThreads)
attention_decode_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, T* __restrict__ o,
                        const Params p) {
  constexpr int LPP = lanes_per_pos<T, D>();
  constexpr int GROUPS = 32 / LPP;          // positions a warp works on at a time
  constexpr int kSlots = slots<T, D>();
  constexpr int DPL = D / LPP;
  constexpr int REC = D + 2;
  static_assert(DPL % softmax::Elem<T>::kPerVec == 0, "a lane's share of a row must be whole 16-byte vectors");
  extern __shared__ __align__(16) float sm[];
  float* q_s = sm;                          // [G][D], already multiplied by scale * log2(e)
  float* part = sm + G * D;                 // [kSlots][G][REC]
  float* mine = part + kSlots * G * REC;    // [G][REC]: this CTA's merged partial

  const uint32_t rank = ptx::cluster_ctarank(), splits = ptx::cluster_nctarank();
  const int unit = blockIdx.x / splits;     // flattened (batch, KV head)
  const int b = unit / p.heads_kv, g = unit % p.heads_kv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = lane / LPP, sub = lane % LPP, slot = warp * GROUPS + half;  // `half`: this lane's group in the warp
  const int h0 = g * p.group + p.head_base;  // first query head handled here

  for (int i = tid; i < G * D; i += kThreads) {
    const int hh = i / D, dd = i % D;
    q_s[i] = hh < p.heads_here
                 ? softmax::Elem<T>::load1(q + (static_cast<int64_t>(b) * p.heads_q + h0 + hh) * D + dd) * p.scale_log2
                 : 0.f;
  }
  __syncthreads();

  // this CTA's positions: a contiguous range, a multiple of 32 long except for the last CTA
  const int chunk = ((p.seq_len + static_cast<int>(splits) - 1) / static_cast<int>(splits) + 31) & ~31;
  const int p_begin = static_cast<int>(rank) * chunk;
  const int p_end = min(p.seq_len, p_begin + chunk);
  const int64_t cache_off = (static_cast<int64_t>(b) * p.heads_kv + g) * p.max_seq * D;
  const T* kbase = kc + cache_off;
  const T* vbase = vc + cache_off;

  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[h][e] = 0.f;
  }
  float qr[G][DPL];  // this lane's share of every query row
#pragma unroll
  for (int h = 0; h < G; ++h)
#pragma unroll
    for (int e = 0; e < DPL; ++e) qr[h][e] = q_s[h * D + sub * DPL + e];

  // Slot s of the CTA takes positions p_begin + s + kSlots * it.  The lane groups of a warp run
  // the same number of iterations (the shuffles below are executed by the whole warp): the trip
  // count follows the first group's position, the others are predicated.
  float kf[DPL], vf[DPL], kn[DPL], vn[DPL];
#pragma unroll
  for (int e = 0; e < DPL; ++e) kf[e] = vf[e] = kn[e] = vn[e] = 0.f;
  const int first = p_begin + warp * GROUPS;
  if (first + half < p_end) {
    load_row<T, DPL>(kbase + static_cast<int64_t>(first + half) * D, sub, kf);
    load_row<T, DPL>(vbase + static_cast<int64_t>(first + half) * D, sub, vf);
  }
  for (int base = first; base < p_end; base += kSlots) {
    const int pos = base + half;
    const bool valid = pos < p_end;
    if (pos + kSlots < p_end) {  // the next row of this slot is in flight while this one is used
      load_row<T, DPL>(kbase + static_cast<int64_t>(pos + kSlots) * D, sub, kn);
      load_row<T, DPL>(vbase + static_cast<int64_t>(pos + kSlots) * D, sub, vn);
    }
    float s[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int e = 0; e < DPL; e += 2) {
        d0 = fmaf(qr[h][e], kf[e], d0);
        d1 = fmaf(qr[h][e + 1], kf[e + 1], d1);
      }
      s[h] = d0 + d1;
    }
    // sum over the lanes of this position (xor offsets below LPP stay inside the lane group)
#pragma unroll
    for (int off = LPP / 2; off > 0; off >>= 1)
#pragma unroll
      for (int h = 0; h < G; ++h) s[h] += __shfl_xor_sync(0xffffffffu, s[h], off);
    if (valid) {
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float m_new = fmaxf(m[h], s[h]);
        const float alpha = ptx::ex2_approx(m[h] - m_new);  // first row: 2^(-inf) = 0
        const float pr = ptx::ex2_approx(s[h] - m_new);
        m[h] = m_new;
        l[h] = fmaf(l[h], alpha, pr);
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[h][e] = fmaf(pr, vf[e], acc[h][e] * alpha);
      }
    }
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      kf[e] = kn[e];
      vf[e] = vn[e];
    }
  }

  // slot records -> shared memory
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float* rec = part + (slot * G + h) * REC;
#pragma unroll
    for (int e = 0; e < DPL; ++e) rec[sub * DPL + e] = acc[h][e];
    if (sub == 0) {
      rec[D] = m[h];
      rec[D + 1] = l[h];
    }
  }
  __syncthreads();
  // merge the slots: thread t handles output element (h, dd)
  for (int i = tid; i < G * D; i += kThreads) {
    const int hh = i / D, dd = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int sl = 0; sl < kSlots; ++sl) mm = fmaxf(mm, part[(sl * G + hh) * REC + D]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int sl = 0; sl < kSlots; ++sl) {
      const float* rec = part + (sl * G + hh) * REC;
      const float w = rec[D] == -INFINITY ? 0.f : ptx::ex2_approx(rec[D] - mm);  // an empty slot carries no weight
      ll = fmaf(rec[D + 1], w, ll);
      oo = fmaf(rec[dd], w, oo);
    }
    mine[hh * REC + dd] = oo;
    if (dd == 0) {
      mine[hh * REC + D] = mm;
      mine[hh * REC + D + 1] = ll;
    }
  }
  // merge across the cluster through distributed shared memory (every CTA writes its share of the result)
  ptx::cluster_sync_all();
  cluster_merge<T, G, D, kThreads>(mine, part, rank, splits, p.heads_here, o + (static_cast<int64_t>(b) * p.heads_q + h0) * D);
  ptx::cluster_sync_all();  // nobody leaves while its shared memory may still be read
}

// ===========================================================================
// 16-bit caches: the same operator on tensor cores.  With 16-bit storage the FP32 pipe
// cannot keep up with HBM once several query heads share a cache row (8 heads: ~145
// instructions per row and warp above), so the query heads of a group become the M
// dimension of mma.sync m16n8k16 tiles: S[16 heads x 16 positions] = Q K^T and
// O[16 heads x D] += P V, f32 accumulation, online softmax on the accumulator fragments.
// (tcgen05 needs 64 or 128 rows per tile; 16 padded rows per (batch, KV head) is what a
// decode step has, so this is the one place the warp-level MMA is the right size.)
//
// Per CTA 4 or 8 warps; each warp streams its own tiles of 16 positions through a cp.async
// ring of 2 or 3 stages in shared memory (K and V rows padded by 16 bytes: conflict-free
// ldmatrix), keeps its own running (max, sum, O) and the partial results are merged as
// above: warps through shared memory, CTAs of the cluster through distributed shared memory.
// The ring is started before anything else is read; Q goes from global memory straight into
// the A fragments.
// ===========================================================================
namespace mma {
// warps per CTA: 4 for large launches (several CTAs per SM), 8 when a launch has at most one CTA per SM
constexpr int kTilePos = 16;   // positions per tile
constexpr int kRows = 16;      // query heads per pass (rows of the MMA tile)

template <int D>
constexpr int pitch_bytes() { return D * 2 + 16; }
template <int D>
constexpr int stage_bytes() { return 2 * kTilePos * pitch_bytes<D>(); }   // K tile + V tile
// ring (a warp's record for the merge later overlays its own part of it, the CTA's merged record the rest of warp 0's):
// without a separate record three 4-warp CTAs fit one SM.
// 4 warps x 2 stages when several CTAs share an SM (large batches: the other CTAs hide the latencies);
// 8 warps x 3 stages when a launch has at most one CTA per SM (a few sequences): a single warp per
// scheduler spends ~2900 cycles on a tile (the MMA, ldmatrix and shuffle latencies in a row), so the
// lone CTA needs two warps per scheduler and 136 KiB of loads in flight to draw its share of HBM.
template <int D, int STAGES, int WARPS>
constexpr int smem_bytes() { return WARPS * STAGES * stage_bytes<D>(); }

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool kIsBf16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (kIsBf16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool kIsBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kIsBf16) return ptx::pack_bf16x2(lo, hi);
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T, int D, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_mma_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, T* __restrict__ o,
                            const Params p) {
  constexpr bool kIsBf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
  constexpr int kWarps = WARPS, kThreads = WARPS * 32;
  constexpr int PITCH = pitch_bytes<D>();
  constexpr int KSTEPS = D / 16;      // k-steps of Q K^T; pairs of 8-wide output tiles of P V
  constexpr int REC = D + 2;
  constexpr int CHUNKS = D * 2 / 16;  // 16-byte pieces per cache row
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* ring = smem_raw;                                           // [warp][stage][K | V][16 rows][PITCH]
  constexpr int WARP_FLOATS = STAGES * stage_bytes<D>() / 4;              // a warp's ring share, reused for its record [16][REC]
  static_assert(2 * kRows * REC <= WARP_FLOATS, "a warp's record and the CTA's merged record must fit into a ring share");
  float* part = reinterpret_cast<float*>(ring);                       // warp w's record at part + w * WARP_FLOATS
  float* mine = part + kRows * REC;                                   // the CTA's merged record [16][REC], behind warp 0's

  const uint32_t rank = ptx::cluster_ctarank(), splits = ptx::cluster_nctarank();
  const int unit = blockIdx.x / splits;
  const int b = unit / p.heads_kv, g = unit % p.heads_kv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gr = lane >> 2, tq = lane & 3;   // fragment row group and column pair
  const int h0 = g * p.group + p.head_base;

  const int chunk = ((p.seq_len + static_cast<int>(splits) - 1) / static_cast<int>(splits) + 63) & ~63;
  const int p_begin = static_cast<int>(rank) * chunk;
  const int p_end = min(p.seq_len, p_begin + chunk);
  const int n_tiles = p_end > p_begin ? (p_end - p_begin + kTilePos - 1) / kTilePos : 0;
  const int64_t cache_off = (static_cast<int64_t>(b) * p.heads_kv + g) * p.max_seq * D;
  const uint8_t* kbase = reinterpret_cast<const uint8_t*>(kc + cache_off);
  const uint8_t* vbase = reinterpret_cast<const uint8_t*>(vc + cache_off);
  const uint32_t ring_w = ptx::smem_u32(ring) + warp * STAGES * stage_bytes<D>();

  auto prefetch = [&](int tile, int stage) {  // this warp's tile `tile` of the CTA's range into its ring stage
    const int row0 = p_begin + tile * kTilePos;
    const uint32_t dst = ring_w + stage * stage_bytes<D>();
#pragma unroll
    for (int c = lane; c < kTilePos * CHUNKS; c += 32) {
      const int r = c / CHUNKS, cc = c % CHUNKS;
      const bool ok = row0 + r < p_end;
      const int64_t src = (static_cast<int64_t>(ok ? row0 + r : p_begin)) * (D * 2) + cc * 16;
      cp_async_16(dst + r * PITCH + cc * 16, kbase + src, ok);
      cp_async_16(dst + kTilePos * PITCH + r * PITCH + cc * 16, vbase + src, ok);
    }
  };

  float oacc[2 * KSTEPS][4];
#pragma unroll
  for (int j = 0; j < 2 * KSTEPS; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows gr and gr + 8 (this thread's share of the sums)
  const float sl2 = p.scale_log2;

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {  // the first tiles are on their way before anything else is read
    if (warp + i * kWarps < n_tiles) prefetch(warp + i * kWarps, i);
    cp_async_commit();
  }
  // A fragments of Q for every k-step, straight from global memory (all loads independent, rows beyond
  // heads_here zero): a0 (row gr, k 2tq..), a1 (row gr+8, ..), a2 (row gr, k 2tq+8..), a3 (row gr+8, ..)
  uint32_t qa[KSTEPS][4];
  {
    const uint32_t* r0 = reinterpret_cast<const uint32_t*>(q + (static_cast<int64_t>(b) * p.heads_q + h0 + gr) * D);
    const uint32_t* r1 = r0 + 8 * (D / 2);
    const bool ok0 = gr < p.heads_here, ok1 = gr + 8 < p.heads_here;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = ok0 ? __ldg(r0 + kk * 8 + tq) : 0u;
      qa[kk][1] = ok1 ? __ldg(r1 + kk * 8 + tq) : 0u;
      qa[kk][2] = ok0 ? __ldg(r0 + kk * 8 + tq + 4) : 0u;
      qa[kk][3] = ok1 ? __ldg(r1 + kk * 8 + tq + 4) : 0u;
    }
  }
  int stage = 0;
  for (int t = warp; t < n_tiles; t += kWarps, stage = stage + 1 == STAGES ? 0 : stage + 1) {
    if (t + (STAGES - 1) * kWarps < n_tiles) prefetch(t + (STAGES - 1) * kWarps, stage == 0 ? STAGES - 1 : stage - 1);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();  // everything but the newest STAGES - 1 groups: this tile has landed
    __syncwarp();
    const uint32_t ks = ring_w + stage * stage_bytes<D>();
    const uint32_t vs = ks + kTilePos * PITCH;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t kb[4];  // (positions 0-7, k lo), (0-7, k hi), (8-15, k lo), (8-15, k hi)
      ldmatrix_x4(ks + ((lane & 7) + ((lane >> 4) & 1) * 8) * PITCH + (kk * 16 + ((lane >> 3) & 1) * 8) * 2, kb);
      mma_16816<kIsBf16>(s[0], qa[kk], kb[0], kb[1]);
      mma_16816<kIsBf16>(s[1], qa[kk], kb[2], kb[3]);
    }
    // scale to log2 units; positions past the end of the range carry no weight
    const int pos = p_begin + t * kTilePos + 2 * tq;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int pp = pos + j * 8 + (e & 1);
        s[j][e] = pp < p_end ? s[j][e] * sl2 : -INFINITY;
      }
    float t0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    float t1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);  // finite: a tile has at least one valid position
    const float a0 = ptx::ex2_approx(m0 - n0), a1 = ptx::ex2_approx(m1 - n1);  // first tile: 2^(-inf) = 0
    m0 = n0;
    m1 = n1;
    uint32_t pa[4];
    {
      const float p00 = ptx::ex2_approx(s[0][0] - n0), p01 = ptx::ex2_approx(s[0][1] - n0);
      const float p02 = ptx::ex2_approx(s[0][2] - n1), p03 = ptx::ex2_approx(s[0][3] - n1);
      const float p10 = ptx::ex2_approx(s[1][0] - n0), p11 = ptx::ex2_approx(s[1][1] - n0);
      const float p12 = ptx::ex2_approx(s[1][2] - n1), p13 = ptx::ex2_approx(s[1][3] - n1);
      l0 = fmaf(l0, a0, (p00 + p01) + (p10 + p11));
      l1 = fmaf(l1, a1, (p02 + p03) + (p12 + p13));
      pa[0] = pack2<kIsBf16>(p00, p01);  // row gr,     positions 2tq..
      pa[1] = pack2<kIsBf16>(p02, p03);  // row gr + 8, positions 2tq..
      pa[2] = pack2<kIsBf16>(p10, p11);  // row gr,     positions 2tq + 8..
      pa[3] = pack2<kIsBf16>(p12, p13);  // row gr + 8, positions 2tq + 8..
    }
#pragma unroll
    for (int j = 0; j < 2 * KSTEPS; ++j) {
      oacc[j][0] *= a0;
      oacc[j][1] *= a0;
      oacc[j][2] *= a1;
      oacc[j][3] *= a1;
    }
#pragma unroll
    for (int jj = 0; jj < KSTEPS; ++jj) {
      uint32_t vb[4];  // (positions 0-7, d lo), (8-15, d lo), (0-7, d hi), (8-15, d hi), transposed on load
      ldmatrix_x4_trans(vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (jj * 16 + ((lane >> 4) & 1) * 8) * 2, vb);
      mma_16816<kIsBf16>(oacc[2 * jj], pa, vb[0], vb[1]);
      mma_16816<kIsBf16>(oacc[2 * jj + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();  // the stage is refilled at the top of the next iteration; every lane is done reading it
  }
  cp_async_wait<0>();
  __syncwarp();  // the warp's ring share is free: it now receives the warp's record
  // this thread's share of the row sums -> the whole row's
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // warp records -> shared memory: row r of warp w at part[(w * 16 + r) * REC]: O[D], max, sum
  {
    float* r0 = part + warp * WARP_FLOATS + gr * REC;
    float* r1 = part + warp * WARP_FLOATS + (gr + 8) * REC;
#pragma unroll
    for (int j = 0; j < 2 * KSTEPS; ++j) {
      r0[j * 8 + 2 * tq] = oacc[j][0];
      r0[j * 8 + 2 * tq + 1] = oacc[j][1];
      r1[j * 8 + 2 * tq] = oacc[j][2];
      r1[j * 8 + 2 * tq + 1] = oacc[j][3];
    }
    if (tq == 0) {
      r0[D] = m0;
      r0[D + 1] = l0;
      r1[D] = m1;
      r1[D + 1] = l1;
    }
  }
  __syncthreads();
  for (int i = tid; i < kRows * D; i += kThreads) {
    const int hh = i / D, dd = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, part[w * WARP_FLOATS + hh * REC + D]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* rec = part + w * WARP_FLOATS + hh * REC;
      const float wgt = rec[D] == -INFINITY ? 0.f : ptx::ex2_approx(rec[D] - mm);  // a warp without tiles carries no weight
      ll = fmaf(rec[D + 1], wgt, ll);
      oo = fmaf(rec[dd], wgt, oo);
    }
    mine[hh * REC + dd] = oo;
    if (dd == 0) {
      mine[hh * REC + D] = mm;
      mine[hh * REC + D + 1] = ll;
    }
  }
  ptx::cluster_sync_all();
  cluster_merge<T, kRows, D, kThreads>(mine, part, rank, splits, p.heads_here, o + (static_cast<int64_t>(b) * p.heads_q + h0) * D);
  ptx::cluster_sync_all();  // nobody leaves while its shared memory may still be read
}

}  // namespace mma
// ===========================================================================
// f32 caches on tensor cores, for groups of several query heads (one head per cache is served as
// well by the FP32-pipe kernel above).  The same structure as the 16-bit kernel: the heads of a
// group are the M = 16 rows, a warp streams its own tiles of 8 positions through a cp.async ring,
// online softmax on the accumulator fragments, warp records merged through shared memory and the
// CTAs of the cluster through distributed shared memory.  The arithmetic keeps f32 accuracy (the
// oracle is matched to 1e-5): mma.sync.m16n8k8.tf32 with every operand split into hi + lo and three
// products per product, as in gemm_tf32x3.cuh.  B fragments are plain 32-bit loads from rows padded
// by 16 bytes (32 banks); the accumulator fragment of S is the A fragment of P V with the k index
// tq -> position 2tq, tq + 4 -> position 2tq + 1, applied to the V row addresses.
// ===========================================================================
namespace tf32 {

constexpr int kTilePos = 8;
constexpr int kRows = 16;

template <int D>
constexpr int pitch_words() { return D + 4; }
template <int D>
constexpr int stage_bytes() { return 2 * kTilePos * pitch_words<D>() * 4; }  // K tile + V tile
template <int D, int STAGES, int WARPS>
constexpr int smem_bytes() { return WARPS * STAGES * stage_bytes<D>(); }

__device__ __forceinline__ void split(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;          // what the tensor core reads of x
  lo = __float_as_uint(x - __uint_as_float(hi));  // exact; the tensor core reads its top 11 bits
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int D, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_tf32_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc,
                             float* __restrict__ o, const Params p) {
  namespace cp = mma;  // cp.async helpers
  constexpr int kWarps = WARPS, kThreads = WARPS * 32;
  constexpr int PW = pitch_words<D>();
  constexpr int KSTEPS = D / 8;      // k-steps of Q K^T; 8-wide output tiles of P V
  constexpr int REC = D + 2;
  constexpr int CHUNKS = D / 4;      // 16-byte pieces per cache row
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* ring = smem_raw;                                           // [warp][stage][K | V][8 rows][PW floats]
  constexpr int WARP_FLOATS = STAGES * stage_bytes<D>() / 4;          // a warp's ring share, reused for its record [16][REC]
  static_assert(2 * kRows * REC <= WARP_FLOATS, "a warp's record and the CTA's merged record must fit into a ring share");
  float* part = reinterpret_cast<float*>(ring);                       // warp w's record at part + w * WARP_FLOATS
  float* mine = part + kRows * REC;                                   // the CTA's merged record [16][REC], behind warp 0's

  const uint32_t rank = ptx::cluster_ctarank(), splits = ptx::cluster_nctarank();
  const int unit = blockIdx.x / splits;
  const int b = unit / p.heads_kv, g = unit % p.heads_kv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gr = lane >> 2, tq = lane & 3;   // fragment row group and column pair
  const int h0 = g * p.group + p.head_base;

  const int chunk = ((p.seq_len + static_cast<int>(splits) - 1) / static_cast<int>(splits) + 63) & ~63;
  const int p_begin = static_cast<int>(rank) * chunk;
  const int p_end = min(p.seq_len, p_begin + chunk);
  const int n_tiles = p_end > p_begin ? (p_end - p_begin + kTilePos - 1) / kTilePos : 0;
  const int64_t cache_off = (static_cast<int64_t>(b) * p.heads_kv + g) * p.max_seq * D;
  const float* kbase = kc + cache_off;
  const float* vbase = vc + cache_off;
  const uint32_t ring_w = ptx::smem_u32(ring) + warp * STAGES * stage_bytes<D>();

  auto prefetch = [&](int tile, int stage) {  // this warp's tile `tile` of the CTA's range into its ring stage
    const int row0 = p_begin + tile * kTilePos;
    const uint32_t dst = ring_w + stage * stage_bytes<D>();
#pragma unroll
    for (int c = lane; c < kTilePos * CHUNKS; c += 32) {
      const int r = c / CHUNKS, cc = c % CHUNKS;
      const bool ok = row0 + r < p_end;  // rows past the range are zero-filled: they carry no weight, and 0 * V stays finite
      const int64_t src = (static_cast<int64_t>(ok ? row0 + r : p_begin)) * D + cc * 4;
      cp::cp_async_16(dst + (r * PW + cc * 4) * 4, kbase + src, ok);
      cp::cp_async_16(dst + ((kTilePos + r) * PW + cc * 4) * 4, vbase + src, ok);
    }
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {  // the first tiles are on their way before anything else is read
    if (warp + i * kWarps < n_tiles) prefetch(warp + i * kWarps, i);
    cp::cp_async_commit();
  }
  // A fragments of Q (rows beyond heads_here zero): a0 (row gr, k tq), a1 (row gr+8, k tq), a2 (row gr, k tq+4), a3 (row gr+8, k tq+4)
  float qa[KSTEPS][4];
  {
    const float* r0 = q + (static_cast<int64_t>(b) * p.heads_q + h0 + gr) * D;
    const float* r1 = r0 + 8 * D;
    const bool ok0 = gr < p.heads_here, ok1 = gr + 8 < p.heads_here;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = ok0 ? __ldg(r0 + kk * 8 + tq) : 0.f;
      qa[kk][1] = ok1 ? __ldg(r1 + kk * 8 + tq) : 0.f;
      qa[kk][2] = ok0 ? __ldg(r0 + kk * 8 + tq + 4) : 0.f;
      qa[kk][3] = ok1 ? __ldg(r1 + kk * 8 + tq + 4) : 0.f;
    }
  }

  float oacc[KSTEPS][4];
#pragma unroll
  for (int j = 0; j < KSTEPS; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows gr and gr + 8 (this thread's share of the sums)
  const float sl2 = p.scale_log2;

  int stage = 0;
  for (int t = warp; t < n_tiles; t += kWarps, stage = stage + 1 == STAGES ? 0 : stage + 1) {
    if (t + (STAGES - 1) * kWarps < n_tiles) prefetch(t + (STAGES - 1) * kWarps, stage == 0 ? STAGES - 1 : stage - 1);
    cp::cp_async_commit();
    cp::cp_async_wait<STAGES - 1>();  // everything but the newest STAGES - 1 groups: this tile has landed
    __syncwarp();
    const float* ks = reinterpret_cast<const float*>(ring + warp * STAGES * stage_bytes<D>() + stage * stage_bytes<D>());
    const float* vs = ks + kTilePos * PW;
    // Four partial sums (k-steps 4c, 4c+1, 4c+2, 4c+3), their products issued term by term across the four, so
    // that an MMA never waits for the one just before it; (row gr, pos 2tq), (gr, 2tq+1), (gr+8, 2tq), (gr+8, 2tq+1)
    float sp[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) sp[c][e] = 0.f;
#pragma unroll
    for (int k4 = 0; k4 < KSTEPS; k4 += 4) {
      uint32_t ah[4][4], al[4][4], b0h[4], b0l[4], b1h[4], b1l[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int e = 0; e < 4; ++e) split(qa[k4 + c][e], ah[c][e], al[c][e]);
        const float* kr = ks + gr * PW + (k4 + c) * 8 + tq;  // b0 (k tq, position gr), b1 (k tq+4, position gr)
        split(kr[0], b0h[c], b0l[c]);
        split(kr[4], b1h[c], b1l[c]);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) mma_tf32(sp[c], al[c], b0h[c], b1h[c]);  // small terms first
#pragma unroll
      for (int c = 0; c < 4; ++c) mma_tf32(sp[c], ah[c], b0l[c], b1l[c]);
#pragma unroll
      for (int c = 0; c < 4; ++c) mma_tf32(sp[c], ah[c], b0h[c], b1h[c]);
    }
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = (sp[0][e] + sp[1][e]) + (sp[2][e] + sp[3][e]);
    // scale to log2 units; positions past the end of the range carry no weight
    const int pos = p_begin + t * kTilePos + 2 * tq;
    s[0] = pos < p_end ? s[0] * sl2 : -INFINITY;
    s[1] = pos + 1 < p_end ? s[1] * sl2 : -INFINITY;
    s[2] = pos < p_end ? s[2] * sl2 : -INFINITY;
    s[3] = pos + 1 < p_end ? s[3] * sl2 : -INFINITY;
    float t0 = fmaxf(s[0], s[1]), t1 = fmaxf(s[2], s[3]);
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);  // finite: a tile has at least one valid position
    const float a0 = ptx::ex2_approx(m0 - n0), a1 = ptx::ex2_approx(m1 - n1);  // first tile: 2^(-inf) = 0
    m0 = n0;
    m1 = n1;
    const float p0 = ptx::ex2_approx(s[0] - n0), p1 = ptx::ex2_approx(s[1] - n0);
    const float p2 = ptx::ex2_approx(s[2] - n1), p3 = ptx::ex2_approx(s[3] - n1);
    l0 = fmaf(l0, a0, p0 + p1);
    l1 = fmaf(l1, a1, p2 + p3);
    if (__any_sync(0xffffffffu, a0 != 1.0f || a1 != 1.0f)) {  // a maximum moved somewhere in the warp: rescale
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) {
        oacc[j][0] *= a0;
        oacc[j][1] *= a0;
        oacc[j][2] *= a1;
        oacc[j][3] *= a1;
      }
    }
    // O += P V: a0 (row gr, k tq -> position 2tq), a1 (row gr+8, same), a2 (row gr, k tq+4 -> position 2tq+1), a3
    uint32_t ah[4], al[4];
    split(p0, ah[0], al[0]);
    split(p2, ah[1], al[1]);
    split(p1, ah[2], al[2]);
    split(p3, ah[3], al[3]);
    const float* vr = vs + 2 * tq * PW + gr;  // b0 (position 2tq, d 8j + gr), b1 (position 2tq + 1, d 8j + gr)
#pragma unroll
    for (int j0 = 0; j0 < KSTEPS; j0 += 8) {  // eight independent accumulators at a time, term by term
      uint32_t b0h[8], b0l[8], b1h[8], b1l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        split(vr[(j0 + j) * 8], b0h[j], b0l[j]);
        split(vr[PW + (j0 + j) * 8], b1h[j], b1l[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) mma_tf32(oacc[j0 + j], al, b0h[j], b1h[j]);
#pragma unroll
      for (int j = 0; j < 8; ++j) mma_tf32(oacc[j0 + j], ah, b0l[j], b1l[j]);
#pragma unroll
      for (int j = 0; j < 8; ++j) mma_tf32(oacc[j0 + j], ah, b0h[j], b1h[j]);
    }
    __syncwarp();  // the stage is refilled at the top of the next iteration; every lane is done reading it
  }
  cp::cp_async_wait<0>();
  __syncwarp();  // the warp's ring share is free: it now receives the warp's record
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // warp records -> shared memory: row r of warp w at part[w * WARP_FLOATS + r * REC]: O[D], max, sum
  {
    float* r0 = part + warp * WARP_FLOATS + gr * REC;
    float* r1 = part + warp * WARP_FLOATS + (gr + 8) * REC;
#pragma unroll
    for (int j = 0; j < KSTEPS; ++j) {
      r0[j * 8 + 2 * tq] = oacc[j][0];
      r0[j * 8 + 2 * tq + 1] = oacc[j][1];
      r1[j * 8 + 2 * tq] = oacc[j][2];
      r1[j * 8 + 2 * tq + 1] = oacc[j][3];
    }
    if (tq == 0) {
      r0[D] = m0;
      r0[D + 1] = l0;
      r1[D] = m1;
      r1[D + 1] = l1;
    }
  }
  __syncthreads();
  for (int i = tid; i < kRows * D; i += kThreads) {
    const int hh = i / D, dd = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, part[w * WARP_FLOATS + hh * REC + D]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* rec = part + w * WARP_FLOATS + hh * REC;
      const float wgt = rec[D] == -INFINITY ? 0.f : ptx::ex2_approx(rec[D] - mm);  // a warp without tiles carries no weight
      ll = fmaf(rec[D + 1], wgt, ll);
      oo = fmaf(rec[dd], wgt, oo);
    }
    mine[hh * REC + dd] = oo;
    if (dd == 0) {
      mine[hh * REC + D] = mm;
      mine[hh * REC + D + 1] = ll;
    }
  }
  ptx::cluster_sync_all();
  cluster_merge<float, kRows, D, kThreads>(mine, part, rank, splits, p.heads_here, o + (static_cast<int64_t>(b) * p.heads_q + h0) * D);
  ptx::cluster_sync_all();  // nobody leaves while its shared memory may still be read
}

}  // namespace tf32
}  // namespace attn_decode
}  // namespace tsm100
