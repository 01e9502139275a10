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
constexpr int kMaxSplits = 8;

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
  // merge across the cluster through distributed shared memory (rank 0 writes the result)
  ptx::cluster_sync_all();
  if (rank == 0) {
    const uint32_t mine_addr = ptx::smem_u32(mine);
    for (int i = tid; i < G * D; i += kThreads) {
      const int hh = i / D, dd = i % D;
      if (hh >= p.heads_here) continue;
      float mm = -INFINITY;
      for (uint32_t r = 0; r < splits; ++r)
        mm = fmaxf(mm, ptx::ld_shared_cluster_f32(ptx::mapa_shared(mine_addr + (hh * REC + D) * 4, r)));
      float ll = 0.f, oo = 0.f;
      for (uint32_t r = 0; r < splits; ++r) {
        const uint32_t base = ptx::mapa_shared(mine_addr + hh * REC * 4, r);
        const float mr = ptx::ld_shared_cluster_f32(base + D * 4);
        const float w = mr == -INFINITY ? 0.f : ptx::ex2_approx(mr - mm);
        ll = fmaf(ptx::ld_shared_cluster_f32(base + (D + 1) * 4), w, ll);
        oo = fmaf(ptx::ld_shared_cluster_f32(base + dd * 4), w, oo);
      }
      // seq_len == 0: no position contributes; 0 / 0 = NaN, as the five phases give
      softmax::Elem<T>::store1(o + (static_cast<int64_t>(b) * p.heads_q + h0 + hh) * D + dd, oo / ll);
    }
  }
  ptx::cluster_sync_all();  // nobody leaves while its shared memory may still be read
}

}  // namespace attn_decode
}  // namespace tsm100
