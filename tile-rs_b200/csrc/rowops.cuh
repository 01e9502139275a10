// The other bandwidth-bound row operators of tile_std, built on the row-softmax
// skeleton (softmax.cuh): every element is read from HBM once and written once.
//
//   rms_norm   y[r,c] = x[r,c] * rsqrt(mean_c(x[r,:]^2) + eps)
//              __tile_rms_norm_f32(dst, src, eps, rows, cols)
//              (crates/tile_std/src/tile.rs:2063, wrapper :2731-2738); semantics
//              linalg.mul + linalg.reduce addf + rsqrt(sum / cols + eps) + multiply
//              (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1666-1767).  Replaces
//              the lowering at crates/rustc_codegen_tile/src/mlir_to_gpu.rs:920-977.
//   reduce     y[r] = sum_c x[r,c]  or  max_c x[r,c]
//              __tile_reduce_sum_f32 / __tile_reduce_max_f32 (tile.rs:206-209, wrappers
//              :2352-2367: the result is a ROWS x 1 tile); semantics linalg.fill(0 | -inf)
//              + linalg.reduce (mlir_to_linalg.rs:545-550).  The reference's NVIDIA
//              lowering reduces within one warp only (mlir_to_gpu.rs:2059-2092).
//   silu_mul   y = silu(gate) * up,  silu(x) = x / (1 + exp(-x));  up may be absent
//              __tile_silu_f32 + __tile_mul_f32 (tile.rs:229, :184; wrappers :2416-2422,
//              :2272-2282); semantics mlir_to_linalg.rs:774-782 and :425; the fusion of
//              the pair is the reference's own (mlir_to_gpu.rs:542-641).
//
// Roofline: HBM.  Algorithmic bytes per element: rms_norm 2 * sizeof(T); reduce
// sizeof(T) (+ sizeof(T) per row); silu_mul 3 * sizeof(T) (2 * sizeof(T) without up).
#pragma once

#include "softmax.cuh"

namespace tsm100 {
namespace rowops {

using softmax::Elem;
using softmax::Vec16;
using softmax::ld_stream;
using softmax::st_stream;
using softmax::warp_max;
using softmax::warp_sum;

enum : int { kRmsNorm = 0, kReduceSum = 1, kReduceMax = 2 };

// ---------------------------------------------------------------------------
// LANES threads per row (32: one warp, rows of a CTA are independent; 128 or 256:
// the whole CTA), VPT 16-byte vectors per thread (vector k * LANES + lane).  x must
// be 16-byte aligned with cols a multiple of Elem<T>::kPerVec (the host checks);
// cols <= LANES * VPT * kPerVec.  The loads of a group's next row are in flight
// while the current row is reduced and stored.
// ---------------------------------------------------------------------------
template <typename T, int OP, int VPT, int LANES, int THREADS>
__global__ void __launch_bounds__(THREADS)
row_op_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int32_t cols, float eps) {
  constexpr int PV = Elem<T>::kPerVec;
  constexpr int GROUPS = THREADS / LANES;  // rows in flight per CTA
  constexpr int NW = LANES / 32;           // warps per row
  __shared__ float red[2][NW > 1 ? NW : 1];  // alternating slots: one barrier per row
  const int tid = threadIdx.x, lane = tid % LANES, group = tid / LANES;
  const int nvec = cols / PV;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * GROUPS + group;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * GROUPS;
  constexpr bool kIsMax = OP == kReduceMax;
  const float pad = kIsMax ? -INFINITY : 0.f;

  Vec16 raw[VPT];
  if (first < rows) {
    const Vec16* x0 = reinterpret_cast<const Vec16*>(x + first * cols);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = k * LANES + lane;
      if (i < nvec) raw[k] = ld_stream(x0 + i);
    }
  }
  int parity = 0;
  // Every thread of a CTA runs the same number of iterations when LANES == THREADS; with
  // one warp per row nothing below synchronises across warps.
  for (int64_t row = first; row < rows; row += stride, parity ^= 1) {
    Vec16 nxt[VPT];
    const int64_t next_row = row + stride;
    if (next_row < rows) {
      const Vec16* xn = reinterpret_cast<const Vec16*>(x + next_row * cols);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = k * LANES + lane;
        if (i < nvec) nxt[k] = ld_stream(xn + i);
      }
    }
    float v[VPT][PV];
    float acc[4] = {pad, pad, pad, pad};  // four partial results shorten the dependency chain
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = k * LANES + lane;
      if (i < nvec) {
        Elem<T>::unpack(raw[k], v[k]);
#pragma unroll
        for (int e = 0; e < PV; ++e) {
          if (OP == kRmsNorm) acc[e & 3] = fmaf(v[k][e], v[k][e], acc[e & 3]);
          else if (OP == kReduceSum) acc[e & 3] += v[k][e];
          else acc[e & 3] = fmaxf(acc[e & 3], v[k][e]);
        }
      }
    }
    float a = kIsMax ? fmaxf(fmaxf(acc[0], acc[1]), fmaxf(acc[2], acc[3])) : (acc[0] + acc[1]) + (acc[2] + acc[3]);
    a = kIsMax ? warp_max(a) : warp_sum(a);
    if (NW > 1) {
      if ((tid & 31) == 0) red[parity][tid >> 5] = a;
      __syncthreads();
      a = red[parity][0];
#pragma unroll
      for (int w = 1; w < NW; ++w) a = kIsMax ? fmaxf(a, red[parity][w]) : a + red[parity][w];
      // slot `parity` is rewritten two rows later, after the barrier of the next row
    }
    if (OP == kRmsNorm) {
      const float scale = rsqrtf(a / static_cast<float>(cols) + eps);
      Vec16* yr = reinterpret_cast<Vec16*>(y + row * cols);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = k * LANES + lane;
        if (i < nvec) {
#pragma unroll
          for (int e = 0; e < PV; ++e) v[k][e] *= scale;
          st_stream(yr + i, Elem<T>::pack(v[k]));
        }
      }
    } else {
      if (lane == 0) Elem<T>::store1(y + row, a);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) raw[k] = nxt[k];
  }
}

// ---------------------------------------------------------------------------
// Any width, any alignment: one CTA per row, scalar accesses, the row is read
// twice for rms_norm (once for the reductions).
// ---------------------------------------------------------------------------
template <typename T, int OP, int THREADS>
__global__ void __launch_bounds__(THREADS)
row_op_stream_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols, float eps) {
  __shared__ float red[32];
  constexpr bool kIsMax = OP == kReduceMax;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float a = kIsMax ? -INFINITY : 0.f;
    for (int64_t i = threadIdx.x; i < cols; i += THREADS) {
      const float f = Elem<T>::load1(xr + i);
      if (OP == kRmsNorm) a = fmaf(f, f, a);
      else if (OP == kReduceSum) a += f;
      else a = fmaxf(a, f);
    }
    a = softmax::block_reduce<THREADS>(a, red, kIsMax);
    if (OP == kRmsNorm) {
      const float scale = rsqrtf(a / static_cast<float>(cols) + eps);
      T* yr = y + row * cols;
      for (int64_t i = threadIdx.x; i < cols; i += THREADS) Elem<T>::store1(yr + i, Elem<T>::load1(xr + i) * scale);
    } else if (threadIdx.x == 0) {
      Elem<T>::store1(y + row, a);
    }
  }
}

// ---------------------------------------------------------------------------
// y = silu(gate) * up over n elements (a flat range: the operator is element-wise).
// Vector kernel: gate, up, y 16-byte aligned, n a multiple of kPerVec; UNROLL
// independent 16-byte loads per stream and thread are in flight at a time.
// ---------------------------------------------------------------------------
// f32 storage: libm-grade exp and a true divide (the 1e-5 bar).  16-bit storage holds twice
// the elements per byte and the result is rounded to 8 or 11 bits anyway: ex2.approx and an
// approximate divide keep the kernel on the HBM roofline instead of the FP32 pipe.
template <typename T>
__device__ __forceinline__ float silu(float x) {
  if (sizeof(T) == 4) return x / (1.0f + expf(-x));
  return __fdividef(x, 1.0f + __expf(-x));
}

template <typename T, bool HAS_UP, int UNROLL, int THREADS>
__global__ void __launch_bounds__(THREADS)
silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, int64_t nvec) {
  constexpr int PV = Elem<T>::kPerVec;
  const Vec16* g = reinterpret_cast<const Vec16*>(gate);
  const Vec16* u = reinterpret_cast<const Vec16*>(up);
  Vec16* out = reinterpret_cast<Vec16*>(y);
  const int64_t step = static_cast<int64_t>(gridDim.x) * THREADS;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; base < nvec; base += step * UNROLL) {
    Vec16 gv[UNROLL], uv[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const int64_t i = base + k * step;
      if (i < nvec) {
        gv[k] = ld_stream(g + i);
        if (HAS_UP) uv[k] = ld_stream(u + i);
      }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      const int64_t i = base + k * step;
      if (i < nvec) {
        float a[PV], b[PV];
        Elem<T>::unpack(gv[k], a);
        if (HAS_UP) Elem<T>::unpack(uv[k], b);
#pragma unroll
        for (int e = 0; e < PV; ++e) a[e] = HAS_UP ? silu<T>(a[e]) * b[e] : silu<T>(a[e]);
        st_stream(out + i, Elem<T>::pack(a));
      }
    }
  }
}

template <typename T, bool HAS_UP, int THREADS>
__global__ void __launch_bounds__(THREADS)
silu_mul_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, int64_t n) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * THREADS;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; i < n; i += step) {
    const float s = silu<T>(Elem<T>::load1(gate + i));
    Elem<T>::store1(y + i, HAS_UP ? s * Elem<T>::load1(up + i) : s);
  }
}

}  // namespace rowops
}  // namespace tsm100

// ===========================================================================
// The two steps before decode / prefill attention in a transformer layer.
//
//   rope             x[b, s, h, 2i], x[b, s, h, 2i+1] rotated by angle (start_pos + s) * theta^(-2i / d), in place;
//                    x is [batch][seq_len][heads][d] (token-major).
//                    __tile_rope_inplace_f32 (seq_len = 1) and __tile_rope_prefill_f32
//                    (crates/tile_std/src/tile.rs:2113-2115, :2128-2129); arithmetic of the Metal
//                    lowering (crates/rustc_codegen_tile/src/mlir_to_msl.rs:10707-10728, :10883-10908):
//                    freq = 1 / pow(theta, 2 i / d), angle = float(pos) * freq, f32 cos and sin.
//   kv_cache_update  cache[b, h, start_pos + s, :] = src[b, s, h, :]; cache is [batch][heads][max_seq][d].
//                    __tile_kv_cache_update_f32 and __tile_kv_cache_update_prefill_f32 (tile.rs:2117-2119,
//                    :2131-2132; mlir_to_msl.rs:10730-10741, :10910-10926).
// position, start_pos, theta, max_seq and the head count are run-time constants of those kernels.
// ===========================================================================
namespace tsm100 {
namespace rowops {

// one thread per (batch, token, pair index): the angle is computed once and used for every head
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(T* __restrict__ x, int64_t tokens, int32_t seq_len, int32_t heads, int32_t d, int32_t start_pos, float theta) {
  const int half = d / 2;
  const int64_t n = tokens * half;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t tok = idx / half;
    const int i = static_cast<int>(idx % half);
    const int pos = start_pos + static_cast<int>(tok % seq_len);
    const float freq = 1.0f / powf(theta, 2.0f * static_cast<float>(i) / static_cast<float>(d));
    const float angle = static_cast<float>(pos) * freq;
    float s, c;
    sincosf(angle, &s, &c);
    T* p = x + tok * heads * d + 2 * i;
    for (int h = 0; h < heads; ++h, p += d) {
      const float x0 = Elem<T>::load1(p), x1 = Elem<T>::load1(p + 1);
      Elem<T>::store1(p, x0 * c - x1 * s);
      Elem<T>::store1(p + 1, x0 * s + x1 * c);
    }
  }
}

// The same with 16-byte accesses (head_dim a multiple of the vector, 16-byte aligned buffer): one thread per
// (batch, token, vector of a head row); its PV/2 angles are computed once and used for every head, and the
// loads of four heads are in flight together.  Same formula per pair as above.
template <typename T>
__global__ void __launch_bounds__(256)
rope_vec_kernel(T* __restrict__ x, int64_t tokens, int32_t seq_len, int32_t heads, int32_t d, int32_t start_pos, float theta) {
  constexpr int PV = Elem<T>::kPerVec;
  constexpr int HU = 4;
  const int dv = d / PV;
  const int64_t n = tokens * dv;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t tok = idx / dv;
    const int j = static_cast<int>(idx % dv);
    const int pos = start_pos + static_cast<int>(tok % seq_len);
    float c[PV / 2], s[PV / 2];
#pragma unroll
    for (int e = 0; e < PV / 2; ++e) {
      const int i = j * (PV / 2) + e;
      const float freq = 1.0f / powf(theta, 2.0f * static_cast<float>(i) / static_cast<float>(d));
      const float angle = static_cast<float>(pos) * freq;
      sincosf(angle, &s[e], &c[e]);
    }
    Vec16* p = reinterpret_cast<Vec16*>(x + tok * heads * d) + j;
    auto rotate = [&](const Vec16& raw) -> Vec16 {
      float f[PV], r[PV];
      Elem<T>::unpack(raw, f);
#pragma unroll
      for (int e = 0; e < PV / 2; ++e) {
        const float x0 = f[2 * e], x1 = f[2 * e + 1];
        r[2 * e] = x0 * c[e] - x1 * s[e];
        r[2 * e + 1] = x0 * s[e] + x1 * c[e];
      }
      return Elem<T>::pack(r);
    };
    int h = 0;
    for (; h + HU <= heads; h += HU) {
      Vec16 raw[HU];
#pragma unroll
      for (int u = 0; u < HU; ++u) raw[u] = p[static_cast<int64_t>(h + u) * dv];
#pragma unroll
      for (int u = 0; u < HU; ++u) p[static_cast<int64_t>(h + u) * dv] = rotate(raw[u]);
    }
    for (; h < heads; ++h) p[static_cast<int64_t>(h) * dv] = rotate(p[static_cast<int64_t>(h) * dv]);
  }
}

// VEC = elements per access (16 bytes when rows allow it, else 1); I = index arithmetic type: 32-bit when the
// element count allows it (64-bit divisions cost more than the copy)
template <typename T, int VEC, typename I>
__global__ void __launch_bounds__(256)
kv_cache_update_kernel(const T* __restrict__ src, T* __restrict__ cache, int64_t batch, int32_t seq_len, int32_t heads,
                       int32_t d, int32_t start_pos, int32_t max_seq) {
  const I dv = static_cast<I>(d / VEC);
  const I n = static_cast<I>(batch * seq_len * heads) * dv;
  const I stride = static_cast<I>(gridDim.x) * blockDim.x;
  for (I idx = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int dd = static_cast<int>(idx % dv) * VEC;
    I r = idx / dv;
    const I h = r % static_cast<I>(heads);
    r /= static_cast<I>(heads);
    const I si = r % static_cast<I>(seq_len);
    const int64_t b = static_cast<int64_t>(r / static_cast<I>(seq_len));
    const T* s = src + ((b * seq_len + static_cast<int64_t>(si)) * heads + static_cast<int64_t>(h)) * d + dd;
    T* c = cache + ((b * heads + static_cast<int64_t>(h)) * max_seq + start_pos + static_cast<int64_t>(si)) * d + dd;
    if (VEC == 1) *c = *s;
    else *reinterpret_cast<Vec16*>(c) = *reinterpret_cast<const Vec16*>(s);
  }
}

}  // namespace rowops
}  // namespace tsm100
