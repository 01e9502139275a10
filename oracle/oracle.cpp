// CPU oracle for the tile_std matmul / row-softmax / fused-attention hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
// compared with and the timed CPU baseline; nothing on the product path may
// link, load or call it.
//
// PARITY UNPINNED: the reference holds no golden numeric vector, known-answer
// test or data file for these operators (its tests assert emitted text only),
// and its CPU executor for the linalg bridge is not part of its tree.  The
// functions below therefore restate the arithmetic of the linalg operators the
// reference's bridge emits, each citing the emitter lines it follows, and are
// cross-checked against an independent numpy/float64 statement in the tests.
//
// Conventions: every matrix is row-major and contiguous.  bf16 values travel
// as uint16_t bit patterns, widened exactly to f32 on load (arith.extf) and
// narrowed with round-to-nearest-even on store (arith.truncf), as
// crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1249-1303 lowers the casts.
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -shared -fPIC).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// Round-to-nearest-even narrowing; NaN stays NaN (quiet bit forced).
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}

// One softmax row: linalg.softmax dimension(1)
// (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1305-1343):
//   m = max_j x_j ; e_j = exp(x_j - m) ; s = sum_j e_j ; y_j = e_j / s.
template <typename Acc>
inline void softmax_row(const float* x, float* y, int64_t n) {
  Acc m = -std::numeric_limits<Acc>::infinity();
  for (int64_t j = 0; j < n; ++j) m = x[j] > m ? static_cast<Acc>(x[j]) : m;
  Acc s = 0;
  if (sizeof(Acc) == 4) {
    for (int64_t j = 0; j < n; ++j) {
      float e = expf(x[j] - static_cast<float>(m));
      y[j] = e;
      s += e;
    }
    for (int64_t j = 0; j < n; ++j) y[j] = y[j] / static_cast<float>(s);
  } else {
    std::vector<double> e(n);
    for (int64_t j = 0; j < n; ++j) {
      e[j] = std::exp(static_cast<double>(x[j]) - static_cast<double>(m));
      s += e[j];
    }
    for (int64_t j = 0; j < n; ++j) y[j] = static_cast<float>(e[j] / s);
  }
}

// Attention for one (head) slice, restating the decomposition the bridge emits
// for __tile_attention_f32 (mlir_to_linalg.rs:1781-1902): Kt = transpose(K);
// S = Q*Kt (linalg.matmul, f32, zero-filled); S *= (float)(1/sqrt((double)D));
// P = softmax rows; O = P*V.  With `causal`, the mask of
// __tile_causal_mask_f32 (mlir_to_linalg.rs:1191-1244) is applied between the
// scale and the softmax: S[i][j] = -inf where j > i.
// Rows are independent, so the S x S score tile is produced one row at a time;
// per element the sequence of f32 operations is the one written above.
void attention_slice(const float* q, const float* k, const float* v, float* o,
                     int64_t s_q, int64_t s_kv, int64_t d, bool causal) {
  const float scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(d)));
#pragma omp parallel
  {
    std::vector<float> sc(s_kv), p(s_kv), acc(d);
#pragma omp for schedule(dynamic, 8)
    for (int64_t i = 0; i < s_q; ++i) {
      const float* qi = q + i * d;
      const int64_t lim = causal ? (i + 1 < s_kv ? i + 1 : s_kv) : s_kv;
      for (int64_t j = 0; j < lim; ++j) {
        const float* kj = k + j * d;
        float a = 0.f;
        for (int64_t c = 0; c < d; ++c) a += qi[c] * kj[c];
        sc[j] = a * scale;
      }
      // masked entries are -inf: exp(-inf - m) = 0 contributes nothing, so the
      // softmax over the unmasked prefix equals the softmax over the full row.
      softmax_row<float>(sc.data(), p.data(), lim);
      for (int64_t c = 0; c < d; ++c) acc[c] = 0.f;
      for (int64_t j = 0; j < lim; ++j) {
        const float pj = p[j];
        const float* vj = v + j * d;
        for (int64_t c = 0; c < d; ++c) acc[c] += pj * vj[c];
      }
      std::memcpy(o + i * d, acc.data(), sizeof(float) * d);
    }
  }
}

// One rms_norm row (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1666-1767):
//   sq = x * x (linalg.mul) ; s = 0 + sum_j sq_j (linalg.fill 0 + linalg.reduce addf, in
//   index order) ; rs = rsqrt(s / cols + eps) (arith.divf, arith.addf, math.rsqrt) ;
//   y_j = x_j * rs.  Acc = float follows the bridge's f32 arithmetic, Acc = double is the
//   truth the error bound is taken against.
template <typename Acc>
inline void rms_norm_row(const float* x, float* y, int64_t n, float eps) {
  Acc s = 0;
  for (int64_t j = 0; j < n; ++j) {
    const Acc sq = static_cast<Acc>(x[j]) * static_cast<Acc>(x[j]);
    s += sq;
  }
  const Acc var = s / static_cast<Acc>(static_cast<float>(n)) + static_cast<Acc>(eps);
  const Acc rs = static_cast<Acc>(1) / std::sqrt(var);
  for (int64_t j = 0; j < n; ++j) y[j] = static_cast<float>(static_cast<Acc>(x[j]) * rs);
}

// Row reduction (mlir_to_linalg.rs:545-550: linalg.fill(0 | -inf) + linalg.reduce addf |
// maximumf over dimension 1, in index order).
template <typename Acc>
inline float reduce_row(const float* x, int64_t n, bool is_max) {
  if (is_max) {
    float m = -std::numeric_limits<float>::infinity();
    for (int64_t j = 0; j < n; ++j) m = x[j] > m ? x[j] : m;
    return m;
  }
  Acc s = 0;
  for (int64_t j = 0; j < n; ++j) s += static_cast<Acc>(x[j]);
  return static_cast<float>(s);
}

// silu(x) = x / (1 + exp(-x)) (mlir_to_linalg.rs:774-782: negf, math.exp, addf 1, divf).
template <typename Acc>
inline float silu_one(float x) {
  if (sizeof(Acc) == 4) return x / (expf(-x) + 1.0f);
  return static_cast<float>(static_cast<double>(x) / (std::exp(-static_cast<double>(x)) + 1.0));
}

}  // namespace

extern "C" {

int orc_num_threads(void) {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Sets the number of OpenMP threads the functions below use (launchers such as torchrun
// export OMP_NUM_THREADS=1, which would otherwise make a "CPU baseline" single-threaded).
void orc_set_num_threads(int n) {
#if defined(_OPENMP)
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void orc_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}

// C[M,N] = A[M,K] * B[K,N]; linalg.fill 0 then linalg.matmul
// (mlir_to_linalg.rs:1345-1393): C starts at zero and accumulates in f32, k
// ascending for every (i,j).  The i-k-j loop order keeps that per-element
// order while letting the compiler vectorise over j.
// With b_transposed != 0, B is stored [N,K] (the __tile_matmul_transposed_*
// weight layout, crates/tile_std/src/tile.rs:2017-2031).
void orc_gemm_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                  int b_transposed) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    float* ci = c + i * n;
    for (int64_t j = 0; j < n; ++j) ci[j] = 0.f;
    if (!b_transposed) {
      for (int64_t kk = 0; kk < k; ++kk) {
        const float aik = a[i * k + kk];
        const float* bk = b + kk * n;
        for (int64_t j = 0; j < n; ++j) ci[j] += aik * bk[j];
      }
    } else {
      for (int64_t j = 0; j < n; ++j) {
        const float* bj = b + j * k;
        float acc = 0.f;
        for (int64_t kk = 0; kk < k; ++kk) acc += a[i * k + kk] * bj[kk];
        ci[j] = acc;
      }
    }
  }
}

// Same contraction with f64 accumulation: the "truth" the error bounds of the
// f32 configuration are stated against.
void orc_gemm_f64acc(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                     int b_transposed) {
#pragma omp parallel
  {
    std::vector<double> row(n);
#pragma omp for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
      for (int64_t j = 0; j < n; ++j) row[j] = 0.0;
      if (!b_transposed) {
        for (int64_t kk = 0; kk < k; ++kk) {
          const double aik = a[i * k + kk];
          const float* bk = b + kk * n;
          for (int64_t j = 0; j < n; ++j) row[j] += aik * static_cast<double>(bk[j]);
        }
      } else {
        for (int64_t j = 0; j < n; ++j) {
          const float* bj = b + j * k;
          double acc = 0.0;
          for (int64_t kk = 0; kk < k; ++kk) acc += static_cast<double>(a[i * k + kk]) * bj[kk];
          row[j] = acc;
        }
      }
      for (int64_t j = 0; j < n; ++j) c[i * n + j] = static_cast<float>(row[j]);
    }
  }
}

// 16-bit-input contraction (__tile_matmul_f16 family, tile.rs:1982-1986,
// :2593-2601, :2666-2674; accumulate f32 per the comment at :2657-2664) on
// bf16 bit patterns: inputs widened exactly, f32 accumulate, the unrounded f32
// result written to c_f32 and, if c_bf16 != NULL, one RNE narrowing to bf16.
void orc_gemm_bf16(const uint16_t* a, const uint16_t* b, float* c_f32, uint16_t* c_bf16,
                   int64_t m, int64_t n, int64_t k, int b_transposed) {
  std::vector<float> bf(static_cast<size_t>(k) * n);
  orc_bf16_to_f32(b, bf.data(), k * n);
#pragma omp parallel
  {
    std::vector<float> arow(k);
#pragma omp for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
      for (int64_t kk = 0; kk < k; ++kk) arow[kk] = bf16_to_f32(a[i * k + kk]);
      float* ci = c_f32 + i * n;
      for (int64_t j = 0; j < n; ++j) ci[j] = 0.f;
      if (!b_transposed) {
        for (int64_t kk = 0; kk < k; ++kk) {
          const float aik = arow[kk];
          const float* bk = bf.data() + kk * n;
          for (int64_t j = 0; j < n; ++j) ci[j] += aik * bk[j];
        }
      } else {
        for (int64_t j = 0; j < n; ++j) {
          const float* bj = bf.data() + j * k;
          float acc = 0.f;
          for (int64_t kk = 0; kk < k; ++kk) acc += arow[kk] * bj[kk];
          ci[j] = acc;
        }
      }
      if (c_bf16)
        for (int64_t j = 0; j < n; ++j) c_bf16[i * n + j] = f32_to_bf16(ci[j]);
    }
  }
}

// Row softmax, f32 (mlir_to_linalg.rs:1305-1343; the same five steps appear in
// crates/tile_std/src/kernel_ops.rs:245-271 and mlir_to_gpu.rs:1266-1326).
void orc_softmax_f32(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) softmax_row<float>(x + r * cols, y + r * cols, cols);
}

// f64-internal variant, used as the truth for the f32 error bound.
void orc_softmax_f64acc(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) softmax_row<double>(x + r * cols, y + r * cols, cols);
}

// bf16-I/O row softmax: widen, f32 math, unrounded f32 to y_f32 (may be NULL)
// and RNE bf16 to y_bf16 (may be NULL).
void orc_softmax_bf16(const uint16_t* x, float* y_f32, uint16_t* y_bf16, int64_t rows,
                      int64_t cols) {
#pragma omp parallel
  {
    std::vector<float> xr(cols), yr(cols);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      for (int64_t j = 0; j < cols; ++j) xr[j] = bf16_to_f32(x[r * cols + j]);
      softmax_row<float>(xr.data(), yr.data(), cols);
      if (y_f32) std::memcpy(y_f32 + r * cols, yr.data(), sizeof(float) * cols);
      if (y_bf16)
        for (int64_t j = 0; j < cols; ++j) y_bf16[r * cols + j] = f32_to_bf16(yr[j]);
    }
  }
}

// __tile_rms_norm_f32 on an f32 tile; f64acc != 0 selects the truth variant.
void orc_rms_norm_f32(const float* x, float* y, int64_t rows, int64_t cols, float eps, int f64acc) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    if (f64acc) rms_norm_row<double>(x + r * cols, y + r * cols, cols, eps);
    else rms_norm_row<float>(x + r * cols, y + r * cols, cols, eps);
  }
}

// bf16-I/O rms_norm: widen, f32 math, unrounded f32 to y_f32 (may be NULL) and RNE bf16 to
// y_bf16 (may be NULL).
void orc_rms_norm_bf16(const uint16_t* x, float* y_f32, uint16_t* y_bf16, int64_t rows, int64_t cols, float eps) {
#pragma omp parallel
  {
    std::vector<float> xr(cols), yr(cols);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      for (int64_t j = 0; j < cols; ++j) xr[j] = bf16_to_f32(x[r * cols + j]);
      rms_norm_row<float>(xr.data(), yr.data(), cols, eps);
      if (y_f32) std::memcpy(y_f32 + r * cols, yr.data(), sizeof(float) * cols);
      if (y_bf16)
        for (int64_t j = 0; j < cols; ++j) y_bf16[r * cols + j] = f32_to_bf16(yr[j]);
    }
  }
}

// __tile_reduce_sum_f32 / __tile_reduce_max_f32: y[rows].
void orc_reduce_f32(const float* x, float* y, int64_t rows, int64_t cols, int is_max, int f64acc) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    y[r] = f64acc ? reduce_row<double>(x + r * cols, cols, is_max != 0) : reduce_row<float>(x + r * cols, cols, is_max != 0);
}

// __tile_silu_f32 followed by __tile_mul_f32 (linalg.mul, mlir_to_linalg.rs:425); up == NULL
// gives silu alone.
void orc_silu_mul_f32(const float* gate, const float* up, float* y, int64_t n, int f64acc) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    if (f64acc) {
      const double g = gate[i];
      const double s = g / (std::exp(-g) + 1.0);
      y[i] = static_cast<float>(up ? s * static_cast<double>(up[i]) : s);
    } else {
      const float s = silu_one<float>(gate[i]);
      y[i] = up ? s * up[i] : s;
    }
  }
}

// bf16-I/O: widen, f32 math, unrounded f32 and RNE bf16 results (either may be NULL).
void orc_silu_mul_bf16(const uint16_t* gate, const uint16_t* up, float* y_f32, uint16_t* y_bf16, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float s = silu_one<float>(bf16_to_f32(gate[i]));
    const float r = up ? s * bf16_to_f32(up[i]) : s;
    if (y_f32) y_f32[i] = r;
    if (y_bf16) y_bf16[i] = f32_to_bf16(r);
  }
}

// Batched attention on f32 tensors: Q,O [batch][hq][s][d], K,V [batch][hkv][s][d].
// hq == hkv gives __tile_attention_f32 per (batch, head) slice
// (mlir_to_linalg.rs:1781-1902), non-causal unless `causal`.  hq > hkv is the
// grouped-query form of __tile_attention_gqa_* as the NVIDIA emitter defines it
// (mlir_to_gpu.rs:1624-1711): kv_head = h / (hq / hkv), scale 1/sqrt(d); that
// intrinsic is always causal there, so callers pass causal = 1 for it.
void orc_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t batch,
                       int64_t hq, int64_t hkv, int64_t s, int64_t d, int causal) {
  const int64_t group = hq / hkv;
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t h = 0; h < hq; ++h) {
      const int64_t g = h / group;
      attention_slice(q + ((b * hq + h) * s) * d, k + ((b * hkv + g) * s) * d,
                      v + ((b * hkv + g) * s) * d, o + ((b * hq + h) * s) * d, s, s, d,
                      causal != 0);
    }
}

// bf16-input attention: Q,K,V widened to f32, all statistics and accumulation
// in f32, unrounded f32 output to o_f32 and (if non-NULL) RNE bf16 to o_bf16.
// `q_rows`/`q_row0` restrict the computed query rows to [q_row0, q_row0+q_rows)
// of every head so that long sequences can be spot-checked; outputs are then
// [batch][hq][q_rows][d].
void orc_attention_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* o_f32,
                        uint16_t* o_bf16, int64_t batch, int64_t hq, int64_t hkv, int64_t s,
                        int64_t d, int causal, int64_t q_row0, int64_t q_rows) {
  const int64_t group = hq / hkv;
  std::vector<float> qf(static_cast<size_t>(q_rows) * d), kf(static_cast<size_t>(s) * d),
      vf(static_cast<size_t>(s) * d), of(static_cast<size_t>(q_rows) * d);
  const float scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(d)));
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t h = 0; h < hq; ++h) {
      const int64_t g = h / group;
      orc_bf16_to_f32(q + ((b * hq + h) * s + q_row0) * d, qf.data(), q_rows * d);
      if (h % group == 0 || h == 0) {
        orc_bf16_to_f32(k + ((b * hkv + g) * s) * d, kf.data(), s * d);
        orc_bf16_to_f32(v + ((b * hkv + g) * s) * d, vf.data(), s * d);
      }
#pragma omp parallel
      {
        std::vector<float> sc(s), p(s), acc(d);
#pragma omp for schedule(dynamic, 8)
        for (int64_t i = 0; i < q_rows; ++i) {
          const int64_t gi = q_row0 + i;  // global query row decides the mask
          const float* qi = qf.data() + i * d;
          const int64_t lim = causal ? (gi + 1 < s ? gi + 1 : s) : s;
          for (int64_t j = 0; j < lim; ++j) {
            const float* kj = kf.data() + j * d;
            float a = 0.f;
            for (int64_t c = 0; c < d; ++c) a += qi[c] * kj[c];
            sc[j] = a * scale;
          }
          softmax_row<float>(sc.data(), p.data(), lim);
          for (int64_t c = 0; c < d; ++c) acc[c] = 0.f;
          for (int64_t j = 0; j < lim; ++j) {
            const float pj = p[j];
            const float* vj = vf.data() + j * d;
            for (int64_t c = 0; c < d; ++c) acc[c] += pj * vj[c];
          }
          std::memcpy(of.data() + i * d, acc.data(), sizeof(float) * d);
        }
      }
      const int64_t off = ((b * hq + h) * q_rows) * d;
      if (o_f32) std::memcpy(o_f32 + off, of.data(), sizeof(float) * q_rows * d);
      if (o_bf16) orc_f32_to_bf16(of.data(), o_bf16 + off, q_rows * d);
    }
}

// Parity metrics between a result y and the oracle r (n elements):
//   out[0] = max|y-r|, out[1] = max|r|, out[2] = ||y-r||_F, out[3] = ||r||_F,
//   out[4] = max over r_i >= floor of |y_i-r_i|/r_i (0 if none).
void orc_compare_f32(const float* y, const float* r, int64_t n, double floor_r, double* out) {
  double mad = 0, mr = 0, se = 0, sr = 0, mrel = 0;
#pragma omp parallel for reduction(max : mad, mr, mrel) reduction(+ : se, sr) schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const double yi = y[i], ri = r[i];
    const double dlt = std::fabs(yi - ri);
    mad = dlt > mad ? dlt : mad;
    mr = std::fabs(ri) > mr ? std::fabs(ri) : mr;
    se += dlt * dlt;
    sr += ri * ri;
    if (ri >= floor_r && floor_r > 0) {
      const double rel = dlt / ri;
      mrel = rel > mrel ? rel : mrel;
    }
  }
  out[0] = mad;
  out[1] = mr;
  out[2] = std::sqrt(se);
  out[3] = std::sqrt(sr);
  out[4] = mrel;
}

// __tile_attention_decode_f32 with a leading batch: q, o [batch][hq][d], caches
// [batch][hkv][max_seq][d], positions p < seq_len, kv head = h / (hq / hkv).  The five phases
// of crates/rustc_codegen_tile/src/mlir_to_msl.rs:10747-10812: score = (q . K_p) * rsqrt(d),
// max, e = exp(score - max) and its sum, normalise, weighted V sum over positions in order.
// f64acc != 0 keeps every intermediate in double (the truth for the error bound).
void orc_attention_decode_f32(const float* q, const float* kc, const float* vc, float* o, int64_t batch, int64_t hq,
                              int64_t hkv, int64_t seq_len, int64_t max_seq, int64_t d, int f64acc) {
  const int64_t group = hq / hkv;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t h = 0; h < hq; ++h) {
      const float* qh = q + (b * hq + h) * d;
      const float* kh = kc + (b * hkv + h / group) * max_seq * d;
      const float* vh = vc + (b * hkv + h / group) * max_seq * d;
      float* oh = o + (b * hq + h) * d;
      if (f64acc) {
        std::vector<double> sc(seq_len);
        const double scale = 1.0 / std::sqrt(static_cast<double>(d));
        double mx = -std::numeric_limits<double>::infinity();
        for (int64_t p = 0; p < seq_len; ++p) {
          double dot = 0;
          for (int64_t j = 0; j < d; ++j) dot += static_cast<double>(qh[j]) * kh[p * d + j];
          sc[p] = dot * scale;
          mx = sc[p] > mx ? sc[p] : mx;
        }
        double sum = 0;
        for (int64_t p = 0; p < seq_len; ++p) {
          sc[p] = std::exp(sc[p] - mx);
          sum += sc[p];
        }
        for (int64_t j = 0; j < d; ++j) {
          double acc = 0;
          for (int64_t p = 0; p < seq_len; ++p) acc += sc[p] / sum * vh[p * d + j];
          oh[j] = static_cast<float>(acc);
        }
      } else {
        std::vector<float> sc(seq_len);
        const float scale = 1.0f / std::sqrt(static_cast<float>(d));
        float mx = -std::numeric_limits<float>::infinity();
        for (int64_t p = 0; p < seq_len; ++p) {
          float dot = 0.f;
          for (int64_t j = 0; j < d; ++j) dot += qh[j] * kh[p * d + j];
          sc[p] = dot * scale;
          mx = sc[p] > mx ? sc[p] : mx;
        }
        float sum = 0.f;
        for (int64_t p = 0; p < seq_len; ++p) {
          sc[p] = expf(sc[p] - mx);
          sum += sc[p];
        }
        const float inv = 1.0f / sum;
        for (int64_t p = 0; p < seq_len; ++p) sc[p] *= inv;
        for (int64_t j = 0; j < d; ++j) {
          float acc = 0.f;
          for (int64_t p = 0; p < seq_len; ++p) acc += sc[p] * vh[p * d + j];
          oh[j] = acc;
        }
      }
    }
}

// bf16 storage: widen q and the caches exactly, f32 arithmetic as above, unrounded f32 result
// to o_f32 (may be NULL) and RNE bf16 to o_bf16 (may be NULL).
void orc_attention_decode_bf16(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, float* o_f32, uint16_t* o_bf16,
                               int64_t batch, int64_t hq, int64_t hkv, int64_t seq_len, int64_t max_seq, int64_t d) {
  const int64_t nq = batch * hq * d, nkv = batch * hkv * max_seq * d;
  std::vector<float> qf(nq), kf(nkv), vf(nkv), of(nq);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < nq; ++i) qf[i] = bf16_to_f32(q[i]);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < nkv; ++i) {
    kf[i] = bf16_to_f32(kc[i]);
    vf[i] = bf16_to_f32(vc[i]);
  }
  orc_attention_decode_f32(qf.data(), kf.data(), vf.data(), of.data(), batch, hq, hkv, seq_len, max_seq, d, 0);
  if (o_f32) std::memcpy(o_f32, of.data(), sizeof(float) * nq);
  if (o_bf16)
    for (int64_t i = 0; i < nq; ++i) o_bf16[i] = f32_to_bf16(of[i]);
}

// __tile_rope_inplace_f32 / __tile_rope_prefill_f32 on x [batch][seq_len][heads][d], in place
// (crates/rustc_codegen_tile/src/mlir_to_msl.rs:10707-10728, :10883-10908): for pair index i of
// the token at position pos = start_pos + s: freq = 1 / pow(theta, 2 i / d), angle = float(pos) * freq,
// (x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos), all in f32; f64acc != 0 evaluates the same in double.
void orc_rope_f32(float* x, int64_t batch, int64_t seq_len, int64_t heads, int64_t d, int64_t start_pos, float theta, int f64acc) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t s = 0; s < seq_len; ++s)
      for (int64_t i = 0; i < d / 2; ++i) {
        const int64_t pos = start_pos + s;
        double c, sn;
        if (f64acc) {
          const double ang = static_cast<double>(pos) / std::pow(static_cast<double>(theta), 2.0 * i / static_cast<double>(d));
          c = std::cos(ang);
          sn = std::sin(ang);
        } else {
          const float freq = 1.0f / powf(theta, 2.0f * static_cast<float>(i) / static_cast<float>(d));
          const float ang = static_cast<float>(pos) * freq;
          c = cosf(ang);
          sn = sinf(ang);
        }
        for (int64_t h = 0; h < heads; ++h) {
          float* p = x + ((b * seq_len + s) * heads + h) * d + 2 * i;
          if (f64acc) {
            const double x0 = p[0], x1 = p[1];
            p[0] = static_cast<float>(x0 * c - x1 * sn);
            p[1] = static_cast<float>(x0 * sn + x1 * c);
          } else {
            const float x0 = p[0], x1 = p[1], cf = static_cast<float>(c), sf = static_cast<float>(sn);
            p[0] = x0 * cf - x1 * sf;
            p[1] = x0 * sf + x1 * cf;
          }
        }
      }
}

// __tile_kv_cache_update_f32 / _prefill_f32 (mlir_to_msl.rs:10730-10741, :10910-10926), any 4-byte or 2-byte
// element: cache[b][h][start_pos + s][:] = src[b][s][h][:].
void orc_kv_cache_update(const void* src, void* cache, int64_t elem_bytes, int64_t batch, int64_t seq_len, int64_t heads,
                         int64_t d, int64_t start_pos, int64_t max_seq) {
  const char* sp = static_cast<const char*>(src);
  char* cp = static_cast<char*>(cache);
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t s = 0; s < seq_len; ++s)
      for (int64_t h = 0; h < heads; ++h)
        std::memcpy(cp + (((b * heads + h) * max_seq + start_pos + s) * d) * elem_bytes,
                    sp + (((b * seq_len + s) * heads + h) * d) * elem_bytes, d * elem_bytes);
}

// __tile_attention_prefill_f32 (crates/rustc_codegen_tile/src/mlir_to_msl.rs:10928-11010, without its cap of 256
// cache positions): q, o token-major [seq_len][hq][d], caches [hkv][max_seq][d]; the token at index s sits at
// position start_pos + s and sees cache positions 0 .. start_pos + s; scale rsqrt(d); the five phases in f32
// (f64acc != 0: in double).
void orc_attention_prefill_f32(const float* q, const float* kc, const float* vc, float* o, int64_t hq, int64_t hkv,
                               int64_t seq_len, int64_t start_pos, int64_t max_seq, int64_t d, int f64acc) {
  const int64_t group = hq / hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
  for (int64_t s = 0; s < seq_len; ++s)
    for (int64_t h = 0; h < hq; ++h) {
      const int64_t n = start_pos + s + 1;  // visible positions
      const float* qh = q + (s * hq + h) * d;
      const float* kh = kc + (h / group) * max_seq * d;
      const float* vh = vc + (h / group) * max_seq * d;
      float* oh = o + (s * hq + h) * d;
      if (f64acc) {
        std::vector<double> sc(n);
        const double scale = 1.0 / std::sqrt(static_cast<double>(d));
        double mx = -std::numeric_limits<double>::infinity(), sum = 0;
        for (int64_t p = 0; p < n; ++p) {
          double dot = 0;
          for (int64_t j = 0; j < d; ++j) dot += static_cast<double>(qh[j]) * kh[p * d + j];
          sc[p] = dot * scale;
          mx = sc[p] > mx ? sc[p] : mx;
        }
        for (int64_t p = 0; p < n; ++p) {
          sc[p] = std::exp(sc[p] - mx);
          sum += sc[p];
        }
        for (int64_t j = 0; j < d; ++j) {
          double acc = 0;
          for (int64_t p = 0; p < n; ++p) acc += sc[p] / sum * vh[p * d + j];
          oh[j] = static_cast<float>(acc);
        }
      } else {
        std::vector<float> sc(n);
        const float scale = 1.0f / std::sqrt(static_cast<float>(d));
        float mx = -std::numeric_limits<float>::infinity(), sum = 0.f;
        for (int64_t p = 0; p < n; ++p) {
          float dot = 0.f;
          for (int64_t j = 0; j < d; ++j) dot += qh[j] * kh[p * d + j];
          sc[p] = dot * scale;
          mx = sc[p] > mx ? sc[p] : mx;
        }
        for (int64_t p = 0; p < n; ++p) {
          sc[p] = expf(sc[p] - mx);
          sum += sc[p];
        }
        const float inv = 1.0f / sum;
        for (int64_t j = 0; j < d; ++j) {
          float acc = 0.f;
          for (int64_t p = 0; p < n; ++p) acc += sc[p] * inv * vh[p * d + j];
          oh[j] = acc;
        }
      }
    }
}

}  // extern "C"
