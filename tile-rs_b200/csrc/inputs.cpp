// Seeded synthetic inputs, generated on the host so that the GPU path and the
// CPU checker read the very same buffers.  Counter-based: element i of stream
// `seed` depends on (seed, i) only, so any sub-range can be produced alone
// (each rank of a sharded run generates just its shard).
#include <cmath>
#include <cstdint>
#include <cstring>

#include "../../include/tile_sm100.h"

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

inline uint64_t splitmix64(uint64_t z) {
  z += kGolden;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
inline uint64_t draw(uint64_t seed, uint64_t idx) { return splitmix64(seed ^ (idx * kGolden)); }

inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

// Both members of the Box-Muller pair (2p, 2p+1) come from one log / sqrt; a chunk of the index
// range is walked pair by pair, with the ragged first and last elements handled alone.
template <typename Store>
void fill_normal(int64_t n, uint64_t seed, int64_t first_index, double sigma, Store store) {
  const double two_pi = 6.283185307179586476925286766559;
  const int64_t p_lo = first_index >> 1, p_hi = (first_index + n + 1) >> 1;  // pairs that overlap the range
#pragma omp parallel for schedule(static)
  for (int64_t p = p_lo; p < p_hi; ++p) {
    const uint64_t pair = static_cast<uint64_t>(p);
    const double u1 = (static_cast<double>(draw(seed, 2 * pair) >> 40) + 1.0) * (1.0 / 16777216.0);  // (0, 1]
    const double u2 = static_cast<double>(draw(seed, 2 * pair + 1) >> 40) * (1.0 / 16777216.0);       // [0, 1)
    const double rad = std::sqrt(-2.0 * std::log(u1)) * sigma;
    const int64_t i0 = 2 * p - first_index, i1 = i0 + 1;
    if (i0 >= 0 && i0 < n) store(i0, static_cast<float>(rad * std::cos(two_pi * u2)));
    if (i1 >= 0 && i1 < n) store(i1, static_cast<float>(rad * std::sin(two_pi * u2)));
  }
}

}  // namespace

extern "C" {

int32_t tsm100_fill_uniform_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index) {
  if (n < 0 || (n > 0 && !dst)) return TSM100_ERR_INVALID;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t r = draw(seed, static_cast<uint64_t>(first_index + i)) >> 40;  // top 24 bits
    dst[i] = static_cast<float>(static_cast<double>(r) * (2.0 / 16777216.0) - 1.0);
  }
  return TSM100_OK;
}

int32_t tsm100_fill_normal_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index, double sigma) {
  if (n < 0 || first_index < 0 || (n > 0 && !dst)) return TSM100_ERR_INVALID;
  fill_normal(n, seed, first_index, sigma, [dst](int64_t i, float v) { dst[i] = v; });
  return TSM100_OK;
}

int32_t tsm100_fill_normal_bf16(uint16_t* dst, int64_t n, uint64_t seed, int64_t first_index, double sigma, float factor) {
  if (n < 0 || first_index < 0 || (n > 0 && !dst)) return TSM100_ERR_INVALID;
  fill_normal(n, seed, first_index, sigma, [dst, factor](int64_t i, float v) { dst[i] = f32_to_bf16_rne(v * factor); });
  return TSM100_OK;
}

int32_t tsm100_plant_outliers_f32(float* dst, int64_t n, uint64_t seed, int64_t first_index, uint32_t period,
                                  float value) {
  if (n < 0 || (n > 0 && !dst) || period == 0) return TSM100_ERR_INVALID;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    if (draw(seed, static_cast<uint64_t>(first_index + i)) % period == 0) dst[i] = value;
  return TSM100_OK;
}

int32_t tsm100_scale_f32(float* dst, int64_t n, float factor) {
  if (n < 0 || (n > 0 && !dst)) return TSM100_ERR_INVALID;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] *= factor;
  return TSM100_OK;
}

int32_t tsm100_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  if (n < 0 || (n > 0 && (!dst || !src))) return TSM100_ERR_INVALID;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_rne(src[i]);
  return TSM100_OK;
}

int32_t tsm100_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  if (n < 0 || (n > 0 && (!dst || !src))) return TSM100_ERR_INVALID;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t u = static_cast<uint32_t>(src[i]) << 16;
    std::memcpy(&dst[i], &u, 4);
  }
  return TSM100_OK;
}

}  // extern "C"
