// Counter-based noise shared by the fused LM-head sampler and the restricted (top-k / top-p) sampler: both draw the
// same Gumbel variate for a given (seed, row, vocabulary index), so an unrestricted call of either picks the same token.
#pragma once
#include <cstdint>

namespace artb {

__device__ __forceinline__ uint32_t mix32(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

__device__ __forceinline__ float gumbel_noise(uint32_t seed, uint32_t row, uint32_t col) {
  uint32_t h = mix32(seed ^ (row * 0x9e3779b1u));
  h = mix32(h ^ (col * 0x85ebca77u) ^ 0x27d4eb2fu);
  const float u = (static_cast<float>(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(-__logf(u));
}

}  // namespace artb
