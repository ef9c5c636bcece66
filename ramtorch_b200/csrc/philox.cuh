// Philox4x32-10 (Salmon et al., SC'11) for the stochastic-rounding draws.
// Counter/key layout is the one documented in include/rt_b200.h ("Random bits"):
//   key = (seed lo, seed hi), counter = (i >> 3, tensor_id, step, stream);
//   the 4 output words carry the 16-bit draws of elements 8*(i>>3) .. 8*(i>>3)+7.
#pragma once
#include <stdint.h>

namespace rt {

constexpr uint32_t kPhiloxM0 = 0xD2511F53u;
constexpr uint32_t kPhiloxM1 = 0xCD9E8D57u;
constexpr uint32_t kPhiloxW0 = 0x9E3779B9u;
constexpr uint32_t kPhiloxW1 = 0xBB67AE85u;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    // 32x32 -> 64 products; the compiler emits one wide multiply per pair.
    const uint64_t p0 = (uint64_t)kPhiloxM0 * c.x;
    const uint64_t p1 = (uint64_t)kPhiloxM1 * c.z;
    uint4 n;
    n.x = (uint32_t)(p1 >> 32) ^ c.y ^ k.x;
    n.y = (uint32_t)p1;
    n.z = (uint32_t)(p0 >> 32) ^ c.w ^ k.y;
    n.w = (uint32_t)p0;
    c = n;
    k.x += kPhiloxW0;
    k.y += kPhiloxW1;
  }
  return c;
}

// The key schedule (k + r * W per round) depends on the seed only, so the big kernels receive it
// ready-made as a kernel argument: twenty constant-bank operands instead of twenty integer adds
// per Philox call.
struct PhiloxKeys {
  uint32_t k[20];
};
inline PhiloxKeys philox_keys(uint64_t seed) {
  PhiloxKeys out;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    out.k[2 * r] = k0;
    out.k[2 * r + 1] = k1;
    k0 += kPhiloxW0;
    k1 += kPhiloxW1;
  }
  return out;
}
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, const PhiloxKeys& keys) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)kPhiloxM0 * c.x;
    const uint64_t p1 = (uint64_t)kPhiloxM1 * c.z;
    uint4 n;
    n.x = (uint32_t)(p1 >> 32) ^ c.y ^ keys.k[2 * r];
    n.y = (uint32_t)p1;
    n.z = (uint32_t)(p0 >> 32) ^ c.w ^ keys.k[2 * r + 1];
    n.w = (uint32_t)p0;
    c = n;
  }
  return c;
}
__device__ __forceinline__ uint4 draws8(const PhiloxKeys& keys, uint32_t tensor_id, uint32_t step,
                                        uint32_t stream, uint32_t group8) {
  return philox4x32_10(make_uint4(group8, tensor_id, step, stream), keys);
}
__device__ __forceinline__ uint32_t draw1(const PhiloxKeys& keys, uint32_t tensor_id, uint32_t step,
                                          uint32_t stream, int64_t i) {
  const uint4 o = draws8(keys, tensor_id, step, stream, (uint32_t)((uint64_t)i >> 3));
  const uint32_t j = (uint32_t)i & 7u;
  const uint32_t w = (j >> 1) == 0 ? o.x : (j >> 1) == 1 ? o.y : (j >> 1) == 2 ? o.z : o.w;
  return (j & 1u) ? (w >> 16) : (w & 0xFFFFu);
}

// The eight 16-bit draws of group `group8` (= element index >> 3), packed two per word:
// element j of the group uses word j>>1, low half for even j, high half for odd j.
__device__ __forceinline__ uint4 draws8(uint64_t seed, uint32_t tensor_id, uint32_t step,
                                        uint32_t stream, uint32_t group8) {
  return philox4x32_10(make_uint4(group8, tensor_id, step, stream),
                       make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
}

__device__ __forceinline__ uint32_t draw1(uint64_t seed, uint32_t tensor_id, uint32_t step,
                                          uint32_t stream, int64_t i) {
  const uint4 o = draws8(seed, tensor_id, step, stream, (uint32_t)((uint64_t)i >> 3));
  const uint32_t j = (uint32_t)i & 7u;
  const uint32_t w = (j >> 1) == 0 ? o.x : (j >> 1) == 1 ? o.y : (j >> 1) == 2 ? o.z : o.w;
  return (j & 1u) ? (w >> 16) : (w & 0xFFFFu);
}

}  // namespace rt
