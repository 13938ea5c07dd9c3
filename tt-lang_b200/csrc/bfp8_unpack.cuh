// Device-side expansion of one bfloat8_b block (16 values sharing an exponent) to bf16.
// The tile layout is described at the top of bfp8.cu.
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

// 16 sign|magnitude bytes (one block) -> 16 bf16, exact.  A value is (-1)^s * m * 2^(E-133) and a
// bf16 with a zero exponent field is the denormal (-1)^s * mantissa * 2^-133, so the byte is placed
// as sign and mantissa of a bf16 denormal (one byte permute that doubles each byte, one mask) and
// multiplied by 2^E, which is exact: two integer-pipe instructions and one multiply per PAIR of
// values.  2^E itself is a bf16 only up to E = 127; above that the factor is applied as
// 2^127 * 2^(E-127).
__device__ __forceinline__ void unpack_block(const uint4 v, const int E, uint32_t (&o)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  const uint32_t f1 = (uint32_t)(E <= 127 ? E + 127 : 254) << 7;
  const uint32_t f1x2 = f1 | (f1 << 16);
  const __nv_bfloat162 s1 = *reinterpret_cast<const __nv_bfloat162 *>(&f1x2);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const uint32_t x = __byte_perm(w[q >> 1], 0u, (q & 1) ? 0x3322u : 0x1100u) & 0x807f807fu;  // [b, b, b', b']
    const __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&x), s1);
    o[q] = *reinterpret_cast<const uint32_t *>(&y);
  }
  if (E > 127) {
    const uint32_t f2 = (uint32_t)E << 7;   // 2^(E-127)
    const uint32_t f2x2 = f2 | (f2 << 16);
    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&f2x2);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&o[q]), s2);
      o[q] = *reinterpret_cast<const uint32_t *>(&y);
    }
  }
}
