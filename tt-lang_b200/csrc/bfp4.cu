// bfloat4_b block-float weights: host packer / unpacker, device unpack kernel and the bfp4-weight matmul.
//
// The reference fixes the tile size only: a 32x32 bfloat4_b tile takes 576 bytes = 512 value bytes + 64
// shared-exponent bytes (python/ttl/dtype_utils.py:178-179, dtype alias :82-83).  The layout used here completes that the same
// way as for bfloat8_b (csrc/bfp8.cu) - a design choice of this library, applied identically by the CPU packer,
// the CPU oracle and the GPU kernel; byte-compatibility with Tenstorrent tensors is not claimed:
//
//   * tiles in row-major tile order, four 16x16 faces per tile (face f = 2*(r/16) + (c/16)), a block = one face
//     row = 16 consecutive elements of one matrix row;
//   * bytes [0, 64) of a tile: block exponents, index f*16 + (r%16), the largest biased fp32 exponent among the
//     block's values (0 if all are zero / denormal);
//   * bytes [64, 576): 8 bytes per block at 64 + f*128 + (r%16)*8; value j of the block is the low (j even) or
//     high (j odd) nibble of byte j/2: bit 3 = sign, bits 2..0 = magnitude m, value = (-1)^sign * m * 2^(E - 129)
//     (the largest element of a block has m in [4, 7]);
//   * m = |x| * 2^(129 - E) rounded to nearest, ties to even, saturated at 7.
#include <cuda_bf16.h>

#include <cmath>
#include <cstring>

#include "ctx.h"

int ttlb_launch_gemm_bf16_ex(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                             int64_t m, int64_t n, int64_t k, bool multicast, cudaStream_t stream);

int ttlb_launch_gemm_bf16_full(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, bool multicast, const void *bias, int64_t ldbias,
                               cudaStream_t stream);

namespace {

inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

// sign | 3-bit magnitude of x for block exponent E
inline uint8_t quantise4(uint32_t bits, int E) {
  const int e = (int)((bits >> 23) & 0xff);
  const uint8_t sign = (uint8_t)((bits >> 31) << 3);
  if (e == 0 || E == 0) return sign;                       // zero / denormal input
  const uint32_t sig = (bits & 0x7fffffu) | 0x800000u;     // 24-bit significand, value = sig * 2^(e-150)
  const int shift = 21 + (E - e);                          // m = sig >> shift, rounded
  uint32_t m;
  if (shift >= 32) {
    m = 0;
  } else {
    const uint32_t q = sig >> shift;
    const uint32_t rem = sig & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    m = q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
  }
  if (m > 7u) m = 7u;
  return (uint8_t)(sign | m);
}

// One thread per block of 16 values (8 packed bytes in, 32 bytes of bf16 out); a 256-thread CTA expands 4
// consecutive tiles of one tile row.  m * 2^(E-129) has a 3-bit significand: exact in bf16, denormals included.
__global__ void __launch_bounds__(256) ttlb_unpack_bfp4_kernel(const uint8_t *__restrict__ tiles, int tile_cols_total,
                                                             int tile_col0, int tile_rows, int tile_cols,
                                                             __nv_bfloat16 *__restrict__ out, long long ld) {
  const int blk = threadIdx.x & 63;
  const int tc = blockIdx.x * 4 + (threadIdx.x >> 6);
  if (tc >= tile_cols) return;
  const int f = blk >> 4, fr = blk & 15;
  for (int tr = blockIdx.y; tr < tile_rows; tr += gridDim.y) {
    const uint8_t *tile = tiles + ((long long)tr * tile_cols_total + tile_col0 + tc) * TTLB_BFP4_TILE_BYTES;
    const int E = tile[blk];
    const uint2 v = __ldcs(reinterpret_cast<const uint2 *>(tile + 64 + f * 128 + fr * 8));
    const uint32_t w[2] = {v.x, v.y};
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint32_t lo = (w[q >> 2] >> ((q & 3) * 8)) & 0xfu, hi = (w[q >> 2] >> ((q & 3) * 8 + 4)) & 0xfu;
      const float x0 = ldexpf((float)(lo & 7u), E - 129), x1 = ldexpf((float)(hi & 7u), E - 129);
      const __nv_bfloat162 y = __floats2bfloat162_rn((lo & 8u) ? -x0 : x0, (hi & 8u) ? -x1 : x1);
      o[q] = *reinterpret_cast<const uint32_t *>(&y);
    }
    const long long row = (long long)tr * 32 + (f >> 1) * 16 + fr;
    const long long col = (long long)tc * 32 + (f & 1) * 16;
    uint4 *dst = reinterpret_cast<uint4 *>(out + row * ld + col);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

int check_args(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total, int64_t tile_col0, int64_t k, int64_t n) {
  if (!tiles || ((uintptr_t)tiles % 16)) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp4: tile pointer null or misaligned");
  if (k <= 0 || n <= 0 || (k % 32) || (n % 32))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp4: K and N must be positive multiples of 32");
  if (tile_col0 < 0 || tile_cols_total <= 0 || tile_col0 + n / 32 > tile_cols_total)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp4: column window exceeds the packed matrix");
  return TTLB_OK;
}

int launch_unpack(ttlb_ctx *ctx, const uint8_t *tiles, int64_t tile_cols_total, int64_t tile_col0, int64_t tile_rows,
                  int64_t tile_cols, void *out, int64_t ld, cudaStream_t s) {
  const unsigned gx = (unsigned)((tile_cols + 3) / 4);
  const unsigned gy = (unsigned)(tile_rows < 65535 ? tile_rows : 65535);
  ttlb_unpack_bfp4_kernel<<<dim3(gx, gy), 256, 0, s>>>(tiles, (int)tile_cols_total, (int)tile_col0, (int)tile_rows,
                                                         (int)tile_cols, reinterpret_cast<__nv_bfloat16 *>(out), ld);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}

}  // namespace

extern "C" int ttlb_pack_bfp4_b(const float *src, int64_t rows, int64_t cols, uint8_t *dst_tiles) {
  if (!src || !dst_tiles || rows <= 0 || cols <= 0 || (rows % 32) || (cols % 32)) return TTLB_ERR_INVALID_ARG;
  const int64_t tcs = cols / 32;
  for (int64_t tr = 0; tr < rows / 32; ++tr)
    for (int64_t tc = 0; tc < tcs; ++tc) {
      uint8_t *tile = dst_tiles + (tr * tcs + tc) * TTLB_BFP4_TILE_BYTES;
      for (int f = 0; f < 4; ++f)
        for (int fr = 0; fr < 16; ++fr) {
          const float *p = src + (tr * 32 + (f >> 1) * 16 + fr) * cols + tc * 32 + (f & 1) * 16;
          int E = 0;
          for (int j = 0; j < 16; ++j) {
            const int e = (int)((f32_bits(p[j]) >> 23) & 0xff);
            if (e == 0xff) return TTLB_ERR_INVALID_ARG;  // inf / nan cannot be represented
            if (e > E) E = e;
          }
          tile[f * 16 + fr] = (uint8_t)E;
          uint8_t *q = tile + 64 + f * 128 + fr * 8;
          for (int j = 0; j < 16; j += 2)
            q[j >> 1] = (uint8_t)(quantise4(f32_bits(p[j]), E) | (quantise4(f32_bits(p[j + 1]), E) << 4));
        }
    }
  return TTLB_OK;
}

extern "C" int ttlb_unpack_bfp4_b(const uint8_t *tiles, int64_t rows, int64_t cols, float *dst) {
  if (!tiles || !dst || rows <= 0 || cols <= 0 || (rows % 32) || (cols % 32)) return TTLB_ERR_INVALID_ARG;
  const int64_t tcs = cols / 32;
  for (int64_t tr = 0; tr < rows / 32; ++tr)
    for (int64_t tc = 0; tc < tcs; ++tc) {
      const uint8_t *tile = tiles + (tr * tcs + tc) * TTLB_BFP4_TILE_BYTES;
      for (int f = 0; f < 4; ++f)
        for (int fr = 0; fr < 16; ++fr) {
          const int E = tile[f * 16 + fr];
          const uint8_t *q = tile + 64 + f * 128 + fr * 8;
          float *p = dst + (tr * 32 + (f >> 1) * 16 + fr) * cols + tc * 32 + (f & 1) * 16;
          for (int j = 0; j < 16; ++j) {
            const int nib = (q[j >> 1] >> ((j & 1) * 4)) & 0xf;
            const float mag = std::ldexp((float)(nib & 7), E - 129);
            p[j] = (nib & 8) ? -mag : mag;
          }
        }
    }
  return TTLB_OK;
}

extern "C" int ttlb_unpack_bfp4_b_device(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total, int64_t tile_col0,
                                         int64_t k, int64_t n, void *out_bf16, int64_t ld, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  int rc = check_args(ctx, tiles, tile_cols_total, tile_col0, k, n);
  if (rc) return rc;
  if (!out_bf16 || ((uintptr_t)out_bf16 % 16) || (ld % 8) || ld < n)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp4: output null, misaligned or pitch too small");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "bfp4: cannot select device %d", ctx->device);
  return launch_unpack(ctx, reinterpret_cast<const uint8_t *>(tiles), tile_cols_total, tile_col0, k / 32, n / 32, out_bf16,
                       ld, reinterpret_cast<cudaStream_t>(stream));
}

// C = act(A x W + bias) with W stored as bfloat4_b tiles: the weight window is expanded to bf16 in the context's
// scratch (the same buffer the bfloat8_b path uses), then the tensor-core GEMM runs on it with the bias / activation
// epilogue of ttlb_matmul_bf16_epilogue (bias NULL and act 0: the plain product).
extern "C" int ttlb_matmul_bfp4w_epilogue(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, const void *bias, int64_t ldbias,
                                          int act, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_bfp4w: null descriptor");
  if (act < TTLB_ACT_NONE || act > TTLB_ACT_TANH) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: unknown activation %d", act);
  if (!bias && ldbias != 0) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: a bias pitch without a bias");
  if (d->m == 0 || d->n == 0) return TTLB_OK;
  int rc = check_args(ctx, d->b_tiles, d->b_tile_cols, d->b_tile_col0, d->k, d->n);
  if (rc) return rc;
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "matmul_bfp4w: cannot select device %d", ctx->device);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const size_t need = (size_t)d->k * (size_t)d->n * 2;
  if (ctx->scratch_bytes < need) {
    if (ctx->scratch) {
      TTLB_CUDA_CHECK(ctx, cudaStreamSynchronize(s));
      TTLB_CUDA_CHECK(ctx, cudaFree(ctx->scratch));
      ctx->scratch = nullptr;
      ctx->scratch_bytes = 0;
    }
    TTLB_CUDA_CHECK(ctx, cudaMalloc(&ctx->scratch, need));
    ctx->scratch_bytes = need;
  }
  rc = launch_unpack(ctx, reinterpret_cast<const uint8_t *>(d->b_tiles), d->b_tile_cols, d->b_tile_col0, d->k / 32, d->n / 32,
                     ctx->scratch, d->n, s);
  if (rc) return rc;
  ctx->gemm_act = act;
  rc = ttlb_launch_gemm_bf16_full(ctx, d->a, d->lda, ctx->scratch, d->n, d->c, d->ldc, d->m, d->n, d->k, false, bias, ldbias, s);
  ctx->gemm_act = 0;
  return rc;
}

extern "C" int ttlb_matmul_bfp4w(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, void *stream) {
  return ttlb_matmul_bfp4w_epilogue(ctx, d, nullptr, 0, TTLB_ACT_NONE, stream);
}
