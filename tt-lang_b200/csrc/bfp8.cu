// bfloat8_b block-float weights: host packer/unpacker, device unpack kernel and the
// bfp8-weight matmul (ttlb_matmul_bfp8w).
//
// What the reference fixes about the format is the tile size only: a 32x32 bfloat8_b tile
// takes 1088 bytes = 1024 value bytes + 64 shared-exponent bytes, i.e. one exponent per 16
// values (python/ttl/dtype_utils.py:174-175).  The layout used here completes that as
// follows (a design choice of this library, applied identically by the CPU packer, the
// CPU oracle and the GPU kernels; byte-compatibility with Tenstorrent tensors is not claimed):
//
//   * a matrix [R, C] (R, C multiples of 32) is stored as tiles in row-major tile order;
//   * a tile is split into four 16x16 faces in row-major face order
//     (face f = 2*(r/16) + (c/16)), each face stored row-major;
//   * a block is one face row: 16 consecutive elements of one matrix row;
//   * bytes [0, 64) of a tile: block exponents, index f*16 + (r%16); a block exponent is the
//     largest biased fp32 exponent among the block's values (0 if all are zero/denormal);
//   * bytes [64, 1088): one byte per value at 64 + f*256 + (r%16)*16 + (c%16):
//     bit 7 = sign, bits 6..0 = magnitude m, value = (-1)^sign * m * 2^(E - 133)
//     (so the largest element of a block has m in [64, 127]);
//   * m = |x| * 2^(133 - E) rounded to nearest, ties to even, saturated at 127.
#include <cuda_bf16.h>

#include <cmath>
#include <cstring>

#include "bfp8_unpack.cuh"
#include "ctx.h"

int ttlb_launch_gemm_bf16(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k, cudaStream_t stream);
int ttlb_launch_gemm_bf16_ex(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                             int64_t m, int64_t n, int64_t k, bool multicast, cudaStream_t stream);

int ttlb_launch_gemm_bf16_full(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, bool multicast, const void *bias, int64_t ldbias,
                               cudaStream_t stream);

int ttlb_launch_gemm_bfp8w_tmem(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, bool publish, cudaStream_t stream);

namespace {

inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

// magnitude byte of x for block exponent E
inline uint8_t quantise(uint32_t bits, int E) {
  const int e = (int)((bits >> 23) & 0xff);
  if (e == 0 || E == 0) return (uint8_t)((bits >> 31) << 7);  // zero / denormal input
  const uint32_t sig = (bits & 0x7fffffu) | 0x800000u;        // 24-bit significand, value = sig * 2^(e-150)
  const int shift = 17 + (E - e);                              // m = sig >> shift, rounded
  uint32_t m;
  if (shift >= 32) {
    m = 0;
  } else {
    const uint32_t q = sig >> shift;
    const uint32_t rem = sig & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    m = q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
  }
  if (m > 127u) m = 127u;
  return (uint8_t)(((bits >> 31) << 7) | m);
}

// One thread per block of 16 values; a 256-thread CTA expands 4 consecutive tiles of one tile row
// (blockIdx.y = tile row, blockIdx.x = group of 4 tile columns): no integer division.
__global__ void __launch_bounds__(256) ttlb_unpack_bfp8_kernel(const uint8_t *__restrict__ tiles, int tile_cols_total,
                                                             int tile_col0, int tile_rows, int tile_cols,
                                                             __nv_bfloat16 *__restrict__ out, long long ld) {
  const int blk = threadIdx.x & 63;
  const int tc = blockIdx.x * 4 + (threadIdx.x >> 6);
  if (tc >= tile_cols) return;
  const int f = blk >> 4, fr = blk & 15;
  for (int tr = blockIdx.y; tr < tile_rows; tr += gridDim.y) {
    const uint8_t *tile = tiles + ((long long)tr * tile_cols_total + tile_col0 + tc) * TTLB_BFP8_TILE_BYTES;
    const int E = tile[blk];
    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(tile + 64 + f * 256 + fr * 16));
    uint32_t o[8];
    unpack_block(v, E, o);
    const long long row = (long long)tr * 32 + (f >> 1) * 16 + fr;
    const long long col = (long long)tc * 32 + (f & 1) * 16;
    uint4 *dst = reinterpret_cast<uint4 *>(out + row * ld + col);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace

extern "C" int ttlb_pack_bfp8_b(const float *src, int64_t rows, int64_t cols, uint8_t *dst_tiles) {
  if (!src || !dst_tiles || rows <= 0 || cols <= 0 || (rows % 32) || (cols % 32)) return TTLB_ERR_INVALID_ARG;
  const int64_t tcs = cols / 32;
  for (int64_t tr = 0; tr < rows / 32; ++tr)
    for (int64_t tc = 0; tc < tcs; ++tc) {
      uint8_t *tile = dst_tiles + (tr * tcs + tc) * TTLB_BFP8_TILE_BYTES;
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
          uint8_t *q = tile + 64 + f * 256 + fr * 16;
          for (int j = 0; j < 16; ++j) q[j] = quantise(f32_bits(p[j]), E);
        }
    }
  return TTLB_OK;
}

extern "C" int ttlb_unpack_bfp8_b(const uint8_t *tiles, int64_t rows, int64_t cols, float *dst) {
  if (!tiles || !dst || rows <= 0 || cols <= 0 || (rows % 32) || (cols % 32)) return TTLB_ERR_INVALID_ARG;
  const int64_t tcs = cols / 32;
  for (int64_t tr = 0; tr < rows / 32; ++tr)
    for (int64_t tc = 0; tc < tcs; ++tc) {
      const uint8_t *tile = tiles + (tr * tcs + tc) * TTLB_BFP8_TILE_BYTES;
      for (int f = 0; f < 4; ++f)
        for (int fr = 0; fr < 16; ++fr) {
          const int E = tile[f * 16 + fr];
          const uint8_t *q = tile + 64 + f * 256 + fr * 16;
          float *p = dst + (tr * 32 + (f >> 1) * 16 + fr) * cols + tc * 32 + (f & 1) * 16;
          for (int j = 0; j < 16; ++j) {
            const float mag = std::ldexp((float)(q[j] & 0x7f), E - 133);
            p[j] = (q[j] & 0x80) ? -mag : mag;
          }
        }
    }
  return TTLB_OK;
}

static int launch_unpack(ttlb_ctx *ctx, const uint8_t *tiles, int64_t tile_cols_total, int64_t tile_col0,
                         int64_t tile_rows, int64_t tile_cols, void *out, int64_t ld, cudaStream_t s) {
  const unsigned gx = (unsigned)((tile_cols + 3) / 4);
  const unsigned gy = (unsigned)(tile_rows < 65535 ? tile_rows : 65535);
  ttlb_unpack_bfp8_kernel<<<dim3(gx, gy), 256, 0, s>>>(tiles, (int)tile_cols_total, (int)tile_col0, (int)tile_rows,
                                                         (int)tile_cols, reinterpret_cast<__nv_bfloat16 *>(out), ld);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}

static int check_bfp8_args(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total, int64_t tile_col0, int64_t k,
                           int64_t n) {
  if (!tiles || ((uintptr_t)tiles % 16)) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp8: tile pointer null or misaligned");
  if (k <= 0 || n <= 0 || (k % 32) || (n % 32))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp8: K and N must be positive multiples of 32");
  if (tile_col0 < 0 || tile_cols_total <= 0 || tile_col0 + n / 32 > tile_cols_total)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp8: column window exceeds the packed matrix");
  return TTLB_OK;
}

extern "C" int ttlb_unpack_bfp8_b_device(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total, int64_t tile_col0,
                                         int64_t k, int64_t n, void *out_bf16, int64_t ld, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  int rc = check_bfp8_args(ctx, tiles, tile_cols_total, tile_col0, k, n);
  if (rc) return rc;
  if (!out_bf16 || ((uintptr_t)out_bf16 % 16) || (ld % 8) || ld < n)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "bfp8: output null, misaligned or pitch too small");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "bfp8: cannot select device %d", ctx->device);
  return launch_unpack(ctx, reinterpret_cast<const uint8_t *>(tiles), tile_cols_total, tile_col0, k / 32, n / 32,
                       out_bf16, ld, reinterpret_cast<cudaStream_t>(stream));
}

static int matmul_bfp8w_impl(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, bool multicast, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_bfp8w: null descriptor");
  if (d->m == 0 || d->n == 0) return TTLB_OK;
  int rc = check_bfp8_args(ctx, d->b_tiles, d->b_tile_cols, d->b_tile_col0, d->k, d->n);
  if (rc) return rc;
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "matmul_bfp8w: cannot select device %d", ctx->device);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Unpack inside the GEMM mainloop (no scratch) when selected and the output fills the SM pairs.
  const bool fused_ok = d->m > 0 && d->m <= 0x7fffffff && d->n <= 0x7fffffff && d->k <= 0x7fffffff;
  if (fused_ok && (ctx->bfp8_mode == 2 ||
                   (ctx->bfp8_mode == 1 && ((d->m + 255) / 256) * ((d->n + 255) / 256) >= ctx->sm_count / 2))) {
    if (!d->a || !d->c) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null operand");
    if ((d->lda % 8) || (d->ldc % 8) || ((uintptr_t)d->a % 16) || ((uintptr_t)d->c % 16))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG,
                       "matmul: pointers must be 16-byte aligned and K, N and the row pitches multiples of 8");
    if (d->lda < d->k || d->ldc < d->n)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: row pitch smaller than the row");
    return ttlb_launch_gemm_bfp8w_tmem(ctx, d, multicast, s);
  }
  // otherwise expand the weight window to bf16 in scratch memory owned by the context, then run the bf16 GEMM
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
  // Column chunks: the expansion of chunk i+1 (HBM-bound, on a side stream) runs under the GEMM of chunk i
  // (tensor-bound, on the caller's stream).  Events order them: fork from the caller's stream, one event per
  // expanded chunk, every side-stream kernel is waited for by a GEMM, so the side stream has joined again when
  // the call returns.  Chunks are multiples of 256 columns and large enough to keep the two-CTA GEMM.
  int chunks = 1;
  if (!multicast && ctx->bfp8_chunks > 1) {
    for (int c = ctx->bfp8_chunks > 4 ? 4 : ctx->bfp8_chunks; c > 1; --c)
      if (d->n % (256 * c) == 0 && ((d->m + 255) / 256) * (d->n / c / 256) >= ctx->sm_count / 2) {
        chunks = c;
        break;
      }
  }
  const uint8_t *tiles = reinterpret_cast<const uint8_t *>(d->b_tiles);
  if (chunks == 1) {
    rc = launch_unpack(ctx, tiles, d->b_tile_cols, d->b_tile_col0, d->k / 32, d->n / 32, ctx->scratch, d->n, s);
    if (rc) return rc;
    return ttlb_launch_gemm_bf16_ex(ctx, d->a, d->lda, ctx->scratch, d->n, d->c, d->ldc, d->m, d->n, d->k, multicast, s);
  }
  if (!ctx->side_stream) {
    TTLB_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    TTLB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming));
    for (cudaEvent_t &e : ctx->ev_chunk) TTLB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  const int64_t nc = d->n / chunks;   // columns per chunk
  __nv_bfloat16 *wb = reinterpret_cast<__nv_bfloat16 *>(ctx->scratch);
  // the side stream starts after everything already queued on the caller's stream (earlier users of the
  // scratch buffer included)
  TTLB_CUDA_CHECK(ctx, cudaEventRecord(ctx->ev_fork, s));
  TTLB_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->ev_fork, 0));
  for (int i = 0; i < chunks; ++i) {
    rc = launch_unpack(ctx, tiles, d->b_tile_cols, d->b_tile_col0 + i * (nc / 32), d->k / 32, nc / 32, wb + i * nc, d->n,
                       ctx->side_stream);
    if (rc) return rc;
    TTLB_CUDA_CHECK(ctx, cudaEventRecord(ctx->ev_chunk[i], ctx->side_stream));
  }
  for (int i = 0; i < chunks; ++i) {
    TTLB_CUDA_CHECK(ctx, cudaStreamWaitEvent(s, ctx->ev_chunk[i], 0));
    rc = ttlb_launch_gemm_bf16_ex(ctx, d->a, d->lda, wb + i * nc, d->n,
                                  reinterpret_cast<__nv_bfloat16 *>(d->c) + i * nc, d->ldc, d->m, nc, d->k, false, s);
    if (rc) return rc;
  }
  return TTLB_OK;
}

extern "C" int ttlb_set_bfp8_chunks(ttlb_ctx *ctx, int chunks) {
  if (!ctx || chunks < 1 || chunks > 4) return TTLB_ERR_INVALID_ARG;
  ctx->bfp8_chunks = chunks;
  return TTLB_OK;
}

extern "C" int ttlb_set_bfp8_mode(ttlb_ctx *ctx, int mode) {
  if (!ctx || mode < 0 || mode > 2) return TTLB_ERR_INVALID_ARG;
  ctx->bfp8_mode = mode;
  return TTLB_OK;
}

extern "C" int ttlb_matmul_bfp8w(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, void *stream) {
  return matmul_bfp8w_impl(ctx, d, false, stream);
}

// The quantised linear layer with bias and activation: weights expanded to bf16 in the context's scratch, then
// the bf16 GEMM with the bias / activation epilogue.
extern "C" int ttlb_matmul_bfp8w_epilogue(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, const void *bias, int64_t ldbias,
                                          int act, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_bfp8w: null descriptor");
  if (act < TTLB_ACT_NONE || act > TTLB_ACT_TANH) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: unknown activation %d", act);
  if (!bias && ldbias != 0) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: a bias pitch without a bias");
  if (d->m == 0 || d->n == 0) return TTLB_OK;
  int rc = check_bfp8_args(ctx, d->b_tiles, d->b_tile_cols, d->b_tile_col0, d->k, d->n);
  if (rc) return rc;
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "matmul_bfp8w: cannot select device %d", ctx->device);
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

extern "C" int ttlb_matmul_bfp8w_multicast(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, void *stream) {
  return matmul_bfp8w_impl(ctx, d, true, stream);
}

int ttlb_set_pub_peers(ttlb_ctx *ctx, void *const *peers, int n_peers);

extern "C" int ttlb_matmul_bfp8w_peers(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, void *const *peers, int n_peers,
                                       void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_bfp8w: null descriptor");
  int rc = ttlb_set_pub_peers(ctx, peers, n_peers);
  if (rc) return rc;
  ttlb_gemm_bfp8_desc own = *d;
  own.c = peers[0];
  rc = matmul_bfp8w_impl(ctx, &own, true, stream);
  ctx->pub_n_peers = 0;
  return rc;
}

// Context-free launch of the unpack kernel (used by the allocation-free entry point).
int ttlb_bfp8_unpack_launch_raw(const uint8_t *tiles, int64_t tile_cols_total, int64_t tile_col0, int64_t tile_rows,
                                int64_t tile_cols, void *out, int64_t ld, int sm_count, cudaStream_t s) {
  (void)sm_count;
  const unsigned gx = (unsigned)((tile_cols + 3) / 4);
  const unsigned gy = (unsigned)(tile_rows < 65535 ? tile_rows : 65535);
  ttlb_unpack_bfp8_kernel<<<dim3(gx, gy), 256, 0, s>>>(tiles, (int)tile_cols_total, (int)tile_col0, (int)tile_rows,
                                                         (int)tile_cols, reinterpret_cast<__nv_bfloat16 *>(out), ld);
  return cudaGetLastError() == cudaSuccess ? TTLB_OK : TTLB_ERR_CUDA;
}
