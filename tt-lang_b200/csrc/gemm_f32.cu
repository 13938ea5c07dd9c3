// fp32 matmul for tile programs on float32 tensors (ttlb_matmul_f32).
//
// The reference's matmul examples run their kernels on float32 tensors
// (examples/singlecore_matmul.py:73-75, examples/multicore_matmul.py:118-120) and compare with an
// fp32 golden at rtol 1e-4, which rules out TF32 tensor cores.  This is a plain CUDA-core kernel -
// 64x64 output tile per 256-thread CTA, 4x4 outputs per thread, K stepped by 16 through shared
// memory, fp32 FMA accumulation in ascending K order - kept for coverage of fp32 programs; the
// benchmarked matmul path is the bf16 tensor-core kernel.
#include "ctx.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) ttlb_gemm_f32_kernel(const float *__restrict__ a, long long lda,
                                                          const float *__restrict__ b, long long ldb,
                                                          float *__restrict__ c, long long ldc, int m, int n, int k) {
  __shared__ float sa[TK][TM + 4];
  __shared__ float sb[TK][TN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += TK) {
    // A tile 64x16: 1024 elements, 4 per thread; B tile 16x64
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      const int ar = e >> 4, ac = e & 15;
      const int gr = row0 + ar, gc = k0 + ac;
      sa[ac][ar] = (gr < m && gc < k) ? a[(long long)gr * lda + gc] : 0.f;
      const int br = e >> 6, bc = e & 63;
      const int hr = k0 + br, hc = col0 + bc;
      sb[br][bc] = (hr < k && hc < n) ? b[(long long)hr * ldb + hc] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx * 4 + j;
      if (gc < n) c[(long long)gr * ldc + gc] = acc[i][j];
    }
  }
}

}  // namespace

extern "C" int ttlb_matmul_f32(ttlb_ctx *ctx, const ttlb_gemm_desc *d, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_f32: null descriptor");
  if (d->m == 0 || d->n == 0) return TTLB_OK;
  if (!d->a || !d->b || !d->c) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_f32: null operand");
  if (d->m < 0 || d->n < 0 || d->k <= 0 || d->m > 0x7fffffff || d->n > 0x7fffffff || d->k > 0x7fffffff)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_f32: bad shape");
  if (d->lda < d->k || d->ldb < d->n || d->ldc < d->n)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_f32: row pitch smaller than the row");
  if (((uintptr_t)d->a % 4) || ((uintptr_t)d->b % 4) || ((uintptr_t)d->c % 4))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul_f32: misaligned pointer");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "matmul_f32: cannot select device %d", ctx->device);
  const long long gx = (d->n + TN - 1) / TN, gy = (d->m + TM - 1) / TM;
  if (gy > 65535) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "matmul_f32: more than 65535 row tiles");
  ttlb_gemm_f32_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float *>(d->a), d->lda, reinterpret_cast<const float *>(d->b), d->ldb,
      reinterpret_cast<float *>(d->c), d->ldc, (int)d->m, (int)d->n, (int)d->k);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
