// Context management for the ttlb200 C ABI (include/ttlb200.h).
#include "ctx.h"
#include "eltwise_jit.h"

extern "C" {

const char *ttlb_version(void) { return "ttlb200 0.1 (sm_100a)"; }

int ttlb_init(int device_ordinal, ttlb_ctx **out) {
  if (!out) return TTLB_ERR_INVALID_ARG;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) return TTLB_ERR_CUDA;  // no CPU fallback exists
  if (device_ordinal < 0 || device_ordinal >= n) return TTLB_ERR_INVALID_ARG;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return TTLB_ERR_CUDA;
  if (prop.major != 10) return TTLB_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
  ttlb_ctx *ctx = new ttlb_ctx();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  ttlb_device_guard g(device_ordinal);
  if (!g.ok || cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess ||
      cudaMemset(ctx->d_status, 0, sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->h_status, sizeof(int)) != cudaSuccess) {
    if (ctx->d_status) cudaFree(ctx->d_status);
    delete ctx;
    return TTLB_ERR_CUDA;
  }
  *ctx->h_status = 0;
  *out = ctx;
  return TTLB_OK;
}

void ttlb_destroy(ttlb_ctx *ctx) {
  if (!ctx) return;
  {
    ttlb_device_guard g(ctx->device);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->reduce_scratch) cudaFree(ctx->reduce_scratch);
    if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    for (cudaEvent_t e : ctx->ev_chunk)
      if (e) cudaEventDestroy(e);
    ttlb_jit_cache_destroy(ctx->jit);
  }
  delete ctx;
}

const char *ttlb_last_error(ttlb_ctx *ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int64_t ttlb_launch_count(ttlb_ctx *ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
