// Internal context shared by the C-ABI entry points (not installed; the public
// surface is include/ttlb200.h).
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "ttlb200.h"

struct ttlb_jit_cache;

struct ttlb_ctx {
  int device = 0;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int64_t launches = 0;
  std::string err;
  // Device-side status word for kernels with bounded waits (GEMM / attention):
  // 0 = ok, otherwise a code telling which wait gave up.
  int *d_status = nullptr;
  int *h_status = nullptr;  // pinned mirror
  // Element-wise programs: specialised (NVRTC) kernels cached per program signature.
  ttlb_jit_cache *jit = nullptr;
  int eltwise_mode = TTLB_ELTWISE_AUTO;
  int eltwise_last_path = -1;
  // tcgen05 kernels: opt-in shared memory set once per context; bound for device-side waits
  bool gemm_attr_set = false;
  bool gemm2_attr_set = false;
  int gemm_variant = 1;  // 0: always one-CTA 128x256 tiles; 1: two-CTA (cta_group::2) 256x256 tiles for large outputs
  bool gemm_tmem_attr_set = false;
  int gemm_act = 0;  // activation of the GEMM being launched (set by ttlb_matmul_bf16_epilogue around its launch)
  // output region in each GPU's copy of a shared buffer, for the GEMM being launched (ttlb_matmul_*_peers)
  void *pub_peers[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int pub_n_peers = 0;
  int bfp8_mode = 1;  // 0: unpack kernel + bf16 GEMM; 1: unpack inside the GEMM mainloop for large outputs; 2: always inside
  bool attn_attr_set = false;
  long long wait_limit_cycles = 4000000000LL;  // ~2 s at 1.9 GHz
  // Scratch in HBM owned by the context (bf16 expansion of bfloat8_b weights); grows on demand.
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  // Reductions over rows: partial rows, per-column-group partials and arrival counters (one allocation).
  void *reduce_scratch = nullptr;
  // bfp8-weight matmul: the weight expansion of column chunk i+1 runs on this stream under the GEMM of chunk i
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr;
  cudaEvent_t ev_chunk[4] = {nullptr, nullptr, nullptr, nullptr};
  int bfp8_chunks = 1;  // column chunks of the two-step bfp8 path (1: no overlap; measured: overlap gains nothing)
};

inline int ttlb_fail(ttlb_ctx *ctx, int code, const char *fmt, ...) {
  if (ctx) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    ctx->err = buf;
  }
  return code;
}

#define TTLB_CUDA_CHECK(ctx, expr)                                                     \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ttlb_fail((ctx), TTLB_ERR_CUDA, "%s failed: %s", #expr,                   \
                       cudaGetErrorString(e__));                                       \
  } while (0)

// RAII guard: make the context's device current for the duration of a call.
struct ttlb_device_guard {
  int prev = -1;
  bool ok = true;
  explicit ttlb_device_guard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
  }
  ~ttlb_device_guard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};
