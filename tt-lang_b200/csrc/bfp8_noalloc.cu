// ttlb_matmul_bfp8w_noalloc: the bfp8-weight matmul for callers that must not allocate.
//
// Who cannot allocate: code that runs after a serving process has handed all of the GPU's free
// memory to its own pool (a cudaMalloc there fails even though memory is "free" inside the pool),
// code on a latency-critical path (cudaMalloc and cudaFree synchronise the device and take an
// unbounded time), and plugins that are only allowed to touch the buffers they are given.  The
// regular entry point, ttlb_matmul_bfp8w, expands the weight window to bf16 in scratch memory that
// it cudaMallocs (and regrows) inside the context, and creating a context allocates as well.  This
// variant needs no context and calls no allocating routine: its scratch is a fixed array in the
// library's device image.
//
// Cost and limits, so that nobody is surprised:
//   * every GPU that loads this library holds the 32 MiB array (plus a 4-byte status word) from
//     the moment the library's device code is loaded until the process exits, whether or not
//     this entry point is ever called;
//   * the weight window may have at most TTLB_NOALLOC_MAX_WEIGHT_ELEMS = 16 Mi values
//     (k * n <= 16,777,216, e.g. 4096 x 4096 or 8192 x 2048); larger windows are rejected;
//   * all calls on one GPU share the array: two calls whose kernels may overlap on the GPU (two
//     streams, two threads) race on it - serialise them;
//   * the first call on a device that passes the argument checks looks up the array's device address and
//     raises the GEMM kernel's shared-memory limit (under a lock); make that first call before any stream
//     capture begins;
//   * with check == 0 a bounded device-side wait that ran out goes unreported: the status word is private to
//     this entry point and the next call clears it.  Pass check != 0 where that matters.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "ttlb200.h"

int ttlb_gemm_bf16_launch_raw(const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc, int64_t m,
                              int64_t n, int64_t k, int sm_count, int *d_status, long long wait_limit, bool *attr_set,
                              cudaStream_t stream);
int ttlb_gemm_bf16_raw_prepare();
int ttlb_bfp8_unpack_launch_raw(const uint8_t *tiles, int64_t tile_cols_total, int64_t tile_col0, int64_t tile_rows,
                                int64_t tile_cols, void *out, int64_t ld, int sm_count, cudaStream_t s);

namespace {

constexpr size_t kScratchBytes = (size_t)TTLB_NOALLOC_MAX_WEIGHT_ELEMS * 2;  // bf16 expansion of the window

// In host code these names are only handles for cudaGetSymbolAddress: they are not device
// addresses and must never be passed to a kernel as they stand.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];
static __device__ int g_noalloc_status;

constexpr int kMaxDevices = 64;
struct DeviceSetup {
  bool ready = false;
  void *scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int *status = nullptr;    // device address of g_noalloc_status on this device
  int sm_count = 0;
  bool gemm_attr_set = false;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

int fail(char *err, size_t err_len, int code, const char *msg) {
  if (err && err_len) snprintf(err, err_len, "%s", msg);
  return code;
}

}  // namespace

extern "C" int ttlb_matmul_bfp8w_noalloc(const ttlb_gemm_bfp8_desc *d, void *stream, int check, char *err,
                                         size_t err_len) {
  if (err && err_len) err[0] = 0;
  if (!d) return fail(err, err_len, TTLB_ERR_INVALID_ARG, "matmul_bfp8w_noalloc: null descriptor");
  if (d->m == 0 || d->n == 0) return TTLB_OK;
  if (!d->a || !d->b_tiles || !d->c) return fail(err, err_len, TTLB_ERR_INVALID_ARG, "matmul_bfp8w_noalloc: null tensor");
  if (d->m < 0 || d->n < 0 || d->k <= 0 || (d->k % 32) || (d->n % 32) || d->m > 0x7fffffff)
    return fail(err, err_len, TTLB_ERR_INVALID_ARG, "matmul_bfp8w_noalloc: k and n must be positive multiples of 32");
  if ((int64_t)d->k * d->n > (int64_t)TTLB_NOALLOC_MAX_WEIGHT_ELEMS) {
    if (err && err_len)
      snprintf(err, err_len,
               "matmul_bfp8w_noalloc: weight window %lld x %lld = %lld values exceeds the fixed scratch of %lld "
               "values; use ttlb_matmul_bfp8w or split the columns",
               (long long)d->k, (long long)d->n, (long long)d->k * d->n, (long long)TTLB_NOALLOC_MAX_WEIGHT_ELEMS);
    return TTLB_ERR_UNSUPPORTED;
  }
  if (d->b_tile_col0 < 0 || d->b_tile_cols <= 0 || d->b_tile_col0 + d->n / 32 > d->b_tile_cols)
    return fail(err, err_len, TTLB_ERR_INVALID_ARG, "matmul_bfp8w_noalloc: column window exceeds the packed matrix");
  if ((d->lda % 8) || (d->ldc % 8) || d->lda < d->k || d->ldc < d->n || ((uintptr_t)d->a % 16) ||
      ((uintptr_t)d->c % 16) || ((uintptr_t)d->b_tiles % 16))
    return fail(err, err_len, TTLB_ERR_INVALID_ARG, "matmul_bfp8w_noalloc: misaligned pointer or bad row pitch");

  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: no current CUDA device");
  DeviceSetup *su = &g_setup[dev];
  {
    // set-up, once per device, with that device current
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!su->ready) {
      int major = 0;
      if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
        return fail(err, err_len, TTLB_ERR_UNSUPPORTED, "matmul_bfp8w_noalloc: the kernels are built for sm_100a only");
      if (cudaDeviceGetAttribute(&su->sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: cannot query the device");
      void *p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p)
        return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: cudaGetSymbolAddress(scratch) failed");
      su->scratch = p;
      e = cudaGetSymbolAddress(&p, g_noalloc_status);
      if (e != cudaSuccess || !p)
        return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: cudaGetSymbolAddress(status) failed");
      su->status = reinterpret_cast<int *>(p);
      // the GEMM kernel's shared-memory limit is raised here, under the lock, not by whichever thread launches first
      if (ttlb_gemm_bf16_raw_prepare() != TTLB_OK)
        return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: cannot raise the GEMM kernel's shared-memory limit");
      su->gemm_attr_set = true;
      su->ready = true;
    }
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the status word keeps whatever the previous call left: it must start at zero
  if (cudaMemsetAsync(su->status, 0, sizeof(int), s) != cudaSuccess)
    return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: cudaMemsetAsync failed");
  // the scratch itself needs no clearing: the unpack below overwrites all k x n values the GEMM reads
  int rc = ttlb_bfp8_unpack_launch_raw(reinterpret_cast<const uint8_t *>(d->b_tiles), d->b_tile_cols, d->b_tile_col0,
                                       d->k / 32, d->n / 32, su->scratch, d->n, su->sm_count, s);
  if (rc) return fail(err, err_len, rc, "matmul_bfp8w_noalloc: unpack launch failed");
  rc = ttlb_gemm_bf16_launch_raw(d->a, d->lda, su->scratch, d->n, d->c, d->ldc, d->m, d->n, d->k, su->sm_count,
                                 su->status, 4000000000LL, &su->gemm_attr_set, s);
  if (rc) return fail(err, err_len, rc, "matmul_bfp8w_noalloc: GEMM launch failed");
  if (check) {
    int code = 0;
    if (cudaMemcpyAsync(&code, su->status, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
      return fail(err, err_len, TTLB_ERR_CUDA, "matmul_bfp8w_noalloc: reading the status word failed");
    if (code != 0) return fail(err, err_len, TTLB_ERR_TIMEOUT, "matmul_bfp8w_noalloc: a bounded device-side wait ran out");
  }
  return TTLB_OK;
}
