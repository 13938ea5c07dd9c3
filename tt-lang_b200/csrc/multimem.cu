// Switch-replicated stores (NVLink multicast): write a local bf16 region once and have the NVSwitch
// deliver it to the same offset of every GPU bound to the multicast object (ttlb_multimem_bcast).
// Used to publish an output shard to all ranks of a sharded matmul / attention without a per-peer copy.
// `mc_dst` is the multicast address of the destination (e.g. torch symmetric memory's multicast_ptr
// plus the byte offset of the region); it is written with multimem.st, never read.
#include "ctx.h"

namespace {

__global__ void __launch_bounds__(256) ttlb_multimem_bcast_kernel(const uint4 *__restrict__ src, uint4 *mc_dst,
                                                                long long rows, long long vec_per_row,
                                                                long long src_ld_vec, long long dst_ld_vec) {
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row, c = i - r * vec_per_row;
    const uint4 v = __ldcs(src + r * src_ld_vec + c);
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst + r * dst_ld_vec + c),
                 "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w))
                 : "memory");
  }
}

}  // namespace

extern "C" int ttlb_multimem_bcast(ttlb_ctx *ctx, const void *src, int64_t src_ld_bytes, void *mc_dst,
                                   int64_t dst_ld_bytes, int64_t rows, int64_t row_bytes, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (rows == 0 || row_bytes == 0) return TTLB_OK;
  if (!src || !mc_dst || rows < 0 || row_bytes < 0)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "multimem_bcast: null pointer or negative size");
  if ((row_bytes % 16) || (src_ld_bytes % 16) || (dst_ld_bytes % 16) || ((uintptr_t)src % 16) || ((uintptr_t)mc_dst % 16) ||
      src_ld_bytes < row_bytes || dst_ld_bytes < row_bytes)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "multimem_bcast: rows, pitches and pointers must be multiples of 16 bytes");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "multimem_bcast: cannot select device %d", ctx->device);
  const long long total = rows * (row_bytes / 16);
  long long grid = (total + 255) / 256;
  const long long cap = (long long)ctx->sm_count * 8;
  if (grid > cap) grid = cap;
  ttlb_multimem_bcast_kernel<<<(unsigned)grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4 *>(src), reinterpret_cast<uint4 *>(mc_dst), rows, row_bytes / 16, src_ld_bytes / 16,
      dst_ld_bytes / 16);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
