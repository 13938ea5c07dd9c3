// bf16 GEMM on the 5th-generation tensor cores (ttlb_matmul_bf16).
//
//   C[M,N] (bf16) = A[M,K] (bf16, row-major) x B[K,N] (bf16, row-major), fp32 accumulation.
//
// This is the GPU form of the tile program `for k: out_blk.store(a_blk @ b_blk, acc=True)`
// (examples/singlecore_matmul.py:36-45) and of the Tensix loop it compiles to,
// `matmul_tiles(cb0, cb1, 0, 0, 0)` over the K tiles into a DST accumulator
// (examples/metal_examples/multicore_matmul/metal/kernels/mm_compute.cpp:30-65).
// The circular buffers become a ring of shared-memory stages guarded by mbarriers
// (reserve/push = wait empty / TMA arrive on full; wait/pop = wait full / UMMA commit on
// empty), DST becomes a TMEM accumulator.
//
// Persistent, warp-specialised, one CTA per SM, 192 threads:
//   warp 0      TMA producer: A tile 128x64 (K-major) and B tile 64x256 (N-major, as four
//               64x64 boxes) per stage, 128-byte swizzle, 4 stages of 48 KB
//   warp 1      UMMA issuer: tcgen05.mma 128x256x16, fp32 accumulators in TMEM, two
//               accumulator buffers (2 x 256 columns) so the epilogue of tile i overlaps
//               the main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld -> bf16 -> global stores (each thread owns one row)
// B is consumed straight from its row-major layout (MN-major operand), no transpose pass.
// Tiles are rasterised in bands of 16 M-tiles so the CTAs of one wave share A rows and B
// columns in L2.
#include <cuda_bf16.h>

#include <mutex>

#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;

ttlb_encode_tiled_fn ttlb_get_encode_tiled() {
  static ttlb_encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<ttlb_encode_tiled_fn>(p);
  });
  return fn;
}

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;         // 16 KB
constexpr int B_CHUNK_BYTES = BK * 64 * 2;   // 8 KB: one 64-column slice of the B tile
constexpr int B_BYTES = BK * BN * 2;         // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GROUP_M = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
// Publishing epilogue (the output goes to every GPU of a group): each epilogue warp stages 32 rows x 128 columns
// (256 bytes per row) so that a store instruction covers whole 256-byte row segments.
constexpr int PUB_COLS = 128;
constexpr int PUB_WARP_BYTES = 32 * PUB_COLS * 2;  // 8 KB
constexpr int SMEM_BYTES_PUB = SMEM_BYTES + 4 * PUB_WARP_BYTES;
constexpr int MAX_PEERS = 8;

struct GemmParams {
  __nv_bfloat16 *c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n;
  int *status;
  long long wait_limit;
  // 0: plain stores to `c`.  1: `c` is an NVLink multicast address, stored with multimem.st (the switch
  // replicates every store to all GPUs of the group).  2: the same tile is stored to `peer_c[0..n_peers)`, the
  // output region in every GPU's copy of the buffer (peer-mapped memory, this GPU's own copy included).
  int multicast;
  __nv_bfloat16 *peer_c[MAX_PEERS] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_peers = 0;
  const __nv_bfloat16 *bias = nullptr;  // optional [m, n] matrix added to the product before rounding
  long long ldbias = 0;                 // 0: the bias is one row of n values, added to every output row
  int act = 0;                          // TTLB_ACT_*: applied to product + bias before the rounding
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

// ACT: the instantiation with the activation epilogue (its transcendental code costs registers; the plain
// instantiation is the kernel the matmul configurations are measured with)
// PUB: the instantiation whose epilogue publishes the tile to several GPUs through a shared-memory stage
template <bool ACT, bool PUB = false>
__global__ void __launch_bounds__(THREADS, 1)
ttlb_gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  // barrier layout (8 bytes each): full[4] empty[4] tmem_full[2] tmem_empty[2]; then tmem ptr, abort flag
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw)) + STAGES * STAGE_BYTES;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + 8 * (2 * STAGES + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int fail = 0;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !fail; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit)) {
            fail = 1;
            break;
          }
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          tma_load_2d(sa, &map_a, kb * BK, tm * BM, full_bar(stage));
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(sb + j * B_CHUNK_BYTES, &map_b, tn * BN + j * 64, kb * BK, full_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN, false, true);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int t = blockIdx.x; t < num_tiles && !fail; t += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.wait_limit)) {
          fail = 2;
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.wait_limit)) {
            fail = 2;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t da = desc_kmajor_sw128(sa), db = desc_mnmajor_sw128(sb, B_CHUNK_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc, (kb | k) != 0);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (fail) break;
        umma_commit(tfull_bar(acc));
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles && !fail; t += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      // the outcome of the wait is made the same for the whole warp: what follows is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_limit))) {
        fail = 3;
        break;
      }
      tc_fence_after();
      if constexpr (PUB) {
        // tcgen05.ld hands every thread one row; the rows go through a swizzled stage so that each store
        // instruction of the warp writes two whole 256-byte row segments (16 lanes x 16 bytes each) - through
        // NVLink, 16-byte stores scattered over 32 rows reach a small fraction of the link rate
        uint8_t *stage = gen + 256 + (warp - 2) * PUB_WARP_BYTES;
#pragma unroll 1
        for (int half = 0; half < BN / PUB_COLS; ++half) {
#pragma unroll 1
          for (int cc = 0; cc < PUB_COLS / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * PUB_COLS + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              const int unit = cc * 4 + v;  // 16-byte unit within the 256-byte row
              *reinterpret_cast<uint4 *>(stage + lane * (PUB_COLS * 2) + ((unit ^ (lane & 7)) << 4)) = o;
            }
          }
          if (half == BN / PUB_COLS - 1) {
            // every accumulator column has been read: the issuer may start the next tile into this buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
          } else {
            __syncwarp();
          }
          const int unit = lane & 15;
          const long long gcol = (long long)tn * BN + half * PUB_COLS + unit * 8;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rl = 2 * i + (lane >> 4);
            const uint4 o = *reinterpret_cast<const uint4 *>(stage + rl * (PUB_COLS * 2) + ((unit ^ (rl & 7)) << 4));
            const long long grow = (long long)tm * BM + q * 32 + rl;
            if (grow < p.m && gcol < p.n) {
              const long long off = grow * p.ldc + gcol;
              if (p.multicast == 1) {
                st_multimem_16(p.c + off, o);
              } else {
                for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4 *>(p.peer_c[d] + off) = o;
              }
            }
          }
          __syncwarp();
        }
        continue;
      }
      const int row = tm * BM + q * 32 + lane;
      __nv_bfloat16 *crow = p.c + (long long)row * p.ldc + (long long)tn * BN;
      const __nv_bfloat16 *brow = p.bias ? p.bias + (long long)row * p.ldbias + (long long)tn * BN : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if (row < p.m && col0 < p.n) {
          if (col0 + 32 <= p.n) {
            if (brow) add_bias32(r, brow + c * 32);
            if (ACT) apply_act32(r, p.act);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              *reinterpret_cast<uint4 *>(crow + c * 32 + v * 8) = o;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (col0 + e < p.n)
                crow[c * 32 + e] = __float2bfloat16_rn(act1(__uint_as_float(r[e]) + (brow ? __bfloat162float(brow[c * 32 + e]) : 0.f), ACT ? p.act : 0));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  if (fail) atomicCAS(p.status, 0, fail);
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let TMA copies that may still be in flight land before the CTA's
    // shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_map(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
             uint32_t box_inner, uint32_t box_outer) {
  ttlb_encode_tiled_fn enc = ttlb_get_encode_tiled();
  if (!enc) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return TTLB_OK;
}

}  // namespace

int ttlb_make_map_bf16_2d(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  return make_map(ctx, map, ptr, inner, outer, pitch_bytes, box_inner, box_outer);
}
int ttlb_launch_gemm_bf16_2cta(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, const void *bias, int64_t ldbias, bool publish,
                               cudaStream_t stream);
int ttlb_launch_gemm_bf16_full(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, bool multicast, const void *bias, int64_t ldbias,
                               cudaStream_t stream);

// Shared with the bfp8-weight path, which first expands the weights to bf16.
int ttlb_launch_gemm_bf16_ex(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                             int64_t m, int64_t n, int64_t k, bool multicast, cudaStream_t stream);

int ttlb_launch_gemm_bf16(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
  return ttlb_launch_gemm_bf16_ex(ctx, a, lda, b, ldb, c, ldc, m, n, k, false, stream);
}

int ttlb_launch_gemm_bf16_ex(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                             int64_t m, int64_t n, int64_t k, bool multicast, cudaStream_t stream) {
  return ttlb_launch_gemm_bf16_full(ctx, a, lda, b, ldb, c, ldc, m, n, k, multicast, nullptr, 0, stream);
}

// multicast: `c` is a multicast address (the output is published to every GPU of the group); needs n % 32 == 0.
// bias: optional bf16 [m, n] matrix (row pitch ldbias) added to the fp32 product before the rounding to bf16.
int ttlb_launch_gemm_bf16_full(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, bool multicast, const void *bias, int64_t ldbias,
                               cudaStream_t stream) {
  if (m == 0 || n == 0) return TTLB_OK;
  if (bias && (((uintptr_t)bias % 16) || (ldbias % 8) || (ldbias != 0 && ldbias < n)))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG,
                     "matmul: bias must be 16-byte aligned with a row pitch >= N that is a multiple of 8 (or 0: one row)");
  if (multicast && (n % 32))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: a multicast output needs N to be a multiple of 32");
  if (!a || !b || !c) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null operand");
  if (m < 0 || n < 0 || k <= 0) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: bad shape %lldx%lldx%lld",
                                                 (long long)m, (long long)n, (long long)k);
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
    return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "matmul: dimension too large");
  if ((k % 8) || (n % 8) || (lda % 8) || (ldb % 8) || (ldc % 8) || ((uintptr_t)a % 16) || ((uintptr_t)b % 16) ||
      ((uintptr_t)c % 16))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG,
                     "matmul: pointers must be 16-byte aligned and K, N and the row pitches multiples of 8");
  if (lda < k || ldb < n || ldc < n) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: row pitch smaller than the row");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "matmul: cannot select device %d", ctx->device);
  // Two-CTA tiles once there are enough 256x256 tiles to give every SM pair one; smaller outputs
  // spread better as 128x256 tiles.
  if ((!multicast || (!bias && !ctx->gemm_act)) &&
      (ctx->gemm_variant == 2 ||
       (ctx->gemm_variant == 1 && ((m + 255) / 256) * ((n + 255) / 256) >= ctx->sm_count / 2)))
    return ttlb_launch_gemm_bf16_2cta(ctx, a, lda, b, ldb, c, ldc, m, n, k, bias, ldbias, multicast, stream);

  CUtensorMap map_a, map_b;
  int rc = make_map(ctx, &map_a, a, (uint64_t)k, (uint64_t)m, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  rc = make_map(ctx, &map_b, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, 64, BK);
  if (rc) return rc;

  // the attribute is per device, and a context is bound to one device
  if (!ctx->gemm_attr_set) {
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              SMEM_BYTES));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              SMEM_BYTES));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_kernel<false, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_PUB));
    ctx->gemm_attr_set = true;
  }

  GemmParams p;
  p.c = reinterpret_cast<__nv_bfloat16 *>(c);
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.tiles_m = (int)((m + BM - 1) / BM);
  p.tiles_n = (int)((n + BN - 1) / BN);
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  p.multicast = multicast ? 1 : 0;
  if (multicast && ctx->pub_n_peers > 0) {
    // the output region in every GPU's copy of the buffer, given by the caller of ttlb_matmul_*_peers
    p.multicast = 2;
    p.n_peers = ctx->pub_n_peers;
    for (int i = 0; i < ctx->pub_n_peers; ++i) p.peer_c[i] = reinterpret_cast<__nv_bfloat16 *>(ctx->pub_peers[i]);
  }
  if (multicast && (bias || ctx->gemm_act))
    return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "matmul: bias / activation with a published output");
  p.bias = reinterpret_cast<const __nv_bfloat16 *>(bias);
  p.ldbias = ldbias;
  p.act = ctx->gemm_act;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  if (multicast)
    ttlb_gemm_bf16_kernel<false, true><<<grid, THREADS, SMEM_BYTES_PUB, stream>>>(map_a, map_b, p);
  else if (p.act)
    ttlb_gemm_bf16_kernel<true><<<grid, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p);
  else
    ttlb_gemm_bf16_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}

extern "C" int ttlb_matmul_bf16(ttlb_ctx *ctx, const ttlb_gemm_desc *d, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null descriptor");
  return ttlb_launch_gemm_bf16(ctx, d->a, d->lda, d->b, d->ldb, d->c, d->ldc, d->m, d->n, d->k,
                               reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ttlb_matmul_bf16_bias(ttlb_ctx *ctx, const ttlb_gemm_desc *d, const void *bias, int64_t ldbias, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null descriptor");
  if (!bias) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null bias");
  return ttlb_launch_gemm_bf16_full(ctx, d->a, d->lda, d->b, d->ldb, d->c, d->ldc, d->m, d->n, d->k, false, bias, ldbias,
                                    reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ttlb_matmul_bf16_epilogue(ttlb_ctx *ctx, const ttlb_gemm_desc *d, const void *bias, int64_t ldbias, int act,
                                         void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null descriptor");
  if (act < TTLB_ACT_NONE || act > TTLB_ACT_TANH) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: unknown activation %d", act);
  if (!bias && ldbias != 0) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: a bias pitch without a bias");
  ctx->gemm_act = act;
  const int rc = ttlb_launch_gemm_bf16_full(ctx, d->a, d->lda, d->b, d->ldb, d->c, d->ldc, d->m, d->n, d->k, false, bias,
                                            ldbias, reinterpret_cast<cudaStream_t>(stream));
  ctx->gemm_act = 0;
  return rc;
}

extern "C" int ttlb_matmul_bf16_multicast(ttlb_ctx *ctx, const ttlb_gemm_desc *d, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null descriptor");
  return ttlb_launch_gemm_bf16_ex(ctx, d->a, d->lda, d->b, d->ldb, d->c, d->ldc, d->m, d->n, d->k, true,
                                  reinterpret_cast<cudaStream_t>(stream));
}

// Peer pointers of ttlb_matmul_*_peers, checked and parked in the context for the launch that follows.
int ttlb_set_pub_peers(ttlb_ctx *ctx, void *const *peers, int n_peers) {
  if (!peers || n_peers < 1 || n_peers > MAX_PEERS)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: 1 to %d peer outputs", MAX_PEERS);
  for (int i = 0; i < n_peers; ++i) {
    if (!peers[i] || ((uintptr_t)peers[i] % 16))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: peer output %d is null or not 16-byte aligned", i);
    ctx->pub_peers[i] = peers[i];
  }
  ctx->pub_n_peers = n_peers;
  return TTLB_OK;
}

extern "C" int ttlb_matmul_bf16_peers(ttlb_ctx *ctx, const ttlb_gemm_desc *d, void *const *peers, int n_peers, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "matmul: null descriptor");
  int rc = ttlb_set_pub_peers(ctx, peers, n_peers);
  if (rc) return rc;
  rc = ttlb_launch_gemm_bf16_ex(ctx, d->a, d->lda, d->b, d->ldb, peers[0], d->ldc, d->m, d->n, d->k, true,
                                reinterpret_cast<cudaStream_t>(stream));
  ctx->pub_n_peers = 0;
  return rc;
}

extern "C" int ttlb_check_status(ttlb_ctx *ctx, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  ttlb_device_guard g(ctx->device);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  TTLB_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  TTLB_CUDA_CHECK(ctx, cudaStreamSynchronize(s));
  const int code = *ctx->h_status;
  if (code != 0) {
    TTLB_CUDA_CHECK(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), s));
    TTLB_CUDA_CHECK(ctx, cudaStreamSynchronize(s));
    static const char *who[] = {"", "TMA producer", "UMMA issuer", "epilogue", "softmax", "correction", "self-test"};
    return ttlb_fail(ctx, TTLB_ERR_TIMEOUT, "a bounded device-side wait ran out (%s, code %d)",
                     code > 0 && code < 7 ? who[code] : "?", code);
  }
  return TTLB_OK;
}

extern "C" int ttlb_set_gemm_variant(ttlb_ctx *ctx, int variant) {
  if (!ctx || variant < 0 || variant > 2) return TTLB_ERR_INVALID_ARG;
  ctx->gemm_variant = variant;
  return TTLB_OK;
}

extern "C" int ttlb_set_wait_limit(ttlb_ctx *ctx, int64_t cycles) {
  if (!ctx || cycles <= 0) return TTLB_ERR_INVALID_ARG;
  ctx->wait_limit_cycles = cycles;
  return TTLB_OK;
}

// One-time, per-device preparation of the context-free launch below (with that device current).
int ttlb_gemm_bf16_raw_prepare() {
  return cudaFuncSetAttribute(ttlb_gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) ==
                 cudaSuccess
             ? TTLB_OK
             : TTLB_ERR_CUDA;
}

// Context-free launch of the GEMM kernel for callers that bring their own status word and device
// facts (used by the allocation-free bfp8-weight entry point).  Arguments are assumed validated.
int ttlb_gemm_bf16_launch_raw(const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc, int64_t m,
                              int64_t n, int64_t k, int sm_count, int *d_status, long long wait_limit, bool *attr_set,
                              cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  int rc = make_map(nullptr, &map_a, a, (uint64_t)k, (uint64_t)m, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  rc = make_map(nullptr, &map_b, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, 64, BK);
  if (rc) return rc;
  if (!*attr_set) {
    if (cudaFuncSetAttribute(ttlb_gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return TTLB_ERR_CUDA;
    *attr_set = true;
  }
  GemmParams p;
  p.c = reinterpret_cast<__nv_bfloat16 *>(c);
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.tiles_m = (int)((m + BM - 1) / BM);
  p.tiles_n = (int)((n + BN - 1) / BN);
  p.status = d_status;
  p.wait_limit = wait_limit;
  p.multicast = 0;
  const int tiles = p.tiles_m * p.tiles_n;
  ttlb_gemm_bf16_kernel<false><<<tiles < sm_count ? tiles : sm_count, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p);
  return cudaGetLastError() == cudaSuccess ? TTLB_OK : TTLB_ERR_CUDA;
}

// ---- self-test of the bounded-wait machinery ------------------------------------------------
// One CTA initialises an mbarrier that nothing ever arrives on and waits for it with the given
// cycle limit.  The wait must give up, raise the abort flag, and the kernel must record code 6 in the
// status word and return normally - the same path a real kernel takes when a producer never shows
// up - so that the host-side reporting (ttlb_check_status -> TTLB_ERR_TIMEOUT) can be tested without
// ever hanging a GPU.
namespace {
__global__ void ttlb_wait_selftest_kernel(int *status, long long limit) {
  __shared__ unsigned long long bar_storage;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar_storage), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar_storage), 0, &abort_flag, limit);
    if (!ok) atomicCAS(status, 0, 6);
  }
  __syncthreads();
}
}  // namespace

extern "C" int ttlb_selftest_wait_timeout(ttlb_ctx *ctx, int64_t limit_cycles, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "selftest: limit must be in (0, 2e9] cycles");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "selftest: cannot select device %d", ctx->device);
  ttlb_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ctx->d_status, limit_cycles);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
