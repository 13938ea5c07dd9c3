// bfloat8_b-weight GEMM with the block-float unpack INSIDE the mainloop (no bf16 copy of the
// weights in HBM).  A cluster of two CTAs computes a 256x256 output tile with two-CTA UMMAs
// (tcgen05 cta_group::2), as gemm_bf16_2cta.cu does; the difference is the B operand:
//
//   * warp 0 brings, per 64-deep k-block, this CTA's 128 weight columns as PACKED tiles
//     (2 tile rows x 4 tile columns x 1088 bytes; tiles of one tile row are contiguous, so two
//     untiled bulk copies) into a staging ring;
//   * warps 6..13 (256 threads in groups that take the k-blocks in turn, one 16-value block per
//     thread at a time) expand them in registers (bfp8_unpack.cuh) and write bf16 into the UMMA's B
//     slot in the 128-byte-swizzled, column-major ("MN-major") layout a TMA load of a bf16 matrix
//     would have produced, fence the writes towards the async proxy and arrive on the LEADER CTA's
//     "B ready" barrier;
//   * the leader's warp 1 waits for A (TMA bytes of both CTAs) and for B, then issues the UMMAs.
//
// HBM/L2 traffic for the weights is 1.0625 bytes per value instead of 1.0625 + 2 (unpack kernel
// write) + 2 (GEMM read), and no scratch memory is needed.  The price: a weight tile is expanded once
// per 256-row output tile that uses it instead of once, and the expansion shares the SM's
// shared-memory data path with the tensor core.  Per k-block and SM that path carries 128
// wavefronts (128 B each) of TMA writes for A, 68 for the packed tiles, about 84 of converter reads,
// 128 of converter writes and 256 of tensor-core reads, against 512 cycles of UMMA time; measured
// on 4096x8192x28672 this kernel takes 1.55 ms where the unpack kernel plus the bf16 two-CTA GEMM
// take 1.38 ms, so ttlb_matmul_bfp8w uses it only when asked (ttlb_set_bfp8_mode).  A variant whose
// converters read the packed tiles straight from global memory (no staging ring) measured 1.65 ms.
//
// Shared memory per CTA: 5 stages x (16 KB A + 16 KB B + 8.5 KB packed) = 202.5 KB.
// Every wait is bounded; no load is multicast.
#include <cuda_bf16.h>

#include "bfp8_unpack.cuh"
#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int FBM = 256, FBN = 256, FBK = 64, FSTAGES = 5;
constexpr int FA_BYTES = 128 * FBK * 2;       // 16 KB
constexpr int FB_CHUNK = FBK * 64 * 2;        // 8 KB: 64 columns x 64 k
constexpr int FB_BYTES = 2 * FB_CHUNK;        // 16 KB: this CTA's 128 columns
constexpr int TILE_BYTES = 1088;
constexpr int FP_ROW = 4 * TILE_BYTES;        // packed tiles of one tile row: 4352 B
constexpr int FP_BYTES = 2 * FP_ROW;          // 8704 B
constexpr int FTHREADS = 14 * 32;
constexpr int CONV_WARPS = 8;
constexpr int CONV_GROUPS = 2;   // measured on 4096x8192x28672: 1 group 1.59 ms, 2 groups 1.55 ms, 4 groups 1.59 ms
constexpr int FGROUP_M = 8;
constexpr int FSMEM_BYTES = FSTAGES * (FA_BYTES + FB_BYTES + FP_BYTES) + 1024 + 512;

struct FusedParams {
  const uint8_t *tiles;    // packed weights, row-major tile order
  long long tile_cols_total;
  int tile_col0;           // first tile column of the weight slice
  int tile_rows, tile_cols;  // k / 32, n / 32
  __nv_bfloat16 *c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n;
  int *status;
  long long wait_limit;
};

__device__ __forceinline__ void ftile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int per_group = FGROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * FGROUP_M;
  const int rows = min(FGROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

template <int G>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FTHREADS, 1)
ttlb_gemm_bfp8w_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_ring = base, b_ring = base + FSTAGES * FA_BYTES, p_ring = b_ring + FSTAGES * FB_BYTES;
  const uint32_t bars = p_ring + FSTAGES * FP_BYTES;
  uint8_t *gen_b = gbase + FSTAGES * FA_BYTES;
  const uint8_t *gen_p = gen_b + FSTAGES * FB_BYTES;
  uint8_t *gen_bars = gbase + FSTAGES * (FA_BYTES + FB_BYTES + FP_BYTES);
  auto afull_bar = [&](int s) { return bars + 8u * s; };                   // leader: A bytes of both CTAs
  auto pfull_bar = [&](int s) { return bars + 8u * (FSTAGES + s); };       // local: packed bytes
  auto bfull_bar = [&](int s) { return bars + 8u * (2 * FSTAGES + s); };   // leader: 16 converter warps
  auto empty_bar = [&](int s) { return bars + 8u * (3 * FSTAGES + s); };   // local: UMMAs done with the stage
  auto tfull_bar = [&](int a) { return bars + 8u * (4 * FSTAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (4 * FSTAGES + 2 + a); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_bars + 8 * (4 * FSTAGES + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_bars + 8 * (4 * FSTAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + FBK - 1) / FBK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < FSTAGES; ++s) {
      mbar_init(afull_bar(s), 1);
      mbar_init(pfull_bar(s), 1);
      mbar_init(bfull_bar(s), 2 * CONV_WARPS / G);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int fail = 0;
  if (warp == 0) {
    // ---- producer: A by TMA (signals the leader), packed weights by bulk copies (signal locally)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters) {
        int tm, tn;
        ftile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int tc0 = tn * (FBN / 32) + (int)rank * 4;            // first tile column of this CTA's half
        const int ntc = max(0, min(4, p.tile_cols - tc0));          // tile columns that exist
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit)) { fail = 1; break; }
          if (rank == 0) mbar_expect_tx(afull_bar(stage), 2 * FA_BYTES);
          tma_load_2d_2sm(a_ring + stage * FA_BYTES, &map_a, kb * FBK, tm * FBM + (int)rank * 128,
                          afull_bar(stage) & 0xFEFFFFFFu);
          const int ntr = min(2, p.tile_rows - kb * 2);
          if (ntc > 0) {
            mbar_expect_tx(pfull_bar(stage), (uint32_t)(ntr * ntc * TILE_BYTES));
            for (int r = 0; r < ntr; ++r)
              bulk_load(p_ring + stage * FP_BYTES + r * FP_ROW,
                        p.tiles + ((long long)(kb * 2 + r) * p.tile_cols_total + p.tile_col0 + tc0) * TILE_BYTES,
                        (uint32_t)(ntc * TILE_BYTES), pfull_bar(stage));
          } else {
            mbar_arrive(pfull_bar(stage));   // nothing to load for this half: release the converters
          }
          if (++stage == FSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- UMMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(FBM, FBN, false, true);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.wait_limit)) { fail = 2; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * FBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(afull_bar(stage), phase, abort_flag, p.wait_limit)) { fail = 2; break; }
          if (!mbar_wait(bfull_bar(stage), phase, abort_flag, p.wait_limit)) { fail = 2; break; }
          tc_fence_after();
          const uint64_t da = desc_kmajor_sw128(a_ring + stage * FA_BYTES);
          const uint64_t db = desc_mnmajor_sw128(b_ring + stage * FB_BYTES, FB_CHUNK);
#pragma unroll
          for (int k = 0; k < FBK / 16; ++k)
            umma_f16_2sm(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc, (kb | k) != 0);
          umma_commit_2sm(empty_bar(stage));
          if (++stage == FSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (fail) break;
        umma_commit_2sm(tfull_bar(acc));
      }
    }
  } else if (warp < 6) {
    // ---- epilogue: this CTA's 128 accumulator rows
    const int q = warp & 3;
    int local = 0;
    for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
      int tm, tn;
      ftile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      // the outcome of the wait is made the same for the whole warp: what follows is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_limit))) { fail = 3; break; }
      tc_fence_after();
      const int row = tm * FBM + (int)rank * 128 + q * 32 + lane;
      __nv_bfloat16 *crow = p.c + (long long)row * p.ldc + (long long)tn * FBN;
#pragma unroll 1
      for (int c = 0; c < FBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * FBN + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * FBN + c * 32;
        if (row < p.m && col0 < p.n) {   // n is a multiple of 32: a 32-column group is all in or all out
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            *reinterpret_cast<uint4 *>(crow + c * 32 + v * 8) = o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(tempty_bar(acc), 0);
    }
  } else {
    // ---- converters: packed tiles -> swizzled bf16 B slot.  G groups of 8/G warps take the k-blocks
    // in turn, so the latency of one k-block's chain (wait, read, expand, write, proxy fence, remote
    // arrive) is spread over G k-block times.
    constexpr int W = CONV_WARPS / G;            // warps per group
    const int cw = warp - 6;                     // 0..7
    const int group = cw / W, tig = (cw % W) * 32 + lane;   // thread in group
    long long it = 0;                            // k-blocks seen so far (all tiles)
    for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters) {
      int tm, tn;
      ftile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int tc_first = tn * (FBN / 32) + (int)rank * 4;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((int)(it % G) != group) continue;
        const int stage = (int)(it % FSTAGES);
        const uint32_t phase = (uint32_t)((it / FSTAGES) & 1);
        if (!mbar_wait(pfull_bar(stage), phase, abort_flag, p.wait_limit)) { fail = 4; break; }
        const uint8_t *ps = gen_p + stage * FP_BYTES;
        uint8_t *bs = gen_b + stage * FB_BYTES;
#pragma unroll
        for (int j = 0; j < 2 * G; ++j) {
          const int u = j * (32 * W) + tig;      // 0..511: tile = u / 64 (tile row = tile / 4), block = u % 64
          const int tile_i = u >> 6, blk = u & 63, trow = tile_i >> 2, tcol = tile_i & 3;
          const int f = blk >> 4, fr = blk & 15;
          const int kk = trow * 32 + (f >> 1) * 16 + fr;         // k row within the slot
          const int g0 = (tcol & 1) * 4 + (f & 1) * 2;           // first of the block's two 16-byte column groups
          const uint32_t rowoff = (uint32_t)((tcol >> 1) * FB_CHUNK + kk * 128);
          uint32_t o[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
          if (tc_first + tcol < p.tile_cols && kb * 2 + trow < p.tile_rows) {
            const uint8_t *tile = ps + trow * FP_ROW + tcol * TILE_BYTES;
            const int E = tile[blk];
            const uint4 v = *reinterpret_cast<const uint4 *>(tile + 64 + blk * 16);
            unpack_block(v, E, o);
          }
          *reinterpret_cast<uint4 *>(bs + rowoff + ((g0 ^ (kk & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4 *>(bs + rowoff + (((g0 + 1) ^ (kk & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async();
        __syncwarp();
        // every lane has fenced its own writes; the arrive (default semantics: release) publishes them.
        // An explicit cluster-scope release on this arrive was measured at half the speed.
        if (lane == 0) mbar_arrive_remote(bfull_bar(stage), 0);
      }
    }
  }

  if (fail) atomicCAS(p.status, 0, fail);
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

}  // namespace

int ttlb_make_map_bf16_2d(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// Arguments are validated by the caller (matmul_bfp8w_impl in bfp8.cu).
int ttlb_launch_gemm_bfp8w_fused(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, cudaStream_t stream) {
  CUtensorMap map_a;
  int rc = ttlb_make_map_bf16_2d(ctx, &map_a, d->a, (uint64_t)d->k, (uint64_t)d->m, (uint64_t)d->lda * 2, FBK, 128);
  if (rc) return rc;
  if (!ctx->gemm_fused_attr_set) {
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bfp8w_2cta_kernel<CONV_GROUPS>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, FSMEM_BYTES));
    ctx->gemm_fused_attr_set = true;
  }
  FusedParams p;
  p.tiles = reinterpret_cast<const uint8_t *>(d->b_tiles);
  p.tile_cols_total = d->b_tile_cols;
  p.tile_col0 = (int)d->b_tile_col0;
  p.tile_rows = (int)(d->k / 32);
  p.tile_cols = (int)(d->n / 32);
  p.c = reinterpret_cast<__nv_bfloat16 *>(d->c);
  p.ldc = d->ldc;
  p.m = (int)d->m;
  p.n = (int)d->n;
  p.k = (int)d->k;
  p.tiles_m = (int)((d->m + FBM - 1) / FBM);
  p.tiles_n = (int)((d->n + FBN - 1) / FBN);
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  const int tiles = p.tiles_m * p.tiles_n;
  int clusters = ctx->sm_count / 2;
  if (clusters > tiles) clusters = tiles;
  ttlb_gemm_bfp8w_2cta_kernel<CONV_GROUPS><<<clusters * 2, FTHREADS, FSMEM_BYTES, stream>>>(map_a, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
