// bf16 GEMM with two-CTA tensor-core instructions (tcgen05 cta_group::2): a cluster of two CTAs on
// neighbouring SMs computes one 256x256 output tile.  Each CTA loads its own 128 rows of A and only
// HALF of the B tile (128 of the 256 columns); the UMMA issued by the leader CTA reads both halves,
// so per SM the shared-memory traffic for B (TMA writes and UMMA reads) is halved compared with the
// one-CTA 128x256 kernel, and 6 stages of 32 KB fit where 4 stages of 48 KB did.
//
// Roles per CTA (192 threads) are those of the one-CTA kernel (gemm_bf16.cu); differences:
//   * TMA loads use the cta_group::2 form and signal the LEADER's "full" barrier, which the leader
//     arms with the byte count of both CTAs;
//   * only the leader's warp 1 issues UMMAs (M = 256); tcgen05.commit arrives on the barrier at
//     the same offset in both CTAs, so each CTA's producer and epilogue wait locally;
//   * each CTA's epilogue drains its own 128 TMEM lanes; "accumulator free" arrivals of both CTAs
//     go to the leader (remote mbarrier arrive).
// No TMA load is multicast.  All waits are bounded as in the one-CTA kernel.
#include <cuda_bf16.h>

#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM2 = 256, BN2 = 256, BK2 = 64;
constexpr int A2_BYTES = 128 * BK2 * 2;        // this CTA's 128 rows of A: 16 KB
constexpr int B2_CHUNK = BK2 * 64 * 2;         // 8 KB: one 64-column slice
constexpr int B2_BYTES = BK2 * 128 * 2;        // this CTA's 128 columns of B: 16 KB
constexpr int STAGE2_BYTES = A2_BYTES + B2_BYTES;
constexpr int THREADS2 = 192;
// 6 stages x 32 KB; measured on 8192^3: 4 stages 1489, 6 stages 1522, 7 stages 1519 TFLOP/s, and
// rasterisation groups of 4 / 8 / 16 / 32 tile rows 1481 / 1522 / 1511 / 1410 TFLOP/s
constexpr int STAGES2_DEFAULT = 6, GROUP_M2_DEFAULT = 8;
constexpr int smem2_bytes(int stages) { return stages * STAGE2_BYTES + 1024 + 256; }
// the publishing epilogue passes 32 rows x 128 columns per warp through a swizzled stage
constexpr int PUB2_COLS = 128;
constexpr int PUB2_WARP_BYTES = 32 * PUB2_COLS * 2;   // 8 KB
constexpr int smem2_bytes_pub(int stages) { return smem2_bytes(stages) + 4 * PUB2_WARP_BYTES; }
constexpr int MAX_PEERS2 = 8;

struct Gemm2Params {
  __nv_bfloat16 *c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n;  // in 256x256 tiles
  int *status;
  long long wait_limit;
  const __nv_bfloat16 *bias = nullptr;  // optional [m, n] matrix added to the product before rounding
  long long ldbias = 0;                 // 0: the bias is one row of n values, added to every output row
  int act = 0;                          // TTLB_ACT_*: applied to product + bias before the rounding
  // 0: c is this GPU's output.  1: c is a multicast address (multimem.st: the switch replicates every store to all GPUs
  // of the group).  2: every tile is stored to peer_c[0 .. n_peers), the output in every GPU's copy of a shared buffer
  // (peer-mapped memory, this GPU's own copy included).  Peer memory is only ever written.
  int multicast = 0;
  __nv_bfloat16 *peer_c[MAX_PEERS2] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_peers = 0;
};

template <int GROUP_M2>
__device__ __forceinline__ void tile_coords2(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int per_group = GROUP_M2 * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M2;
  const int rows = min(GROUP_M2, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

// PUB: the instantiation whose epilogue publishes the output to several GPUs through a shared-memory stage
template <int STAGES2, int GROUP_M2, bool ACT, bool PUB = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS2, 1)
ttlb_gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES2 * STAGE2_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES2 + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES2 + 2 + a); };
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw)) + STAGES2 * STAGE2_BYTES;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + 8 * (2 * STAGES2 + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + 8 * (2 * STAGES2 + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + BK2 - 1) / BK2;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);    // used in the leader only: armed there with both CTAs' bytes
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // used in the leader only: 4 epilogue warps of each CTA
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // the peer's barriers are initialised before anything can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int fail = 0;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters) {
        int tm, tn;
        tile_coords2<GROUP_M2>(t, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit)) { fail = 1; break; }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE2_BYTES);
          const uint32_t sa = base + stage * STAGE2_BYTES, sb = sa + A2_BYTES;
          const uint32_t lbar = full_bar(stage) & 0xFEFFFFFFu;   // the leader CTA's barrier
          tma_load_2d_2sm(sa, &map_a, kb * BK2, tm * BM2 + (int)rank * 128, lbar);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_2d_2sm(sb + j * B2_CHUNK, &map_b, tn * BN2 + (int)rank * 128 + j * 64, kb * BK2, lbar);
          if (++stage == STAGES2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM2, BN2, false, true);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.wait_limit)) { fail = 2; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.wait_limit)) { fail = 2; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE2_BYTES, sb = sa + A2_BYTES;
          const uint64_t da = desc_kmajor_sw128(sa), db = desc_mnmajor_sw128(sb, B2_CHUNK);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k)
            umma_f16_2sm(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc, (kb | k) != 0);
          umma_commit_2sm(empty_bar(stage));
          if (++stage == STAGES2) { stage = 0; phase ^= 1u; }
        }
        if (fail) break;
        umma_commit_2sm(tfull_bar(acc));
      }
    }
  } else {
    const int q = warp & 3;
    int local = 0;
    for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
      int tm, tn;
      tile_coords2<GROUP_M2>(t, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      // the outcome of the wait is made the same for the whole warp: what follows is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_limit))) { fail = 3; break; }
      tc_fence_after();
      if constexpr (PUB) {
        // tcgen05.ld hands every thread one row; the rows go through a swizzled stage so that each store
        // instruction of the warp writes two whole 256-byte row segments (16 lanes x 16 bytes each) - through
        // NVLink, 16-byte stores scattered over 32 rows reach a small fraction of the link rate
        uint8_t *stage = gen + 256 + (warp - 2) * PUB2_WARP_BYTES;
#pragma unroll 1
        for (int half = 0; half < BN2 / PUB2_COLS; ++half) {
#pragma unroll 1
          for (int cc = 0; cc < PUB2_COLS / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN2 + half * PUB2_COLS + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              const int unit = cc * 4 + v;  // 16-byte unit within the 256-byte row
              *reinterpret_cast<uint4 *>(stage + lane * (PUB2_COLS * 2) + ((unit ^ (lane & 7)) << 4)) = o;
            }
          }
          if (half == BN2 / PUB2_COLS - 1) {
            // every accumulator column has been read: the issuer may start the next tile into this buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(tempty_bar(acc), 0);
          } else {
            __syncwarp();
          }
          const int unit = lane & 15;
          const long long gcol = (long long)tn * BN2 + half * PUB2_COLS + unit * 8;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rl = 2 * i + (lane >> 4);
            const uint4 o = *reinterpret_cast<const uint4 *>(stage + rl * (PUB2_COLS * 2) + ((unit ^ (rl & 7)) << 4));
            const long long grow = (long long)tm * BM2 + (int)rank * 128 + q * 32 + rl;
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
      const int row = tm * BM2 + (int)rank * 128 + q * 32 + lane;
      __nv_bfloat16 *crow = p.c + (long long)row * p.ldc + (long long)tn * BN2;
      const __nv_bfloat16 *brow = p.bias ? p.bias + (long long)row * p.ldbias + (long long)tn * BN2 : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN2 / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN2 + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN2 + c * 32;
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
      if (lane == 0) mbar_arrive_remote(tempty_bar(acc), 0);
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
  cluster_sync();   // neither CTA frees tensor memory or exits while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

}  // namespace

int ttlb_make_map_bf16_2d(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// Two-CTA launch; arguments are validated by the caller (ttlb_launch_gemm_bf16_ex).  publish: c is a multicast address,
// or - when the context holds peer pointers (ttlb_matmul_bf16_peers) - the output is stored to each of them; n % 8 == 0,
// no bias, no activation.
int ttlb_launch_gemm_bf16_2cta(ttlb_ctx *ctx, const void *a, int64_t lda, const void *b, int64_t ldb, void *c, int64_t ldc,
                               int64_t m, int64_t n, int64_t k, const void *bias, int64_t ldbias, bool publish,
                               cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  int rc = ttlb_make_map_bf16_2d(ctx, &map_a, a, (uint64_t)k, (uint64_t)m, (uint64_t)lda * 2, BK2, 128);
  if (rc) return rc;
  rc = ttlb_make_map_bf16_2d(ctx, &map_b, b, (uint64_t)n, (uint64_t)k, (uint64_t)ldb * 2, 64, BK2);
  if (rc) return rc;
  if (!ctx->gemm2_attr_set) {
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, false>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(STAGES2_DEFAULT)));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(STAGES2_DEFAULT)));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, false, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes_pub(STAGES2_DEFAULT)));
    ctx->gemm2_attr_set = true;
  }
  Gemm2Params p;
  p.c = reinterpret_cast<__nv_bfloat16 *>(c);
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.tiles_m = (int)((m + BM2 - 1) / BM2);
  p.tiles_n = (int)((n + BN2 - 1) / BN2);
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  p.bias = reinterpret_cast<const __nv_bfloat16 *>(bias);
  p.ldbias = ldbias;
  p.act = ctx->gemm_act;
  const int tiles = p.tiles_m * p.tiles_n;
  int clusters = ctx->sm_count / 2;
  if (clusters > tiles) clusters = tiles;
  if (publish) {
    if (bias || p.act) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "matmul: bias / activation with a published output");
    p.multicast = 1;
    if (ctx->pub_n_peers > 0) {
      p.multicast = 2;
      p.n_peers = ctx->pub_n_peers;
      for (int i = 0; i < ctx->pub_n_peers; ++i) p.peer_c[i] = reinterpret_cast<__nv_bfloat16 *>(ctx->pub_peers[i]);
    }
    ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, false, true>
        <<<clusters * 2, THREADS2, smem2_bytes_pub(STAGES2_DEFAULT), stream>>>(map_a, map_b, p);
  } else if (p.act)
    ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, true>
        <<<clusters * 2, THREADS2, smem2_bytes(STAGES2_DEFAULT), stream>>>(map_a, map_b, p);
  else
    ttlb_gemm_bf16_2cta_kernel<STAGES2_DEFAULT, GROUP_M2_DEFAULT, false>
        <<<clusters * 2, THREADS2, smem2_bytes(STAGES2_DEFAULT), stream>>>(map_a, map_b, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
