// Fused causal attention forward (ttlb_attention): O = softmax(scale * Q K^T + mask) V,
// bf16 in/out, fp32 scores, fp32 row max / row sum (online softmax), head_dim 128.
//
// The reference has no attention kernel (its README names a flash-attention test that is not
// in the tree); this is the tile program "for each KV block: S = Q @ K^T; online-softmax update;
// O += P @ V" written directly as a B200 kernel.
//
// One CTA per (batch*head, 128-query tile), 576 threads:
//   warp 0      TMA producer: Q tile once; K and V blocks (128 keys) through 2-stage rings
//   warp 1      UMMA issuer: S_j = Q K_j^T (128x128x128) into one of two TMEM score buffers,
//               then O += P_{j-1} V_{j-1} accumulated in TMEM, so the tensor pipe computes the
//               next scores while the softmax warps work.  P is read from TENSOR MEMORY (the A
//               operand of the second UMMA), not from shared memory.
//   warps 2..17 softmax: thread (row, one of four 32-column parts) reads its 32 scores with
//               tcgen05.ld, exchanges the row max with the three partner warps through shared
//               memory, writes P (bf16 pairs) with tcgen05.st over the first 64 columns of the
//               score buffer it came from, and keeps only the running max and sum.  O is
//               rescaled LAZILY: the max used for the exponentials is raised only when the true
//               max has grown by more than 2^8 (P stays below 256, exact enough in bf16 / fp32);
//               when it is, the threads wait for the last PV UMMA and multiply their 32 columns
//               of O in tensor memory by the correction.  At the end they read O once, divide by
//               the row sum and store bf16.  Four softmax warps per scheduler hide each other's
//               barrier and TMEM latency.
// The shared-memory data path is the scarce resource (a 128x128x128 UMMA reads 512 wavefronts of
// 128 bytes in its 512 cycles when both operands are in shared memory); keeping P out of shared
// memory removes a quarter of the kernel's traffic on it.
// UMMAs of one thread execute in issue order, which is what frees the buffers: S_{j+2} is issued
// after P_j V_j and so cannot overwrite the P_j that aliases S_j's buffer.
// Heavy (late) query tiles are scheduled first.  All waits are bounded.
#include <cuda_bf16.h>

#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;    // 32 KB: a 128 x 128 bf16 tile (Q, K block, V block, P)
constexpr int CHUNK_BYTES = 128 * 64 * 2;    // 16 KB: 128 rows x 64 elements (one 128-byte swizzle span)
constexpr int KV_STAGES = 2;
constexpr int NPART = 4;                      // column parts per row: softmax thread = (row, part)
constexpr int PCOLS = 128 / NPART;            // score / output columns per softmax thread
constexpr int ATT_THREADS = 64 + 128 * NPART;
constexpr int OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = OFF_K + KV_STAGES * TILE_BYTES,
              OFF_X = OFF_V + KV_STAGES * TILE_BYTES;  // X: row-max exchange
constexpr int XCH_BYTES = 2 * NPART * 128 * 4;   // [parity][part][row] floats
constexpr int OFF_BAR = OFF_X + XCH_BYTES;
constexpr int ATT_SMEM = OFF_BAR + 512 + 1024;
constexpr float RESCALE_THRESHOLD = 8.0f;   // in log2 units

struct AttnParams {
  __nv_bfloat16 *o;
  int seq, bh, q_tiles;
  int causal;
  float scale_log2e;
  int *status;
  long long wait_limit;
};

// barrier indices
enum {
  B_QFULL = 0,
  B_KFULL = 1,    // [2]
  B_KEMPTY = 3,   // [2]
  B_VFULL = 5,    // [2]
  B_VEMPTY = 7,   // [2]
  B_SFULL = 9,    // [2]
  B_PFULL = 11,   // [2]  count 4*NPART (one arrival per softmax warp)
  B_ODONE = 13,   //      a PV UMMA has completed (waited on only by a rescale, see there)
  B_OFINAL = 14,  //      the last PV UMMA has completed
  B_XCH = 15,     // [4]  count 32*NPART (all threads that share a TMEM lane quarter)
  B_COUNT = 19
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(ATT_THREADS, 1)
ttlb_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
  auto bar = [&](int i) { return base + OFF_BAR + 8u * i; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + OFF_BAR + 8 * B_COUNT);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + OFF_BAR + 8 * B_COUNT + 8);
  float *xch = reinterpret_cast<float *>(gen + OFF_X);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy tiles first: with a causal mask the last query tile has the most KV blocks
  const int qt = p.q_tiles - 1 - (int)(blockIdx.x % p.q_tiles);
  const int bh = (int)(blockIdx.x / p.q_tiles);
  const int kv_total = (p.seq + BKV - 1) / BKV;
  const int nblk = p.causal ? min(qt + 1, kv_total) : kv_total;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < B_COUNT; ++i) {
      uint32_t count = 1;
      if (i == B_PFULL || i == B_PFULL + 1) count = 4 * NPART;
      if (i >= B_XCH) count = 32 * NPART;
      mbar_init(bar(i), count);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_o = tmem_base + 256;  // S[2] at columns 0 / 128, O at 256

  int fail = 0;
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(B_QFULL), TILE_BYTES);
      tma_load_3d(base + OFF_Q, &map_q, 0, qt * BQ, bh, bar(B_QFULL));
      tma_load_3d(base + OFF_Q + CHUNK_BYTES, &map_q, 64, qt * BQ, bh, bar(B_QFULL));
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(bar(B_KEMPTY + s), ph ^ 1u, abort_flag, p.wait_limit)) { fail = 1; break; }
        mbar_expect_tx(bar(B_KFULL + s), TILE_BYTES);
        tma_load_3d(base + OFF_K + s * TILE_BYTES, &map_k, 0, j * BKV, bh, bar(B_KFULL + s));
        tma_load_3d(base + OFF_K + s * TILE_BYTES + CHUNK_BYTES, &map_k, 64, j * BKV, bh, bar(B_KFULL + s));
        if (!mbar_wait(bar(B_VEMPTY + s), ph ^ 1u, abort_flag, p.wait_limit)) { fail = 1; break; }
        mbar_expect_tx(bar(B_VFULL + s), TILE_BYTES);
        tma_load_3d(base + OFF_V + s * TILE_BYTES, &map_v, 0, j * BKV, bh, bar(B_VFULL + s));
        tma_load_3d(base + OFF_V + s * TILE_BYTES + CHUNK_BYTES, &map_v, 64, j * BKV, bh, bar(B_VFULL + s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);  // Q (K-major) x K^T (K-major)
      constexpr uint32_t idesc_o = idesc_bf16(BQ, HD, false, true);    // P (tensor memory) x V (N-major)
      if (!mbar_wait(bar(B_QFULL), 0, abort_flag, p.wait_limit)) fail = 2;
      auto issue_pv = [&](int j) -> bool {  // PV_j = P_j V_j
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(bar(B_PFULL + s), ph, abort_flag, p.wait_limit)) return false;
        if (!mbar_wait(bar(B_VFULL + s), ph, abort_flag, p.wait_limit)) return false;
        tc_fence_after();
        const uint32_t sv = base + OFF_V + s * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // P_j: 16 keys = 8 columns (two bf16 per column) of score buffer s
          const uint64_t db = desc_mnmajor_sw128(sv, CHUNK_BYTES) + (uint64_t)(kk * 128);
          umma_f16_ts(tm_o, tm_s + s * BKV + kk * 8, db, idesc_o, (j | kk) != 0);
        }
        umma_commit(bar(B_ODONE));
        umma_commit(bar(B_VEMPTY + s));
        return true;
      };
      for (int j = 0; j < nblk && !fail; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait(bar(B_KFULL + s), ph, abort_flag, p.wait_limit)) { fail = 2; break; }
        tc_fence_after();
        const uint32_t sk = base + OFF_K + s * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t da = desc_kmajor_sw128(base + OFF_Q + (kk >> 2) * CHUNK_BYTES) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = desc_kmajor_sw128(sk + (kk >> 2) * CHUNK_BYTES) + (uint64_t)((kk & 3) * 2);
          umma_f16(tm_s + s * BKV, da, db, idesc_s, kk != 0);
        }
        umma_commit(bar(B_SFULL + s));
        umma_commit(bar(B_KEMPTY + s));
        if (j > 0 && !issue_pv(j - 1)) { fail = 2; break; }
      }
      if (!fail && !issue_pv(nblk - 1)) fail = 2;
      if (!fail) umma_commit(bar(B_OFINAL));
    }
  } else {
    // ---- softmax warps: thread = (query row, one of NPART column parts) -------------------
    const int q = warp & 3;               // TMEM lane quarter this warp may access
    const int part = (warp - 2) >> 2;     // which PCOLS-wide slice of the key / head-dim columns
    const int row = q * 32 + lane;        // row inside the query tile
    const int q_idx = qt * BQ + row;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const float sl2e = p.scale_log2e;
    const uint32_t my_o = tm_o + lane_addr + part * PCOLS;
    float m_used = -INFINITY, l_run = 0.f;

    for (int j = 0; j < nblk; ++j) {
      const int s = j & 1;
      if (!mbar_wait(bar(B_SFULL + s), (uint32_t)((j >> 1) & 1), abort_flag, p.wait_limit)) { fail = 4; break; }
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld_32x32(tm_s + lane_addr + s * BKV + part * PCOLS, sr);
      tmem_ld_wait_dep(sr);

      const int key0 = j * BKV + part * PCOLS;
      if ((p.causal && j == qt) || (j + 1) * BKV > p.seq) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int key = key0 + c;
          if ((p.causal && key > q_idx) || key >= p.seq) sr[c] = 0xff800000u;  // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        mx0 = max3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
      }
      const float mx = fmaxf(mx0, mx1);
      // exchange the row max with the partner warps (the other column parts of the same rows)
      float *xrow = xch + (j & 1) * NPART * 128 + row;
      xrow[part * 128] = mx;
      mbar_arrive(bar(B_XCH + q));
      if (!mbar_wait(bar(B_XCH + q), (uint32_t)(j & 1), abort_flag, p.wait_limit)) { fail = 4; break; }
      float m_new = fmaxf(m_used, mx);
#pragma unroll
      for (int k = 1; k < NPART; ++k) m_new = fmaxf(m_new, xrow[((part + k) & (NPART - 1)) * 128]);
      // raise the max used for the exponentials only when the true max has moved far; all threads
      // of a row take the same decision from the same numbers
      float alpha = 1.0f;
      const bool raise = (m_new - m_used) * sl2e > RESCALE_THRESHOLD;
      if (raise) {
        alpha = fast_exp2((m_used - m_new) * sl2e);   // 0 on the first block
        m_used = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // O *= alpha, after PV_{j-1} has landed and before PV_j is released.  The parity test is
        // unambiguous: S_j, which this thread has read, was issued after PV_{j-2}, and UMMAs complete
        // in order, so the barrier is in phase j-1 or later.
        if (!mbar_wait(bar(B_ODONE), (uint32_t)((j - 1) & 1), abort_flag, p.wait_limit)) { fail = 4; break; }
        tc_fence_after();
        uint32_t r[32];
        tmem_ld_32x32(my_o, r);
        tmem_ld_wait_dep(r);
#pragma unroll
        for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
        tmem_st_32x32(my_o, r);
        tmem_st_wait();
      }
      const float neg = -m_used * sl2e;
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), sl2e, neg));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), sl2e, neg));
        rs0 += p0;
        rs1 += p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + (rs0 + rs1);
      // P_j over the first 64 columns of score buffer s: every thread of this lane quarter has read
      // its scores (it arrived on the exchange barrier after its load completed)
      tmem_st_32x16(tm_s + lane_addr + s * BKV + part * (PCOLS / 2), pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PFULL + s));
    }
    if (!fail) {
      const int slot = nblk & 1;
      float *xrow = xch + slot * NPART * 128 + row;
      xrow[part * 128] = l_run;
      mbar_arrive(bar(B_XCH + q));
      if (!mbar_wait(bar(B_XCH + q), (uint32_t)slot, abort_flag, p.wait_limit) ||
          !mbar_wait(bar(B_OFINAL), 0, abort_flag, p.wait_limit))
        fail = 4;
      uint32_t o[32];
      if (!fail) {
        tc_fence_after();
        tmem_ld_32x32(my_o, o);
        tmem_ld_wait_dep(o);
      }
      if (!fail && q_idx < p.seq) {
        float l_tot = l_run;
#pragma unroll
        for (int k = 1; k < NPART; ++k) l_tot += xrow[((part + k) & (NPART - 1)) * 128];
        const float inv = 1.0f / l_tot;
        __nv_bfloat16 *dst = p.o + ((long long)bh * p.seq + q_idx) * HD + part * PCOLS;
#pragma unroll
        for (int u = 0; u < PCOLS / 8; ++u) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[8 * u + 0]) * inv, __uint_as_float(o[8 * u + 1]) * inv);
          v.y = pack_bf16x2(__uint_as_float(o[8 * u + 2]) * inv, __uint_as_float(o[8 * u + 3]) * inv);
          v.z = pack_bf16x2(__uint_as_float(o[8 * u + 4]) * inv, __uint_as_float(o[8 * u + 5]) * inv);
          v.w = pack_bf16x2(__uint_as_float(o[8 * u + 6]) * inv, __uint_as_float(o[8 * u + 7]) * inv);
          *reinterpret_cast<uint4 *>(dst + 8 * u) = v;
        }
      }
    }
  }

  if (fail) atomicCAS(p.status, 0, fail);
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_map3(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t seq, uint64_t bh) {
  ttlb_encode_tiled_fn enc = ttlb_get_encode_tiled();
  if (!enc) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)HD, seq, bh};
  cuuint64_t strides[2] = {(cuuint64_t)HD * 2, seq * HD * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return TTLB_OK;
}

}  // namespace

extern "C" int ttlb_attention(ttlb_ctx *ctx, const ttlb_attn_desc *d, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: null descriptor");
  if (d->batch_heads == 0 || d->seq == 0) return TTLB_OK;
  if (!d->q || !d->k || !d->v || !d->o) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: null tensor");
  if (d->head_dim != HD) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "attention: head_dim %d (128 only)", (int)d->head_dim);
  if (d->batch_heads < 0 || d->seq < 0 || d->seq > (1 << 24) || d->batch_heads > (1 << 24))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: bad shape");
  if (((uintptr_t)d->q % 16) || ((uintptr_t)d->k % 16) || ((uintptr_t)d->v % 16) || ((uintptr_t)d->o % 16))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: tensors must be 16-byte aligned");
  if (!(d->scale > 0.f) || d->scale != d->scale) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: scale must be positive");
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "attention: cannot select device %d", ctx->device);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map3(ctx, &mq, d->q, (uint64_t)d->seq, (uint64_t)d->batch_heads))) return rc;
  if ((rc = make_map3(ctx, &mk, d->k, (uint64_t)d->seq, (uint64_t)d->batch_heads))) return rc;
  if ((rc = make_map3(ctx, &mv, d->v, (uint64_t)d->seq, (uint64_t)d->batch_heads))) return rc;
  if (!ctx->attn_attr_set) {
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));
    ctx->attn_attr_set = true;
  }
  AttnParams p;
  p.o = reinterpret_cast<__nv_bfloat16 *>(d->o);
  p.seq = (int)d->seq;
  p.bh = (int)d->batch_heads;
  p.q_tiles = (int)((d->seq + BQ - 1) / BQ);
  p.causal = d->causal ? 1 : 0;
  p.scale_log2e = d->scale * 1.4426950408889634f;
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  const long long grid = (long long)p.q_tiles * p.bh;
  if (grid > 0x7fffffffLL) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "attention: too many tiles");
  ttlb_attention_kernel<<<(unsigned)grid, ATT_THREADS, ATT_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(mq, mk, mv, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
