// Fused causal attention forward (ttlb_attention): O = softmax(scale * Q K^T + mask) V,
// bf16 in/out, fp32 scores, fp32 row max / row sum (online softmax), head_dim 128.
//
// The reference has no attention kernel (its README names a flash-attention test that is not
// in the tree); this is the tile program "for each KV block: S = Q @ K^T; online-softmax update;
// O += P @ V" written directly as a B200 kernel.
//
// One CTA per (batch*head, PAIR of 128-query tiles), 384 threads.  The two query tiles A and B
// share every K / V block (loaded once) and take turns on the tensor pipe, so the softmax of one
// tile runs under the UMMAs of the other:
//   warp 0      TMA producer: Q_A, Q_B once; K and V blocks (128 keys) through 2-stage rings
//   warp 1      UMMA issuer.  Per KV block j and tile T: S_T = Q_T K_j^T (128x128x128) into T's
//               score buffer in tensor memory, and O_T += P_T V_j with P_T read FROM TENSOR MEMORY
//               (A operand) and O_T accumulated in tensor memory.  Issue order
//               ... PV_A(j), S_A(j+1), PV_B(j), S_B(j+1) ...; UMMAs execute in issue order, which is
//               what makes S_T(j+1) safe to overwrite the P_T(j) that aliases its buffer.
//   warps 2, 3  idle: with warps 0 and 1 they form the warpgroup that gives its registers away (setmaxnreg:
//               56 per thread there, 224 per softmax thread - the softmax holds a row's 128 scores, its 16 packed
//               probabilities and the running statistics in registers and schedules better with room to spare)
//   warps 4..11 softmax, 4 warps per tile, ONE THREAD PER QUERY ROW: the thread reads its 128 scores with
//               tcgen05.ld, takes their maximum without talking to any other thread, writes P (bf16 pairs)
//               with tcgen05.st over the first 64 columns of the score buffer - keys [0, 64) first, so that
//               the first half of P*V runs under the second half of the exponentials - and keeps only the
//               running max and sum.  O is rescaled LAZILY: the max used for the exponentials is
//               raised only when the true max has grown by more than 2^8 (P stays below 256, exact
//               enough in bf16 and fp32); when it is, the warp waits for the last PV UMMA of
//               its tile and multiplies its rows of O in tensor memory by the correction.
//               At the end the threads read O once, divide by the row sum and store bf16.
//               (Two threads per row - 16 softmax warps - cost an exchange of the row maximum through shared
//               memory in every block and were 4 % slower; a polynomial exp2 on the FMA pipe for part of
//               the exponentials was slower in both layouts: the softmax warps are bound by instruction
//               issue and by the chain score -> P -> next score, not by the special-function unit.
//               The scale-and-subtract and the row sum use packed fp32 pairs (fma / add .f32x2).
//               Measured and not kept: scores in two 64-key halves with the second half computed ahead
//               (twice as many, less efficient UMMAs: the tensor pipe became the limit); one UMMA
//               issuer thread per tile (their instructions interleave and the pipe switches accumulator
//               at every instruction).)
// Tensor memory: S_A, S_B, O_A, O_B, 128 columns each.  Shared memory: Q_A, Q_B, K[2], V[2] of 32 KB.
// The shared-memory data path is the scarce resource (a 128x128x128 UMMA with both operands in
// shared memory reads 512 wavefronts of 128 bytes in its 512 cycles): P and O never touch it, and
// each K / V block written by the TMA serves two query tiles.
// Heavy (late) query tiles are scheduled first.  All waits are bounded.
#include <cuda_bf16.h>

#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;    // 32 KB: a 128 x 128 bf16 tile (Q tile, K block, V block)
constexpr int CHUNK_BYTES = 128 * 64 * 2;    // 16 KB: 128 rows x 64 elements (one 128-byte swizzle span)
constexpr int KV_STAGES = 2;
constexpr int NT = 2;                         // query tiles per CTA
constexpr int NPART = 1;                      // one softmax thread per query row: it sees all 128 scores of a block
constexpr int SM_WARP0 = 4;                   // warps 0-3: TMA producer, UMMA issuer, two idle (the register donors)
constexpr int ATT_THREADS = SM_WARP0 * 32 + NT * NPART * 128;
// Registers move from the first warpgroup to the softmax warps (setmaxnreg); 128 * REG_LOW + 256 * REG_HIGH must not
// exceed what the CTA was launched with (384 threads x 168), or the raise would wait for registers for ever.
constexpr int REG_LOW = 56, REG_HIGH = 224;
static_assert(128 * REG_LOW + 256 * REG_HIGH <= ATT_THREADS * 168, "register pool of the CTA exceeded");
constexpr int OFF_Q = 0, OFF_K = NT * TILE_BYTES, OFF_V = OFF_K + KV_STAGES * TILE_BYTES,
              OFF_BAR = OFF_V + KV_STAGES * TILE_BYTES;
constexpr int ATT_SMEM = OFF_BAR + 512 + 1024;
constexpr float RESCALE_THRESHOLD = 8.0f;    // in log2 units

constexpr int MAX_PEERS = 8;

struct AttnParams {
  // pub == 0: plain stores to `o`.  1: `o` is an NVLink multicast address, stored with multimem.st (the switch
  // replicates every store to all GPUs of the group).  2: every row is stored to `peer_o[0..n_peers)`, the output
  // in every GPU's copy of a shared buffer (peer-mapped memory, this GPU's own copy included).
  int pub = 0;
  __nv_bfloat16 *peer_o[MAX_PEERS] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_peers = 0;
  __nv_bfloat16 *o;
  int seq, bh, q_tiles, q_pairs;
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
  B_SFULL = 9,    // [NT]
  B_PFULL = 11,   // [NT][2]  count 4 (the tile's softmax warps): keys [0, 64) / [64, 128) of P are written
  B_ODONE = 15,   // [NT]  a PV UMMA of the tile has completed
  B_COUNT = 17
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// ---- packed fp32 pairs: one instruction works on two values (fma / add .f32x2), which halves the issue slots the
// softmax spends on the scale-and-subtract and on the row sum
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
typedef unsigned long long f2_t;
__device__ __forceinline__ f2_t f2_pack(float lo, float hi) {
  f2_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f2_t f2_pack_u(uint32_t lo, uint32_t hi) {
  f2_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(f2_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2_t f2_fma(f2_t a, f2_t b, f2_t c) {
  f2_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f2_t f2_add(f2_t a, f2_t b) {
  f2_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 32 scores -> 32 probabilities exp2(s * scale - max * scale) as 16 bf16 pairs; the row sum is kept as a pair
__device__ __forceinline__ void exp_pack32(const uint32_t (&src)[32], f2_t sl2e2, f2_t neg2, f2_t &rs2, uint32_t (&pk)[16]) {
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    float a0, a1;
    f2_unpack(f2_fma(f2_pack_u(src[c], src[c + 1]), sl2e2, neg2), a0, a1);
    const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
    rs2 = f2_add(rs2, f2_pack(p0, p1));
    pk[c >> 1] = pack_bf16x2(p0, p1);
  }
}

// PUB: the instantiation whose epilogue publishes the output to several GPUs through a shared-memory stage
template <bool PUB>
__global__ void __launch_bounds__(ATT_THREADS, 1)
ttlb_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
  auto bar = [&](int i) { return base + OFF_BAR + 8u * i; };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + OFF_BAR + 8 * B_COUNT);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + OFF_BAR + 8 * B_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy pairs first: with a causal mask the last query tiles have the most KV blocks
  const int pr = p.q_pairs - 1 - (int)(blockIdx.x % p.q_pairs);
  const int bh = (int)(blockIdx.x / p.q_pairs);
  const int kv_total = (p.seq + BKV - 1) / BKV;
  // KV blocks of tile T (0 when the tile does not exist)
  auto blocks_of = [&](int t) {
    const int qt = 2 * pr + t;
    if (qt >= p.q_tiles) return 0;
    return p.causal ? min(qt + 1, kv_total) : kv_total;
  };
  const int n_a = blocks_of(0), n_b = blocks_of(1);
  const int nblk = max(n_a, n_b);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < B_COUNT; ++i) {
      uint32_t count = 1;
      if (i >= B_PFULL && i < B_PFULL + 2 * NT) count = 4;
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
  const uint32_t tm_s = tmem_base, tm_o = tmem_base + NT * BKV;  // S_A, S_B at columns 0 / 128; O_A, O_B at 256 / 384

  int fail = 0;
  // every role branch starts with its own register move: after a join the lower limit would apply to all
  if (warp == 0) {
    reg_dec<REG_LOW>();
    if (lane == 0) {
      mbar_expect_tx(bar(B_QFULL), (n_b > 0 ? 2 : 1) * TILE_BYTES);
      for (int t = 0; t < NT; ++t) {
        if (t == 1 && n_b == 0) break;
        tma_load_3d(base + OFF_Q + t * TILE_BYTES, &map_q, 0, (2 * pr + t) * BQ, bh, bar(B_QFULL));
        tma_load_3d(base + OFF_Q + t * TILE_BYTES + CHUNK_BYTES, &map_q, 64, (2 * pr + t) * BQ, bh, bar(B_QFULL));
      }
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
    reg_dec<REG_LOW>();
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);  // Q (K-major) x K^T (K-major)
      constexpr uint32_t idesc_o = idesc_bf16(BQ, HD, false, true);    // P (tensor memory) x V (N-major)
      const int n_of[NT] = {n_a, n_b};
      auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T; the caller has waited for K_j
        const uint32_t sk = base + OFF_K + (j & 1) * TILE_BYTES, sq = base + OFF_Q + t * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t da = desc_kmajor_sw128(sq + (kk >> 2) * CHUNK_BYTES) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = desc_kmajor_sw128(sk + (kk >> 2) * CHUNK_BYTES) + (uint64_t)((kk & 3) * 2);
          umma_f16(tm_s + t * BKV, da, db, idesc_s, kk != 0);
        }
        umma_commit(bar(B_SFULL + t));
      };
      auto issue_pv = [&](int t, int j) -> bool {  // O_t (+)= P_t V_j; the caller has waited for V_j
        const uint32_t sv = base + OFF_V + (j & 1) * TILE_BYTES;
        // P arrives in two steps: keys [0,64) first, then [64,128); the first half of the product runs under the
        // second half of the exponentials
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(bar(B_PFULL + t * 2 + h), (uint32_t)(j & 1), abort_flag, p.wait_limit)) return false;
          tc_fence_after();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int kk = h * 4 + i;   // 16 keys = 8 columns (two bf16 per column) of P
            const uint64_t db = desc_mnmajor_sw128(sv, CHUNK_BYTES) + (uint64_t)(kk * 128);
            umma_f16_ts(tm_o + t * HD, tm_s + t * BKV + kk * 8, db, idesc_o, (j | h | i) != 0);
          }
        }
        umma_commit(bar(B_ODONE + t));
        return true;
      };
      if (!mbar_wait(bar(B_QFULL), 0, abort_flag, p.wait_limit) ||
          !mbar_wait(bar(B_KFULL), 0, abort_flag, p.wait_limit)) fail = 2;
      if (!fail) {
        tc_fence_after();
        for (int t = 0; t < NT; ++t)
          if (n_of[t] > 0) issue_s(t, 0);
        umma_commit(bar(B_KEMPTY));
      }
      for (int j = 0; j < nblk && !fail; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(B_VFULL + s), (uint32_t)((j >> 1) & 1), abort_flag, p.wait_limit)) { fail = 2; break; }
        const bool more = j + 1 < nblk;
        bool k_ready = false;
        for (int t = 0; t < NT && !fail; ++t) {
          if (j < n_of[t] && !issue_pv(t, j)) { fail = 2; break; }
          if (t == NT - 1) umma_commit(bar(B_VEMPTY + s));
          if (j + 1 < n_of[t]) {
            if (!k_ready) {
              if (!mbar_wait(bar(B_KFULL + (s ^ 1)), (uint32_t)(((j + 1) >> 1) & 1), abort_flag, p.wait_limit)) { fail = 2; break; }
              tc_fence_after();
              k_ready = true;
            }
            issue_s(t, j + 1);
          }
        }
        if (!fail && more) umma_commit(bar(B_KEMPTY + (s ^ 1)));
      }
    }
  } else if (warp < SM_WARP0) {
    reg_dec<REG_LOW>();
  } else {
    reg_inc<REG_HIGH>();
    // ---- softmax warps: thread = (tile, query row); four warps per tile ------------------------
    const int t = (warp - SM_WARP0) >> 2;          // query tile of the pair
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;          // row inside the query tile
    const int qt = 2 * pr + t;
    const int q_idx = qt * BQ + row;
    const int n_t = t == 0 ? n_a : n_b;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t my_s = tm_s + lane_addr + t * BKV, my_o = tm_o + lane_addr + t * HD;
    const float sl2e = p.scale_log2e;
    float m_used = -INFINITY, l_run = 0.f;

    for (int j = 0; j < n_t; ++j) {
      // the outcome of a wait is made the same for the whole warp: what follows is warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(bar(B_SFULL + t), (uint32_t)(j & 1), abort_flag, p.wait_limit))) { fail = 4; break; }
      tc_fence_after();
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld_32x32(my_s, s0);
      tmem_ld_32x32(my_s + 32, s1);
      tmem_ld_32x32(my_s + 64, s2);
      tmem_ld_32x32(my_s + 96, s3);
      tmem_ld_wait_dep(s0);
      tmem_ld_wait_dep(s1);
      tmem_ld_wait_dep(s2);
      tmem_ld_wait_dep(s3);

      const int key0 = j * BKV;
      if ((p.causal && j >= qt) || (j + 1) * BKV > p.seq) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if ((p.causal && key0 + c > q_idx) || key0 + c >= p.seq) s0[c] = 0xff800000u;  // -inf
          if ((p.causal && key0 + 32 + c > q_idx) || key0 + 32 + c >= p.seq) s1[c] = 0xff800000u;
          if ((p.causal && key0 + 64 + c > q_idx) || key0 + 64 + c >= p.seq) s2[c] = 0xff800000u;
          if ((p.causal && key0 + 96 + c > q_idx) || key0 + 96 + c >= p.seq) s3[c] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        mx0 = max3(mx0, __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
        mx1 = max3(mx1, __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
        mx2 = max3(mx2, __uint_as_float(s2[c]), __uint_as_float(s2[c + 1]));
        mx3 = max3(mx3, __uint_as_float(s3[c]), __uint_as_float(s3[c + 1]));
      }
      const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
      // raise the max used for the exponentials only when the true max has moved far
      float alpha = 1.0f;
      const bool raise = (m_new - m_used) * sl2e > RESCALE_THRESHOLD;
      if (raise) {
        alpha = fast_exp2((m_used - m_new) * sl2e);   // 0 on the first block
        m_used = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // O_t *= alpha (1 for the rows that keep their max), after the last PV UMMA of this tile has landed and
        // before the next is released
        if (!__all_sync(0xffffffffu, mbar_wait(bar(B_ODONE + t), (uint32_t)((j - 1) & 1), abort_flag, p.wait_limit))) { fail = 4; break; }
        tc_fence_after();
#pragma unroll 1
        for (int h = 0; h < HD / 16; ++h) {   // 16 columns at a time: this path must not cost registers
          uint32_t r[16];
          tmem_ld_32x16_sync(my_o + h * 16, r);
#pragma unroll
          for (int c = 0; c < 16; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
          tmem_st_32x16(my_o + h * 16, r);
        }
        tmem_st_wait();
      }
      const f2_t neg2 = f2_pack(-m_used * sl2e, -m_used * sl2e), sl2e2 = f2_pack(sl2e, sl2e);
      f2_t rs2 = f2_pack(0.f, 0.f);
      uint32_t pk[16];
      // P (bf16 pairs) over the first 64 columns of the tile's score buffer; this thread is the only reader of its
      // row of scores, which are all in registers by now
      exp_pack32(s0, sl2e2, neg2, rs2, pk);
      tmem_st_32x16(my_s, pk);
      exp_pack32(s1, sl2e2, neg2, rs2, pk);
      tmem_st_32x16(my_s + 16, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PFULL + t * 2));
      exp_pack32(s2, sl2e2, neg2, rs2, pk);
      tmem_st_32x16(my_s + 32, pk);
      exp_pack32(s3, sl2e2, neg2, rs2, pk);
      tmem_st_32x16(my_s + 48, pk);
      float rs0, rs1;
      f2_unpack(rs2, rs0, rs1);
      l_run = l_run * alpha + (rs0 + rs1);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PFULL + t * 2 + 1));
    }
    if (!fail && n_t > 0) {
      // O / l -> bf16
      if (!__all_sync(0xffffffffu, mbar_wait(bar(B_ODONE + t), (uint32_t)((n_t - 1) & 1), abort_flag, p.wait_limit))) fail = 4;
      if (!fail) {
        tc_fence_after();
        const float inv = 1.0f / l_run;
        __nv_bfloat16 *dst = p.o + ((long long)bh * p.seq + q_idx) * HD;
        if constexpr (PUB) {
          // tcgen05.ld hands every thread one row (256 bytes); the rows go through a swizzled stage in the tile's
          // own Q buffer - every score UMMA of the tile has completed, nothing reads Q any more - so that each
          // store instruction of the warp writes two whole rows instead of 16 bytes to each of 32 rows, which
          // through NVLink reaches a small fraction of the link rate
          uint8_t *stage = gen + OFF_Q + t * TILE_BYTES + q * (32 * HD * 2);
#pragma unroll 1
          for (int h = 0; h < HD / 32; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(my_o + h * 32, r);
            tmem_ld_wait_dep(r);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * u + 0]) * inv, __uint_as_float(r[8 * u + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]) * inv, __uint_as_float(r[8 * u + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]) * inv, __uint_as_float(r[8 * u + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]) * inv, __uint_as_float(r[8 * u + 7]) * inv);
              const int unit = h * 4 + u;   // 16-byte unit within the 256-byte row
              *reinterpret_cast<uint4 *>(stage + lane * (HD * 2) + ((unit ^ (lane & 7)) << 4)) = v;
            }
          }
          __syncwarp();
          const int unit = lane & 15;
          const long long row0 = (long long)bh * p.seq + qt * BQ + q * 32;
#pragma unroll 2
          for (int i = 0; i < 16; ++i) {
            const int rl = 2 * i + (lane >> 4);
            const uint4 v = *reinterpret_cast<const uint4 *>(stage + rl * (HD * 2) + ((unit ^ (rl & 7)) << 4));
            if (qt * BQ + q * 32 + rl < p.seq) {
              const long long off = (row0 + rl) * HD + unit * 8;
              if (p.pub == 1) {
                st_multimem_16(p.o + off, v);
              } else {
                for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4 *>(p.peer_o[d] + off) = v;
              }
            }
          }
        } else {
#pragma unroll 1
          for (int h = 0; h < HD / 32; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(my_o + h * 32, r);
            tmem_ld_wait_dep(r);
            if (q_idx < p.seq) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * u + 0]) * inv, __uint_as_float(r[8 * u + 1]) * inv);
                v.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]) * inv, __uint_as_float(r[8 * u + 3]) * inv);
                v.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]) * inv, __uint_as_float(r[8 * u + 5]) * inv);
                v.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]) * inv, __uint_as_float(r[8 * u + 7]) * inv);
                *reinterpret_cast<uint4 *>(dst + h * 32 + 8 * u) = v;
              }
            }
          }
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

static int attention_impl(ttlb_ctx *ctx, const ttlb_attn_desc *d, int pub, void *const *peers, int n_peers, void *stream);

extern "C" int ttlb_attention(ttlb_ctx *ctx, const ttlb_attn_desc *d, void *stream) {
  return attention_impl(ctx, d, 0, nullptr, 0, stream);
}

extern "C" int ttlb_attention_multicast(ttlb_ctx *ctx, const ttlb_attn_desc *d, void *stream) {
  return attention_impl(ctx, d, 1, nullptr, 0, stream);
}

extern "C" int ttlb_attention_peers(ttlb_ctx *ctx, const ttlb_attn_desc *d, void *const *peers, int n_peers, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!peers || n_peers < 1 || n_peers > MAX_PEERS)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: 1 to %d peer outputs", MAX_PEERS);
  for (int i = 0; i < n_peers; ++i)
    if (!peers[i] || ((uintptr_t)peers[i] % 16))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: peer output %d is null or not 16-byte aligned", i);
  return attention_impl(ctx, d, 2, peers, n_peers, stream);
}

static int attention_impl(ttlb_ctx *ctx, const ttlb_attn_desc *d, int pub, void *const *peers, int n_peers, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: null descriptor");
  if (d->batch_heads == 0 || d->seq == 0) return TTLB_OK;
  if (!d->q || !d->k || !d->v || (!d->o && pub != 2)) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "attention: null tensor");
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
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM));
    ctx->attn_attr_set = true;
  }
  AttnParams p;
  p.o = reinterpret_cast<__nv_bfloat16 *>(pub == 2 ? peers[0] : d->o);
  p.pub = pub;
  p.n_peers = pub == 2 ? n_peers : 0;
  for (int i = 0; i < p.n_peers; ++i) p.peer_o[i] = reinterpret_cast<__nv_bfloat16 *>(peers[i]);
  p.seq = (int)d->seq;
  p.bh = (int)d->batch_heads;
  p.q_tiles = (int)((d->seq + BQ - 1) / BQ);
  p.q_pairs = (p.q_tiles + NT - 1) / NT;
  p.causal = d->causal ? 1 : 0;
  p.scale_log2e = d->scale * 1.4426950408889634f;
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  const long long grid = (long long)p.q_pairs * p.bh;
  if (grid > 0x7fffffffLL) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "attention: too many tiles");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pub)
    ttlb_attention_kernel<true><<<(unsigned)grid, ATT_THREADS, ATT_SMEM, st>>>(mq, mk, mv, p);
  else
    ttlb_attention_kernel<false><<<(unsigned)grid, ATT_THREADS, ATT_SMEM, st>>>(mq, mk, mv, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}
