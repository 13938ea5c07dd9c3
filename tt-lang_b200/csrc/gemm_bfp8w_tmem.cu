// bfloat8_b-weight GEMM with the block-float unpack inside the mainloop and the expanded weights handed to
// the tensor core THROUGH TENSOR MEMORY: nothing that was expanded ever touches shared memory, no bf16 copy of the
// weights exists in HBM, and the call needs no scratch memory.
//
// The product is computed transposed, C^T = W^T X^T: a cluster of two CTAs owns a 256 (weight columns n) x 256
// (activation rows m) tile of C^T, each CTA 128 of the weight columns.  tcgen05.mma reads its A operand - W^T,
// row = weight column n, 16 k per instruction - from tensor memory and its B operand - X^T, i.e. X as it lies in
// memory, k contiguous - from shared memory, where a TMA load puts it (each CTA loads half of the 256 rows; no load
// is multicast).  Per 64-deep k-block and CTA:
//
//   * warp 0 brings 128 rows of X (16 KB); warp 2 brings this CTA's packed weight tiles with two tiled TMA
//     loads: the value bytes of 2 x 4 tiles (a four-dimensional view of the packed matrix, loaded with the 128-byte
//     swizzle so that the converters' 32-bit loads hit 32 different banks) and their block exponents.  (One thread
//     issuing all five loads of the first version needed 640 cycles per k-block and was the limit.)
//   * warps 12..19, two groups of four that take the k-blocks in turn (a warp serves the 32 tensor-memory lanes of
//     its quarter = one tile column), expand bytes to bf16 PAIRS ALONG k - a block's 16 values lie along n and share
//     an exponent, so a pair (k, k+1) of one column has two exponents: one byte permute takes the column's two
//     bytes out of the two rows' words, one mask leaves sign and magnitude where a bf16 has sign and mantissa -
//     with a zero exponent field that IS (-1)^s m 2^-133, a denormal - and two multiplications by pairs of powers
//     of two (2^(E/2) and 2^(E - E/2): 2^E itself is a bf16 only up to E = 127) make (-1)^s m 2^(E-133) exactly,
//     for every exponent - and write them with tcgen05.st (16 lanes x 256 bits: a thread's registers are two lanes'
//     k-pairs), then arrive on the leader CTA's barrier, on which the X bytes are counted too.  The scale pairs are
//     made once per four lanes and passed round by shuffle;
//   * the leader's warp 1 waits on that one barrier and issues four tcgen05.mma.cta_group::2 (256 x 256 x 16),
//     A from tensor memory.
//
// Tensor memory: the accumulator (256 columns) and eight 32-column A slots.  There is room for one accumulator only,
// so no UMMA runs while a tile's accumulator is being read.  To keep that short, the epilogue warps (4..11, two per
// lane quarter) take registers from the other warpgroups (setmaxnreg: 40 for warps 0..3, 72 for the converters, 144
// for them), read their whole 128-column slice with four tcgen05.ld, release the accumulator, and only then convert to
// bf16, transpose 32 x 32 blocks through shared memory and store 16-byte vectors along the rows of C: 1.36 -> 1.31 ms.
// The loads and the expansion of the next tile's first eight k-blocks run under the epilogue too.  A tensor-memory
// lane holds weight column 4 * (lane % 8) + lane / 8 of its tile column: that is the order in which a thread's
// 32-bit load of four neighbouring columns meets the store's lanes (t/4, t/4 + 8, and the same + 16).
// Shared memory per CTA: 8 stages x (16 KB X + 8 KB value bytes + 512 B exponents) + 20 KB for the epilogue.
// Every wait is bounded.
//
// Measured on 4096 x 8192 x 28672: 1.31 ms (1,471 TFLOP/s) against 1.37 ms for the unpack kernel + bf16 GEMM and
// 1.62-1.69 ms for the earlier in-mainloop kernel, which wrote the expanded weights to shared memory (removed).  In
// cycles the mainloop is at the tensor pipe's rate (506-520 per k-block for 512); what decides the rest is the clock:
// every weight is expanded once per 256 activation rows, 16 times in all, and under the power cap that work lowers the
// clock the tensor pipe runs at - which is why the expansion was cut to two integer-pipe instructions per pair of
// values and is done by eight warps, not sixteen.
#include <cuda_bf16.h>

#include "ctx.h"
#include "sm100.cuh"

using namespace sm100;


namespace {

constexpr int TBN = 256;                    // weight columns per cluster tile (rows of C^T), 128 per CTA
constexpr int TBM = 256;                    // activation rows per tile (columns of C^T): the UMMA's N
constexpr int TBK = 64, TSTAGES = 8;
constexpr int X_BYTES = 128 * TBK * 2;      // 16 KB: this CTA's half of the X rows
constexpr int MANT_BYTES = 2 * 4 * 1024;    // two tile rows x four tile columns of value bytes
constexpr int EXP_BYTES = 2 * 4 * 64;
constexpr int PACKED_TILE = 1088;
constexpr int EPI_WARPS = 8;                 // two per tensor-memory lane quarter, 128 accumulator columns each
constexpr int EPI_WARP0 = 4;                 // warps 0..3: X producer, UMMA issuer, packed-weights producer, one idle
constexpr int CONV_WARP0 = EPI_WARP0 + EPI_WARPS;
constexpr int G = 2;                         // converter groups (four warps each) that take the k-blocks in turn;
                                             // measured on 4096x8192x28672: 1 group 1.54 ms, 2 groups 1.36 ms, 3 groups 1.41-1.45 ms,
                                             // 4 groups 1.45 ms (more warps cost clock under the power cap)
constexpr int TTHREADS = (CONV_WARP0 + 4 * G) * 32;
// Registers move between the warpgroups (setmaxnreg): the epilogue warps hold a whole 128-column slice of the
// accumulator, so that the accumulator is free for the next tile after four loads instead of after the stores.  The
// three figures must fit the pool the CTA is launched with (threads x REG_LAUNCH), or the raise would wait for ever.
constexpr int REG_LAUNCH = 96, REG_LOW = 40, REG_EPI = 144, REG_CONV = 72;
static_assert(TTHREADS == 640 && 65536 / TTHREADS / 8 * 8 == REG_LAUNCH, "launch register count");
static_assert(128 * REG_LOW + EPI_WARPS * 32 * REG_EPI + 4 * G * 32 * REG_CONV <= TTHREADS * REG_LAUNCH, "register pool of the CTA exceeded");
constexpr int T_GROUP_M = 8;
constexpr int A_COLS = TBK / 2;             // 32 tensor-memory columns per k-block (two bf16 per column)
constexpr int EPI_PITCH = 256 + 16;          // publishing epilogue: bytes per row of a transposition tile of 32 activation rows x
                                             // 128 weight columns, one tile per half of the accumulator's columns (four warps each)
constexpr int EPI_PITCH1 = 64 + 16;          // plain epilogue: a warp's own tile of 32 activation rows x 32 weight columns
constexpr int EPI_BYTES = EPI_WARPS * 32 * EPI_PITCH1 > 2 * 32 * EPI_PITCH ? EPI_WARPS * 32 * EPI_PITCH1 : 2 * 32 * EPI_PITCH;
constexpr int MAX_PEERS = 8;
constexpr int TSMEM_BYTES = TSTAGES * (X_BYTES + MANT_BYTES + EXP_BYTES) + EPI_BYTES + 1024 + 512;
static_assert(TBM + TSTAGES * A_COLS <= 512, "tensor memory: accumulator + A slots");

struct TmemParams {
  long long tile_cols_total;
  int tile_col0;             // first tile column of the weight slice
  int tile_rows, tile_cols;  // k / 32, n / 32
  __nv_bfloat16 *c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n;
  int *status;
  long long wait_limit;
  // 0: c is this GPU's output.  1: c is a multicast address (multimem.st: the switch replicates every store to all GPUs
  // of the group).  2: every row segment is stored to peer_c[0 .. n_peers), the output in every GPU's copy of a shared
  // buffer (peer-mapped memory, this GPU's own copy included).  Peer memory is only ever written.
  int pub;
  __nv_bfloat16 *peer_c[MAX_PEERS];
  int n_peers;
};

template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// barrier among the `threads` threads that name barrier `id` (1..15; 0 is __syncthreads')
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void ttile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int per_group = T_GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * T_GROUP_M;
  const int rows = min(T_GROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc] on a pair of CTAs
__device__ __forceinline__ void umma_f16_ts_2sm(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// 16 lanes x 16 columns: thread t gives lane t/4 (registers 0, 1, 4, 5) and lane t/4 + 8 (2, 3, 6, 7) their columns
// 2*(t%4), 2*(t%4)+1 (registers 0..3) and the same + 8 (registers 4..7)
__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// product of two bf16 pairs, denormal operands and results included
__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
  const __nv_bfloat162 d = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
  return *reinterpret_cast<const uint32_t *>(&d);
}

// Block exponents (Ea, Eb) of a row pair -> two bf16 pairs of powers of two whose product is (2^Ea, 2^Eb): 2^E itself is
// a bf16 only up to E = 127, 2^(E/2) and 2^(E - E/2) always are (E <= 254: 255 is not a finite value's exponent).
__device__ __forceinline__ void scale_pairs(uint32_t e4, uint32_t sel, uint32_t &s1, uint32_t &s2) {
  const uint32_t u = __byte_perm(e4, 0u, sel);             // Ea in the low half, Eb in the high half
  const uint32_t h = (u >> 1) & 0x007f007fu;
  s1 = (h + 0x007f007fu) << 7;
  s2 = (u - h + 0x007f007fu) << 7;
}

// PUB: the instantiation whose epilogue publishes the output to several GPUs
template <bool PUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TTHREADS, 1)
ttlb_gemm_bfp8w_tmem_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_mant,
                            const __grid_constant__ CUtensorMap map_exp, const TmemParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_ring = base, m_ring = base + TSTAGES * X_BYTES, e_ring = m_ring + TSTAGES * MANT_BYTES;
  const uint32_t bars = e_ring + TSTAGES * EXP_BYTES + EPI_BYTES;
  uint8_t *gen_epi = gbase + TSTAGES * (X_BYTES + MANT_BYTES + EXP_BYTES);
  uint8_t *gen_bars = gen_epi + EPI_BYTES;
  auto pfull_bar = [&](int s) { return bars + 8u * (TSTAGES + s); };       // local: packed bytes
  // leader: both operands of a k-block - X bytes of both CTAs (+ the arrival that announces them) and 4 converter
  // warps of each CTA
  auto afull_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (3 * TSTAGES + s); };   // local: UMMAs done with the stage
  const uint32_t tfull_bar = bars + 8u * (4 * TSTAGES), tempty_bar = bars + 8u * (4 * TSTAGES + 1);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen_bars + 8 * (4 * TSTAGES + 2));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_bars + 8 * (4 * TSTAGES + 2) + 8);
  volatile uint8_t *epi_ok = reinterpret_cast<volatile uint8_t *>(gen_bars + 8 * (4 * TSTAGES + 2) + 16);   // [2 halves][4 warps]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < TSTAGES; ++s) {
      mbar_init(pfull_bar(s), 1);
      mbar_init(afull_bar(s), 9);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 2 * EPI_WARPS);
    fence_barrier_init();
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_mant);
    prefetch_tensormap(&map_exp);
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
  const uint32_t tmem_a = tmem_base + TBM;

  int fail = 0;
  // every role branch starts with its own register move: after a join the lower limit would apply to all
  if (warp == 0 || warp == 2) {
    reg_dec<REG_LOW>();
    // ---- producers, one thread each: warp 0 brings X by TMA (signals the leader), the last warp the packed weights
    // (two tiled loads per k-block: value bytes and exponents of 2 x 4 tiles; signals locally).  Tiles outside the
    // packed matrix arrive as zeros, which expand to zeros; tiles outside the column window are other columns'
    // weights, whose products are never stored.
    const bool packed = warp == 2;
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters) {
        int tm, tn;
        ttile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int tc0 = p.tile_col0 + tn * (TBN / 32) + (int)rank * 4;   // first tile column of this CTA's half
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit)) { fail = 1; break; }
          if (!packed) {
            if (rank == 0) mbar_expect_tx(afull_bar(stage), 2 * X_BYTES);
            tma_load_2d_2sm(x_ring + stage * X_BYTES, &map_x, kb * TBK, tm * TBM + (int)rank * 128,
                            afull_bar(stage) & 0xFEFFFFFFu);
          } else {
            mbar_expect_tx(pfull_bar(stage), MANT_BYTES + EXP_BYTES);
            tma_load_4d(m_ring + stage * MANT_BYTES, &map_mant, 0, 0, tc0, kb * 2, pfull_bar(stage));
            tma_load_3d(e_ring + stage * EXP_BYTES, &map_exp, 0, tc0, kb * 2, pfull_bar(stage));
          }
          if (++stage == TSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    reg_dec<REG_LOW>();
    // ---- UMMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(TBN, TBM, false, false);   // M = weight columns, N = activation rows
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
        if (!mbar_wait(tempty_bar, (uint32_t)((local & 1) ^ 1), abort_flag, p.wait_limit)) { fail = 2; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(afull_bar(stage), phase, abort_flag, p.wait_limit)) { fail = 2; break; }
          tc_fence_after();
          const uint64_t db = desc_kmajor_sw128(x_ring + stage * X_BYTES);
          const uint32_t ta = tmem_a + stage * A_COLS;
#pragma unroll
          for (int k = 0; k < TBK / 16; ++k)
            umma_f16_ts_2sm(tmem_base, ta + k * 8, db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          umma_commit_2sm(empty_bar(stage));
          if (++stage == TSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (fail) break;
        umma_commit_2sm(tfull_bar);
      }
    }
  } else if (warp < EPI_WARP0) {
    reg_dec<REG_LOW>();
  } else if (warp < CONV_WARP0) {
    reg_inc<REG_EPI>();
    // ---- epilogue: this CTA's 128 weight columns (tensor-memory lanes) x 256 activation rows (columns); a warp takes
    // 128 of the columns of its lane quarter
    const int q = warp & 3, half = (warp - EPI_WARP0) >> 2;
    // This lane holds weight column 4 * (lane % 8) + lane / 8 of its warp's 32.  A block of 32 activation rows is
    // turned round in shared memory (row = activation row) so that global stores are 16-byte vectors along the rows of
    // C; the next block's tcgen05.ld is in flight meanwhile.  Plain epilogue: every warp for itself, 32 weight columns
    // (64-byte row segments).  Publishing epilogue: the four warps that share a half of the accumulator's columns work
    // on one tile of 128 weight columns and store two whole 256-byte row segments per instruction, which is what
    // NVLink needs (at home it measured 1 % slower than the plain one).  The four warps wait for the same barrier
    // with the same limit, so they reach the named barriers together or not at all.
    uint8_t *st = PUB ? gen_epi + half * (32 * EPI_PITCH) : gen_epi + (warp - EPI_WARP0) * (32 * EPI_PITCH1);
    const int my_n = (PUB ? q * 32 : 0) + 4 * (lane & 7) + (lane >> 3);
    const int wq = (warp - EPI_WARP0) & 3;                // publishing: this warp stores rows 8 * wq .. 8 * wq + 7 of a block
    const uint32_t my_acc = tmem_base + ((uint32_t)(q * 32) << 16) + half * 128;
    int local = 0;
    for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters, ++local) {
      int tm, tn;
      ttile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      // the outcome of the wait is made the same for the whole warp: what follows is warp-collective
      bool ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar, (uint32_t)(local & 1), abort_flag, p.wait_limit));
      if constexpr (PUB) {
        // the four warps of a half meet at named barriers below: they must all go on or all give up (a warp whose wait
        // ran out a moment before the barrier completed would otherwise leave the other three waiting for ever)
        if (lane == 0) epi_ok[half * 4 + wq] = ok ? 1 : 0;
        named_barrier(1 + half, 128);
        ok = epi_ok[half * 4] & epi_ok[half * 4 + 1] & epi_ok[half * 4 + 2] & epi_ok[half * 4 + 3];
      }
      if (!ok) { fail = 3; break; }
      tc_fence_after();
      const int colb = tn * TBN + (int)rank * 128 + (PUB ? 8 * (lane & 15) : q * 32 + 8 * (lane & 3));
      auto emit = [&](const uint32_t (&r)[32], int c) {
        constexpr int PITCH = PUB ? EPI_PITCH : EPI_PITCH1;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          *reinterpret_cast<__nv_bfloat16 *>(st + i * PITCH + my_n * 2) = __float2bfloat16_rn(__uint_as_float(r[i]));
        if constexpr (PUB) named_barrier(1 + half, 128); else __syncwarp();
        const int row0 = tm * TBM + half * 128 + c * 32;
        if (colb < p.n) {   // n is a multiple of 32: a group of 8 columns is all in or all out
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            // publishing: 16 lanes per row, this warp's 8 rows; plain: 4 lanes per row, all 32 rows
            const int rl = PUB ? 8 * wq + 2 * g + (lane >> 4) : 8 * g + (lane >> 2);
            const int row = row0 + rl;
            const uint4 v = *reinterpret_cast<const uint4 *>(st + rl * PITCH + 16 * (PUB ? (lane & 15) : (lane & 3)));
            if (row < p.m) {
              const long long off = (long long)row * p.ldc + colb;
              if constexpr (!PUB) {
                *reinterpret_cast<uint4 *>(p.c + off) = v;
              } else if (p.pub == 1) {
                st_multimem_16(p.c + off, v);
              } else {
                for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4 *>(p.peer_c[d] + off) = v;
              }
            }
          }
        }
        if constexpr (PUB) named_barrier(1 + half, 128); else __syncwarp();
      };
      // the whole slice into registers, then the accumulator is free: the next tile's UMMAs run under the stores
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld_32x32(my_acc, r0);
      tmem_ld_32x32(my_acc + 32, r1);
      tmem_ld_32x32(my_acc + 64, r2);
      tmem_ld_32x32(my_acc + 96, r3);
      tmem_ld_wait_dep(r0);
      tmem_ld_wait_dep(r1);
      tmem_ld_wait_dep(r2);
      tmem_ld_wait_dep(r3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(tempty_bar, 0);
      emit(r0, 0);
      emit(r1, 1);
      emit(r2, 2);
      emit(r3, 3);
    }
  } else {
    reg_dec<REG_CONV>();
    // ---- converters: packed value bytes -> bf16 pairs along k -> tensor memory.  G groups take the k-blocks in
    // turn, so the latency of one k-block's chain (wait, read, expand, store, remote arrive) is spread over G.
    const int cw = warp - CONV_WARP0;            // 0 .. 4G-1
    const int group = cw >> 2, q = warp & 3;     // q: tensor-memory lane quarter = tile column of this CTA's four
    const int t4 = lane & 3, j = lane >> 2;      // this thread: k rows 4*t4 .. 4*t4+3 of a 16-row face, columns 4j .. 4j+3
    const int face_lo = j >> 2;                  // 0: columns 0..15 of the tile, 1: columns 16..31
    const uint32_t cbyte = (uint32_t)((j & 3) * 4);
    long long it = 0;                            // k-blocks seen so far (all tiles)
    for (int t = cluster_id; t < num_tiles && !fail; t += n_clusters) {
      int tm, tn;
      ttile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((int)(it % G) != group) continue;
        const int stage = (int)(it % TSTAGES);
        const uint32_t phase = (uint32_t)((it / TSTAGES) & 1);
        if (!__all_sync(0xffffffffu, mbar_wait(pfull_bar(stage), phase, abort_flag, p.wait_limit))) { fail = 4; break; }
        const uint8_t *ms = gbase + TSTAGES * X_BYTES + stage * MANT_BYTES;
        const uint8_t *es = gbase + TSTAGES * (X_BYTES + MANT_BYTES) + stage * EXP_BYTES;
        // Scale pairs.  The four lanes that share this thread's rows and face column (lanes j & 3 = 0..3 of the
        // group) need the same eight - (tile row, face row) u = 0..3 x row pairs (0,1), (2,3): each lane makes two
        // of them, u = (j & 3) >> 1 and that + 2, row pair (j & 3) & 1, and they go round by shuffle.
        const int sr = j & 3;
        const uint32_t e_lo = *reinterpret_cast<const uint32_t *>(es + q * 64 + (2 * (sr >> 1) + face_lo) * 16 + 4 * t4);
        const uint32_t e_hi = *reinterpret_cast<const uint32_t *>(es + (4 + q) * 64 + (2 * (sr >> 1) + face_lo) * 16 + 4 * t4);
        const uint32_t psel = (sr & 1) ? 0x4342u : 0x4140u;
        uint32_t my1_lo, my2_lo, my1_hi, my2_hi;
        scale_pairs(e_lo, psel, my1_lo, my2_lo);
        scale_pairs(e_hi, psel, my1_hi, my2_hi);
        const int grp = lane & ~12;                  // lane of the group with j & 3 = 0 (lane = 4 * j + t4)
        uint32_t sc1[4][2], sc2[4][2];               // [u][row pair]
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            const int src = grp + 4 * (2 * (u & 1) + pr);
            sc1[u][pr] = __shfl_sync(0xffffffffu, u < 2 ? my1_lo : my1_hi, src);
            sc2[u][pr] = __shfl_sync(0xffffffffu, u < 2 ? my2_lo : my2_hi, src);
          }
        }
#pragma unroll
        for (int trow = 0; trow < 2; ++trow) {
          uint32_t o[2][8];   // [lane half of the store][register]
          const uint8_t *tile = ms + (trow * 4 + q) * 1024;
#pragma unroll
          for (int kf = 0; kf < 2; ++kf) {     // rows 0..15 / 16..31 of the tile row
            const int f = 2 * kf + face_lo;
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = 4 * t4 + i;                       // row of the face
              const int row128 = 2 * f + (r >> 3);            // 128-byte row of the tile's value bytes
              const int chunk = (r & 7) ^ row128;             // the TMA load's swizzle: 16-byte chunk ^ (row % 8)
              w[i] = *reinterpret_cast<const uint32_t *>(tile + row128 * 128 + chunk * 16 + cbyte);
            }
            // A byte is sign | magnitude m and means (-1)^s m 2^(E-133); placed as sign and mantissa of a bf16 with a
            // zero exponent field it IS (-1)^s m 2^-133 (a denormal): two multiplications by powers of two, both
            // exact, finish the job.  The byte permute doubles the column's byte of row r into the low half and
            // that of row r+1 into the high half.
            const int u = trow * 2 + kf;
#pragma unroll
            for (int a = 0; a < 4; ++a) {   // column 4j + a: lane j (+8 for a odd) of lane half a/2
              const uint32_t sel = 0x4400u + 0x1111u * a;
              const uint32_t x01 = __byte_perm(w[0], w[1], sel) & 0x807f807fu, x23 = __byte_perm(w[2], w[3], sel) & 0x807f807fu;
              o[a >> 1][kf * 4 + (a & 1) * 2 + 0] = hmul2_bf16(hmul2_bf16(x01, sc1[u][0]), sc2[u][0]);
              o[a >> 1][kf * 4 + (a & 1) * 2 + 1] = hmul2_bf16(hmul2_bf16(x23, sc1[u][1]), sc2[u][1]);
            }
          }
          const uint32_t ta = tmem_a + stage * A_COLS + trow * 16 + ((uint32_t)(q * 32) << 16);
          tmem_st_16x256b_x2(ta, o[0]);
          tmem_st_16x256b_x2(ta + (16u << 16), o[1]);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(afull_bar(stage), 0);
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

int make_map_u8(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint32_t rank, const cuuint64_t *dims,
                const cuuint64_t *strides, const cuuint32_t *box, CUtensorMapSwizzle swizzle) {
  ttlb_encode_tiled_fn enc = ttlb_get_encode_tiled();
  if (!enc) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ttlb_fail(ctx, TTLB_ERR_CUDA, "cuTensorMapEncodeTiled (packed weights) failed: %d", (int)r);
  return TTLB_OK;
}

}  // namespace

int ttlb_make_map_bf16_2d(ttlb_ctx *ctx, CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer,
                          uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// Arguments are validated by the caller (matmul_bfp8w_impl in bfp8.cu).  publish: d->c is a multicast address, or - when
// the context holds peer pointers (ttlb_matmul_bfp8w_peers) - the output is stored to each of them.
int ttlb_launch_gemm_bfp8w_tmem(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *d, bool publish, cudaStream_t stream) {
  CUtensorMap map_x, map_mant, map_exp;
  int rc = ttlb_make_map_bf16_2d(ctx, &map_x, d->a, (uint64_t)d->k, (uint64_t)d->m, (uint64_t)d->lda * 2, TBK, 128);
  if (rc) return rc;
  const uint8_t *tiles = reinterpret_cast<const uint8_t *>(d->b_tiles);
  {
    // value bytes: [tile row][tile column][8 rows of 128 bytes]; tiles 1088 bytes apart, first byte 64 past the tile's start
    const cuuint64_t dims[4] = {128, 8, (cuuint64_t)d->b_tile_cols, (cuuint64_t)(d->k / 32)};
    const cuuint64_t strides[3] = {128, PACKED_TILE, (cuuint64_t)d->b_tile_cols * PACKED_TILE};
    const cuuint32_t box[4] = {128, 8, 4, 2};
    rc = make_map_u8(ctx, &map_mant, tiles + 64, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[3] = {64, (cuuint64_t)d->b_tile_cols, (cuuint64_t)(d->k / 32)};
    const cuuint64_t strides[2] = {PACKED_TILE, (cuuint64_t)d->b_tile_cols * PACKED_TILE};
    const cuuint32_t box[3] = {64, 4, 2};
    rc = make_map_u8(ctx, &map_exp, tiles, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  TmemParams p;
  p.tile_cols_total = d->b_tile_cols;
  p.tile_col0 = (int)d->b_tile_col0;
  p.tile_rows = (int)(d->k / 32);
  p.tile_cols = (int)(d->n / 32);
  p.c = reinterpret_cast<__nv_bfloat16 *>(d->c);
  p.ldc = d->ldc;
  p.m = (int)d->m;
  p.n = (int)d->n;
  p.k = (int)d->k;
  p.tiles_m = (int)((d->m + TBM - 1) / TBM);
  p.tiles_n = (int)((d->n + TBN - 1) / TBN);
  p.status = ctx->d_status;
  p.wait_limit = ctx->wait_limit_cycles;
  p.pub = publish ? 1 : 0;
  p.n_peers = 0;
  for (int i = 0; i < MAX_PEERS; ++i) p.peer_c[i] = nullptr;
  if (publish && ctx->pub_n_peers > 0) {
    p.pub = 2;
    p.n_peers = ctx->pub_n_peers;
    for (int i = 0; i < ctx->pub_n_peers; ++i) p.peer_c[i] = reinterpret_cast<__nv_bfloat16 *>(ctx->pub_peers[i]);
  }
  const int tiles_out = p.tiles_m * p.tiles_n;
  int clusters = ctx->sm_count / 2;
  if (clusters > tiles_out) clusters = tiles_out;
  if (!ctx->gemm_tmem_attr_set) {
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bfp8w_tmem_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              TSMEM_BYTES));
    TTLB_CUDA_CHECK(ctx, cudaFuncSetAttribute(ttlb_gemm_bfp8w_tmem_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              TSMEM_BYTES));
    ctx->gemm_tmem_attr_set = true;
  }
  if (p.pub)
    ttlb_gemm_bfp8w_tmem_kernel<true><<<clusters * 2, TTHREADS, TSMEM_BYTES, stream>>>(map_x, map_mant, map_exp, p);
  else
    ttlb_gemm_bfp8w_tmem_kernel<false><<<clusters * 2, TTHREADS, TSMEM_BYTES, stream>>>(map_x, map_mant, map_exp, p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return TTLB_OK;
}

