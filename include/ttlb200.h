/*
 * ttlb200 — C ABI of the B200 (sm_100a) execution backend for tt-lang tile programs.
 *
 * Style follows the reference's own C API (include/ttlang-c/Dialects.h:17-28,
 * include/ttlang-c/TTLAttrs.h:19-34): extern "C", plain value types, no exceptions
 * across the boundary.  Every entry point returns 0 (TTLB_OK) or a negative
 * TTLB_ERR_* code; a human-readable reason is kept per context and read with
 * ttlb_last_error().
 *
 * What this library replaces: the device-dispatch boundary of the reference,
 * run_kernel_on_device(kernel_specs, tensors, cb_configs, core_ranges)
 * (python/ttl/kernel_runner.py:188-255), which hands a compiled tile program to
 * ttnn.generic_op.  Here a recognised tile program is handed, as a plain
 * descriptor, to a hand-written CUDA kernel.
 *
 * Conventions
 *  - Tensors are row-major 2-D arrays; "32x32 tiles" are an indexing convention
 *    (tile (r,c) = elements [32r:32r+32, 32c:32c+32], python/sim/tensoraccessor.py:125-159),
 *    except bfloat8_b weights which are physically tiled (1088-byte tiles).
 *  - Device pointers are borrowed: the caller keeps them alive until the stream
 *    has synchronised.  Outputs are written in place.  Nothing user-visible is
 *    allocated inside the library.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *  - A context is bound to one device and used by one thread at a time
 *    (the reference is single-threaded too: python/ttl/ttl_api.py:71).
 */
#ifndef TTLB200_H
#define TTLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TTLB_EXPORT __declspec(dllexport)
#else
#define TTLB_EXPORT __attribute__((visibility("default")))
#endif

/* ---- status codes ------------------------------------------------------- */
#define TTLB_OK 0
#define TTLB_ERR_INVALID_ARG (-1)
#define TTLB_ERR_UNSUPPORTED (-2)
#define TTLB_ERR_CUDA (-3)
#define TTLB_ERR_TIMEOUT (-4) /* a bounded device-side wait ran out */
#define TTLB_ERR_NCCL (-5)

/* ---- element types (python/ttl/dtype_utils.py:151-181 gives the tile byte sizes) */
#define TTLB_BF16 0   /* 2048-byte tiles */
#define TTLB_F32 1    /* 4096-byte tiles */
#define TTLB_BFP8_B 2 /* 1088-byte tiles: 64 shared exponents + 1024 sign/mantissa bytes */

#define TTLB_BFP4_B 3 /* 576-byte tiles: 64 shared exponents + 512 bytes of sign/3-bit-mantissa nibbles */

#define TTLB_TILE 32
#define TTLB_BFP8_TILE_BYTES 1088
#define TTLB_BFP4_TILE_BYTES 576

typedef struct ttlb_ctx ttlb_ctx;

/* Library version string, static storage. */
TTLB_EXPORT const char *ttlb_version(void);

/* Create / destroy a context bound to CUDA device `device_ordinal`.
 * Replaces ttnn.open_device / close_device in user code
 * (python/sim/ttnnsim.py:218-226).  ttlb_init fails with TTLB_ERR_CUDA when no
 * usable sm_100 device is present: there is no CPU fallback.
 * A context is used by one host thread and ONE STREAM at a time: the bf16 expansion of block-float weights, the
 * partial rows and arrival counters of reductions over rows and the status word are scratch memory owned by the
 * context and shared by all its launches without ordering between streams.  Callers that want concurrent streams on
 * one GPU create one context per stream. */
TTLB_EXPORT int ttlb_init(int device_ordinal, ttlb_ctx **out);
TTLB_EXPORT void ttlb_destroy(ttlb_ctx *ctx);

/* Context-owned message of the last failing call (valid until the next call). */
TTLB_EXPORT const char *ttlb_last_error(ttlb_ctx *ctx);

/* Number of kernels this context has launched since creation. */
TTLB_EXPORT int64_t ttlb_launch_count(ttlb_ctx *ctx);

/* ------------------------------------------------------------------------ *
 * Fused element-wise / broadcast tile programs.
 *
 * Replaces the fused compute kernel the reference generates for a chain of
 * element-wise ops (lib/Dialect/TTL/Transforms/ConvertTTLToCompute.cpp:113-229;
 * op table include/ttlang/Dialect/TTL/TTLElementwiseOps.def:61-82) together
 * with its reader/writer data-movement kernels, and the simulator's per-tile
 * torch ops (python/sim/block.py:870-1010, python/sim/ttnnsim.py:67-109).
 *
 * The expression is an accumulator program: LOAD sets the accumulator from an
 * input, a binary op combines the accumulator with an input (arg >= 0) or with
 * the value popped from a two-deep stack (arg == TTLB_ARG_STACK), PUSH saves the
 * accumulator.  The final accumulator is the output element.
 * ------------------------------------------------------------------------ */
#define TTLB_MAX_IN 6
#define TTLB_MAX_OPS 32
#define TTLB_ARG_STACK (-1)

enum ttlb_opcode {
  TTLB_OP_LOAD = 0, /* acc = in[arg] */
  TTLB_OP_ADD = 1,  /* acc = acc + x */
  TTLB_OP_SUB = 2,  /* acc = acc - x */
  TTLB_OP_RSUB = 3, /* acc = x - acc */
  TTLB_OP_MUL = 4,
  TTLB_OP_DIV = 5,  /* acc = acc / x */
  TTLB_OP_RDIV = 6, /* acc = x / acc */
  TTLB_OP_MAX = 7,
  TTLB_OP_MIN = 8,
  /* The remaining block operators of the simulator (python/sim/block.py:975-1010, torch semantics of
   * python/sim/ttnnsim.py:424-450); executed by the specialised kernel only. */
  TTLB_OP_FLOORDIV = 9,   /* floor(acc / x) as torch.floor_divide computes it */
  TTLB_OP_RFLOORDIV = 10, /* floor(x / acc) */
  TTLB_OP_MOD = 11,       /* remainder with the sign of the divisor (torch.remainder) */
  TTLB_OP_RMOD = 12,
  TTLB_OP_POW = 13,       /* acc ** x */
  TTLB_OP_RPOW = 14,      /* x ** acc */
  TTLB_OP_EXP = 16,
  TTLB_OP_LOG = 17,
  TTLB_OP_SQRT = 18,
  TTLB_OP_RSQRT = 19,
  TTLB_OP_TANH = 20,
  TTLB_OP_SIGMOID = 21,
  TTLB_OP_NEG = 22,
  TTLB_OP_ABS = 23,
  TTLB_OP_RELU = 24,
  TTLB_OP_PUSH = 32, /* push acc on the stack */
  /* Unary math functions of the specification's Appendix B
   * (docs/sphinx/specs/TTLangSpecification.md:700-748) beyond the compiler's op table; executed by the
   * specialised kernel only.  `arg` is unused. */
  TTLB_OP_EXP2 = 40,
  TTLB_OP_EXPM1 = 41,
  TTLB_OP_LOGP1 = 42, /* log(1 + x) */
  TTLB_OP_SQUARE = 43,
  TTLB_OP_RECIP = 44,
  TTLB_OP_TAN = 45,
  TTLB_OP_ATAN = 46,
  TTLB_OP_ATANH = 47,
  TTLB_OP_SIN = 48,
  TTLB_OP_ASIN = 49,
  TTLB_OP_ASINH = 50,
  TTLB_OP_COS = 51,
  TTLB_OP_ACOS = 52,
  TTLB_OP_ACOSH = 53,
  TTLB_OP_GELU = 54,        /* 0.5 x (1 + erf(x / sqrt 2)) */
  TTLB_OP_SILU = 55,        /* x / (1 + exp(-x)) */
  TTLB_OP_SOFTSIGN = 56,    /* x / (1 + |x|) */
  TTLB_OP_HARDSIGMOID = 57, /* clamp(x / 6 + 1/2, 0, 1) */
  /* Functions with scalar parameters: `arg` is the index of the first parameter in `imm`. */
  TTLB_OP_RSUB_IMM = 64,   /* p0 - x */
  TTLB_OP_RELU_MAX = 65,   /* relu(min(x, p0)) */
  TTLB_OP_RELU_MIN = 66,   /* relu(max(x, p0)) */
  TTLB_OP_LEAKY_RELU = 67, /* x >= 0 ? x : p0 x (also prelu) */
  TTLB_OP_ELU = 68,        /* x > 0 ? x : p0 (exp(x) - 1) */
  TTLB_OP_CELU = 69,       /* max(0, x) + min(0, p0 (exp(x p1) - 1)), p1 = 1 / p0 */
  TTLB_OP_SOFTPLUS = 70,   /* x p0 > p2 ? x : log(1 + exp(x p0)) p1, p1 = 1 / p0 */
  TTLB_OP_HARDTANH = 71,   /* min(max(x, p0), p1) */
  TTLB_OP_SELU = 72,       /* p0 (x > 0 ? x : p1 (exp(x) - 1)) */
  TTLB_OP_POW_IMM = 73     /* x ** p0 (block ** integer, python/sim/block.py:986-989); x*x and x*x*x for p0 = 2, 3 */
};
#define TTLB_MAX_IMM 8

/* How an input is indexed from an output element (i, j):
 *  SAME  index = i + off                 (same-shape operand, optionally shifted)
 *  ZERO  index = off                     (one fixed row / column: a degenerate tensor dim -
 *                                         [1,N] row vector, [N,1] column, [1,1] scalar,
 *                                         python/sim/copyhandlers.py:103-131 - or the first
 *                                         row / column of one fixed tile)
 *  TILE  index = off + (i mod 32)        (one fixed tile repeated over the tile
 *                                         grid: the simulator's tile-grid
 *                                         broadcast, python/sim/ttnnsim.py:67-109)
 *  FIRST index = off + (i - i mod 32)    (element 0 of the tile that i falls in: the hardware
 *                                         broadcast convention, a FULL source tile whose first
 *                                         row / column / element carries the data, ttl.bcast
 *                                         Row / Col / Scalar, TTLOps.td:570-597,
 *                                         test/python/test_bcast_ops.py:31-55) */
enum ttlb_index_mode { TTLB_IDX_SAME = 0, TTLB_IDX_ZERO = 1, TTLB_IDX_TILE = 2, TTLB_IDX_FIRST = 3 };

typedef struct {
  const void *ptr; /* element (0,0) of the tensor */
  int64_t ld;      /* row pitch in elements */
  int32_t row_mode, col_mode;
  int64_t row_off, col_off; /* in elements */
} ttlb_operand;

typedef struct {
  int16_t opcode;
  int16_t arg;
} ttlb_instr;

typedef struct {
  int32_t dtype;         /* TTLB_BF16 or TTLB_F32: type of every input and of the output */
  int32_t round_each_op; /* 1: round the accumulator to `dtype` after every op (what the
                            simulator does on bf16 tensors, python/sim/block.py:856-864);
                            0: fp32 intermediates, one final rounding */
  int32_t n_in, n_ops;
  ttlb_operand in[TTLB_MAX_IN];
  ttlb_instr ops[TTLB_MAX_OPS];
  void *out;      /* element (0,0) of the output tensor */
  int64_t out_ld; /* row pitch in elements */
  int64_t row0, col0, rows, cols; /* rectangle of the output to compute, in elements;
                                     col0 and cols must be multiples of 8 */
  float imm[TTLB_MAX_IMM];        /* scalar parameters of the TTLB_OP_*_IMM-style functions */
} ttlb_eltwise_desc;

TTLB_EXPORT int ttlb_eltwise(ttlb_ctx *ctx, const ttlb_eltwise_desc *desc, void *stream);

/* How ttlb_eltwise executes a program.  The reference generates one C++ compute
 * kernel per tile program and has the device runtime compile it
 * (python/ttl/ttl_api.py:425-440, 556-559); likewise a program is normally run by a
 * kernel specialised for it (the streaming skeleton instantiated for the program's
 * operand addressing and op sequence, compiled once for sm_100a with NVRTC and
 * cached in the context).  The generic kernel interprets the same program on the
 * GPU and needs no run-time compiler.
 *   AUTO         specialised kernel; generic kernel if NVRTC cannot be loaded
 *   GENERIC      always the generic (interpreting) kernel
 *   SPECIALISED  specialised kernel or an error */
#define TTLB_ELTWISE_AUTO 0
#define TTLB_ELTWISE_GENERIC 1
#define TTLB_ELTWISE_SPECIALISED 2
TTLB_EXPORT int ttlb_eltwise_set_mode(ttlb_ctx *ctx, int mode);
/* Which kernel the last successful ttlb_eltwise used: TTLB_ELTWISE_GENERIC or
 * TTLB_ELTWISE_SPECIALISED; -1 before the first launch. */
TTLB_EXPORT int ttlb_eltwise_last_path(ttlb_ctx *ctx);
/* CUDA source of the specialised kernel for `desc` (no GPU needed).  Writes at most
 * `len` bytes including the terminating NUL; returns the full length needed, or a
 * negative status for an invalid descriptor. */
TTLB_EXPORT int64_t ttlb_eltwise_source(const ttlb_eltwise_desc *desc, char *buf, size_t len);

/* ------------------------------------------------------------------------ *
 * Reductions: `ttl.math.reduce_sum(expr, scaler, dims)` / `ttl.math.reduce_max(...)`.
 *
 * The functions are specified (docs/sphinx/specs/TTLangSpecification.md:750-755: "scaled sum /
 * maximum reduction over specified dimensions", dims=[0] over rows, dims=[0,1] over rows and
 * columns) but implemented by neither the reference compiler nor its simulator.  Meaning used
 * here: the values of the element-wise program `src` over the rectangle
 * [src.row0, +src.rows) x [src.col0, +src.cols) are combined in fp32 along the reduced
 * dimension(s), the result is multiplied by the scaler and rounded once to `src.dtype`.
 *   dims = ROWS          result[j]   = s * reduce_i value(i, j)   -> out[0 .. fill_rows) x [0 .. cols)
 *   dims = COLS          result[i]   = s * reduce_j value(i, j)   -> out[0 .. rows) x [0 .. fill_cols)
 *   dims = ROWS | COLS   result      = s * reduce_ij value(i, j)  -> out[0 .. fill_rows) x [0 .. fill_cols)
 * Along a reduced dimension the result is written at index 0 and indices 1 .. fill-1 are set to
 * zero: fill = 1 for a degenerate output ([1,N] row vector, [N,1] column, [1,1] scalar), fill = 32
 * for an output of full tiles, which then has the layout ttl.math.broadcast expects of its source
 * on hardware (data in the first row / column / element, test/python/test_bcast_ops.py:31-55).
 * Sums are formed in a fixed order (the same inputs give the same bits on every launch).
 * `src.out`, `src.out_ld` are ignored.  Partial results of a reduction over rows pass through
 * scratch memory owned by the context (allocated on first use).
 * ------------------------------------------------------------------------ */
#define TTLB_REDUCE_SUM 0
#define TTLB_REDUCE_MAX 1
#define TTLB_REDUCE_ROWS 1 /* `dims` contains 0 */
#define TTLB_REDUCE_COLS 2 /* `dims` contains 1 */

typedef struct {
  ttlb_eltwise_desc src; /* the values to reduce; cols and col0 multiples of 8 (bf16) or 4 (fp32) */
  int32_t op;            /* TTLB_REDUCE_SUM / TTLB_REDUCE_MAX */
  int32_t dims;          /* TTLB_REDUCE_ROWS, TTLB_REDUCE_COLS or both */
  const void *scaler;    /* one element of src.dtype in device memory; NULL = 1.0 */
  void *out;             /* where result element (0, 0) goes; src.dtype */
  int64_t out_ld;        /* row pitch of the output in elements */
  int32_t fill_rows, fill_cols; /* 1..32, see above (ignored along a dimension that is kept) */
} ttlb_reduce_desc;

TTLB_EXPORT int ttlb_reduce(ttlb_ctx *ctx, const ttlb_reduce_desc *desc, void *stream);
/* CUDA source of the kernel specialised for `desc` (no GPU needed); same contract as
 * ttlb_eltwise_source. */
TTLB_EXPORT int64_t ttlb_reduce_source(const ttlb_reduce_desc *desc, char *buf, size_t len);

/* ------------------------------------------------------------------------ *
 * Row-resident fusion: up to three reductions over columns followed by an element-wise program, all over
 * the same rows, in ONE kernel that reads every operand once.
 *
 * A tile program such as row softmax - m = reduce_max(x), d = reduce_sum(exp(x - m)), y = exp(x - m) / d -
 * passes m and d on through circular buffers; run launch by launch it reads x three times.  Here one CTA
 * holds a whole row of every operand in registers, forms the reductions one after the other (each result
 * scaled and rounded to `dtype` exactly as ttlb_reduce would store it) and then evaluates `final`.  An
 * operand whose row_mode is TTLB_IDX_PHASE stands for the result of the earlier reduction number row_off
 * (0-based) of the same call, one value per row, used for every column; its ptr is ignored.
 * Requirements: every phase has dims = TTLB_REDUCE_COLS and the same dtype and rectangle as `final`
 * (row0, rows, col0, cols); cols <= 2048 vectors of 16 bytes; phase[].out may be NULL (result not stored)
 * or receives the result as ttlb_reduce would write it.  Sums have a fixed order.
 * No counterpart in the reference compiler, which fuses element-wise chains only
 * (lib/Dialect/TTL/IR/TTLOpsUtils.cpp:9-63).
 * ------------------------------------------------------------------------ */
#define TTLB_MAX_PHASES 3
#define TTLB_IDX_PHASE 4

typedef struct {
  int32_t n_phases; /* 1..TTLB_MAX_PHASES */
  ttlb_reduce_desc phase[TTLB_MAX_PHASES];
  ttlb_eltwise_desc final;
} ttlb_rowfused_desc;

TTLB_EXPORT int ttlb_rowfused(ttlb_ctx *ctx, const ttlb_rowfused_desc *desc, void *stream);
TTLB_EXPORT int64_t ttlb_rowfused_source(const ttlb_rowfused_desc *desc, char *buf, size_t len);

/* ------------------------------------------------------------------------ *
 * Matmul tile programs: C[M,N] = A[M,K] x B[K,N], bf16 in, fp32 accumulate,
 * bf16 out, all row-major.
 *
 * Replaces the accumulate-over-K program `out_blk.store(a_blk @ b_blk, acc=True)`
 * (examples/singlecore_matmul.py:36-45, examples/multicore_matmul.py:92-139) and
 * the Tensix kernels it stands for: reader / matmul_tiles compute / writer
 * (examples/metal_examples/multicore_matmul/metal/kernels/mm_reader.cpp:39-68,
 * mm_compute.cpp:30-65, mm_writer.cpp:29-42).
 * To compute a sub-rectangle of a larger output, pass pointers to its first
 * element and the full row pitches.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void *a; /* bf16 [m, k] */
  int64_t lda;   /* row pitches in elements */
  const void *b; /* bf16 [k, n] */
  int64_t ldb;
  void *c; /* bf16 [m, n] */
  int64_t ldc;
  int64_t m, n, k; /* k, n and the pitches must be multiples of 8 */
} ttlb_gemm_desc;

TTLB_EXPORT int ttlb_matmul_bf16(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, void *stream);
/* The same program on float32 tensors (the reference's matmul examples call their kernels with
 * fp32 tensors and check against an fp32 golden at rtol 1e-4: examples/singlecore_matmul.py:73-88).
 * a, b, c are fp32; fp32 FMA accumulation on the CUDA cores, no alignment requirement beyond 4 bytes. */
TTLB_EXPORT int ttlb_matmul_f32(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, void *stream);

/* ------------------------------------------------------------------------ *
 * bfloat8_b block-float weights (quantised inference GEMM):
 * C[M,N] = A[M,K] (bf16) x W[K,N] where W is stored as 1088-byte bfloat8_b tiles.
 *
 * The reference only fixes the tile size, 1088 bytes = 1024 value bytes + 64 shared
 * exponents, one per 16 values (python/ttl/dtype_utils.py:174-175); it has no
 * pack/unpack code of its own.  The complete byte layout used by this library is
 * written down at the top of csrc/bfp8.cu: tiles in row-major tile order, four
 * 16x16 faces per tile, a block = 16 consecutive values of one face row, exponent =
 * largest biased fp32 exponent of the block, value byte = sign | 7-bit magnitude,
 * value = (-1)^s * m * 2^(E-133), round-to-nearest-even, saturating.
 * ------------------------------------------------------------------------ */
/* Host-side packer / unpacker (plain CPU code; rows and cols multiples of 32).
 * dst_tiles must hold (rows/32)*(cols/32)*1088 bytes.  Inf/NaN inputs are rejected. */
TTLB_EXPORT int ttlb_pack_bfp8_b(const float *src, int64_t rows, int64_t cols, uint8_t *dst_tiles);
TTLB_EXPORT int ttlb_unpack_bfp8_b(const uint8_t *tiles, int64_t rows, int64_t cols, float *dst);
/* Device-side unpack of the column window [32*tile_col0, 32*tile_col0 + n) of a packed
 * [k, 32*tile_cols_total] matrix into a row-major bf16 [k, n] array of pitch ld (exact:
 * every bfloat8_b value is representable in bf16). */
TTLB_EXPORT int ttlb_unpack_bfp8_b_device(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total,
                                          int64_t tile_col0, int64_t k, int64_t n, void *out_bf16, int64_t ld,
                                          void *stream);

typedef struct {
  const void *a; /* bf16 [m, k] activations, row-major */
  int64_t lda;
  const void *b_tiles;  /* packed bfloat8_b weights of a [k, 32*b_tile_cols] matrix (device memory) */
  int64_t b_tile_cols;  /* tile columns of the whole packed matrix */
  int64_t b_tile_col0;  /* first tile column used: output column j reads weight column 32*b_tile_col0 + j */
  void *c; /* bf16 [m, n] */
  int64_t ldc;
  int64_t m, n, k; /* n and k multiples of 32 */
} ttlb_gemm_bfp8_desc;

/* Expands the weight window to bf16 in scratch memory owned by the context (allocated on
 * first use, grown when a larger window arrives), then runs the tensor-core GEMM. */
TTLB_EXPORT int ttlb_matmul_bfp8w(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, void *stream);

/* bfloat4_b weights: 576-byte tiles = 512 value bytes + 64 shared exponents (python/ttl/dtype_utils.py:178-179;
 * the reference has no pack / unpack code for it either).  Same structure as bfloat8_b with 4-bit values: two values
 * per byte (even index in the low nibble), nibble = sign | 3-bit magnitude, value = (-1)^s * m * 2^(E-129); the full
 * layout is written at the top of csrc/bfp4.cu.  The matmul expands the weight window to bf16 in the context's
 * scratch, then runs the tensor-core GEMM; the descriptor is the bfloat8_b one with b_tiles pointing at bfloat4_b
 * tiles. */
TTLB_EXPORT int ttlb_pack_bfp4_b(const float *src, int64_t rows, int64_t cols, uint8_t *dst_tiles);
TTLB_EXPORT int ttlb_unpack_bfp4_b(const uint8_t *tiles, int64_t rows, int64_t cols, float *dst);
TTLB_EXPORT int ttlb_unpack_bfp4_b_device(ttlb_ctx *ctx, const void *tiles, int64_t tile_cols_total,
                                          int64_t tile_col0, int64_t k, int64_t n, void *out_bf16, int64_t ld,
                                          void *stream);
TTLB_EXPORT int ttlb_matmul_bfp4w(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, void *stream);
/* ... with the bias / activation epilogue (arguments as for ttlb_matmul_bf16_epilogue, TTLB_ACT_* below). */
TTLB_EXPORT int ttlb_matmul_bfp4w_epilogue(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, const void *bias,
                                           int64_t ldbias, int act, void *stream);

/* No counterpart in the reference: an addition of this library for callers that must not
 * allocate.  Same result as ttlb_matmul_bfp8w, but no context is needed and no cudaMalloc,
 * cudaFree or other allocating routine is called: the bf16 expansion of the weight window goes
 * into a fixed 32 MiB array in the library's device image.
 *
 * For: code that runs after the process has given all free GPU memory to its own pool, code on a
 * latency-critical path (allocation synchronises the device), plugins restricted to the buffers
 * they are handed.
 * Limits: k * n <= TTLB_NOALLOC_MAX_WEIGHT_ELEMS (larger windows return TTLB_ERR_UNSUPPORTED with
 * a message); every GPU that loads the library holds the 32 MiB until process exit; all calls on
 * one GPU share the array, so calls that can overlap on the GPU race - serialise them.  The first
 * call on a device does a one-time set-up (symbol address look-up, kernel attribute); make it
 * before any stream capture.  The current CUDA device is used.
 * check != 0: synchronise `stream` and return TTLB_ERR_TIMEOUT if a bounded device wait ran out; with check == 0
 * such a timeout is not reported at all (the status word is private to this entry point and cleared by its next call).
 * err / err_len: optional buffer that receives a message on failure. */
#define TTLB_NOALLOC_MAX_WEIGHT_ELEMS (16 * 1024 * 1024)
TTLB_EXPORT int ttlb_matmul_bfp8w_noalloc(const ttlb_gemm_bfp8_desc *desc, void *stream, int check, char *err,
                                          size_t err_len);

/* ------------------------------------------------------------------------ *
 * Fused attention forward: O = softmax(scale * Q K^T + causal mask) V per (batch, head),
 * online softmax with fp32 row max / row sum, bf16 in and out.
 *
 * The reference has no attention kernel or example (README.md:83 names a flash-attention
 * test that is not in its tree); this entry point is the flash-attention tile program
 * (per KV block: S = Q @ K^T, running max/sum update, O += P @ V) as one kernel.
 * Q, K, V, O are contiguous [batch_heads, seq, head_dim] arrays (a [B, H, S, D] tensor
 * with B and H flattened); head_dim must be 128.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void *q, *k, *v; /* bf16 [batch_heads, seq, head_dim] */
  void *o;               /* bf16 [batch_heads, seq, head_dim] */
  int64_t batch_heads, seq, head_dim;
  int32_t causal; /* 1: key j is visible to query i only if j <= i */
  float scale;    /* multiplies Q K^T, e.g. 1/sqrt(head_dim) */
} ttlb_attn_desc;

TTLB_EXPORT int ttlb_attention(ttlb_ctx *ctx, const ttlb_attn_desc *desc, void *stream);

/* ------------------------------------------------------------------------ *
 * Publishing an output shard to every GPU of the box through the NVSwitch.
 *
 * No counterpart in the reference (it is single-chip).  `mc_dst` is a multicast address: memory
 * that is bound, at the same offset, on every GPU of a multicast group (for instance
 * torch.distributed._symmetric_memory's multicast_ptr plus a byte offset).  The region
 * [rows x row_bytes] at `src` (pitch src_ld_bytes) is written once with multimem.st and the switch
 * replicates it to all GPUs, this one included.  Completion on the stream means the stores were
 * issued; a cross-rank barrier after it makes them visible everywhere.
 * ------------------------------------------------------------------------ */
/* The matmuls with the publication fused into the epilogue: desc->c is the multicast address of
 * the output region (same pitch); every output tile is stored once with multimem.st while the tensor
 * cores work on the next tile, and arrives in the output buffer of every GPU.  The epilogue passes the tile
 * through shared memory so that each store instruction of a warp covers two whole 256-byte row segments
 * (16-byte stores scattered over 32 rows reach a small fraction of the NVLink rate).  n must be a multiple
 * of 32.  Nothing is written through the ordinary (unicast) mapping. */
TTLB_EXPORT int ttlb_matmul_bf16_multicast(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, void *stream);
TTLB_EXPORT int ttlb_matmul_bfp8w_multicast(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, void *stream);
/* The same publication without the switch's replication: `peers[0..n_peers)` (1..8) are the addresses of the
 * output region in every GPU's copy of the buffer - peer-mapped memory of the other GPUs and this GPU's own copy,
 * all with the pitch desc->ldc; desc->c is ignored.  The epilogue stores every tile to each of them with ordinary
 * 16-byte stores, row-contiguous (256 bytes per row segment).  Peer memory is only ever written, never read.
 * No counterpart in the reference (it is single-chip). */
TTLB_EXPORT int ttlb_matmul_bf16_peers(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, void *const *peers, int n_peers,
                                       void *stream);
TTLB_EXPORT int ttlb_matmul_bfp8w_peers(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, void *const *peers, int n_peers,
                                        void *stream);
/* ttlb_attention with the same two ways of publishing the output of this rank's heads: desc->o is the multicast
 * address of the output (multicast), or `peers` are the addresses of the output in every GPU's copy of a shared
 * buffer and desc->o is ignored (peers).  The epilogue stages every tile's rows in shared memory and stores whole
 * 128-byte half rows. */
TTLB_EXPORT int ttlb_attention_multicast(ttlb_ctx *ctx, const ttlb_attn_desc *desc, void *stream);
TTLB_EXPORT int ttlb_attention_peers(ttlb_ctx *ctx, const ttlb_attn_desc *desc, void *const *peers, int n_peers,
                                     void *stream);
TTLB_EXPORT int ttlb_multimem_bcast(ttlb_ctx *ctx, const void *src, int64_t src_ld_bytes, void *mc_dst,
                                    int64_t dst_ld_bytes, int64_t rows, int64_t row_bytes, void *stream);

/* C = A x B + bias: `bias` is a bf16 [m, n] matrix (row pitch ldbias elements, 16-byte aligned, pitch a
 * multiple of 8), added to the fp32 product before the single rounding to bf16.  The tile program is the
 * specification's "matmul with bias" (docs/sphinx/specs/TTLangSpecification.md:232-324):
 * y_blk.store(c_blk, acc=True) followed by y_blk.store(a_blk @ b_blk, acc=True) over the K tiles. */
TTLB_EXPORT int ttlb_matmul_bf16_bias(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, const void *bias, int64_t ldbias,
                                      void *stream);

/* C = act(A x B + bias): bias and activation applied to the fp32 accumulators in the GEMM epilogue, one rounding.
 * bias: NULL, a bf16 [m, n] matrix (ldbias >= n), or with ldbias == 0 one row of n values added to every output
 * row (the bias vector of a linear layer).  The tile program: the product accumulated over the K tiles into a
 * block of an intermediate circular buffer, then `y_blk.store(act(p_blk + broadcast(bias_blk, dims=[0])))`, in a
 * kernel with fp32_dest_acc_en=True (without it every op rounds to bf16 and the program runs as a GEMM into a
 * temporary plus an element-wise launch). */
#define TTLB_ACT_NONE 0
#define TTLB_ACT_RELU 1
#define TTLB_ACT_GELU 2
#define TTLB_ACT_SILU 3
#define TTLB_ACT_SIGMOID 4
#define TTLB_ACT_TANH 5
TTLB_EXPORT int ttlb_matmul_bf16_epilogue(ttlb_ctx *ctx, const ttlb_gemm_desc *desc, const void *bias, int64_t ldbias,
                                          int act, void *stream);

/* The same epilogue for bfloat8_b weights (a quantised linear layer with bias and activation): the weight window
 * is expanded to bf16 in the context's scratch, then the bf16 GEMM runs with the bias / activation epilogue. */
TTLB_EXPORT int ttlb_matmul_bfp8w_epilogue(ttlb_ctx *ctx, const ttlb_gemm_bfp8_desc *desc, const void *bias,
                                           int64_t ldbias, int act, void *stream);

/* Which tensor-core GEMM kernel the bf16 / bfp8-weight matmuls use:
 *   0  always one CTA per 128x256 output tile (tcgen05 cta_group::1)
 *   1  (default) a cluster of two CTAs per 256x256 tile (cta_group::2: each CTA stages half of the
 *      B tile) when the output has at least one such tile per SM pair; smaller outputs, and the
 *      multicast-epilogue entry points, keep the one-CTA kernel
 *   2  the two-CTA kernel for every shape (testing) */
TTLB_EXPORT int ttlb_set_gemm_variant(ttlb_ctx *ctx, int variant);

/* How ttlb_matmul_bfp8w expands the block-float weights:
 *   0  a separate unpack kernel writes bf16 into scratch owned by the context, then the bf16 GEMM
 *   1  inside the GEMM mainloop (packed tiles are staged in shared memory, expanded in registers and written
 *      to tensor memory, from where the tensor core reads them as an operand of the transposed product; no
 *      scratch, no bf16 copy in HBM, nothing allocated) when the output has at least one 256x256 tile per SM
 *      pair, mode 0 otherwise.  Same bits as mode 0; the default (4096x8192x28672: 1.31 ms against 1.37 ms).
 *   2  inside the mainloop for every shape (testing) */
TTLB_EXPORT int ttlb_set_bfp8_mode(ttlb_ctx *ctx, int mode);
/* Mode 0 can work in up to `chunks` (1..4) column chunks: the expansion of chunk i+1 runs on a stream owned
 * by the context under the GEMM of chunk i; both are ordered against `stream` by events and the side stream
 * has joined again when ttlb_matmul_bfp8w returns.  Default 1 (expand everything, then one GEMM): on
 * 4096x8192x28672 the overlap measured 1.395 ms with 2 or 4 chunks against 1.365 ms with 1 - the GEMM runs
 * at the power cap, so work moved under it is not free, and smaller GEMMs have longer tails. */
TTLB_EXPORT int ttlb_set_bfp8_chunks(ttlb_ctx *ctx, int chunks);

/* Kernels that wait on hardware barriers (matmul, attention) bound every wait; when
 * one runs out the kernel unwinds normally and records which role gave up.
 * ttlb_check_status synchronises `stream`, returns TTLB_ERR_TIMEOUT if that happened
 * since the last check (and clears the record), else TTLB_OK.  The reference's
 * simulator bounds its waits the same way (CB_DEFAULT_TIMEOUT / COPY_PIPE_TIMEOUT,
 * python/sim/constants.py:47-48). */
TTLB_EXPORT int ttlb_check_status(ttlb_ctx *ctx, void *stream);
/* Self-test of that machinery: launches one CTA that waits, with the given limit (at most 2e9
 * cycles), on a barrier nothing ever arrives on.  The wait gives up, the kernel returns normally,
 * and the next ttlb_check_status reports TTLB_ERR_TIMEOUT.  Never hangs by construction. */
TTLB_EXPORT int ttlb_selftest_wait_timeout(ttlb_ctx *ctx, int64_t limit_cycles, void *stream);
/* Bound of a device-side wait in SM clock cycles (default 4e9, about two seconds). */
TTLB_EXPORT int ttlb_set_wait_limit(ttlb_ctx *ctx, int64_t cycles);

#ifdef __cplusplus
}
#endif

#endif /* TTLB200_H */
