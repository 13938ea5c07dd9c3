// Fused element-wise / broadcast streaming kernel (ttlb_eltwise).
//
// One thread owns one 16-byte vector of the output (8 bf16 or 4 fp32 elements of one
// row).  All inputs of that vector are fetched first (up to TTLB_MAX_IN independent
// 16-byte loads in flight per thread), then the accumulator program is run on
// registers only: the accumulator, the two stack slots and the fetched inputs are all
// statically indexed, the only data-dependent control flow is a warp-uniform switch
// on the opcode.  Streaming operands use evict-first loads and the output an
// evict-first store; broadcast operands (row vector, column, scalar, repeated tile)
// go through the normal cached path since every row / column re-reads them.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "ctx.h"
#include "eltwise_jit.h"

namespace {

struct EltParams {
  ttlb_operand in[TTLB_MAX_IN];
  ttlb_instr ops[TTLB_MAX_OPS];
  int n_in, n_ops, round_each;
  void *out;
  long long out_ld, row0, col0;
  unsigned vpr;  // 16-byte vectors per row of the output rectangle
  unsigned long long items;
};

template <bool BF16>
struct Elem;
template <>
struct Elem<true> {
  using T = __nv_bfloat16;
  static constexpr int VEC = 8;
};
template <>
struct Elem<false> {
  using T = float;
  static constexpr int VEC = 4;
};

template <bool BF16>
__device__ __forceinline__ uint4 load_operand(const ttlb_operand &o, long long gi, long long gj) {
  using T = typename Elem<BF16>::T;
  long long r = o.row_mode == TTLB_IDX_SAME    ? gi + o.row_off
                : o.row_mode == TTLB_IDX_ZERO  ? o.row_off
                : o.row_mode == TTLB_IDX_FIRST ? o.row_off + (gi & ~31LL)
                                               : o.row_off + (gi & 31);
  const T *rowp = reinterpret_cast<const T *>(o.ptr) + r * o.ld;
  if (o.col_mode == TTLB_IDX_ZERO || o.col_mode == TTLB_IDX_FIRST) {   // one element for the whole vector
    const T *ep = rowp + (o.col_mode == TTLB_IDX_ZERO ? o.col_off : o.col_off + (gj & ~31LL));
    if constexpr (BF16) {
      unsigned h = *reinterpret_cast<const unsigned short *>(ep);
      unsigned hh = h | (h << 16);
      return make_uint4(hh, hh, hh, hh);
    } else {
      unsigned w = *reinterpret_cast<const unsigned *>(ep);
      return make_uint4(w, w, w, w);
    }
  }
  long long c = o.col_mode == TTLB_IDX_SAME ? gj + o.col_off : o.col_off + (gj & 31);
  const uint4 *vp = reinterpret_cast<const uint4 *>(rowp + c);
  if (o.row_mode == TTLB_IDX_SAME && o.col_mode == TTLB_IDX_SAME) return __ldcs(vp);
  return __ldg(vp);
}

template <bool BF16>
__device__ __forceinline__ void unpack(const uint4 &v, float (&x)[Elem<BF16>::VEC]) {
  if constexpr (BF16) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    x[0] = __uint_as_float(v.x);
    x[1] = __uint_as_float(v.y);
    x[2] = __uint_as_float(v.z);
    x[3] = __uint_as_float(v.w);
  }
}

__device__ __forceinline__ float round_bf16(float a) {
  return __bfloat162float(__float2bfloat16_rn(a));
}

// NaN-propagating max / min, as torch.maximum / torch.minimum.
__device__ __forceinline__ float nan_max(float a, float b) { return (a > b || a != a) ? a : b; }
__device__ __forceinline__ float nan_min(float a, float b) { return (a < b || a != a) ? a : b; }

template <bool BF16>
__global__ void __launch_bounds__(256, 4) ttlb_eltwise_kernel(const __grid_constant__ EltParams p) {
  constexpr int VEC = Elem<BF16>::VEC;
  using T = typename Elem<BF16>::T;
  const unsigned long long stride = (unsigned long long)gridDim.x * 256ull;
  for (unsigned long long w = (unsigned long long)blockIdx.x * 256ull + threadIdx.x; w < p.items;
       w += stride) {
    const unsigned long long i = w / p.vpr;
    const unsigned jv = (unsigned)(w - i * p.vpr);
    const long long gi = p.row0 + (long long)i;
    const long long gj = p.col0 + (long long)jv * VEC;

    uint4 raw[TTLB_MAX_IN];
#pragma unroll
    for (int k = 0; k < TTLB_MAX_IN; ++k) {
      raw[k] = make_uint4(0, 0, 0, 0);
      if (k < p.n_in) raw[k] = load_operand<BF16>(p.in[k], gi, gj);
    }

    float acc[VEC], s0[VEC], s1[VEC], x[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = s0[e] = s1[e] = 0.f;

    for (int pc = 0; pc < p.n_ops; ++pc) {
      const int op = p.ops[pc].opcode;
      const int arg = p.ops[pc].arg;
      if (op <= TTLB_OP_MIN) {  // LOAD or binary: fetch the operand
        if (arg >= 0) {
          uint4 v = raw[0];
#pragma unroll
          for (int k = 1; k < TTLB_MAX_IN; ++k)
            if (arg == k) v = raw[k];
          unpack<BF16>(v, x);
        } else {  // pop
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            x[e] = s0[e];
            s0[e] = s1[e];
          }
        }
      }
#define TTLB_EACH(expr)                 \
  _Pragma("unroll") for (int e = 0; e < VEC; ++e) { \
    const float a = acc[e];             \
    const float b = x[e];               \
    (void)a;                            \
    (void)b;                            \
    acc[e] = (expr);                    \
  }                                     \
  break;
      switch (op) {
        case TTLB_OP_LOAD: TTLB_EACH(b)
        case TTLB_OP_ADD: TTLB_EACH(a + b)
        case TTLB_OP_SUB: TTLB_EACH(a - b)
        case TTLB_OP_RSUB: TTLB_EACH(b - a)
        case TTLB_OP_MUL: TTLB_EACH(a * b)
        case TTLB_OP_DIV: TTLB_EACH(a / b)
        case TTLB_OP_RDIV: TTLB_EACH(b / a)
        case TTLB_OP_MAX: TTLB_EACH(nan_max(a, b))
        case TTLB_OP_MIN: TTLB_EACH(nan_min(a, b))
        case TTLB_OP_EXP: TTLB_EACH(expf(a))
        case TTLB_OP_LOG: TTLB_EACH(logf(a))
        case TTLB_OP_SQRT: TTLB_EACH(sqrtf(a))
        case TTLB_OP_RSQRT: TTLB_EACH(1.0f / sqrtf(a))
        case TTLB_OP_TANH: TTLB_EACH(tanhf(a))
        case TTLB_OP_SIGMOID: TTLB_EACH(1.0f / (1.0f + expf(-a)))
        case TTLB_OP_NEG: TTLB_EACH(-a)
        case TTLB_OP_ABS: TTLB_EACH(fabsf(a))
        case TTLB_OP_RELU: TTLB_EACH(a < 0.f ? 0.f : a)
        case TTLB_OP_PUSH:
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            s1[e] = s0[e];
            s0[e] = acc[e];
          }
          break;
        default: break;
      }
#undef TTLB_EACH
      if (BF16 && p.round_each && op != TTLB_OP_PUSH && op != TTLB_OP_LOAD) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = round_bf16(acc[e]);
      }
    }

    T *outp = reinterpret_cast<T *>(p.out) + gi * p.out_ld + gj;
    uint4 o;
    if constexpr (BF16) {
      unsigned wds[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        wds[q] = *reinterpret_cast<unsigned *>(&h);
      }
      o = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    } else {
      o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                     __float_as_uint(acc[3]));
    }
    __stcs(reinterpret_cast<uint4 *>(outp), o);
  }
}

bool is_binary(int op) { return op >= TTLB_OP_ADD && op <= TTLB_OP_RPOW; }
bool is_unary(int op) {
  return (op >= TTLB_OP_EXP && op <= TTLB_OP_RELU) || (op >= TTLB_OP_EXP2 && op <= TTLB_OP_HARDSIGMOID);
}
// Functions with scalar parameters: how many entries of `imm` they read (0: not such a function).
int imm_params(int op) {
  switch (op) {
    case TTLB_OP_RSUB_IMM: case TTLB_OP_RELU_MAX: case TTLB_OP_RELU_MIN: case TTLB_OP_LEAKY_RELU: case TTLB_OP_ELU:
    case TTLB_OP_POW_IMM:
      return 1;
    case TTLB_OP_CELU: case TTLB_OP_HARDTANH: case TTLB_OP_SELU:
      return 2;
    case TTLB_OP_SOFTPLUS:
      return 3;
  }
  return 0;
}

}  // namespace

// Host-side validation shared by every execution path.  Returns 1 for "valid but empty".
static int validate_eltwise(ttlb_ctx *ctx, const ttlb_eltwise_desc *d, bool need_out = true) {
  if (!d) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: null descriptor");
  if (d->dtype != TTLB_BF16 && d->dtype != TTLB_F32)
    return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "eltwise: dtype %d (bf16 and f32 only)", d->dtype);
  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  const int esz = d->dtype == TTLB_BF16 ? 2 : 4;
  if (d->n_in < 1 || d->n_in > TTLB_MAX_IN)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: n_in=%d outside [1,%d]", d->n_in, TTLB_MAX_IN);
  if (d->n_ops < 1 || d->n_ops > TTLB_MAX_OPS)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: n_ops=%d outside [1,%d]", d->n_ops,
                     TTLB_MAX_OPS);
  if (d->rows < 0 || d->cols < 0 || d->row0 < 0 || d->col0 < 0)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: negative rectangle");
  if (need_out) {
    if (!d->out) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: null output");
    if ((d->cols % vec) || (d->col0 % vec) || (d->out_ld % vec) || ((uintptr_t)d->out % 16))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG,
                       "eltwise: output must be 16-byte aligned (col0, cols, ld multiples of %d)", vec);
    if (d->out_ld < d->col0 + d->cols)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: rectangle exceeds the output pitch");
  } else if ((d->cols % vec) || (d->col0 % vec)) {
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: col0 and cols must be multiples of %d", vec);
  }
  for (int k = 0; k < d->n_in; ++k) {
    const ttlb_operand &o = d->in[k];
    if (!o.ptr) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d is null", k);
    if (o.row_mode < 0 || o.row_mode > 3 || o.col_mode < 0 || o.col_mode > 3)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d has a bad index mode", k);
    if (o.col_mode == TTLB_IDX_SAME || o.col_mode == TTLB_IDX_TILE) {
      if ((o.ld % vec) || (o.col_off % vec) || ((uintptr_t)o.ptr % 16))
        return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d is not 16-byte aligned", k);
    } else if ((uintptr_t)o.ptr % esz) {
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d is misaligned", k);
    }
    if (o.row_mode == TTLB_IDX_SAME && d->row0 + o.row_off < 0)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d row offset underflows", k);
    if (o.col_mode == TTLB_IDX_SAME && d->col0 + o.col_off < 0)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d col offset underflows", k);
    if ((o.row_mode == TTLB_IDX_TILE && o.row_off < 0) || (o.col_mode == TTLB_IDX_TILE && o.col_off < 0) ||
        (o.row_mode == TTLB_IDX_ZERO && o.row_off < 0) || (o.col_mode == TTLB_IDX_ZERO && o.col_off < 0))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d tile offset is negative", k);
    if ((o.row_mode == TTLB_IDX_FIRST && d->row0 + o.row_off < 0) || (o.col_mode == TTLB_IDX_FIRST && d->col0 + o.col_off < 0))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: input %d tile offset underflows", k);
  }
  // Walk the program once: operand indices in range, stack never under/overflows,
  // first instruction defines the accumulator.
  int depth = 0;
  for (int pc = 0; pc < d->n_ops; ++pc) {
    const int op = d->ops[pc].opcode, arg = d->ops[pc].arg;
    if (pc == 0 && op != TTLB_OP_LOAD)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: program must start with LOAD");
    if (op == TTLB_OP_LOAD || is_binary(op)) {
      if (arg == TTLB_ARG_STACK) {
        if (op == TTLB_OP_LOAD || depth == 0)
          return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: op %d pops an empty stack", pc);
        --depth;
      } else if (arg < 0 || arg >= d->n_in) {
        return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: op %d names input %d of %d", pc, arg,
                         d->n_in);
      }
    } else if (op == TTLB_OP_PUSH) {
      if (++depth > 2)
        return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "eltwise: expression needs a stack deeper than 2");
    } else if (const int np = imm_params(op)) {
      if (arg < 0 || arg + np > TTLB_MAX_IMM)
        return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: op %d reads parameters %d..%d of %d", pc, arg, arg + np - 1,
                         TTLB_MAX_IMM);
    } else if (!is_unary(op)) {
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: unknown opcode %d at %d", op, pc);
    }
  }
  if (depth != 0) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: %d value(s) left on the stack", depth);

  if (d->rows == 0 || d->cols == 0) return 1;  // empty program: nothing to do
  return TTLB_OK;
}

extern "C" int ttlb_eltwise_set_mode(ttlb_ctx *ctx, int mode) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  if (mode < TTLB_ELTWISE_AUTO || mode > TTLB_ELTWISE_SPECIALISED)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "eltwise: unknown mode %d", mode);
  ctx->eltwise_mode = mode;
  return TTLB_OK;
}

extern "C" int ttlb_eltwise_last_path(ttlb_ctx *ctx) { return ctx ? ctx->eltwise_last_path : -1; }

extern "C" int64_t ttlb_eltwise_source(const ttlb_eltwise_desc *d, char *buf, size_t len) {
  const int rc = validate_eltwise(nullptr, d);
  if (rc < 0) return rc;
  const std::string src = ttlb_eltwise_jit_source(d);
  if (buf && len) {
    const size_t n = src.size() < len - 1 ? src.size() : len - 1;
    memcpy(buf, src.data(), n);
    buf[n] = 0;
  }
  return (int64_t)src.size() + 1;
}

extern "C" int ttlb_eltwise(ttlb_ctx *ctx, const ttlb_eltwise_desc *d, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  {
    const int rc = validate_eltwise(ctx, d);
    if (rc < 0) return rc;
    if (rc == 1) return TTLB_OK;
  }
  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "eltwise: cannot select device %d", ctx->device);
  if (ctx->eltwise_mode != TTLB_ELTWISE_GENERIC) {
    const int rc = ttlb_eltwise_jit_launch(ctx, &ctx->jit, d, s);
    if (rc == TTLB_OK) {
      ctx->launches += 1;
      ctx->eltwise_last_path = TTLB_ELTWISE_SPECIALISED;
      return TTLB_OK;
    }
    // AUTO falls back to the generic GPU kernel only when the run-time compiler is absent
    if (ctx->eltwise_mode == TTLB_ELTWISE_SPECIALISED || ttlb_eltwise_jit_available()) return rc;
  }
  for (int pc = 0; pc < d->n_ops; ++pc)
    if (d->ops[pc].opcode >= TTLB_OP_EXP2 || (d->ops[pc].opcode >= TTLB_OP_FLOORDIV && d->ops[pc].opcode <= TTLB_OP_RPOW))
      return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED,
                       "eltwise: opcode %d is implemented by the specialised kernel only (NVRTC is needed)", d->ops[pc].opcode);
  const unsigned long long vpr = (unsigned long long)(d->cols / vec);
  if (vpr > 0xffffffffull) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "eltwise: row too long");
  EltParams p;
  for (int k = 0; k < TTLB_MAX_IN; ++k) p.in[k] = d->in[k < d->n_in ? k : 0];
  for (int k = 0; k < TTLB_MAX_OPS; ++k) p.ops[k] = d->ops[k];
  p.n_in = d->n_in;
  p.n_ops = d->n_ops;
  p.round_each = d->round_each_op ? 1 : 0;
  p.out = d->out;
  p.out_ld = d->out_ld;
  p.row0 = d->row0;
  p.col0 = d->col0;
  p.vpr = (unsigned)vpr;
  p.items = vpr * (unsigned long long)d->rows;

  const unsigned long long want = (p.items + 255ull) / 256ull;
  // Persistent-style grid: a whole number of waves of resident CTAs (4 per SM).
  const unsigned long long resident = (unsigned long long)ctx->sm_count * 4ull;
  const unsigned grid = (unsigned)(want < resident ? want : resident * 2ull < want ? resident * 2ull : resident);
  if (d->dtype == TTLB_BF16)
    ttlb_eltwise_kernel<true><<<grid, 256, 0, s>>>(p);
  else
    ttlb_eltwise_kernel<false><<<grid, 256, 0, s>>>(p);
  TTLB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->launches += 1;
  ctx->eltwise_last_path = TTLB_ELTWISE_GENERIC;
  return TTLB_OK;
}

// --------------------------------------------------------------------------- //
// Reductions
// --------------------------------------------------------------------------- //
namespace {
constexpr size_t kReducePartialFloats = 4u << 20;  // 16 MiB of partial rows
constexpr unsigned kReduceMaxGroups = 8192;        // column groups of 256 vectors
}  // namespace

static int validate_reduce(ttlb_ctx *ctx, const ttlb_reduce_desc *r) {
  if (!r) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: null descriptor");
  const int rc = validate_eltwise(ctx, &r->src, false);
  if (rc < 0) return rc;
  const ttlb_eltwise_desc *d = &r->src;
  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  const int esz = d->dtype == TTLB_BF16 ? 2 : 4;
  if (r->op != TTLB_REDUCE_SUM && r->op != TTLB_REDUCE_MAX)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: unknown op %d", r->op);
  if (r->dims < 1 || r->dims > 3) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: dims=%d (1: rows, 2: columns, 3: both)", r->dims);
  if (!r->out) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: null output");
  if (r->scaler && ((uintptr_t)r->scaler % esz)) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: scaler is misaligned");
  if ((r->dims & TTLB_REDUCE_ROWS) && (r->fill_rows < 1 || r->fill_rows > 32))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: fill_rows=%d outside [1,32]", r->fill_rows);
  if ((r->dims & TTLB_REDUCE_COLS) && (r->fill_cols < 1 || r->fill_cols > 32))
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: fill_cols=%d outside [1,32]", r->fill_cols);
  if (r->dims == TTLB_REDUCE_ROWS) {
    // the result row is stored as 16-byte vectors
    if (((uintptr_t)r->out % 16) || (r->fill_rows > 1 && (r->out_ld % vec)))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: output must be 16-byte aligned (ld a multiple of %d)", vec);
    if (r->fill_rows > 1 && r->out_ld < d->cols) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: result exceeds the output pitch");
  } else {
    if ((uintptr_t)r->out % esz) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: output is misaligned");
    if ((d->rows > 1 || r->fill_rows > 1) && r->out_ld < r->fill_cols)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: result exceeds the output pitch");
  }
  if (d->rows > 0xffffffffll || d->cols / vec > 0xffffffffll) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "reduce: region too large");
  if (rc == 1) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "reduce: empty region");
  return TTLB_OK;
}

extern "C" int64_t ttlb_reduce_source(const ttlb_reduce_desc *r, char *buf, size_t len) {
  if (!r) return TTLB_ERR_INVALID_ARG;
  ttlb_reduce_desc c = *r;
  if (!c.out) c.out = reinterpret_cast<void *>(16);  // source generation needs no buffers
  for (int k = 0; k < c.src.n_in && k < TTLB_MAX_IN; ++k)
    if (!c.src.in[k].ptr) c.src.in[k].ptr = reinterpret_cast<const void *>(16);
  const int rc = validate_reduce(nullptr, &c);
  if (rc < 0) return rc;
  const std::string src = ttlb_reduce_jit_source(&c);
  if (buf && len) {
    const size_t n = src.size() < len - 1 ? src.size() : len - 1;
    memcpy(buf, src.data(), n);
    buf[n] = 0;
  }
  return (int64_t)src.size() + 1;
}

extern "C" int ttlb_reduce(ttlb_ctx *ctx, const ttlb_reduce_desc *r, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  {
    const int rc = validate_reduce(ctx, r);
    if (rc < 0) return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "reduce: cannot select device %d", ctx->device);
  const size_t counter_bytes = (kReduceMaxGroups + 64) * sizeof(unsigned);
  const size_t partial2_bytes = kReduceMaxGroups * sizeof(float);
  if ((r->dims & TTLB_REDUCE_ROWS) && !ctx->reduce_scratch) {
    void *p = nullptr;
    TTLB_CUDA_CHECK(ctx, cudaMalloc(&p, counter_bytes + partial2_bytes + kReducePartialFloats * sizeof(float)));
    cudaError_t e = cudaMemset(p, 0, counter_bytes);  // arrival counters start at zero; kernels leave them zero
    if (e != cudaSuccess) {
      cudaFree(p);
      return ttlb_fail(ctx, TTLB_ERR_CUDA, "reduce: cudaMemset failed: %s", cudaGetErrorString(e));
    }
    ctx->reduce_scratch = p;
  }
  char *base = static_cast<char *>(ctx->reduce_scratch);
  const int rc = ttlb_reduce_jit_launch(ctx, &ctx->jit, r, reinterpret_cast<float *>(base + counter_bytes + partial2_bytes),
                                        kReducePartialFloats, reinterpret_cast<float *>(base + counter_bytes),
                                        reinterpret_cast<unsigned *>(base), kReduceMaxGroups, s);
  if (rc == TTLB_OK) ctx->launches += 1;
  return rc;
}

// --------------------------------------------------------------------------- //
// Row-resident fusion
// --------------------------------------------------------------------------- //
// Checks a stage's program with the stand-ins for earlier results replaced by an ordinary operand.
static int validate_stage(ttlb_ctx *ctx, const ttlb_eltwise_desc *d, int stage, bool need_out) {
  ttlb_eltwise_desc c = *d;
  for (int k = 0; k < c.n_in && k < TTLB_MAX_IN; ++k) {
    if (c.in[k].row_mode != TTLB_IDX_PHASE) continue;
    if (c.in[k].row_off < 0 || c.in[k].row_off >= stage)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: stage %d reads the result of reduction %lld, which is not earlier",
                       stage, (long long)c.in[k].row_off);
    c.in[k].ptr = reinterpret_cast<const void *>(16);
    c.in[k].row_mode = c.in[k].col_mode = TTLB_IDX_ZERO;
    c.in[k].row_off = c.in[k].col_off = 0;
  }
  return validate_eltwise(ctx, &c, need_out);
}

static int validate_rowfused(ttlb_ctx *ctx, const ttlb_rowfused_desc *f) {
  if (!f) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: null descriptor");
  if (f->n_phases < 1 || f->n_phases > TTLB_MAX_PHASES)
    return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: n_phases=%d outside [1,%d]", f->n_phases, TTLB_MAX_PHASES);
  int rc = validate_stage(ctx, &f->final, f->n_phases, true);
  if (rc < 0) return rc;
  if (rc == 1) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: empty region");
  const ttlb_eltwise_desc *d = &f->final;
  const int esz = d->dtype == TTLB_BF16 ? 2 : 4;
  for (int ph = 0; ph < f->n_phases; ++ph) {
    const ttlb_reduce_desc &R = f->phase[ph];
    rc = validate_stage(ctx, &R.src, ph, false);
    if (rc < 0) return rc;
    if (R.src.dtype != d->dtype || R.src.row0 != d->row0 || R.src.rows != d->rows || R.src.col0 != d->col0 ||
        R.src.cols != d->cols)
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: reduction %d has another element type or rectangle than the final stage", ph);
    if (R.dims != TTLB_REDUCE_COLS) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "rowfused: reduction %d is not over columns only", ph);
    if (R.op != TTLB_REDUCE_SUM && R.op != TTLB_REDUCE_MAX) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: unknown op %d", R.op);
    if (R.scaler && ((uintptr_t)R.scaler % esz)) return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: scaler is misaligned");
    if (R.out && (((uintptr_t)R.out % esz) || R.fill_cols < 1 || R.fill_cols > 32 || (d->rows > 1 && R.out_ld < R.fill_cols)))
      return ttlb_fail(ctx, TTLB_ERR_INVALID_ARG, "rowfused: bad output of reduction %d", ph);
  }
  if (d->rows > 0xffffffffll) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "rowfused: too many rows");
  if (d->cols / (d->dtype == TTLB_BF16 ? 8 : 4) > 2048)
    return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "rowfused: rows longer than 2048 16-byte vectors do not fit on chip");
  return TTLB_OK;
}

extern "C" int64_t ttlb_rowfused_source(const ttlb_rowfused_desc *f, char *buf, size_t len) {
  if (!f) return TTLB_ERR_INVALID_ARG;
  ttlb_rowfused_desc c = *f;
  if (!c.final.out) c.final.out = reinterpret_cast<void *>(16);  // source generation needs no buffers
  for (int st = 0; st <= c.n_phases && st <= TTLB_MAX_PHASES; ++st) {
    ttlb_eltwise_desc *d = st < c.n_phases ? &c.phase[st].src : &c.final;
    for (int k = 0; k < d->n_in && k < TTLB_MAX_IN; ++k)
      if (!d->in[k].ptr) d->in[k].ptr = reinterpret_cast<const void *>(16);  // equal geometry = one operand
  }
  const int rc = validate_rowfused(nullptr, &c);
  if (rc < 0) return rc;
  const std::string src = ttlb_rowfused_jit_source(&c);
  if (src.empty()) return TTLB_ERR_UNSUPPORTED;
  if (buf && len) {
    const size_t n = src.size() < len - 1 ? src.size() : len - 1;
    memcpy(buf, src.data(), n);
    buf[n] = 0;
  }
  return (int64_t)src.size() + 1;
}

extern "C" int ttlb_rowfused(ttlb_ctx *ctx, const ttlb_rowfused_desc *f, void *stream) {
  if (!ctx) return TTLB_ERR_INVALID_ARG;
  const int rc = validate_rowfused(ctx, f);
  if (rc < 0) return rc;
  ttlb_device_guard g(ctx->device);
  if (!g.ok) return ttlb_fail(ctx, TTLB_ERR_CUDA, "rowfused: cannot select device %d", ctx->device);
  const int rl = ttlb_rowfused_jit_launch(ctx, &ctx->jit, f, reinterpret_cast<cudaStream_t>(stream));
  if (rl == TTLB_OK) ctx->launches += 1;
  return rl;
}
