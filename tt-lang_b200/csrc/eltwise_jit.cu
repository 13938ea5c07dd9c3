// Per-program specialisation of the fused element-wise kernel.
//
// The reference emits one C++ compute kernel per tile program and lets the device
// runtime compile it (python/ttl/ttl_api.py:425-440, 556-559: generated source is
// written out and JIT-compiled by tt-metal, cached by content hash).  The B200
// counterpart: the hand-written streaming skeleton below is instantiated for one
// accumulator program - operand addressing modes and the op sequence become
// straight-line code - compiled for sm_100a with NVRTC (loaded at run time with
// dlopen, so the library itself has no link dependency on it) and cached per context.
//
// Geometry: a CTA is BX x BY threads (BX*BY = 256); thread (tx, ty) owns the
// 16-byte column vector cv = blockIdx.x*BX + tx and walks rows
// r = blockIdx.y*BY + ty, += gridDim.y*BY.  No integer division anywhere.  Operands
// that do not depend on the row (row vectors, scalars) are fetched once before the
// row loop; streaming operands use evict-first loads, the output evict-first stores.
// --fmad=false keeps `a*b + c` as two roundings, which is what the simulator computes.
#include <dlfcn.h>

#include <cstdlib>
#include <functional>

#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "ctx.h"
#include "eltwise_jit.h"

namespace {

// ---- NVRTC through dlopen --------------------------------------------------
typedef struct _nvrtcProgram *nvrtcProgram;
struct Nvrtc {
  void *h = nullptr;
  int (*CreateProgram)(nvrtcProgram *, const char *, const char *, int, const char *const *,
                       const char *const *) = nullptr;
  int (*CompileProgram)(nvrtcProgram, int, const char *const *) = nullptr;
  int (*GetCUBINSize)(nvrtcProgram, size_t *) = nullptr;
  int (*GetCUBIN)(nvrtcProgram, char *) = nullptr;
  int (*GetProgramLogSize)(nvrtcProgram, size_t *) = nullptr;
  int (*GetProgramLog)(nvrtcProgram, char *) = nullptr;
  int (*DestroyProgram)(nvrtcProgram *) = nullptr;
  bool ok = false;
};

Nvrtc &nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    for (const char *nm : names) {
      n.h = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (n.h) break;
    }
    if (!n.h) return;
#define TTLB_SYM(field, name)                                    \
  n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.h, name)); \
  if (!n.field) return;
    TTLB_SYM(CreateProgram, "nvrtcCreateProgram")
    TTLB_SYM(CompileProgram, "nvrtcCompileProgram")
    TTLB_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    TTLB_SYM(GetCUBIN, "nvrtcGetCUBIN")
    TTLB_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    TTLB_SYM(GetProgramLog, "nvrtcGetProgramLog")
    TTLB_SYM(DestroyProgram, "nvrtcDestroyProgram")
#undef TTLB_SYM
    n.ok = true;
  });
  return n;
}

// ---- launch parameters (must match the struct in the generated source) ------
struct JitParams {
  const void *in[TTLB_MAX_IN];
  long long ld[TTLB_MAX_IN];
  long long roff[TTLB_MAX_IN];
  long long coff[TTLB_MAX_IN];
  void *out;
  long long out_ld, row0, col0;
  unsigned vpr, rows, bx_log2, pad;
  float imm[TTLB_MAX_IMM];
};

const char *kPrelude = R"SRC(
typedef unsigned int u32;
typedef long long i64;
struct JitParams {
  const void* in[6]; i64 ld[6]; i64 roff[6]; i64 coff[6];
  void* out; i64 out_ld, row0, col0; u32 vpr, rows, bx_log2, pad; float imm[8];
};
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v; asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v; asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ u32 pack_bf16x2(float lo, float hi) {
  u32 r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
// NaN-propagating like torch.maximum / torch.minimum: one instruction each
__device__ __forceinline__ float nan_max(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ float nan_min(float a, float b) { float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
// a // b and a % b the way torch computes them on floating-point tensors (floor division through fmod with the
// quotient fixed up, remainder with the sign of the divisor): the simulator's `//` and `%` are torch's
// RB rounds an intermediate to bfloat16 when the program runs with per-op rounding on bfloat16 tensors: torch
// evaluates these two algorithms in the tensor's own type, step by step, and so must this code to give the same bits.
__device__ __forceinline__ float rb_bf16(float x) { return __uint_as_float(pack_bf16x2(x, 0.0f) << 16); }
__device__ __forceinline__ float floor_div(float a, float b) {
  if (b == 0.0f) return a / b;
  const float mod = RB(fmodf(a, b));
  float div = RB(RB(a - mod) / b);
  if (mod != 0.0f && ((b < 0.0f) != (mod < 0.0f))) div = RB(div - 1.0f);
  if (div == 0.0f) return copysignf(0.0f, a / b);
  float fl = floorf(div);
  if (RB(div - fl) > 0.5f) fl = RB(fl + 1.0f);
  return fl;
}
__device__ __forceinline__ float py_mod(float a, float b) {
  float mod = RB(fmodf(a, b));
  if (mod != 0.0f && ((b < 0.0f) != (mod < 0.0f))) mod = RB(mod + b);
  return mod;
}
// block ** integer: torch squares and cubes by multiplying (the cube in the tensor's type, hence RB), else pow()
__device__ __forceinline__ float pow_imm(float a, float n) { return n == 2.0f ? a * a : n == 3.0f ? RB(a * a) * a : powf(a, n); }
)SRC";

const char *binary_expr(int op) {
  switch (op) {
    case TTLB_OP_ADD: return "a + b";
    case TTLB_OP_SUB: return "a - b";
    case TTLB_OP_RSUB: return "b - a";
    case TTLB_OP_MUL: return "a * b";
    case TTLB_OP_DIV: return "a / b";
    case TTLB_OP_RDIV: return "b / a";
    case TTLB_OP_MAX: return "nan_max(a, b)";
    case TTLB_OP_MIN: return "nan_min(a, b)";
    case TTLB_OP_FLOORDIV: return "floor_div(a, b)";
    case TTLB_OP_RFLOORDIV: return "floor_div(b, a)";
    case TTLB_OP_MOD: return "py_mod(a, b)";
    case TTLB_OP_RMOD: return "py_mod(b, a)";
    case TTLB_OP_POW: return "powf(a, b)";
    case TTLB_OP_RPOW: return "powf(b, a)";
  }
  return nullptr;
}

const char *unary_expr(int op) {
  switch (op) {
    case TTLB_OP_EXP: return "expf(a)";
    case TTLB_OP_LOG: return "logf(a)";
    case TTLB_OP_SQRT: return "sqrtf(a)";
    case TTLB_OP_RSQRT: return "1.0f / sqrtf(a)";
    case TTLB_OP_TANH: return "tanhf(a)";
    case TTLB_OP_SIGMOID: return "1.0f / (1.0f + expf(-a))";
    case TTLB_OP_NEG: return "-a";
    case TTLB_OP_ABS: return "fabsf(a)";
    case TTLB_OP_RELU: return "(a < 0.f ? 0.f : a)";
    case TTLB_OP_EXP2: return "exp2f(a)";
    case TTLB_OP_EXPM1: return "expm1f(a)";
    case TTLB_OP_LOGP1: return "log1pf(a)";
    case TTLB_OP_SQUARE: return "a * a";
    case TTLB_OP_RECIP: return "1.0f / a";
    case TTLB_OP_TAN: return "tanf(a)";
    case TTLB_OP_ATAN: return "atanf(a)";
    case TTLB_OP_ATANH: return "atanhf(a)";
    case TTLB_OP_SIN: return "sinf(a)";
    case TTLB_OP_ASIN: return "asinf(a)";
    case TTLB_OP_ASINH: return "asinhf(a)";
    case TTLB_OP_COS: return "cosf(a)";
    case TTLB_OP_ACOS: return "acosf(a)";
    case TTLB_OP_ACOSH: return "acoshf(a)";
    case TTLB_OP_GELU: return "0.5f * a * (1.0f + erff(a * 0.70710678118654752f))";
    case TTLB_OP_SILU: return "a / (1.0f + expf(-a))";
    case TTLB_OP_SOFTSIGN: return "a / (1.0f + fabsf(a))";
    case TTLB_OP_HARDSIGMOID: return "fminf(fmaxf(a * (1.0f / 6.0f) + 0.5f, 0.0f), 1.0f)";
    // with scalar parameters P0.. (entries of p.imm starting at the instruction's arg)
    case TTLB_OP_RSUB_IMM: return "P0 - a";
    case TTLB_OP_RELU_MAX: return "fmaxf(nan_min(a, P0), 0.0f)";
    case TTLB_OP_RELU_MIN: return "fmaxf(nan_max(a, P0), 0.0f)";
    case TTLB_OP_LEAKY_RELU: return "(a >= 0.0f ? a : a * P0)";
    case TTLB_OP_ELU: return "(a > 0.0f ? a : P0 * expm1f(a))";
    case TTLB_OP_CELU: return "(fmaxf(a, 0.0f) + fminf(0.0f, P0 * expm1f(a * P1)))";
    case TTLB_OP_SOFTPLUS: return "(a * P0 > P2 ? a : log1pf(expf(a * P0)) * P1)";
    case TTLB_OP_HARDTANH: return "fminf(fmaxf(a, P0), P1)";
    case TTLB_OP_SELU: return "P0 * (a > 0.0f ? a : P1 * expm1f(a))";
    case TTLB_OP_POW_IMM: return "pow_imm(a, P0)";
  }
  return nullptr;
}

// `var` is the register the 16-byte vector lands in, `gi` the name of the row index.
void emit_load(std::ostringstream &s, const ttlb_eltwise_desc *d, int k, bool bf16, const char *indent,
               const std::string &var, const std::string &gi, const std::string &gj = "gj") {
  const ttlb_operand &o = d->in[k];
  const int esz = bf16 ? 2 : 4;
  const std::string ks = std::to_string(k);
  std::string row = o.row_mode == TTLB_IDX_SAME    ? "(" + gi + " + p.roff[" + ks + "])"
                    : o.row_mode == TTLB_IDX_ZERO  ? "p.roff[" + ks + "]"
                    : o.row_mode == TTLB_IDX_FIRST ? "(p.roff[" + ks + "] + (" + gi + " & ~31LL))"
                                                   : "(p.roff[" + ks + "] + (" + gi + " & 31))";
  s << indent << "{ const char* rp = (const char*)p.in[" << k << "] + " << row << " * p.ld[" << k << "] * " << esz
    << ";\n";
  if (o.col_mode == TTLB_IDX_ZERO || o.col_mode == TTLB_IDX_FIRST) {   // one element for the whole vector
    const std::string ec = o.col_mode == TTLB_IDX_ZERO ? "p.coff[" + ks + "]" : "(p.coff[" + ks + "] + (" + gj + " & ~31LL))";
    s << indent << "  rp += " << ec << " * " << esz << ";\n";
    if (bf16)
      s << indent << "  u32 h = *(const unsigned short*)rp; h |= h << 16; " << var << " = make_uint4(h, h, h, h); }\n";
    else
      s << indent << "  u32 w = *(const u32*)rp; " << var << " = make_uint4(w, w, w, w); }\n";
    return;
  }
  std::string col = o.col_mode == TTLB_IDX_SAME ? "(" + gj + " + p.coff[" + ks + "])"
                                                : "(p.coff[" + ks + "] + (" + gj + " & 31))";
  const bool stream = o.row_mode == TTLB_IDX_SAME && o.col_mode == TTLB_IDX_SAME;
  s << indent << "  " << var << " = " << (stream ? "ld_stream" : "ld_cached") << "(rp + " << col << " * " << esz
    << "); }\n";
}

void emit_unpack(std::ostringstream &s, const std::string &var, const char *dst, bool bf16) {
  static const char *comp[4] = {"x", "y", "z", "w"};
  for (int q = 0; q < 4; ++q) {
    if (bf16) {
      s << "        " << dst << "[" << 2 * q << "] = __uint_as_float(" << var << "." << comp[q] << " << 16); " << dst
        << "[" << 2 * q + 1 << "] = __uint_as_float(" << var << "." << comp[q] << " & 0xffff0000u);\n";
    } else {
      s << "        " << dst << "[" << q << "] = __uint_as_float(" << var << "." << comp[q] << ");\n";
    }
  }
}

// The op sequence of the program as straight-line code: leaves the value of the V elements of one
// 16-byte vector in `acc[V]`.  `var(k)` names the register holding operand k's vector.
template <class VarFn>
void emit_ops(std::ostringstream &s, const ttlb_eltwise_desc *d, VarFn var, bool bf16, bool rnd,
              const std::string &imm = "p.imm", int start_pc = 0, const std::string &start_from = "") {
  s << "      float acc[V], x[V], stk0[V], stk1[V];\n"
       "      (void)x; (void)stk0; (void)stk1;\n";
  if (start_pc > 0)   // the first start_pc ops were evaluated by an earlier stage: continue from its values
    s << "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) acc[e] = " << start_from << "[e];\n";
  int depth = 0;
  for (int pc = start_pc; pc < d->n_ops; ++pc) {
    const int op = d->ops[pc].opcode, arg = d->ops[pc].arg;
    s << "      {  // op " << pc << "\n";
    if (op == TTLB_OP_LOAD) {
      emit_unpack(s, var(arg), "acc", bf16);
    } else if (op == TTLB_OP_PUSH) {
      s << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) stk" << depth << "[e] = acc[e];\n";
      ++depth;
    } else if (const char *be = binary_expr(op)) {
      if (arg >= 0) {
        emit_unpack(s, var(arg), "x", bf16);
      } else {
        --depth;
        s << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) x[e] = stk" << depth << "[e];\n";
      }
      s << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) { const float a = acc[e], b = x[e]; acc[e] = "
        << be << "; }\n";
    } else if (const char *ue = unary_expr(op)) {
      if (op >= TTLB_OP_RSUB_IMM)
        s << "        const float P0 = " << imm << "[" << arg << "], P1 = " << imm << "[" << (arg + 1 < TTLB_MAX_IMM ? arg + 1 : arg)
          << "], P2 = " << imm << "[" << (arg + 2 < TTLB_MAX_IMM ? arg + 2 : arg) << "]; (void)P1; (void)P2;\n";
      s << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) { const float a = acc[e]; acc[e] = " << ue
        << "; }\n";
    }
    if (rnd && op != TTLB_OP_LOAD && op != TTLB_OP_PUSH) {
      s << "        _Pragma(\"unroll\") for (int e = 0; e < V; e += 2) { const u32 w = pack_bf16x2(acc[e], acc[e + 1]); "
           "acc[e] = __uint_as_float(w << 16); acc[e + 1] = __uint_as_float(w & 0xffff0000u); }\n";
    }
    s << "      }\n";
  }
}

// Rows handled per loop iteration: all their loads are issued before any arithmetic, so a
// thread keeps U x (streaming operands) 16-byte loads in flight.  Bounded by registers.
int rows_per_iteration(const ttlb_eltwise_desc *d) {
  // operands that cost a 16-byte load per row; one element per row (a column vector) is a 2- or 4-byte load
  int streaming = 0;
  for (int k = 0; k < d->n_in; ++k)
    if (d->in[k].row_mode != TTLB_IDX_ZERO && (d->in[k].col_mode == TTLB_IDX_SAME || d->in[k].col_mode == TTLB_IDX_TILE))
      ++streaming;
  if (const char *e = getenv("TTLB200_ELTWISE_ROWS")) {   // tuning knob: rows in flight per thread
    const int v = atoi(e);
    if (v >= 1 && v <= 8) return v;
  }
  int u = 8 / (streaming > 0 ? streaming : 1);
  return u < 1 ? 1 : u > 4 ? 4 : u;
}

}  // namespace

std::string ttlb_eltwise_jit_key(const ttlb_eltwise_desc *d) {
  std::ostringstream k;
  k << d->dtype << ':' << (d->round_each_op ? 1 : 0) << ':' << d->n_in << ':';
  for (int i = 0; i < d->n_in; ++i) k << d->in[i].row_mode << d->in[i].col_mode << ',';
  k << ':';
  for (int i = 0; i < d->n_ops; ++i) k << d->ops[i].opcode << '/' << d->ops[i].arg << ',';
  return k.str();
}

std::string ttlb_eltwise_jit_source(const ttlb_eltwise_desc *d) {
  const bool bf16 = d->dtype == TTLB_BF16;
  const int V = bf16 ? 8 : 4;
  const bool rnd = bf16 && d->round_each_op;
  std::ostringstream s;
  {
    // tuning knobs: cache operators of the streaming load / store (defaults: evict-first both ways)
    std::string pre = kPrelude;
    const char *ld = getenv("TTLB200_ELTWISE_LD"), *st = getenv("TTLB200_ELTWISE_ST");
    auto swap = [&](const std::string &from, const std::string &to) {
      const size_t at = pre.find(from);
      if (at != std::string::npos) pre.replace(at, from.size(), to);
    };
    if (ld && *ld) swap("ld.global.cs.v4.u32", std::string("ld.global.") + ld + ".v4.u32");
    if (st && *st) swap("st.global.cs.v4.u32", std::string(st) == "default" ? "st.global.v4.u32" : std::string("st.global.") + st + ".v4.u32");
    s << (rnd ? "#define RB(x) rb_bf16(x)\n" : "#define RB(x) (x)\n") << pre;
  }
  s << "#define V " << V << "\n";
  int min_ctas = 0;   // tuning knob: ask the compiler to fit this many CTAs per SM
  if (const char *e = getenv("TTLB200_ELTWISE_MIN_CTAS")) min_ctas = atoi(e);
  s << "extern \"C\" __global__ void __launch_bounds__(256" << (min_ctas > 0 ? ", " + std::to_string(min_ctas) : std::string())
    << ") ttlb_eltwise_jit(const __grid_constant__ JitParams p) {\n"
       "  const u32 tx = threadIdx.x & ((1u << p.bx_log2) - 1u), ty = threadIdx.x >> p.bx_log2;\n"
       "  const u32 by = 256u >> p.bx_log2;\n"
       "  const u32 cv = (blockIdx.x << p.bx_log2) + tx;\n"
       "  if (cv >= p.vpr) return;\n"
       "  const i64 gj = p.col0 + (i64)cv * V;\n";
  const int U = rows_per_iteration(d);
  auto var = [&](int k, int u) {
    return d->in[k].row_mode == TTLB_IDX_ZERO ? "v" + std::to_string(k) : "v" + std::to_string(k) + "_" + std::to_string(u);
  };
  // row-invariant operands: fetched once
  for (int k = 0; k < d->n_in; ++k)
    if (d->in[k].row_mode == TTLB_IDX_ZERO) {
      s << "  uint4 v" << k << ";\n";
      emit_load(s, d, k, bf16, "  ", "v" + std::to_string(k), "0");
    }
  s << "  const u32 rstride = gridDim.y * by;\n"
       "  for (u32 r = blockIdx.y * by + ty; r < p.rows; r += rstride * " << U << ") {\n";
  for (int u = 0; u < U; ++u) {
    s << "    const i64 gi" << u << " = p.row0 + (i64)r + (i64)rstride * " << u << ";\n";
    if (u) s << "    const bool ok" << u << " = r + rstride * " << u << " < p.rows;\n";
  }
  for (int u = 0; u < U; ++u)
    for (int k = 0; k < d->n_in; ++k)
      if (d->in[k].row_mode != TTLB_IDX_ZERO) {
        s << "    uint4 " << var(k, u) << " = make_uint4(0, 0, 0, 0);\n";
        if (u) s << "    if (ok" << u << ")\n";
        emit_load(s, d, k, bf16, "    ", var(k, u), "gi" + std::to_string(u));
      }
  for (int u = 0; u < U; ++u) {
    s << "    " << (u ? "if (ok" + std::to_string(u) + ") " : "") << "{  // row " << u << "\n";
    emit_ops(s, d, [&](int k) { return var(k, u); }, bf16, rnd);
    s << "      uint4 o;\n";
    if (bf16) {
      s << "      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);\n"
           "      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);\n";
    } else {
      s << "      o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]);\n"
           "      o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]);\n";
    }
    s << "      st_stream((char*)p.out + (gi" << u << " * p.out_ld + gj) * " << (bf16 ? 2 : 4) << ", o);\n";
    s << "    }\n";
  }
  s << "  }\n}\n";
  return s.str();
}

bool ttlb_eltwise_jit_available() { return nvrtc().ok; }

struct JitKernel {
  cudaKernel_t kern;
  int blocks_per_sm;  // resident 256-thread CTAs per SM
};

struct ttlb_jit_cache {
  std::map<std::string, JitKernel> kernels;
  std::vector<cudaLibrary_t> libs;
};

void ttlb_jit_cache_destroy(ttlb_jit_cache *c) {
  if (!c) return;
  for (cudaLibrary_t l : c->libs) cudaLibraryUnload(l);
  delete c;
}

// Compiles `src` (entry point `name`) for sm_100a unless `key` is already in the cache.
static int get_kernel(ttlb_ctx *ctx, ttlb_jit_cache **cachep, const std::string &key, const std::string &src,
                      const char *name, JitKernel *out, int threads = 256) {
  Nvrtc &n = nvrtc();
  if (!n.ok) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "%s: NVRTC (libnvrtc.so.12) is not available", name);
  if (!*cachep) *cachep = new ttlb_jit_cache();
  ttlb_jit_cache *cache = *cachep;
  auto it = cache->kernels.find(key);
  if (it != cache->kernels.end()) {
    *out = it->second;
    return TTLB_OK;
  }
  nvrtcProgram prog;
  if (n.CreateProgram(&prog, src.c_str(), "ttlb_jit.cu", 0, nullptr, nullptr) != 0)
    return ttlb_fail(ctx, TTLB_ERR_CUDA, "%s: nvrtcCreateProgram failed", name);
  const char *opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "-lineinfo", "--std=c++17"};
  const int rc = n.CompileProgram(prog, 4, opts);
  if (rc != 0) {
    size_t ls = 0;
    n.GetProgramLogSize(prog, &ls);
    std::string log(ls, '\0');
    if (ls) n.GetProgramLog(prog, log.data());
    n.DestroyProgram(&prog);
    return ttlb_fail(ctx, TTLB_ERR_CUDA, "%s: NVRTC compile failed: %.400s", name, log.c_str());
  }
  size_t cs = 0;
  n.GetCUBINSize(prog, &cs);
  std::vector<char> cubin(cs);
  n.GetCUBIN(prog, cubin.data());
  n.DestroyProgram(&prog);
  cudaLibrary_t lib;
  TTLB_CUDA_CHECK(ctx, cudaLibraryLoadData(&lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  cudaKernel_t kern;
  cudaError_t e = cudaLibraryGetKernel(&kern, lib, name);
  if (e != cudaSuccess) {
    cudaLibraryUnload(lib);
    return ttlb_fail(ctx, TTLB_ERR_CUDA, "%s: cudaLibraryGetKernel failed: %s", name, cudaGetErrorString(e));
  }
  cache->libs.push_back(lib);
  JitKernel jk;
  jk.kern = kern;
  jk.blocks_per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&jk.blocks_per_sm, reinterpret_cast<const void *>(kern), threads, 0) !=
          cudaSuccess ||
      jk.blocks_per_sm < 1) {
    cudaGetLastError();
    jk.blocks_per_sm = 4;
  }
  cache->kernels[key] = jk;
  *out = jk;
  return TTLB_OK;
}

// Returns TTLB_OK and launches, or an error (the caller may then use the interpreter).
int ttlb_eltwise_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cachep, const ttlb_eltwise_desc *d, cudaStream_t stream) {
  JitKernel jk;
  {
    const std::string key = ttlb_eltwise_jit_key(d);
    const bool cached = *cachep && (*cachep)->kernels.count(key);
    const int rc = get_kernel(ctx, cachep, key, cached ? std::string() : ttlb_eltwise_jit_source(d), "ttlb_eltwise_jit", &jk);
    if (rc != TTLB_OK) return rc;
  }

  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  JitParams p{};
  for (int k = 0; k < d->n_in; ++k) {
    p.in[k] = d->in[k].ptr;
    p.ld[k] = d->in[k].ld;
    p.roff[k] = d->in[k].row_off;
    p.coff[k] = d->in[k].col_off;
  }
  p.out = d->out;
  p.out_ld = d->out_ld;
  p.row0 = d->row0;
  p.col0 = d->col0;
  p.vpr = (unsigned)(d->cols / vec);
  p.rows = (unsigned)d->rows;
  for (int k = 0; k < TTLB_MAX_IMM; ++k) p.imm[k] = d->imm[k];
  unsigned bx_log2 = 0;
  while (bx_log2 < 8 && (1u << bx_log2) < p.vpr) ++bx_log2;
  p.bx_log2 = bx_log2;
  const unsigned bx = 1u << bx_log2, by = 256u / bx;
  const unsigned gx = (p.vpr + bx - 1) / bx;
  const unsigned row_blocks = (p.rows + by - 1) / by;
  // exactly one wave of resident CTAs: no tail wave at reduced occupancy
  unsigned gy = (unsigned)(ctx->sm_count * jk.blocks_per_sm) / (gx ? gx : 1);
  if (gy < 1) gy = 1;
  if (gy > row_blocks) gy = row_blocks;
  if (gy > 65535u) gy = 65535u;
  void *args[] = {&p};
  TTLB_CUDA_CHECK(ctx, cudaLaunchKernel(reinterpret_cast<const void *>(jk.kern), dim3(gx, gy, 1), dim3(256, 1, 1), args, 0,
                                        stream));
  return TTLB_OK;
}

// --------------------------------------------------------------------------- //
// Reductions (ttlb_reduce): the same per-program specialisation, with the store
// replaced by a running sum / maximum.
//
// Over rows (ROWS, ROWS|COLS): the element-wise geometry - a thread owns one 16-byte
// column vector and walks rows - with V running values per thread.  A CTA combines its
// threads' values through shared memory, writes one partial row to scratch, and the
// last CTA of a column group to finish (a counter in scratch) combines the partial rows
// in index order, scales, rounds and stores: one launch, fixed summation order.
// Over columns only (COLS): one warp per row, lanes stride over the row's 16-byte
// vectors with several loads in flight, then a butterfly of shuffles.
// --------------------------------------------------------------------------- //
namespace {

struct RedParams {
  JitParams p;
  const void *scaler;
  void *out;
  long long out_ld;
  float *partial;     // [gridDim.y][ncols]
  float *partial2;    // [gridDim.x]
  unsigned *counter;  // [gridDim.x] arrivals per column group, zero between launches
  unsigned *counter2; // arrivals of column groups (ROWS|COLS), zero between launches
  unsigned fill_rows, fill_cols, ncols, pad;
};

const char *kRedPrelude = R"SRC(
struct RedParams {
  JitParams p; const void* scaler; void* out; i64 out_ld;
  float* partial; float* partial2; u32* counter; u32* counter2;
  u32 fill_rows, fill_cols, ncols, pad;
};
)SRC";

int cols_in_flight(const ttlb_eltwise_desc *d) {
  int streaming = 0;
  for (int k = 0; k < d->n_in; ++k)
    if (d->in[k].col_mode == TTLB_IDX_SAME || d->in[k].col_mode == TTLB_IDX_TILE) ++streaming;
  int u = 8 / (streaming > 0 ? streaming : 1);
  return u < 1 ? 1 : u > 4 ? 4 : u;
}

}  // namespace

std::string ttlb_reduce_jit_key(const ttlb_reduce_desc *r) {
  std::ostringstream k;
  k << "red" << r->op << '/' << r->dims << ':' << ttlb_eltwise_jit_key(&r->src);
  return k.str();
}

std::string ttlb_reduce_jit_source(const ttlb_reduce_desc *r) {
  const ttlb_eltwise_desc *d = &r->src;
  const bool bf16 = d->dtype == TTLB_BF16;
  const int V = bf16 ? 8 : 4;
  const bool rnd = bf16 && d->round_each_op;
  const bool is_max = r->op == TTLB_REDUCE_MAX;
  const char *init = is_max ? "__uint_as_float(0xff800000u)" : "0.0f";
  std::ostringstream s;
  s << (rnd ? "#define RB(x) rb_bf16(x)\n" : "#define RB(x) (x)\n") << kPrelude << kRedPrelude;
  s << "#define V " << V << "\n#define ESZ " << (bf16 ? 2 : 4) << "\n";
  s << "#define COMB(a, b) " << (is_max ? "nan_max((a), (b))" : "((a) + (b))") << "\n";
  if (bf16)
    s << "__device__ __forceinline__ float ld_elem(const void* q) { return __uint_as_float(((u32)*(const unsigned short*)q) << 16); }\n"
         "__device__ __forceinline__ void st_elem(void* base, i64 idx, float x) { ((unsigned short*)base)[idx] = "
         "(unsigned short)(pack_bf16x2(x, 0.0f) & 0xffffu); }\n";
  else
    s << "__device__ __forceinline__ float ld_elem(const void* q) { return *(const float*)q; }\n"
         "__device__ __forceinline__ void st_elem(void* base, i64 idx, float x) { ((float*)base)[idx] = x; }\n";
  s << "extern \"C\" __global__ void __launch_bounds__(256) ttlb_reduce_jit(const __grid_constant__ RedParams q) {\n"
       "  const JitParams& p = q.p;\n"
       "  const float sc = q.scaler ? ld_elem(q.scaler) : 1.0f;\n";

  if (r->dims == TTLB_REDUCE_COLS) {
    const int U = cols_in_flight(d);
    auto var = [&](int k, int u) { return "v" + std::to_string(k) + "_" + std::to_string(u); };
    s << "  const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;\n"
         "  for (u32 r = blockIdx.x * 8u + warp; r < p.rows; r += gridDim.x * 8u) {\n"
         "    const i64 gi = p.row0 + (i64)r;\n"
         "    float racc = " << init << ";\n"
         "    for (u32 c = lane; c < p.vpr; c += 32u * " << U << ") {\n";
    for (int u = 0; u < U; ++u) {
      s << "      const i64 gj" << u << " = p.col0 + (i64)(c + 32u * " << u << ") * V;\n";
      if (u) s << "      const bool ok" << u << " = c + 32u * " << u << " < p.vpr;\n";
    }
    for (int u = 0; u < U; ++u)
      for (int k = 0; k < d->n_in; ++k) {
        s << "      uint4 " << var(k, u) << " = make_uint4(0, 0, 0, 0);\n";
        if (u) s << "      if (ok" << u << ")\n";
        emit_load(s, d, k, bf16, "      ", var(k, u), "gi", "gj" + std::to_string(u));
      }
    for (int u = 0; u < U; ++u) {
      s << "      " << (u ? "if (ok" + std::to_string(u) + ") " : "") << "{\n";
      emit_ops(s, d, [&](int k) { return var(k, u); }, bf16, rnd);
      s << "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) racc = COMB(racc, acc[e]);\n"
           "      }\n";
    }
    s << "    }\n"
         "    _Pragma(\"unroll\") for (int o = 16; o; o >>= 1) { const float y = __shfl_xor_sync(0xffffffffu, racc, o); "
         "racc = COMB(racc, y); }\n"
         "    if (lane < q.fill_cols) st_elem(q.out, (i64)r * q.out_ld + lane, lane == 0 ? racc * sc : 0.0f);\n"
         "  }\n}\n";
    return s.str();
  }

  // ---- over rows (and optionally columns) --------------------------------
  const int U = rows_per_iteration(d);
  auto var = [&](int k, int u) {
    return d->in[k].row_mode == TTLB_IDX_ZERO ? "v" + std::to_string(k) : "v" + std::to_string(k) + "_" + std::to_string(u);
  };
  s << "  __shared__ float sm[256 * V];\n"
       "  __shared__ u32 s_last;\n"
       "  const u32 bx = 1u << p.bx_log2, tx = threadIdx.x & (bx - 1u), ty = threadIdx.x >> p.bx_log2;\n"
       "  const u32 by = 256u >> p.bx_log2;\n"
       "  const u32 cv = (blockIdx.x << p.bx_log2) + tx;\n"
       "  const bool colok = cv < p.vpr;\n"
       "  const i64 gj = p.col0 + (i64)cv * V;\n"
       "  float racc[V];\n"
       "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) racc[e] = " << init << ";\n"
       "  if (colok) {\n";
  for (int k = 0; k < d->n_in; ++k)
    if (d->in[k].row_mode == TTLB_IDX_ZERO) {
      s << "  uint4 v" << k << ";\n";
      emit_load(s, d, k, bf16, "  ", "v" + std::to_string(k), "0");
    }
  s << "  const u32 rstride = gridDim.y * by;\n"
       "  for (u32 r = blockIdx.y * by + ty; r < p.rows; r += rstride * " << U << ") {\n";
  for (int u = 0; u < U; ++u) {
    s << "    const i64 gi" << u << " = p.row0 + (i64)r + (i64)rstride * " << u << ";\n";
    if (u) s << "    const bool ok" << u << " = r + rstride * " << u << " < p.rows;\n";
  }
  for (int u = 0; u < U; ++u)
    for (int k = 0; k < d->n_in; ++k)
      if (d->in[k].row_mode != TTLB_IDX_ZERO) {
        s << "    uint4 " << var(k, u) << " = make_uint4(0, 0, 0, 0);\n";
        if (u) s << "    if (ok" << u << ")\n";
        emit_load(s, d, k, bf16, "    ", var(k, u), "gi" + std::to_string(u));
      }
  for (int u = 0; u < U; ++u) {
    s << "    " << (u ? "if (ok" + std::to_string(u) + ") " : "") << "{  // row " << u << "\n";
    emit_ops(s, d, [&](int k) { return var(k, u); }, bf16, rnd);
    s << "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) racc[e] = COMB(racc[e], acc[e]);\n"
         "    }\n";
  }
  s << "  }\n  }\n";
  // CTA-level combine over ty (in index order), one partial row per CTA
  s << "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) sm[(ty * bx + tx) * V + e] = racc[e];\n"
       "  __syncthreads();\n"
       "  if (ty == 0) {\n"
       "    for (u32 t = 1; t < by; ++t)\n"
       "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) racc[e] = COMB(racc[e], sm[(t * bx + tx) * V + e]);\n"
       "    if (colok) {\n"
       "      float4* dst = (float4*)(q.partial + (size_t)blockIdx.y * q.ncols + (size_t)cv * V);\n"
       "      _Pragma(\"unroll\") for (int e = 0; e < V; e += 4) dst[e >> 2] = make_float4(racc[e], racc[e + 1], racc[e + 2], racc[e + 3]);\n"
       "    }\n"
       "  }\n"
       "  __threadfence();\n"
       "  __syncthreads();\n"
       "  if (threadIdx.x == 0) s_last = (atomicAdd(&q.counter[blockIdx.x], 1u) == gridDim.y - 1u) ? 1u : 0u;\n"
       "  __syncthreads();\n"
       "  if (!s_last) return;\n"
       "  __threadfence();\n"
       "  float tot[V];\n"
       "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) tot[e] = " << init << ";\n"
       "  if (colok) {\n"   // the CTA's `by` thread rows share the partial rows, then combine in thread-row order
       "    for (u32 g = ty; g < gridDim.y; g += by) {\n"
       "      const float4* src = (const float4*)(q.partial + (size_t)g * q.ncols + (size_t)cv * V);\n"
       "      _Pragma(\"unroll\") for (int e = 0; e < V; e += 4) { const float4 f = __ldcg(src + (e >> 2)); "
       "tot[e] = COMB(tot[e], f.x); tot[e + 1] = COMB(tot[e + 1], f.y); tot[e + 2] = COMB(tot[e + 2], f.z); "
       "tot[e + 3] = COMB(tot[e + 3], f.w); }\n"
       "    }\n"
       "  }\n"
       "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) sm[(ty * bx + tx) * V + e] = tot[e];\n"
       "  __syncthreads();\n"
       "  if (ty == 0)\n"
       "    for (u32 t = 1; t < by; ++t)\n"
       "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) tot[e] = COMB(tot[e], sm[(t * bx + tx) * V + e]);\n";
  if (r->dims == TTLB_REDUCE_ROWS) {
    s << "  if (ty == 0 && colok) {\n"
         "    uint4 o, z = make_uint4(0, 0, 0, 0);\n"
         "    _Pragma(\"unroll\") for (int e = 0; e < V; ++e) tot[e] = tot[e] * sc;\n";
    if (bf16)
      s << "    o.x = pack_bf16x2(tot[0], tot[1]); o.y = pack_bf16x2(tot[2], tot[3]);\n"
           "    o.z = pack_bf16x2(tot[4], tot[5]); o.w = pack_bf16x2(tot[6], tot[7]);\n";
    else
      s << "    o.x = __float_as_uint(tot[0]); o.y = __float_as_uint(tot[1]);\n"
           "    o.z = __float_as_uint(tot[2]); o.w = __float_as_uint(tot[3]);\n";
    s << "    *(uint4*)((char*)q.out + (i64)cv * V * ESZ) = o;\n"
         "    for (u32 rr = 1; rr < q.fill_rows; ++rr) *(uint4*)((char*)q.out + ((i64)rr * q.out_ld + (i64)cv * V) * ESZ) = z;\n"
         "  }\n"
         "  if (threadIdx.x == 0) q.counter[blockIdx.x] = 0u;\n"
         "}\n";
    return s.str();
  }
  // ROWS | COLS: fold the column group, then the column groups
  s << "  float t = " << init << ";\n"
       "  if (ty == 0 && colok) { _Pragma(\"unroll\") for (int e = 0; e < V; ++e) t = COMB(t, tot[e]); }\n"
       "  __syncthreads();\n"
       "  if (ty == 0) sm[tx] = t;\n"
       "  __syncthreads();\n"
       "  if (threadIdx.x == 0) {\n"
       "    float c = sm[0];\n"
       "    for (u32 i = 1; i < bx; ++i) c = COMB(c, sm[i]);\n"
       "    q.partial2[blockIdx.x] = c;\n"
       "    q.counter[blockIdx.x] = 0u;\n"
       "    __threadfence();\n"
       "    if (atomicAdd(q.counter2, 1u) == gridDim.x - 1u) {\n"
       "      __threadfence();\n"
       "      float res = " << init << ";\n"
       "      for (u32 g = 0; g < gridDim.x; ++g) res = COMB(res, __ldcg(q.partial2 + g));\n"
       "      for (u32 rr = 0; rr < q.fill_rows; ++rr)\n"
       "        for (u32 cc = 0; cc < q.fill_cols; ++cc) st_elem(q.out, (i64)rr * q.out_ld + cc, (rr | cc) ? 0.0f : res * sc);\n"
       "      *q.counter2 = 0u;\n"
       "    }\n"
       "  }\n"
       "}\n";
  return s.str();
}

int ttlb_reduce_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cachep, const ttlb_reduce_desc *r, float *partial,
                           size_t partial_floats, float *partial2, unsigned *counters, unsigned max_groups,
                           cudaStream_t stream) {
  const ttlb_eltwise_desc *d = &r->src;
  JitKernel jk;
  {
    const std::string key = ttlb_reduce_jit_key(r);
    const bool cached = *cachep && (*cachep)->kernels.count(key);
    const int rc = get_kernel(ctx, cachep, key, cached ? std::string() : ttlb_reduce_jit_source(r), "ttlb_reduce_jit", &jk);
    if (rc != TTLB_OK) return rc;
  }
  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  RedParams q{};
  JitParams &p = q.p;
  for (int k = 0; k < d->n_in; ++k) {
    p.in[k] = d->in[k].ptr;
    p.ld[k] = d->in[k].ld;
    p.roff[k] = d->in[k].row_off;
    p.coff[k] = d->in[k].col_off;
  }
  p.row0 = d->row0;
  p.col0 = d->col0;
  p.vpr = (unsigned)(d->cols / vec);
  p.rows = (unsigned)d->rows;
  for (int k = 0; k < TTLB_MAX_IMM; ++k) p.imm[k] = d->imm[k];
  q.scaler = r->scaler;
  q.out = r->out;
  q.out_ld = r->out_ld;
  q.fill_rows = (unsigned)r->fill_rows;
  q.fill_cols = (unsigned)r->fill_cols;
  q.ncols = (unsigned)d->cols;
  const unsigned resident = (unsigned)(ctx->sm_count * jk.blocks_per_sm);
  void *args[] = {&q};
  if (r->dims == TTLB_REDUCE_COLS) {
    unsigned gx = (p.rows + 7u) / 8u;
    if (gx > resident) gx = resident;
    TTLB_CUDA_CHECK(ctx, cudaLaunchKernel(reinterpret_cast<const void *>(jk.kern), dim3(gx, 1, 1), dim3(256, 1, 1), args,
                                          0, stream));
    return TTLB_OK;
  }
  // One warp wide (32 vectors = 512 contiguous bytes per row), 8 thread rows: the CTA folds 8 rows in
  // shared memory before it writes a partial row, and a column group is 256 columns, so that there are
  // few partial rows and many groups to finish them in parallel.
  unsigned bx_log2 = 0;
  while (bx_log2 < 5 && (1u << bx_log2) < p.vpr) ++bx_log2;
  p.bx_log2 = bx_log2;
  const unsigned bx = 1u << bx_log2, by = 256u / bx;
  const unsigned gx = (p.vpr + bx - 1) / bx;
  if (gx > max_groups) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "reduce: %lld columns are too many", (long long)d->cols);
  const unsigned row_blocks = (p.rows + by - 1) / by;
  unsigned gy = resident / gx;
  const size_t fit = partial_floats / (size_t)d->cols;  // partial rows the scratch holds
  if (fit < 1) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "reduce: %lld columns are too many", (long long)d->cols);
  if (gy > fit) gy = (unsigned)fit;
  if (gy > row_blocks) gy = row_blocks;
  if (gy < 1) gy = 1;
  if (gy > 65535u) gy = 65535u;
  q.partial = partial;
  q.partial2 = partial2;
  q.counter = counters;
  q.counter2 = counters + max_groups;
  TTLB_CUDA_CHECK(ctx, cudaLaunchKernel(reinterpret_cast<const void *>(jk.kern), dim3(gx, gy, 1), dim3(256, 1, 1), args, 0,
                                        stream));
  return TTLB_OK;
}

// --------------------------------------------------------------------------- //
// Row-resident fusion (ttlb_rowfused): reductions over columns, then an element-wise
// program, over the same rows in one kernel.  A CTA of 256 threads owns a row at a
// time: thread t holds the 16-byte vectors t, t+256, ... of every operand in registers
// (all loads of a row are issued before any arithmetic), each reduction is folded per
// thread, by shuffles per warp and through shared memory per CTA in a fixed order, its
// scaled and rounded result is broadcast to the threads as the operand of the next
// stage, and the final program is evaluated from the same registers and stored.
// --------------------------------------------------------------------------- //
namespace {

struct RowParams {
  JitParams p;  // the distinct memory operands of all stages; out / out_ld: the final output
  const void *scaler[TTLB_MAX_PHASES];
  void *red_out[TTLB_MAX_PHASES];
  long long red_ld[TTLB_MAX_PHASES];
  unsigned red_fill[TTLB_MAX_PHASES];
  unsigned pad;
  float imm[TTLB_MAX_PHASES + 1][TTLB_MAX_IMM];
};

const char *kRowPrelude = R"SRC(
struct RowParams {
  JitParams p; const void* scaler[3]; void* red_out[3]; i64 red_ld[3]; u32 red_fill[3]; u32 pad; float imm[4][8];
};
)SRC";

// The distinct memory operands of all stages, and for every (stage, operand) where it lives.
struct RowLayout {
  ttlb_eltwise_desc g;                               // g.in[0 .. g.n_in): the distinct operands
  int where[TTLB_MAX_PHASES + 1][TTLB_MAX_IN];       // >= 0: index into g.in; < 0: result of phase -(v + 1)
  bool ok = true;
};

RowLayout row_layout(const ttlb_rowfused_desc *f) {
  RowLayout L;
  L.g = f->final;
  L.g.n_in = 0;
  for (int st = 0; st <= f->n_phases; ++st) {
    const ttlb_eltwise_desc *d = st < f->n_phases ? &f->phase[st].src : &f->final;
    for (int k = 0; k < d->n_in; ++k) {
      const ttlb_operand &o = d->in[k];
      if (o.row_mode == TTLB_IDX_PHASE) {
        L.where[st][k] = -(int)o.row_off - 1;
        continue;
      }
      int found = -1;
      for (int n = 0; n < L.g.n_in; ++n) {
        const ttlb_operand &x = L.g.in[n];
        if (x.ptr == o.ptr && x.ld == o.ld && x.row_mode == o.row_mode && x.col_mode == o.col_mode &&
            x.row_off == o.row_off && x.col_off == o.col_off)
          found = n;
      }
      if (found < 0) {
        if (L.g.n_in == TTLB_MAX_IN) {
          L.ok = false;
          return L;
        }
        found = L.g.n_in++;
        L.g.in[found] = o;
      }
      L.where[st][k] = found;
    }
  }
  return L;
}

bool per_vector(const ttlb_operand &o) { return o.col_mode != TTLB_IDX_ZERO; }

bool takes_operand(int op) { return op <= TTLB_OP_RPOW; }   // LOAD and the binary ops name an input (or the stack)
int n_imm(int op) {
  switch (op) {
    case TTLB_OP_RSUB_IMM: case TTLB_OP_RELU_MAX: case TTLB_OP_RELU_MIN: case TTLB_OP_LEAKY_RELU: case TTLB_OP_ELU:
    case TTLB_OP_POW_IMM: return 1;
    case TTLB_OP_CELU: case TTLB_OP_HARDTANH: case TTLB_OP_SELU: return 2;
    case TTLB_OP_SOFTPLUS: return 3;
  }
  return 0;
}

// Stage `st` may continue from the values reduction `a` computed when its program starts with the whole
// program of `a` (same ops on the same operands with the same parameters and rounding): exp(x - max) of a
// softmax is then evaluated once.  Returns the reduction to continue from, or -1.
int continue_from(const ttlb_rowfused_desc *f, const RowLayout &L, int st) {
  const ttlb_eltwise_desc *d = st < f->n_phases ? &f->phase[st].src : &f->final;
  int best = -1, best_n = 1;   // continuing from a bare LOAD saves nothing
  for (int a = 0; a < st && a < f->n_phases; ++a) {
    const ttlb_eltwise_desc *e = &f->phase[a].src;
    if (e->n_ops > d->n_ops || e->n_ops <= best_n || (e->round_each_op != 0) != (d->round_each_op != 0)) continue;
    bool same = true;
    for (int pc = 0; pc < e->n_ops && same; ++pc) {
      const int op = e->ops[pc].opcode, arg = e->ops[pc].arg;
      if (op != d->ops[pc].opcode) same = false;
      else if (takes_operand(op)) {
        const int arg2 = d->ops[pc].arg;
        if ((arg < 0) != (arg2 < 0)) same = false;
        else if (arg >= 0 && L.where[a][arg] != L.where[st][arg2]) same = false;
      } else {
        for (int i = 0; i < n_imm(op) && same; ++i)
          if (e->imm[arg + i] != d->imm[d->ops[pc].arg + i]) same = false;
      }
    }
    if (same) {
      best = a;
      best_n = e->n_ops;
    }
  }
  return best;
}

}  // namespace

static int rowfused_threads(const ttlb_rowfused_desc *f);

std::string ttlb_rowfused_jit_key(const ttlb_rowfused_desc *f, const RowLayout &L, int vpt) {
  std::ostringstream k;
  k << "rowf" << vpt << 't' << rowfused_threads(f) << ':' << f->n_phases << ':';
  for (int n = 0; n < L.g.n_in; ++n) k << L.g.in[n].row_mode << L.g.in[n].col_mode << ',';
  for (int st = 0; st <= f->n_phases; ++st) {
    const ttlb_eltwise_desc *d = st < f->n_phases ? &f->phase[st].src : &f->final;
    k << '|';
    if (st < f->n_phases) k << f->phase[st].op << (f->phase[st].out ? 'w' : '-') << (f->phase[st].scaler ? 's' : '-');
    k << d->dtype << (d->round_each_op ? 1 : 0) << 'c' << continue_from(f, L, st) << ':';
    for (int i = 0; i < d->n_in; ++i) k << L.where[st][i] << ',';
    k << ':';
    for (int i = 0; i < d->n_ops; ++i) k << d->ops[i].opcode << '/' << d->ops[i].arg << ',';
  }
  return k.str();
}

// Threads per CTA of the row-resident kernel: 256, or 512 / 1024 for long rows so that a thread holds at most
// two vectors per operand (fewer registers per thread, more resident warps).  TTLB200_ROWFUSED_THREADS overrides.
static int rowfused_threads(const ttlb_rowfused_desc *f) {
  if (const char *e = getenv("TTLB200_ROWFUSED_THREADS")) {
    const int t = atoi(e);
    if (t == 128 || t == 256 || t == 512 || t == 1024) return t;
  }
  const int vec = f->final.dtype == TTLB_BF16 ? 8 : 4;
  const long long vpr = f->final.cols / vec;
  int t = 256;
  while (t < 1024 && vpr > 2LL * t) t *= 2;
  return t;
}
static int rowfused_vpt(const ttlb_rowfused_desc *f) {
  const int vec = f->final.dtype == TTLB_BF16 ? 8 : 4;
  const long long vpr = f->final.cols / vec;
  const int t = rowfused_threads(f);
  return (int)((vpr + t - 1) / t);
}

std::string ttlb_rowfused_jit_source(const ttlb_rowfused_desc *f) {
  const RowLayout L = row_layout(f);
  if (!L.ok) return std::string();
  const bool bf16 = f->final.dtype == TTLB_BF16;
  const int V = bf16 ? 8 : 4;
  const int VPT = rowfused_vpt(f);
  const int T = rowfused_threads(f);
  std::ostringstream s;
  s << (bf16 && f->final.round_each_op ? "#define RB(x) rb_bf16(x)\n" : "#define RB(x) (x)\n") << kPrelude << kRowPrelude;
  s << "#define V " << V << "\n#define ESZ " << (bf16 ? 2 : 4) << "\n";
  if (bf16)
    s << "__device__ __forceinline__ float ld_elem(const void* q) { return __uint_as_float(((u32)*(const unsigned short*)q) << 16); }\n"
         "__device__ __forceinline__ void st_elem(void* base, i64 idx, float x) { ((unsigned short*)base)[idx] = "
         "(unsigned short)(pack_bf16x2(x, 0.0f) & 0xffffu); }\n";
  else
    s << "__device__ __forceinline__ float ld_elem(const void* q) { return *(const float*)q; }\n"
         "__device__ __forceinline__ void st_elem(void* base, i64 idx, float x) { ((float*)base)[idx] = x; }\n";
  // TTLB200_ROWFUSED_MIN_CTAS=n asks the compiler to fit n CTAs per SM (fewer registers, possibly spills)
  int min_ctas = 0;
  if (const char *e = getenv("TTLB200_ROWFUSED_MIN_CTAS")) min_ctas = atoi(e);
  s << "extern \"C\" __global__ void __launch_bounds__(" << T << (min_ctas > 0 ? ", " + std::to_string(min_ctas) : std::string())
    << ") ttlb_rowfused_jit(const __grid_constant__ RowParams q) {\n"
       "  const JitParams& p = q.p;\n"
       "  __shared__ float sm[" << T / 32 << "];\n"
       "  const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;\n";
  for (int j = 0; j < VPT; ++j)
    s << "  const u32 cv" << j << " = threadIdx.x + " << T << "u * " << j << "; const bool ok" << j << " = cv" << j
      << " < p.vpr; const i64 gj" << j << " = p.col0 + (i64)cv" << j << " * V;\n";
  for (int ph = 0; ph < f->n_phases; ++ph)
    s << "  const float sc" << ph << " = q.scaler[" << ph << "] ? ld_elem(q.scaler[" << ph << "]) : 1.0f;\n";
  // Registers g*: the row being worked on; h*: the CTA's next row, whose loads are issued before the
  // arithmetic of the current row starts (a CTA works on one row at a time, so without this its loads and
  // its arithmetic would take turns).
  auto loads = [&](const char *pre, const std::string &gi, const std::string &cond) {
    for (int n = 0; n < L.g.n_in; ++n) {
      if (!per_vector(L.g.in[n])) {
        if (!cond.empty()) s << "    if (" << cond << ")\n";
        emit_load(s, &L.g, n, bf16, "    ", pre + std::to_string(n), gi, "gj0");
        continue;
      }
      for (int j = 0; j < VPT; ++j) {
        s << "    if (ok" << j << (cond.empty() ? "" : " && " + cond) << ")\n";
        emit_load(s, &L.g, n, bf16, "    ", pre + std::to_string(n) + "_" + std::to_string(j), gi, "gj" + std::to_string(j));
      }
    }
  };
  auto each_reg = [&](const std::function<void(const std::string &)> &fn) {
    for (int n = 0; n < L.g.n_in; ++n) {
      if (!per_vector(L.g.in[n])) fn(std::to_string(n));
      else
        for (int j = 0; j < VPT; ++j) fn(std::to_string(n) + "_" + std::to_string(j));
    }
  };
  each_reg([&](const std::string &r) { s << "  uint4 g" << r << " = make_uint4(0, 0, 0, 0);\n"; });
  s << "  if (blockIdx.x < p.rows) {\n    const i64 gi0 = p.row0 + (i64)blockIdx.x;\n";
  loads("g", "gi0", "");
  s << "  }\n"
       "  for (u32 r = blockIdx.x; r < p.rows; r += gridDim.x) {\n"
       "    const i64 gi = p.row0 + (i64)r;\n"
       "    const bool more = r + gridDim.x < p.rows;\n"
       "    const i64 gin = gi + (i64)gridDim.x;\n";
  each_reg([&](const std::string &r) { s << "    uint4 h" << r << " = make_uint4(0, 0, 0, 0);\n"; });
  loads("h", "gin", "more");
  auto var = [&](int st, int k, int j) -> std::string {
    const int w = L.where[st][k];
    if (w < 0) return "phv" + std::to_string(-w - 1);
    return per_vector(L.g.in[w]) ? "g" + std::to_string(w) + "_" + std::to_string(j) : "g" + std::to_string(w);
  };
  int from[TTLB_MAX_PHASES + 1];
  bool saved[TTLB_MAX_PHASES] = {false, false, false};
  for (int st = 0; st <= f->n_phases; ++st) {
    from[st] = continue_from(f, L, st);
    if (from[st] >= 0) saved[from[st]] = true;
  }
  auto start_pc = [&](int st) { return from[st] >= 0 ? f->phase[from[st]].src.n_ops : 0; };
  auto start_var = [&](int st, int j) {
    return from[st] >= 0 ? "sv" + std::to_string(from[st]) + "_" + std::to_string(j) : std::string();
  };
  for (int ph = 0; ph < f->n_phases; ++ph) {
    const ttlb_reduce_desc &R = f->phase[ph];
    const bool is_max = R.op == TTLB_REDUCE_MAX;
    const std::string P = std::to_string(ph);
    if (saved[ph])
      for (int j = 0; j < VPT; ++j) s << "    float sv" << P << "_" << j << "[V];\n";
    auto comb = [&](const std::string &a, const std::string &b) {
      return is_max ? "nan_max(" + a + ", " + b + ")" : "(" + a + " + " + b + ")";
    };
    s << "    float racc" << P << " = " << (is_max ? "__uint_as_float(0xff800000u)" : "0.0f") << ";\n";
    for (int j = 0; j < VPT; ++j) {
      s << "    if (ok" << j << ") {\n";
      emit_ops(s, &R.src, [&](int k) { return var(ph, k, j); }, bf16, bf16 && R.src.round_each_op, "q.imm[" + P + "]",
               start_pc(ph), start_var(ph, j));
      if (saved[ph]) s << "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) sv" << P << "_" << j << "[e] = acc[e];\n";
      s << "      _Pragma(\"unroll\") for (int e = 0; e < V; ++e) racc" << P << " = " << comb("racc" + P, "acc[e]") << ";\n"
           "    }\n";
    }
    s << "    _Pragma(\"unroll\") for (int o = 16; o; o >>= 1) { const float y = __shfl_xor_sync(0xffffffffu, racc" << P
      << ", o); racc" << P << " = " << comb("racc" + P, "y") << "; }\n"
         "    if (lane == 0) sm[warp] = racc" << P << ";\n"
         "    __syncthreads();\n"
         "    float res" << P << " = sm[0];\n"
         "    _Pragma(\"unroll\") for (int w = 1; w < " << T / 32 << "; ++w) res" << P << " = " << comb("res" + P, "sm[w]") << ";\n"
         "    __syncthreads();\n"
         "    res" << P << " = res" << P << " * sc" << P << ";\n";
    if (bf16)
      s << "    uint4 phv" << P << "; { u32 h = pack_bf16x2(res" << P << ", 0.0f) & 0xffffu; res" << P
        << " = __uint_as_float(h << 16); h |= h << 16; phv" << P << " = make_uint4(h, h, h, h); }\n";
    else
      s << "    uint4 phv" << P << "; { const u32 w = __float_as_uint(res" << P << "); phv" << P << " = make_uint4(w, w, w, w); }\n";
    if (R.out)
      s << "    if (threadIdx.x < q.red_fill[" << P << "]) st_elem(q.red_out[" << P << "], (i64)r * q.red_ld[" << P
        << "] + threadIdx.x, threadIdx.x == 0 ? res" << P << " : 0.0f);\n";
  }
  const std::string FP = std::to_string(f->n_phases);
  for (int j = 0; j < VPT; ++j) {
    s << "    if (ok" << j << ") {\n";
    emit_ops(s, &f->final, [&](int k) { return var(f->n_phases, k, j); }, bf16, bf16 && f->final.round_each_op,
             "q.imm[" + FP + "]", start_pc(f->n_phases), start_var(f->n_phases, j));
    s << "      uint4 o;\n";
    if (bf16)
      s << "      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);\n"
           "      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);\n";
    else
      s << "      o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]);\n"
           "      o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]);\n";
    s << "      st_stream((char*)p.out + (gi * p.out_ld + gj" << j << ") * ESZ, o);\n"
         "    }\n";
  }
  each_reg([&](const std::string &r) { s << "    g" << r << " = h" << r << ";\n"; });
  s << "  }\n}\n";
  return s.str();
}

int ttlb_rowfused_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cachep, const ttlb_rowfused_desc *f, cudaStream_t stream) {
  const RowLayout L = row_layout(f);
  if (!L.ok) return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "rowfused: more than %d distinct operands", TTLB_MAX_IN);
  const int vpt = rowfused_vpt(f);
  int vectors = 0;
  for (int n = 0; n < L.g.n_in; ++n) vectors += per_vector(L.g.in[n]) ? vpt : 1;
  if (vpt > 8 || vectors > 24)
    return ttlb_fail(ctx, TTLB_ERR_UNSUPPORTED, "rowfused: a row of the operands does not fit in registers (%d vectors per thread)",
                     vectors);
  JitKernel jk;
  {
    const std::string key = ttlb_rowfused_jit_key(f, L, vpt);
    const bool cached = *cachep && (*cachep)->kernels.count(key);
    const int rc = get_kernel(ctx, cachep, key, cached ? std::string() : ttlb_rowfused_jit_source(f), "ttlb_rowfused_jit", &jk,
                              rowfused_threads(f));
    if (rc != TTLB_OK) return rc;
  }
  const ttlb_eltwise_desc *d = &f->final;
  const int vec = d->dtype == TTLB_BF16 ? 8 : 4;
  RowParams q{};
  JitParams &p = q.p;
  for (int n = 0; n < L.g.n_in; ++n) {
    p.in[n] = L.g.in[n].ptr;
    p.ld[n] = L.g.in[n].ld;
    p.roff[n] = L.g.in[n].row_off;
    p.coff[n] = L.g.in[n].col_off;
  }
  p.out = d->out;
  p.out_ld = d->out_ld;
  p.row0 = d->row0;
  p.col0 = d->col0;
  p.vpr = (unsigned)(d->cols / vec);
  p.rows = (unsigned)d->rows;
  for (int ph = 0; ph < f->n_phases; ++ph) {
    q.scaler[ph] = f->phase[ph].scaler;
    q.red_out[ph] = f->phase[ph].out;
    q.red_ld[ph] = f->phase[ph].out_ld;
    q.red_fill[ph] = (unsigned)f->phase[ph].fill_cols;
    for (int k = 0; k < TTLB_MAX_IMM; ++k) q.imm[ph][k] = f->phase[ph].src.imm[k];
  }
  for (int k = 0; k < TTLB_MAX_IMM; ++k) q.imm[f->n_phases][k] = d->imm[k];
  unsigned grid = (unsigned)(ctx->sm_count * jk.blocks_per_sm);
  if (grid > p.rows) grid = p.rows;
  void *args[] = {&q};
  TTLB_CUDA_CHECK(ctx, cudaLaunchKernel(reinterpret_cast<const void *>(jk.kern), dim3(grid, 1, 1),
                                        dim3((unsigned)rowfused_threads(f), 1, 1), args, 0, stream));
  return TTLB_OK;
}
