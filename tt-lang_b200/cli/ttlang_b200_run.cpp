// ttlang-b200-run: run a recognised tile program from its launch plan, without Python.
//
//   ttlang-b200-run plan.json [--steps N] [--warmup W] [--device D]
//
// The reference ships its compiler drivers as native tools next to the Python front end
// (tools/ttlang-translate/ttlang-translate.cpp:24-29 registers the translations and hands over to MLIR's
// translate main).  This is the run-time counterpart for the B200 backend: `python -m ttl_b200.translate
// program.py --emit DIR` writes, per kernel call, a plan (the launches the program was recognised as, with their
// operand addressing and op sequences) and the raw bytes of every argument tensor; this tool loads them into
// device memory, issues the launches through the C ABI of libttlb200 (include/ttlb200.h), times them with CUDA
// events on the launching stream, and writes every tensor a launch wrote to `<file>.out`.
//
// Supported launch kinds: eltwise, reduce_sum / reduce_max, row_fused, matmul_bf16 (optional bias / activation),
// matmul_f32, matmul_bfp8w.
// One JSON line on stdout: {"launches": n, "steps": k, "ms_per_step": t, "outputs": [...]}.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "ttlb200.h"

namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true / false / null) -------------------------
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;
  const Json &at(const std::string &k) const {
    auto it = obj.find(k);
    if (it == obj.end()) {
      fprintf(stderr, "plan: missing key \"%s\"\n", k.c_str());
      exit(2);
    }
    return it->second;
  }
  bool has(const std::string &k) const { return obj.count(k) != 0 && obj.at(k).kind != Null; }
  int64_t i() const { return (int64_t)num; }
};

struct Parser {
  const std::string &s;
  size_t p = 0;
  explicit Parser(const std::string &text) : s(text) {}
  [[noreturn]] void die(const char *what) {
    fprintf(stderr, "plan: %s at byte %zu\n", what, p);
    exit(2);
  }
  void ws() {
    while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r')) ++p;
  }
  Json value() {
    ws();
    if (p >= s.size()) die("unexpected end");
    Json j;
    const char c = s[p];
    if (c == '{') {
      j.kind = Json::Obj;
      ++p;
      ws();
      if (s[p] == '}') { ++p; return j; }
      for (;;) {
        ws();
        Json k = value();
        if (k.kind != Json::Str) die("object key must be a string");
        ws();
        if (s[p++] != ':') die("expected ':'");
        j.obj[k.str] = value();
        ws();
        if (s[p] == ',') { ++p; continue; }
        if (s[p] == '}') { ++p; return j; }
        die("expected ',' or '}'");
      }
    }
    if (c == '[') {
      j.kind = Json::Arr;
      ++p;
      ws();
      if (s[p] == ']') { ++p; return j; }
      for (;;) {
        j.arr.push_back(value());
        ws();
        if (s[p] == ',') { ++p; continue; }
        if (s[p] == ']') { ++p; return j; }
        die("expected ',' or ']'");
      }
    }
    if (c == '"') {
      j.kind = Json::Str;
      ++p;
      while (p < s.size() && s[p] != '"') {
        if (s[p] == '\\' && p + 1 < s.size()) ++p;
        j.str.push_back(s[p++]);
      }
      if (p >= s.size()) die("unterminated string");
      ++p;
      return j;
    }
    if (!s.compare(p, 4, "true")) { j.kind = Json::Bool; j.b = true; p += 4; return j; }
    if (!s.compare(p, 5, "false")) { j.kind = Json::Bool; p += 5; return j; }
    if (!s.compare(p, 4, "null")) { p += 4; return j; }
    char *end = nullptr;
    j.num = strtod(s.c_str() + p, &end);
    if (end == s.c_str() + p) die("unexpected character");
    j.kind = Json::Num;
    p = (size_t)(end - s.c_str());
    return j;
  }
};

struct Tensor {
  int64_t rows = 0, cols = 0, bytes = 0;
  std::string dtype, file;
  void *dev = nullptr;
  bool written = false;
  int64_t ld() const { return cols; }
  int esz() const { return dtype == "f32" ? 4 : 2; }
};

#define CUDA_OK(expr)                                                                   \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s failed: %s\n", #expr, cudaGetErrorString(e__));               \
      exit(3);                                                                          \
    }                                                                                   \
  } while (0)

const int kTempBase = 1000;   // tensor indices from here on name temporaries of the plan

}  // namespace

int main(int argc, char **argv) {
  std::string plan_path;
  int steps = 1, warmup = 0, device = 0;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--steps" && i + 1 < argc) steps = atoi(argv[++i]);
    else if (a == "--warmup" && i + 1 < argc) warmup = atoi(argv[++i]);
    else if (a == "--device" && i + 1 < argc) device = atoi(argv[++i]);
    else if (a == "-h" || a == "--help") { printf("usage: ttlang-b200-run plan.json [--steps N] [--warmup W] [--device D]\n"); return 0; }
    else plan_path = a;
  }
  if (plan_path.empty() || steps < 1) { fprintf(stderr, "usage: ttlang-b200-run plan.json [--steps N] [--warmup W] [--device D]\n"); return 2; }
  std::ifstream f(plan_path);
  if (!f) { fprintf(stderr, "cannot open %s\n", plan_path.c_str()); return 2; }
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string text = ss.str();
  Parser parser(text);
  const Json plan = parser.value();
  const std::string dir = plan_path.find('/') == std::string::npos ? "." : plan_path.substr(0, plan_path.rfind('/'));

  ttlb_ctx *ctx = nullptr;
  int rc = ttlb_init(device, &ctx);
  if (rc != TTLB_OK) { fprintf(stderr, "ttlb_init(%d) failed (%d): no usable B200; this backend has no CPU fallback\n", device, rc); return 3; }
  CUDA_OK(cudaSetDevice(device));

  // tensors: the kernel call's arguments, then the plan's temporaries
  std::vector<Tensor> args, temps;
  auto load = [&](const Json &jt, bool temp) {
    Tensor t;
    t.rows = jt.at("shape").arr[0].i();
    t.cols = jt.at("shape").arr[1].i();
    t.dtype = jt.at("dtype").str;
    if (t.dtype == "bfp8_b") t.bytes = (t.rows / 32) * (t.cols / 32) * 1088;
    else t.bytes = t.rows * t.cols * t.esz();
    if (t.bytes > 0) CUDA_OK(cudaMalloc(&t.dev, (size_t)t.bytes));
    if (temp || !jt.has("file")) {
      if (t.bytes > 0) CUDA_OK(cudaMemset(t.dev, 0, (size_t)t.bytes));
    } else {
      t.file = dir + "/" + jt.at("file").str;
      std::ifstream in(t.file, std::ios::binary);
      std::vector<char> host((size_t)t.bytes);
      if (!in || !in.read(host.data(), t.bytes)) { fprintf(stderr, "cannot read %lld bytes from %s\n", (long long)t.bytes, t.file.c_str()); exit(2); }
      CUDA_OK(cudaMemcpy(t.dev, host.data(), (size_t)t.bytes, cudaMemcpyHostToDevice));
    }
    return t;
  };
  for (const Json &jt : plan.at("tensors").arr) args.push_back(load(jt, false));
  if (plan.has("temps"))
    for (const Json &jt : plan.at("temps").arr) temps.push_back(load(jt, true));
  auto tensor = [&](int64_t idx) -> Tensor & {
    if (idx >= kTempBase) {
      if ((size_t)(idx - kTempBase) >= temps.size()) { fprintf(stderr, "plan: temporary %lld does not exist\n", (long long)idx); exit(2); }
      return temps[(size_t)(idx - kTempBase)];
    }
    if (idx < 0 || (size_t)idx >= args.size()) { fprintf(stderr, "plan: tensor %lld does not exist\n", (long long)idx); exit(2); }
    return args[(size_t)idx];
  };

  // the element-wise program of a launch (`l`: inputs, opcodes, imm, round_each_op) over rows [row0, +rows) x columns
  // [col0, +cols); operands named in `produced` stand for results of earlier phases of a row-fused launch
  auto fill_program = [&](ttlb_eltwise_desc &d, const Json &l, const Tensor &like, const std::map<int64_t, int> *produced) {
    memset(&d, 0, sizeof(d));
    d.dtype = like.dtype == "f32" ? TTLB_F32 : TTLB_BF16;
    d.round_each_op = l.at("round_each_op").b ? 1 : 0;
    const std::vector<Json> &ins = l.at("inputs").arr;
    const std::vector<Json> &ops = l.at("opcodes").arr;
    d.n_in = (int32_t)ins.size();
    d.n_ops = (int32_t)ops.size();
    if (d.n_in > TTLB_MAX_IN || d.n_ops > TTLB_MAX_OPS) { fprintf(stderr, "plan: launch too large\n"); exit(2); }
    for (int k = 0; k < d.n_in; ++k) {
      const std::vector<Json> &v = ins[(size_t)k].arr;
      const int64_t ti = v[0].i();
      if (produced && produced->count(ti)) {
        d.in[k].ptr = nullptr;
        d.in[k].row_mode = TTLB_IDX_PHASE;
        d.in[k].row_off = produced->at(ti);
        d.in[k].col_mode = TTLB_IDX_ZERO;
        d.in[k].col_off = 0;
        d.in[k].ld = 1;
        continue;
      }
      Tensor &t = tensor(ti);
      d.in[k].ptr = t.dev;
      d.in[k].ld = t.rows > 1 ? t.ld() : t.cols;
      d.in[k].row_mode = (int32_t)v[1].i();
      d.in[k].row_off = v[2].i();
      d.in[k].col_mode = (int32_t)v[3].i();
      d.in[k].col_off = v[4].i();
    }
    for (int k = 0; k < d.n_ops; ++k) {
      d.ops[k].opcode = (int16_t)ops[(size_t)k].arr[0].i();
      d.ops[k].arg = (int16_t)ops[(size_t)k].arr[1].i();
    }
    if (l.has("imm"))
      for (size_t k = 0; k < l.at("imm").arr.size() && k < TTLB_MAX_IMM; ++k) d.imm[k] = (float)l.at("imm").arr[k].num;
  };
  // a reduction launch (`l`: kind reduce_sum / reduce_max, dims, rect_tiles, reduced_tiles, scaler) as a descriptor
  auto fill_reduce = [&](ttlb_reduce_desc &r, const Json &l, const std::map<int64_t, int> *produced, bool with_out) {
    Tensor &out = tensor(l.at("out").i());
    fill_program(r.src, l, out, produced);
    const std::vector<Json> &rt = l.at("rect_tiles").arr;
    const std::vector<Json> &ext = l.at("reduced_tiles").arr;
    bool rows_reduced = false, cols_reduced = false;
    for (const Json &dm : l.at("dims").arr) (dm.i() == 0 ? rows_reduced : cols_reduced) = true;
    r.src.row0 = rows_reduced ? 0 : rt[0].i() * 32;
    r.src.rows = rows_reduced ? ext[0].i() * 32 : (rt[1].i() - rt[0].i()) * 32;
    r.src.col0 = cols_reduced ? 0 : rt[2].i() * 32;
    r.src.cols = cols_reduced ? ext[1].i() * 32 : (rt[3].i() - rt[2].i()) * 32;
    r.op = l.at("kind").str == "reduce_sum" ? TTLB_REDUCE_SUM : TTLB_REDUCE_MAX;
    r.dims = (rows_reduced ? TTLB_REDUCE_ROWS : 0) | (cols_reduced ? TTLB_REDUCE_COLS : 0);
    const int es = out.esz();
    r.out_ld = out.rows > 1 ? out.ld() : out.cols;
    const int64_t orow = out.rows == 1 ? 0 : rt[0].i() * 32, ocol = out.cols == 1 ? 0 : rt[2].i() * 32;
    r.fill_rows = out.rows == 1 ? 1 : 32;
    r.fill_cols = out.cols == 1 ? 1 : 32;
    r.out = with_out ? (char *)out.dev + (orow * r.out_ld + ocol) * es : nullptr;
    r.scaler = nullptr;
    if (l.has("scaler")) {
      const std::vector<Json> &sc = l.at("scaler").arr;
      Tensor &st = tensor(sc[0].i());
      r.scaler = (char *)st.dev + (sc[1].i() * (st.rows > 1 ? st.ld() : 0) + sc[2].i()) * es;
    }
    if (with_out) out.written = true;
  };

  cudaStream_t stream;
  CUDA_OK(cudaStreamCreate(&stream));
  const std::vector<Json> &launches = plan.at("launches").arr;
  auto run_all = [&]() {
    for (const Json &l : launches) {
      const std::string kind = l.at("kind").str;
      const std::vector<Json> &rt = l.at("rect_tiles").arr;
      const int64_t r0 = rt[0].i() * 32, r1 = rt[1].i() * 32, c0 = rt[2].i() * 32, c1 = rt[3].i() * 32;
      Tensor &out = tensor(l.at("out").i());
      out.written = true;
      int st = TTLB_OK;
      if (kind == "eltwise") {
        ttlb_eltwise_desc d;
        fill_program(d, l, out, nullptr);
        d.out = out.dev;
        d.out_ld = out.ld();
        const bool deg_r = out.rows == 1, deg_c = out.cols == 1;
        d.row0 = deg_r ? 0 : r0;
        d.rows = deg_r ? 1 : r1 - r0;
        d.col0 = deg_c ? 0 : c0;
        d.cols = deg_c ? 1 : c1 - c0;
        st = ttlb_eltwise(ctx, &d, stream);
      } else if (kind == "reduce_sum" || kind == "reduce_max") {
        ttlb_reduce_desc r;
        fill_reduce(r, l, nullptr, true);
        st = ttlb_reduce(ctx, &r, stream);
      } else if (kind == "row_fused") {
        // reductions over columns whose results stay on chip, then the element-wise program that reads them
        static ttlb_rowfused_desc f;
        memset(&f, 0, sizeof(f));
        const std::vector<Json> &phases = l.at("phases").arr;
        if (phases.size() > TTLB_MAX_PHASES) { fprintf(stderr, "plan: too many phases\n"); exit(2); }
        std::map<int64_t, int> produced;
        for (size_t i = 0; i < phases.size(); ++i) produced[phases[i].at("out").i()] = (int)i;
        f.n_phases = (int32_t)phases.size();
        for (size_t i = 0; i < phases.size(); ++i) fill_reduce(f.phase[i], phases[i], &produced, false);
        const Json &fin = l.at("final");
        fill_program(f.final, fin, out, &produced);
        f.final.out = out.dev;
        f.final.out_ld = out.ld();
        f.final.row0 = r0;
        f.final.rows = r1 - r0;
        f.final.col0 = c0;
        f.final.cols = c1 - c0;
        st = ttlb_rowfused(ctx, &f, stream);
      } else if (kind == "matmul_bf16" || kind == "matmul_f32") {
        Tensor &a = tensor(l.at("a").i()), &b = tensor(l.at("b").i());
        const int es = a.esz();
        ttlb_gemm_desc g;
        g.a = (char *)a.dev + r0 * a.ld() * es;
        g.lda = a.ld();
        g.b = (char *)b.dev + c0 * es;
        g.ldb = b.ld();
        g.c = (char *)out.dev + (r0 * out.ld() + c0) * es;
        g.ldc = out.ld();
        g.m = r1 - r0;
        g.n = c1 - c0;
        g.k = a.cols;
        if (kind == "matmul_f32") {
          st = ttlb_matmul_f32(ctx, &g, stream);
        } else if (l.has("bias") || l.has("act")) {
          const void *bias = nullptr;
          int64_t ldbias = 0;
          if (l.has("bias")) {
            Tensor &bt = tensor(l.at("bias").i());
            const bool row = bt.rows == 1 && out.rows != 1;
            bias = (char *)bt.dev + ((row ? 0 : r0 * bt.ld()) + c0) * 2;
            ldbias = row ? 0 : bt.ld();
          }
          st = ttlb_matmul_bf16_epilogue(ctx, &g, bias, ldbias, l.has("act") ? (int)l.at("act_code").i() : TTLB_ACT_NONE, stream);
        } else {
          st = ttlb_matmul_bf16(ctx, &g, stream);
        }
      } else if (kind == "matmul_bfp8w") {
        Tensor &a = tensor(l.at("a").i()), &b = tensor(l.at("b").i());
        ttlb_gemm_bfp8_desc g;
        g.a = (char *)a.dev + r0 * a.ld() * 2;
        g.lda = a.ld();
        g.b_tiles = b.dev;
        g.b_tile_cols = b.cols / 32;
        g.b_tile_col0 = c0 / 32;
        g.c = (char *)out.dev + (r0 * out.ld() + c0) * 2;
        g.ldc = out.ld();
        g.m = r1 - r0;
        g.n = c1 - c0;
        g.k = a.cols;
        st = ttlb_matmul_bfp8w(ctx, &g, stream);
      } else {
        fprintf(stderr, "launch kind \"%s\" is not supported by this tool (eltwise, reduce_sum, reduce_max, row_fused, matmul_bf16, matmul_f32, matmul_bfp8w)\n", kind.c_str());
        exit(2);
      }
      if (st != TTLB_OK) { fprintf(stderr, "launch \"%s\" failed (%d): %s\n", kind.c_str(), st, ttlb_last_error(ctx)); exit(3); }
    }
  };

  for (int i = 0; i < warmup; ++i) run_all();
  cudaEvent_t e0, e1;
  CUDA_OK(cudaEventCreate(&e0));
  CUDA_OK(cudaEventCreate(&e1));
  CUDA_OK(cudaStreamSynchronize(stream));
  CUDA_OK(cudaEventRecord(e0, stream));
  for (int i = 0; i < steps; ++i) run_all();
  CUDA_OK(cudaEventRecord(e1, stream));
  CUDA_OK(cudaStreamSynchronize(stream));
  rc = ttlb_check_status(ctx, stream);
  if (rc != TTLB_OK) { fprintf(stderr, "device status: %s\n", ttlb_last_error(ctx)); return 3; }
  float ms = 0;
  CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));

  std::string outs;
  for (Tensor &t : args) {
    if (!t.written || t.file.empty()) continue;
    std::vector<char> host((size_t)t.bytes);
    CUDA_OK(cudaMemcpy(host.data(), t.dev, (size_t)t.bytes, cudaMemcpyDeviceToHost));
    const std::string path = t.file + ".out";
    std::ofstream o(path, std::ios::binary);
    o.write(host.data(), t.bytes);
    outs += (outs.empty() ? "\"" : ", \"") + path + "\"";
  }
  printf("{\"launches\": %zu, \"steps\": %d, \"warmup\": %d, \"ms_per_step\": %.6f, \"outputs\": [%s]}\n", launches.size(), steps, warmup,
         ms / steps, outs.c_str());
  for (Tensor &t : args) if (t.dev) cudaFree(t.dev);
  for (Tensor &t : temps) if (t.dev) cudaFree(t.dev);
  ttlb_destroy(ctx);
  return 0;
}
