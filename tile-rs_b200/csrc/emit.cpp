// The `cuda_sm100` CodegenTarget: merged MLIR text -> one CUDA translation unit.
//
// Stands where the reference's NVIDIA emitter stands
// (crates/rustc_codegen_tile/src/mlir_to_gpu.rs:62-99 behind
// crates/tile_codegen/src/target.rs:57-65), but does not translate intrinsics
// into scalar CUDA line by line.  It recognises what an entry kernel computes
// (row softmax, a matrix product, fused attention, with the casts and masks
// around them) and emits a launcher that instantiates the hand-written sm_100a
// kernels of this library for the shapes the module carries.
//
// Input contract (crates/rustc_codegen_tile/src/mlir_parse.rs:84-213):
//   * an entry kernel is an `llvm.func` whose header (pretty form) or closing
//     line (generic form) carries `hacc.entry`;
//   * a global-memory pointer argument has a type containing `ptr<1>`;
//   * tile shapes and other integers are operands defined by
//     `llvm.mlir.constant`; the first operand of a compute intrinsic is an
//     ignored destination id.
// A non-constant SSA name is never read as a number (the reference's
// parse_const_arg turns `%12` into 12, mlir_parse.rs:1368-1388).
//
// Pure and deterministic: reads the text, touches no file, no environment.
// Anything outside the target's scope is an error, never a TODO comment.
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/tile_sm100.h"

namespace tsm100 {
std::string& last_error_ref();
}

namespace {

struct EmitFailure {
  std::string msg;
};
[[noreturn]] void reject(const std::string& m) { throw EmitFailure{m}; }

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r' || s[a] == '\n')) ++a;
  while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r' || s[b - 1] == '\n')) --b;
  return s.substr(a, b - a);
}

bool starts_with(const std::string& s, const char* p) { return s.compare(0, std::strlen(p), p) == 0; }
bool contains(const std::string& s, const char* p) { return s.find(p) != std::string::npos; }

int count_char(const std::string& s, char c) {
  int n = 0;
  for (char ch : s) n += ch == c;
  return n;
}

// Splits on commas that are not nested inside (), <>, [] or {}.
std::vector<std::string> split_top(const std::string& s) {
  std::vector<std::string> out;
  int depth = 0;
  std::string cur;
  for (char c : s) {
    if (c == '(' || c == '<' || c == '[' || c == '{') ++depth;
    if (c == ')' || c == '>' || c == ']' || c == '}') --depth;
    if (c == ',' && depth == 0) {
      out.push_back(trim(cur));
      cur.clear();
    } else {
      cur.push_back(c);
    }
  }
  if (!trim(cur).empty()) out.push_back(trim(cur));
  return out;
}

// Text between the '(' at `open` and its matching ')'.
std::string paren_body(const std::string& s, size_t open) {
  int depth = 0;
  for (size_t i = open; i < s.size(); ++i) {
    if (s[i] == '(') ++depth;
    if (s[i] == ')' && --depth == 0) return s.substr(open + 1, i - open - 1);
  }
  return s.substr(open + 1);
}

struct Arg {
  std::string name;
  bool is_gm = false;
};

struct Func {
  std::string name;
  std::vector<Arg> args;
  bool is_entry = false;
  std::vector<std::string> body;
};

std::vector<Arg> parse_arg_list(const std::string& inside) {
  std::vector<Arg> out;
  for (const std::string& item : split_top(inside)) {
    const size_t colon = item.find(':');
    if (item.empty() || item[0] != '%' || colon == std::string::npos) continue;
    Arg a;
    a.name = trim(item.substr(0, colon));
    a.is_gm = contains(item.substr(colon + 1), "ptr<1>");
    out.push_back(a);
  }
  return out;
}

std::vector<Func> parse_module(const std::string& text) {
  std::vector<std::string> lines;
  {
    std::istringstream in(text);
    std::string l;
    while (std::getline(in, l)) lines.push_back(trim(l));
  }
  std::vector<Func> funcs;
  for (size_t i = 0; i < lines.size();) {
    const std::string& line = lines[i];
    const size_t at = line.find("llvm.func @");
    if (at != std::string::npos && !starts_with(line, "//")) {
      Func f;
      const size_t name0 = at + std::strlen("llvm.func @");
      const size_t open = line.find('(', name0);
      if (open == std::string::npos) reject("cannot parse function header: " + line);
      f.name = trim(line.substr(name0, open - name0));
      f.args = parse_arg_list(paren_body(line, open));
      f.is_entry = contains(line, "hacc.entry");
      int depth = count_char(line, '{') - count_char(line, '}');
      ++i;
      while (i < lines.size() && depth > 0) {
        depth += count_char(lines[i], '{') - count_char(lines[i], '}');
        if (depth > 0) f.body.push_back(lines[i]);
        ++i;
      }
      funcs.push_back(f);
    } else if (starts_with(line, "\"llvm.func\"()")) {
      // generic form: "llvm.func"() <{sym_name = "k", ...}> ({  ^bb0(%arg0: T, ...):  ...  }) {hacc.entry} : () -> ()
      Func f;
      const size_t sn = line.find("sym_name = \"");
      if (sn != std::string::npos) {
        const size_t b = sn + std::strlen("sym_name = \"");
        f.name = line.substr(b, line.find('"', b) - b);
      }
      int depth = count_char(line, '(') - count_char(line, ')');
      ++i;
      while (i < lines.size() && depth > 0) {
        const std::string& bl = lines[i];
        depth += count_char(bl, '(') - count_char(bl, ')');
        if (depth <= 0) {
          f.is_entry = contains(bl, "hacc.entry");
        } else if (starts_with(bl, "^bb0(")) {
          f.args = parse_arg_list(paren_body(bl, bl.find('(')));
        } else {
          f.body.push_back(bl);
        }
        ++i;
      }
      if (!f.name.empty()) funcs.push_back(f);
    } else {
      ++i;
    }
  }
  return funcs;
}

// ---- one body line -----------------------------------------------------------
struct Call {
  std::string result;  // may be empty
  std::string callee;
  std::vector<std::string> args;
};

std::string result_of(const std::string& line) {
  if (line.empty() || line[0] != '%') return "";
  const size_t eq = line.find('=');
  return eq == std::string::npos ? "" : trim(line.substr(0, eq));
}

// Accepts `%r = llvm.call @f(a, b) : ...` and `%r = "llvm.call"(a, b) <{callee = @f, ...}> : ...`.
bool parse_call(const std::string& line, Call* out) {
  const size_t pretty = line.find("llvm.call @");
  if (pretty != std::string::npos && !contains(line, "\"llvm.call\"")) {
    const size_t n0 = pretty + std::strlen("llvm.call @");
    const size_t open = line.find('(', n0);
    if (open == std::string::npos) return false;
    out->result = result_of(line);
    out->callee = trim(line.substr(n0, open - n0));
    out->args = split_top(paren_body(line, open));
    return true;
  }
  const size_t generic = line.find("\"llvm.call\"(");
  if (generic != std::string::npos) {
    const size_t open = generic + std::strlen("\"llvm.call\"");
    const size_t cal = line.find("callee = @");
    if (cal == std::string::npos) return false;
    size_t e = cal + std::strlen("callee = @");
    size_t n1 = e;
    while (n1 < line.size() && (isalnum(static_cast<unsigned char>(line[n1])) || line[n1] == '_' || line[n1] == '.')) ++n1;
    out->result = result_of(line);
    out->callee = line.substr(e, n1 - e);
    out->args = split_top(paren_body(line, open));
    return true;
  }
  return false;
}

// `%c = llvm.mlir.constant(128 : i32) : i32` or `%c = "llvm.mlir.constant"() <{value = 128 : i32}> : () -> i32`
bool parse_constant(const std::string& line, std::string* name, std::string* literal, bool* is_float) {
  if (!contains(line, "llvm.mlir.constant")) return false;
  *name = result_of(line);
  if (name->empty()) return false;
  std::string lit;
  const size_t v = line.find("value = ");
  if (v != std::string::npos) {
    lit = line.substr(v + std::strlen("value = "));
  } else {
    const size_t open = line.find('(', line.find("llvm.mlir.constant"));
    if (open == std::string::npos) return false;
    lit = paren_body(line, open);
  }
  const size_t colon = lit.find(':');
  std::string ty = colon == std::string::npos ? "" : trim(lit.substr(colon + 1));
  lit = trim(colon == std::string::npos ? lit : lit.substr(0, colon));
  if (lit.empty()) return false;
  *is_float = starts_with(ty, "f") || lit.find('.') != std::string::npos ||
              (lit.find('e') != std::string::npos && !starts_with(lit, "0x"));
  if (lit == "true") lit = "1";
  if (lit == "false") lit = "0";
  *literal = lit;
  return true;
}

// ---- dataflow over tiles -------------------------------------------------------
enum class Dt { F32, F16, BF16 };
const char* dt_enum(Dt d) { return d == Dt::F32 ? "TSM100_F32" : d == Dt::F16 ? "TSM100_F16" : "TSM100_BF16"; }
const char* dt_name(Dt d) { return d == Dt::F32 ? "f32" : d == Dt::F16 ? "f16" : "bf16"; }

bool suffix_dtype(const std::string& callee, Dt* d) {
  auto ends = [&](const char* s) {
    const size_t n = std::strlen(s);
    return callee.size() >= n && callee.compare(callee.size() - n, n, s) == 0;
  };
  if (ends("_bf16")) { *d = Dt::BF16; return true; }
  if (ends("_f16")) { *d = Dt::F16; return true; }
  if (ends("_f32")) { *d = Dt::F32; return true; }
  return false;
}

enum class Kind { Load, Softmax, Matmul, MatmulT, Transpose, Scale, CausalMask, Attention, AttentionGqa,
                  RmsNorm, ReduceSum, ReduceMax, Ewise };

struct Tile {
  Kind kind = Kind::Load;
  Dt dtype = Dt::F32;      // storage type of the data the tile came from (through casts: the load's)
  int arg = -1;            // Load: index among the kernel's pointer arguments
  long rows = 0, cols = 0;
  std::vector<std::string> in;  // producer tiles
  long m = 0, k = 0, n = 0;     // Matmul*
  double scalar = 0;            // Scale: factor; RmsNorm: eps; Ewise scale / fill: the constant; clamp: lo
  double scalar2 = 0;           // Ewise clamp: hi
  std::string ew;               // Ewise: operator name ("add", "exp", "clamp", ...)
  long heads = 0, kv_heads = 0, seq = 0, dim = 0;  // Attention*
  bool narrowed = false;        // the value went through an f32 -> 16-bit cast ...
  Dt narrow_to = Dt::F32;       // ... to this type; only a store of that type may consume it (the store is the rounding)
};

struct Kernel {
  std::string name;
  int nargs = 0;
  std::string op;        // "softmax" | "gemm" | "attention" | "rms_norm" | "reduce" | "silu_mul" | "ewise"
  std::string summary;   // comment line
  std::string body;      // statements of the launcher
  std::string instantiation;  // explicit instantiation(s) of the __global__ kernel(s)
  std::string descriptor;     // the TileKernel descriptor of the kernel, one JSON object
};

struct FuncCtx {
  const Func& f;
  std::map<std::string, long> ints;
  std::map<std::string, double> floats;
  std::map<std::string, int> ptr_alias;  // SSA -> pointer-argument index
  std::map<std::string, Tile> tiles;

  explicit FuncCtx(const Func& fn) : f(fn) {
    int idx = 0;
    for (const Arg& a : f.args)
      if (a.is_gm) ptr_alias[a.name] = idx++;
  }
  int nptr() const {
    int n = 0;
    for (const Arg& a : f.args) n += a.is_gm;
    return n;
  }
  long int_of(const std::string& ssa, const char* what) const {
    auto it = ints.find(ssa);
    if (it == ints.end()) {
      // a literal operand is accepted; an SSA name that is not a known constant is not
      if (!ssa.empty() && (isdigit(static_cast<unsigned char>(ssa[0])))) return std::stol(ssa);
      reject(std::string("kernel ") + f.name + ": " + what + " operand " + ssa + " is not a compile-time integer constant");
    }
    return it->second;
  }
  int ptr_of(const std::string& ssa) const {
    auto it = ptr_alias.find(ssa);
    if (it == ptr_alias.end()) reject("kernel " + f.name + ": " + ssa + " is not a global-memory pointer argument");
    return it->second;
  }
  const Tile& tile_of(const std::string& ssa) const {
    auto it = tiles.find(ssa);
    if (it == tiles.end()) reject("kernel " + f.name + ": tile " + ssa + " has no known producer");
    return it->second;
  }
};

const char* cxx_type(Dt d) { return d == Dt::F32 ? "float" : d == Dt::F16 ? "__half" : "__nv_bfloat16"; }

// The softmax kernel the library's dispatch picks for a row width (ops.cuh), as an
// explicit instantiation directive; empty when the row is not 16-byte-vector aligned.
std::string softmax_instantiation(Dt d, long cols) {
  const long per_vec = d == Dt::F32 ? 4 : 8;
  if (cols % per_vec != 0) return "";
  const long nvec = cols / per_vec;
  const std::string t = cxx_type(d);
  const std::string sig = "(const " + t + "*, " + t + "*, int64_t, int32_t);\n";
  if (nvec <= 256) {
    const long c = nvec <= 32 ? 1 : nvec <= 64 ? 2 : nvec <= 128 ? 4 : 8;
    return "template __global__ void tsm100::softmax::softmax_rows_warp<" + t + ", " + std::to_string(c) + ", 4>" + sig;
  }
  if (nvec <= 2048) {
    const char* shape = nvec <= 512 ? "4, 128" : nvec <= 1024 ? "8, 128" : "8, 256";
    return "template __global__ void tsm100::softmax::softmax_rows_cta<" + t + ", " + shape + ">" + sig;
  }
  return "";
}

// Element-wise intrinsics `__tile_<op>_<dtype>`: 1 = unary, 2 = binary, 0 = not one of them.
// The packed `_4` and `_scalar` variants of the ggml family are other intrinsics.
std::string ewise_name(const std::string& callee) {
  const size_t b = std::strlen("__tile_"), e = callee.rfind('_');
  return (callee.size() > b && e != std::string::npos && e > b) ? callee.substr(b, e - b) : std::string();
}
int ewise_arity(const std::string& callee) {
  if (!starts_with(callee, "__tile_")) return 0;
  const std::string n = ewise_name(callee);
  static const char* kBinary[] = {"add", "sub", "mul", "div", "max", "min"};
  static const char* kUnary[] = {"exp", "log", "neg", "tanh", "abs", "sqrt", "rsqrt", "sigmoid", "silu", "relu"};
  for (const char* k : kBinary)
    if (n == k) return 2;
  for (const char* k : kUnary)
    if (n == k) return 1;
  return 0;
}

std::string float_literal(double v) {
  const float f = static_cast<float>(v);
  if (std::isinf(f)) return f > 0 ? "INFINITY" : "(-INFINITY)";
  if (std::isnan(f)) return "NAN";
  char buf[48];
  snprintf(buf, sizeof buf, "%.9g", static_cast<double>(f));
  std::string s = buf;
  if (s.find('.') == std::string::npos && s.find('e') == std::string::npos) s += ".0";
  return s + "f";
}

// The same for the rms_norm / reduce kernels (ops.cuh: row_op_typed).
std::string row_op_instantiation(Dt d, const char* op, long cols) {
  const long per_vec = d == Dt::F32 ? 4 : 8;
  const std::string t = cxx_type(d);
  const long nvec = cols / per_vec;
  if (cols % per_vec != 0 || nvec > 2048)
    return "template __global__ void tsm100::rowops::row_op_stream_kernel<" + t + ", tsm100::rowops::" + op + ", 512>(const " + t +
           "*, " + t + "*, int64_t, int64_t, float);\n";
  const char* shape = nvec <= 32 ? "1, 32, 128" : nvec <= 64 ? "2, 32, 128" : nvec <= 128 ? "4, 32, 128" : nvec <= 256 ? "8, 32, 128"
                    : nvec <= 512 ? "4, 128, 128" : nvec <= 1024 ? "8, 128, 128" : "8, 256, 256";
  return "template __global__ void tsm100::rowops::row_op_kernel<" + t + ", tsm100::rowops::" + op + ", " + shape + ">(const " + t + "*, " +
         t + "*, int64_t, int32_t, float);\n";
}

// The TileKernel descriptor of one kernel (crates/tile_hal/src/kernel.rs:93-212: name, the ordered
// TileOp sequence, input / output buffer counts, preferred mode), as one JSON object, plus
// what a launcher needs to validate buffers: per pointer argument its role, storage type and
// element count per block.
std::string describe(const Func& f, const FuncCtx& cx, int store_arg, Dt store_dt, long store_rows, long store_cols) {
  auto dt_tag = [](Dt d) { return d == Dt::F32 ? "F32" : d == Dt::F16 ? "F16" : "BF16"; };
  auto camel = [](const std::string& n) {  // "reduce_max" -> "ReduceMax"
    std::string o;
    bool up = true;
    for (char ch : n) {
      if (ch == '_') { up = true; continue; }
      o += up ? static_cast<char>(toupper(static_cast<unsigned char>(ch))) : ch;
      up = false;
    }
    return o;
  };
  std::ostringstream ops;
  bool first = true, uses_matmul = false;
  struct ArgInfo { bool seen = false; bool output = false; Dt dt = Dt::F32; long elems = 0; };
  std::vector<ArgInfo> args(static_cast<size_t>(cx.nptr()));
  auto op = [&](const std::string& body) {
    ops << (first ? "" : ", ") << "{" << body << "}";
    first = false;
  };
  auto rc = [](long r, long c) { return "\"rows\": " + std::to_string(r) + ", \"cols\": " + std::to_string(c); };
  for (const std::string& line : f.body) {
    Call c;
    if (!parse_call(line, &c)) continue;
    const std::string& fn = c.callee;
    Dt dt = Dt::F32;
    const bool has_dt = suffix_dtype(fn, &dt);
    auto it = cx.tiles.find(c.result);
    const Tile* t = it == cx.tiles.end() ? nullptr : &it->second;
    if (starts_with(fn, "__tile_load_") && t) {
      op("\"op\": \"Load\", " + rc(t->rows, t->cols) + ", \"dtype\": \"" + dt_tag(t->dtype) + "\"");
      ArgInfo& a = args[static_cast<size_t>(t->arg)];
      a.seen = true;
      a.dt = t->dtype;
      a.elems = std::max(a.elems, t->rows * t->cols);
    } else if (starts_with(fn, "__tile_store_") && has_dt) {
      op("\"op\": \"Store\", " + rc(store_rows, store_cols) + ", \"dtype\": \"" + dt_tag(store_dt) + "\"");
    } else if (starts_with(fn, "__tile_cast_")) {
      const std::string n = fn.substr(std::strlen("__tile_cast_"));  // "f32_f16"
      const size_t u = n.find('_');
      std::string from = n.substr(0, u), to = u == std::string::npos ? "" : n.substr(u + 1);
      for (char& ch : from) ch = static_cast<char>(toupper(static_cast<unsigned char>(ch)));
      for (char& ch : to) ch = static_cast<char>(toupper(static_cast<unsigned char>(ch)));
      if (t) op("\"op\": \"Cast" + from + "To" + to + "\", " + rc(t->rows, t->cols));
    } else if (t && t->kind == Kind::Softmax) {
      op("\"op\": \"Softmax\", " + rc(t->rows, t->cols));
    } else if (t && (t->kind == Kind::Matmul || t->kind == Kind::MatmulT)) {
      uses_matmul = true;
      op("\"op\": \"Matmul\", \"m\": " + std::to_string(t->m) + ", \"k\": " + std::to_string(t->k) + ", \"n\": " + std::to_string(t->n) +
         (t->kind == Kind::MatmulT ? ", \"b_transposed\": true" : ""));
    } else if (t && t->kind == Kind::Transpose) {
      op("\"op\": \"Transpose\", " + rc(t->cols, t->rows));  // the operand's shape, as the intrinsic states it
    } else if (t && t->kind == Kind::Scale) {
      op("\"op\": \"Scale\", " + rc(t->rows, t->cols) + ", \"scalar\": " + float_literal(t->scalar).substr(0, float_literal(t->scalar).size() - 1));
    } else if (t && t->kind == Kind::CausalMask) {
      op("\"op\": \"CausalMask\", " + rc(t->rows, t->cols));
    } else if (t && (t->kind == Kind::Attention || t->kind == Kind::AttentionGqa)) {
      uses_matmul = true;
      op("\"op\": \"Attention\", \"b\": " + std::to_string(t->heads) + ", \"s\": " + std::to_string(t->seq) + ", \"d\": " + std::to_string(t->dim) +
         (t->kind == Kind::AttentionGqa ? ", \"kv_heads\": " + std::to_string(t->kv_heads) + ", \"causal\": true" : ""));
    } else if (t && t->kind == Kind::RmsNorm) {
      op("\"op\": \"RmsNorm\", " + rc(t->rows, t->cols) + ", \"eps\": " + float_literal(t->scalar).substr(0, float_literal(t->scalar).size() - 1));
    } else if (t && (t->kind == Kind::ReduceSum || t->kind == Kind::ReduceMax)) {
      op(std::string("\"op\": \"") + (t->kind == Kind::ReduceSum ? "ReduceSum" : "ReduceMax") + "\", " + rc(t->rows, t->cols));
    } else if (t && t->kind == Kind::Ewise) {
      auto num = [](double v) { const std::string l = float_literal(v); return l.substr(0, l.size() - 1); };
      std::string extra;
      if (t->ew == "fill") extra = ", \"scalar\": " + num(t->scalar);
      if (t->ew == "clamp") extra = ", \"lo\": " + num(t->scalar) + ", \"hi\": " + num(t->scalar2);
      op("\"op\": \"" + camel(t->ew) + "\", " + rc(t->rows, t->cols) + extra);
    }
  }
  if (store_arg >= 0) {
    ArgInfo& a = args[static_cast<size_t>(store_arg)];
    a.seen = true;
    a.output = true;
    a.dt = store_dt;
    a.elems = std::max(a.elems, store_rows * store_cols);
  }
  int n_in = 0, n_out = 0;
  std::ostringstream aj;
  for (size_t i = 0; i < args.size(); ++i) {
    n_in += args[i].seen && !args[i].output;
    n_out += args[i].output;
    aj << (i ? ", " : "") << "{\"index\": " << i << ", \"role\": \"" << (args[i].output ? "output" : args[i].seen ? "input" : "unused")
       << "\", \"dtype\": \"" << dt_tag(args[i].dt) << "\", \"elements_per_block\": " << args[i].elems << "}";
  }
  std::ostringstream o;
  // TileKernel::inferred_mode (kernel.rs:204-211): General when a matrix product is involved
  o << "{\"name\": \"" << f.name << "\", \"mode\": \"" << (uses_matmul ? "General" : "Vector") << "\", \"num_inputs\": " << n_in
    << ", \"num_outputs\": " << n_out << ", \"ops\": [" << ops.str() << "], \"args\": [" << aj.str() << "]}";
  return o.str();
}

Kernel lower(const Func& f) {
  FuncCtx cx(f);
  Kernel k;
  k.name = f.name;
  k.nargs = cx.nptr();
  std::string stored_tile;
  int store_arg = -1;
  Dt store_dt = Dt::F32;
  long store_rows = 0, store_cols = 0;

  for (const std::string& line : f.body) {
    if (line.empty() || starts_with(line, "//") || starts_with(line, "^") || contains(line, "llvm.return") ||
        contains(line, "llvm.mlir.addressof") || line == "}" || line == "{")
      continue;
    std::string name, lit;
    bool is_float = false;
    if (parse_constant(line, &name, &lit, &is_float)) {
      try {
        if (is_float) {
          if (starts_with(lit, "0x")) {  // bit pattern of an f32
            uint32_t bits = static_cast<uint32_t>(std::stoul(lit, nullptr, 16));
            float v;
            std::memcpy(&v, &bits, 4);
            cx.floats[name] = v;
          } else {
            cx.floats[name] = std::stod(lit);
          }
        } else {
          cx.ints[name] = std::stol(lit, nullptr, 0);
        }
      } catch (...) {
        reject("kernel " + f.name + ": cannot read constant in: " + line);
      }
      continue;
    }
    Call c;
    if (parse_call(line, &c)) {
      const std::string& fn = c.callee;
      Dt dt = Dt::F32;
      const bool has_dt = suffix_dtype(fn, &dt);
      auto need = [&](size_t n) {
        if (c.args.size() != n)
          reject("kernel " + f.name + ": " + fn + " expects " + std::to_string(n) + " operands, got " + std::to_string(c.args.size()));
      };
      if (fn == "__tile_pipe_barrier" || fn == "__tile_pipelined_for_begin" || fn == "__tile_pipelined_for_end" ||
          fn == "__tile_get_block_idx" || fn == "__tile_get_block_num" || fn == "get_block_idx" || fn == "get_block_num") {
        continue;  // scheduling hints and the per-block index: the launcher applies the per-block tile stride
      }
      if (starts_with(fn, "__tile_load_") && has_dt) {
        need(3);
        Tile t;
        t.kind = Kind::Load;
        t.dtype = dt;
        t.arg = cx.ptr_of(c.args[0]);
        t.rows = cx.int_of(c.args[1], "rows");
        t.cols = cx.int_of(c.args[2], "cols");
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_store_") && has_dt) {
        need(4);
        if (!stored_tile.empty()) reject("kernel " + f.name + ": more than one tile store; one operator per kernel is supported");
        store_arg = cx.ptr_of(c.args[0]);
        stored_tile = c.args[1];
        store_dt = dt;
        store_rows = cx.int_of(c.args[2], "rows");
        store_cols = cx.int_of(c.args[3], "cols");
      } else if (starts_with(fn, "__tile_cast_")) {
        need(4);
        // Arithmetic is f32 inside every kernel and values are rounded once, when they are stored.  A cast can
        // therefore be a relabel only where the reference's arith.extf / arith.truncf
        // (crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1249-1303) would not change a value either:
        //  * widening a freshly loaded 16-bit tile (exact), and
        //  * narrowing the result right before a store of the narrow type (the store is that rounding).
        // Anything else - an operator fed with narrowed values, a round trip through a 16-bit type - would need
        // a rounding in the middle of the kernel and is refused instead of being silently skipped.
        const std::string nm = fn.substr(std::strlen("__tile_cast_"));  // "f32_f16"
        const size_t us = nm.find('_');
        Dt from = Dt::F32, to = Dt::F32;
        if (us == std::string::npos || !suffix_dtype("_" + nm.substr(0, us), &from) || !suffix_dtype("_" + nm.substr(us + 1), &to))
          reject("kernel " + f.name + ": unknown cast " + fn);
        Tile t = cx.tile_of(c.args[1]);
        if (t.narrowed)
          reject("kernel " + f.name + ": " + fn + " casts a value that was already narrowed to " + dt_name(t.narrow_to) +
                 "; a round trip through a 16-bit type inside one kernel is not supported (values are rounded once, at the store)");
        if (from != Dt::F32 && to == Dt::F32) {
          if (t.kind != Kind::Load || t.dtype != from)
            reject("kernel " + f.name + ": " + fn + " must widen a freshly loaded " + dt_name(from) + " tile");
        } else if (from == Dt::F32 && to != Dt::F32) {
          t.narrowed = true;
          t.narrow_to = to;
        } else {
          reject("kernel " + f.name + ": " + fn + " is neither a widening nor a narrowing cast");
        }
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_softmax_") && has_dt) {
        need(4);
        Tile t;
        t.kind = Kind::Softmax;
        t.in = {c.args[1]};
        t.rows = cx.int_of(c.args[2], "rows");
        t.cols = cx.int_of(c.args[3], "cols");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_rms_norm_") && has_dt && !contains(fn, "_mul_") && fn.back() != '4') {
        need(5);  // (dst, src, eps, rows, cols)
        Tile t;
        t.kind = Kind::RmsNorm;
        t.in = {c.args[1]};
        auto it = cx.floats.find(c.args[2]);
        t.scalar = it == cx.floats.end() ? 1e-5 : it->second;  // the reference's NVIDIA emitter falls back to 1e-5
        t.rows = cx.int_of(c.args[3], "rows");
        t.cols = cx.int_of(c.args[4], "cols");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if ((starts_with(fn, "__tile_reduce_sum_") || starts_with(fn, "__tile_reduce_max_")) && has_dt) {
        need(4);  // (dst, src, rows, cols) -> a rows x 1 tile
        Tile t;
        t.kind = starts_with(fn, "__tile_reduce_sum_") ? Kind::ReduceSum : Kind::ReduceMax;
        t.in = {c.args[1]};
        t.rows = cx.int_of(c.args[2], "rows");
        t.cols = cx.int_of(c.args[3], "cols");  // width of the reduced tile; the result has one column
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (has_dt && ewise_arity(fn) != 0) {
        // element-wise intrinsics: (dst, a, b, rows, cols) / (dst, src, rows, cols); the reference's
        // SiLU*Mul fusion also accepts the four-operand product (a, b, rows, cols)
        const int arity = ewise_arity(fn);
        Tile t;
        t.kind = Kind::Ewise;
        t.ew = ewise_name(fn);
        size_t o = 1;
        if (arity == 2) {
          if (c.args.size() != 5 && !(t.ew == "mul" && c.args.size() == 4))
            reject("kernel " + f.name + ": " + fn + " expects 5 operands, got " + std::to_string(c.args.size()));
          if (c.args.size() == 4) o = 0;
          t.in = {c.args[o], c.args[o + 1]};
        } else {
          need(4);
          t.in = {c.args[1]};
        }
        t.rows = cx.int_of(c.args[o + arity], "rows");
        t.cols = cx.int_of(c.args[o + arity + 1], "cols");
        t.dtype = cx.tile_of(t.in[0]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_clamp_") && has_dt) {
        need(6);  // (dst, src, lo, hi, rows, cols)
        Tile t;
        t.kind = Kind::Ewise;
        t.ew = "clamp";
        t.in = {c.args[1]};
        auto lo = cx.floats.find(c.args[2]), hi = cx.floats.find(c.args[3]);
        if (lo == cx.floats.end() || hi == cx.floats.end())
          reject("kernel " + f.name + ": clamp bounds must be compile-time float constants");
        t.scalar = lo->second;
        t.scalar2 = hi->second;
        t.rows = cx.int_of(c.args[4], "rows");
        t.cols = cx.int_of(c.args[5], "cols");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_fill_") && has_dt) {
        need(4);  // (dst, scalar, rows, cols)
        Tile t;
        t.kind = Kind::Ewise;
        t.ew = "fill";
        auto it = cx.floats.find(c.args[1]);
        if (it == cx.floats.end()) reject("kernel " + f.name + ": the fill value must be a compile-time float constant");
        t.scalar = it->second;
        t.rows = cx.int_of(c.args[2], "rows");
        t.cols = cx.int_of(c.args[3], "cols");
        t.dtype = dt;
        cx.tiles[c.result] = t;
      } else if ((starts_with(fn, "__tile_matmul_transposed_") || starts_with(fn, "__tile_matmul_")) && has_dt &&
                 !contains(fn, "dequant") && !contains(fn, "_i8")) {
        need(6);
        Tile t;
        t.kind = starts_with(fn, "__tile_matmul_transposed_") ? Kind::MatmulT : Kind::Matmul;
        t.in = {c.args[1], c.args[2]};
        t.m = cx.int_of(c.args[3], "m");
        t.k = cx.int_of(c.args[4], "k");
        t.n = cx.int_of(c.args[5], "n");
        t.rows = t.m;
        t.cols = t.n;
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_transpose_") && has_dt) {
        need(4);
        Tile t;
        t.kind = Kind::Transpose;
        t.in = {c.args[1]};
        t.rows = cx.int_of(c.args[3], "cols");
        t.cols = cx.int_of(c.args[2], "rows");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_scale_") && has_dt) {
        need(5);
        Tile t;
        t.kind = Kind::Scale;
        t.in = {c.args[1]};
        auto it = cx.floats.find(c.args[2]);
        if (it == cx.floats.end()) reject("kernel " + f.name + ": scale factor " + c.args[2] + " is not a compile-time float constant");
        t.scalar = it->second;
        t.rows = cx.int_of(c.args[3], "rows");
        t.cols = cx.int_of(c.args[4], "cols");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_causal_mask_") && has_dt) {
        need(4);
        Tile t;
        t.kind = Kind::CausalMask;
        t.in = {c.args[1]};
        t.rows = cx.int_of(c.args[2], "rows");
        t.cols = cx.int_of(c.args[3], "cols");
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_attention_gqa_") && has_dt) {
        // operand order of the NVIDIA emitter: (dst, q, k, v, num_heads, num_kv_heads, seq_len, head_dim)
        need(8);
        Tile t;
        t.kind = Kind::AttentionGqa;
        t.in = {c.args[1], c.args[2], c.args[3]};
        t.heads = cx.int_of(c.args[4], "num_heads");
        t.kv_heads = cx.int_of(c.args[5], "num_kv_heads");
        t.seq = cx.int_of(c.args[6], "seq_len");
        t.dim = cx.int_of(c.args[7], "head_dim");
        t.rows = t.heads * t.seq;
        t.cols = t.dim;
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else if (starts_with(fn, "__tile_attention_") && has_dt) {
        need(6);
        Tile t;
        t.kind = Kind::Attention;
        t.in = {c.args[1], c.args[2], c.args[3]};
        t.heads = t.kv_heads = 1;
        t.seq = cx.int_of(c.args[4], "seq_len");
        t.dim = cx.int_of(c.args[5], "head_dim");
        t.rows = t.seq;
        t.cols = t.dim;
        t.dtype = cx.tile_of(c.args[1]).dtype;
        cx.tiles[c.result] = t;
      } else {
        reject("kernel " + f.name + ": intrinsic " + fn + " is outside the cuda_sm100 target (matmul, softmax, attention, rms_norm, row reductions, element-wise operators)");
      }
      continue;
    }
    // pointer arithmetic of the #[tile_kernel] prelude: the result aliases its base pointer
    if (contains(line, "llvm.getelementptr")) {
      const std::string res = result_of(line);
      const size_t p = line.find('%', line.find("getelementptr"));
      if (!res.empty() && p != std::string::npos) {
        size_t e = p + 1;
        while (e < line.size() && (isalnum(static_cast<unsigned char>(line[e])) || line[e] == '_')) ++e;
        auto it = cx.ptr_alias.find(line.substr(p, e - p));
        if (it != cx.ptr_alias.end()) cx.ptr_alias[res] = it->second;
      }
      continue;
    }
    // integer arithmetic and conversions feeding that pointer arithmetic carry no tile semantics
    static const char* kScalarOps[] = {"llvm.mul", "llvm.add", "llvm.sub", "llvm.zext", "llvm.sext", "llvm.trunc",
                                       "llvm.shl", "llvm.ptrtoint", "llvm.inttoptr", "llvm.bitcast", "llvm.and",
                                       "llvm.or", "llvm.udiv", "llvm.urem", "llvm.icmp", "llvm.select", "llvm.br",
                                       "llvm.unreachable", "llvm.intr.assume", "llvm.alloca", "llvm.store", "llvm.load"};
    bool scalar = false;
    for (const char* op : kScalarOps) scalar = scalar || contains(line, op);
    if (scalar) continue;
    reject("kernel " + f.name + ": unrecognised operation: " + line);
  }

  if (stored_tile.empty()) reject("kernel " + f.name + ": no tile store; nothing to compute");
  for (const auto& kv : cx.tiles)
    for (const std::string& in : kv.second.in) {
      auto it = cx.tiles.find(in);
      if (it != cx.tiles.end() && it->second.narrowed)
        reject("kernel " + f.name + ": an operator reads a value narrowed to " + dt_name(it->second.narrow_to) +
               " by a cast; it would see the unrounded f32 values here - cast after the operator, or load the narrow type");
    }
  const Tile& root = cx.tile_of(stored_tile);
  if (root.narrowed && root.narrow_to != store_dt)
    reject("kernel " + f.name + ": a value narrowed to " + dt_name(root.narrow_to) + " is stored as " + dt_name(store_dt));
  std::ostringstream body, inst, sum;
  const Dt out_dt = store_dt;

  auto load_of = [&](const std::string& ssa, const char* role) -> const Tile& {
    const Tile& t = cx.tile_of(ssa);
    if (t.kind != Kind::Load) reject("kernel " + f.name + ": the " + role + " operand must come straight from a tile load");
    return t;
  };

  if (root.kind == Kind::Softmax) {
    const Tile& x = load_of(root.in[0], "softmax input");
    if (x.rows != root.rows || x.cols != root.cols || store_rows != root.rows || store_cols != root.cols)
      reject("kernel " + f.name + ": softmax tile shapes disagree between load, op and store");
    if (out_dt != x.dtype) reject("kernel " + f.name + ": softmax input and output storage types differ");
    k.op = "softmax";
    sum << "__tile_softmax on " << root.rows << " x " << root.cols << " " << dt_name(x.dtype) << " tiles, one per block";
    body << "  tsm100_softmax_desc d;\n  d.dtype = " << dt_enum(x.dtype) << ";\n  d.rows = static_cast<int64_t>(blocks) * " << root.rows
         << ";\n  d.cols = " << root.cols << ";\n"
         << "  st = tsm100::ops::softmax(&msg, &d, args[" << x.arg << "], args[" << store_arg << "], stream);\n";
    const std::string direct = softmax_instantiation(x.dtype, root.cols);
    if (!direct.empty())
      inst << direct;
    else
      inst << "template __global__ void tsm100::softmax::softmax_rows_stream<" << cxx_type(x.dtype) << ", 512>(const "
           << cxx_type(x.dtype) << "*, " << cxx_type(x.dtype) << "*, int64_t, int64_t);\n";
  } else if (root.kind == Kind::RmsNorm) {
    const Tile& x = load_of(root.in[0], "rms_norm input");
    if (x.rows != root.rows || x.cols != root.cols || store_rows != root.rows || store_cols != root.cols)
      reject("kernel " + f.name + ": rms_norm tile shapes disagree between load, op and store");
    if (out_dt != x.dtype) reject("kernel " + f.name + ": rms_norm input and output storage types differ");
    k.op = "rms_norm";
    sum << "__tile_rms_norm on " << root.rows << " x " << root.cols << " " << dt_name(x.dtype) << " tiles, one per block";
    char eps_lit[48];
    snprintf(eps_lit, sizeof eps_lit, "%.9gf", static_cast<double>(static_cast<float>(root.scalar)));
    std::string eps_s = eps_lit;
    if (eps_s.find('.') == std::string::npos && eps_s.find('e') == std::string::npos) eps_s.insert(eps_s.size() - 1, ".0");
    body << "  tsm100_rms_norm_desc d;\n  d.dtype = " << dt_enum(x.dtype) << ";\n  d.rows = static_cast<int64_t>(blocks) * " << root.rows
         << ";\n  d.cols = " << root.cols << ";\n  d.eps = " << eps_s << ";\n"
         << "  st = tsm100::ops::rms_norm(&msg, &d, args[" << x.arg << "], args[" << store_arg << "], stream);\n";
    inst << row_op_instantiation(x.dtype, "kRmsNorm", root.cols);
  } else if (root.kind == Kind::ReduceSum || root.kind == Kind::ReduceMax) {
    const Tile& x = load_of(root.in[0], "reduce input");
    if (x.rows != root.rows || x.cols != root.cols || store_rows != root.rows || store_cols != 1)
      reject("kernel " + f.name + ": a row reduction stores a rows x 1 tile of the loaded tile's rows");
    if (out_dt != x.dtype) reject("kernel " + f.name + ": reduce input and output storage types differ");
    const bool is_max = root.kind == Kind::ReduceMax;
    k.op = "reduce";
    sum << "__tile_reduce_" << (is_max ? "max" : "sum") << " on " << root.rows << " x " << root.cols << " " << dt_name(x.dtype)
        << " tiles, one per block";
    body << "  tsm100_reduce_desc d;\n  d.dtype = " << dt_enum(x.dtype) << ";\n  d.kind = "
         << (is_max ? "TSM100_REDUCE_MAX" : "TSM100_REDUCE_SUM") << ";\n  d.rows = static_cast<int64_t>(blocks) * " << root.rows
         << ";\n  d.cols = " << root.cols << ";\n"
         << "  st = tsm100::ops::reduce(&msg, &d, args[" << x.arg << "], args[" << store_arg << "], stream);\n";
    inst << row_op_instantiation(x.dtype, is_max ? "kReduceMax" : "kReduceSum", root.cols);
  } else if (root.kind == Kind::Ewise || root.kind == Kind::Scale) {
    auto is_op = [](const Tile& t, const char* name) { return t.kind == Kind::Ewise && t.ew == name; };
    // silu(gate), or silu(gate) * up with the pair fused as the reference's NVIDIA emitter does:
    // the library's kernel
    const Tile* silu = nullptr;
    const Tile* up = nullptr;
    if (is_op(root, "silu") && cx.tile_of(root.in[0]).kind == Kind::Load) {
      silu = &root;
    } else if (is_op(root, "mul")) {
      const Tile& a = cx.tile_of(root.in[0]);
      const Tile& b = cx.tile_of(root.in[1]);
      if (is_op(a, "silu") && b.kind == Kind::Load && cx.tile_of(a.in[0]).kind == Kind::Load) { silu = &a; up = &b; }
      else if (is_op(b, "silu") && a.kind == Kind::Load && cx.tile_of(b.in[0]).kind == Kind::Load) { silu = &b; up = &a; }
    }
    const Tile* gate = silu ? &cx.tile_of(silu->in[0]) : nullptr;
    if (silu && out_dt == gate->dtype && (!up || up->dtype == gate->dtype)) {
      if (gate->rows != root.rows || gate->cols != root.cols || store_rows != root.rows || store_cols != root.cols ||
          (up && (up->rows != root.rows || up->cols != root.cols)))
        reject("kernel " + f.name + ": silu / mul tile shapes disagree between loads, ops and store");
      k.op = "silu_mul";
      sum << (up ? "__tile_silu * __tile_mul fused" : "__tile_silu") << " on " << root.rows << " x " << root.cols << " "
          << dt_name(gate->dtype) << " tiles, one per block";
      body << "  tsm100_silu_mul_desc d;\n  d.dtype = " << dt_enum(gate->dtype) << ";\n  d.rows = static_cast<int64_t>(blocks) * " << root.rows
           << ";\n  d.cols = " << root.cols << ";\n"
           << "  st = tsm100::ops::silu_mul(&msg, &d, args[" << gate->arg << "], " << (up ? "args[" + std::to_string(up->arg) + "]" : std::string("nullptr"))
           << ", args[" << store_arg << "], stream);\n";
      const std::string t = cxx_type(gate->dtype);
      const long per_vec = gate->dtype == Dt::F32 ? 4 : 8;
      if ((root.rows * root.cols) % per_vec == 0)
        inst << "template __global__ void tsm100::rowops::silu_mul_kernel<" << t << ", " << (up ? "true" : "false") << ", 4, 256>(const " << t
             << "*, const " << t << "*, " << t << "*, int64_t);\n";
      else
        inst << "template __global__ void tsm100::rowops::silu_mul_scalar_kernel<" << t << ", " << (up ? "true" : "false") << ", 256>(const " << t
             << "*, const " << t << "*, " << t << "*, int64_t);\n";
    } else {
      // Any other chain of element-wise operators between loads and the store: one generated
      // kernel, one pass over memory, f32 arithmetic, 16-byte accesses.
      if (store_rows != root.rows || store_cols != root.cols)
        reject("kernel " + f.name + ": element-wise tile shapes disagree between op and store");
      std::vector<std::pair<int, Dt>> inputs;     // distinct loaded pointers in order of first use
      std::map<std::string, std::string> value;   // tile SSA -> C++ value name
      std::map<std::string, std::string> leaf_name;  // loaded tile SSA -> "in<k>" for the summary line
      std::ostringstream stmts, text;
      int next_v = 0;
      std::function<std::string(const std::string&, std::string*)> gen = [&](const std::string& ssa, std::string* expr) -> std::string {
        auto done = value.find(ssa);
        if (done != value.end()) {  // a value used more than once is computed once
          if (expr) *expr = leaf_name.count(ssa) ? leaf_name[ssa] : done->second;
          return done->second;
        }
        const Tile& t = cx.tile_of(ssa);
        if (t.kind != Kind::Load && (t.rows != root.rows || t.cols != root.cols))
          reject("kernel " + f.name + ": element-wise operands must share the stored tile's shape");
        std::string rhs, shown;
        if (t.kind == Kind::Load) {
          if (t.rows != root.rows || t.cols != root.cols)
            reject("kernel " + f.name + ": element-wise operands must share the stored tile's shape (no broadcast)");
          size_t slot = 0;
          while (slot < inputs.size() && inputs[slot].first != t.arg) ++slot;
          if (slot == inputs.size()) inputs.push_back({t.arg, t.dtype});
          else if (inputs[slot].second != t.dtype) reject("kernel " + f.name + ": one pointer is loaded with two storage types");
          rhs = "a" + std::to_string(slot) + "[e]";
          shown = "in" + std::to_string(slot);
          leaf_name[ssa] = shown;
        } else if (t.kind == Kind::Scale) {
          std::string x;
          gen(t.in[0], &x);
          rhs = value[t.in[0]] + " * " + float_literal(t.scalar);
          shown = "scale(" + x + ", " + float_literal(t.scalar) + ")";
        } else if (t.kind == Kind::Ewise) {
          std::string x, y;
          if (!t.in.empty()) gen(t.in[0], &x);
          if (t.in.size() > 1) gen(t.in[1], &y);
          const std::string a = t.in.empty() ? "" : value[t.in[0]], b = t.in.size() > 1 ? value[t.in[1]] : "";
          const std::string& o = t.ew;
          if (o == "add") rhs = a + " + " + b;
          else if (o == "sub") rhs = a + " - " + b;
          else if (o == "mul") rhs = a + " * " + b;
          else if (o == "div") rhs = a + " / " + b;
          else if (o == "max") rhs = "fmaxf(" + a + ", " + b + ")";
          else if (o == "min") rhs = "fminf(" + a + ", " + b + ")";
          else if (o == "exp") rhs = "expf(" + a + ")";
          else if (o == "log") rhs = "logf(" + a + ")";
          else if (o == "neg") rhs = "-" + a;
          else if (o == "tanh") rhs = "tanhf(" + a + ")";
          else if (o == "abs") rhs = "fabsf(" + a + ")";
          else if (o == "sqrt") rhs = "sqrtf(" + a + ")";
          else if (o == "rsqrt") rhs = "tsm100::ewise::op_rsqrt(" + a + ")";
          else if (o == "sigmoid") rhs = "tsm100::ewise::op_sigmoid(" + a + ")";
          else if (o == "silu") rhs = "tsm100::ewise::op_silu(" + a + ")";
          else if (o == "relu") rhs = "tsm100::ewise::op_relu(" + a + ")";
          else if (o == "clamp") rhs = "tsm100::ewise::op_clamp(" + a + ", " + float_literal(t.scalar) + ", " + float_literal(t.scalar2) + ")";
          else if (o == "fill") rhs = float_literal(t.scalar);
          else reject("kernel " + f.name + ": element-wise operator " + o + " has no lowering");
          shown = o + "(" + (o == "fill" ? float_literal(t.scalar) : x) + (y.empty() ? "" : ", " + y) +
                  (o == "clamp" ? ", " + float_literal(t.scalar) + ", " + float_literal(t.scalar2) : "") + ")";
        } else {
          reject("kernel " + f.name + ": an element-wise chain may only consume loaded tiles and other element-wise results");
        }
        const std::string name = "v" + std::to_string(next_v++);
        stmts << "      const float " << name << " = " << rhs << ";\n";
        value[ssa] = name;
        if (expr) *expr = shown;
        return name;
      };
      std::string shown;
      const std::string result = gen(stored_tile, &shown);
      if (inputs.empty()) inputs.push_back({-1, out_dt});  // a pure fill: no input stream
      k.op = "ewise";
      sum << "element-wise chain fused into one pass: out = " << shown << " on " << root.rows << " x " << root.cols << " tiles, one per block";
      const std::string to = cxx_type(out_dt);
      std::ostringstream params, call_args, loads8, loads1, align;
      for (size_t i = 0; i < inputs.size(); ++i) {
        if (inputs[i].first < 0) continue;
        const std::string ti = cxx_type(inputs[i].second);
        params << "const " << ti << "* __restrict__ p" << i << ", ";
        call_args << "static_cast<const " << ti << "*>(args[" << inputs[i].first << "]), ";
        loads8 << "    float a" << i << "[8];\n    tsm100::ewise::load8(p" << i << ", i, a" << i << ");\n";
        loads1 << "    float a" << i << "[1] = {tsm100::ewise::load1(p" << i << ", i)};\n";
        align << " && tsm100::ops::aligned16(args[" << inputs[i].first << "])";
      }
      inst << "// out = " << shown << "\n"
           << "__global__ void __launch_bounds__(256) " << f.name << "_ewise_vec(" << params.str() << to << "* __restrict__ out, int64_t n8) {\n"
           << "  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;\n"
           << "  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += step) {\n"
           << loads8.str() << "    float r[8];\n#pragma unroll\n    for (int e = 0; e < 8; ++e) {\n"
           << stmts.str() << "      r[e] = " << result << ";\n    }\n    tsm100::ewise::store8(out, i, r);\n  }\n}\n"
           << "__global__ void __launch_bounds__(256) " << f.name << "_ewise_scalar(" << params.str() << to << "* __restrict__ out, int64_t n) {\n"
           << "  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;\n"
           << "  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {\n"
           << loads1.str() << "    const int e = 0;\n" << stmts.str() << "    tsm100::ewise::store1(out, i, " << result << ");\n  }\n}\n";
      body << "  const int64_t n = static_cast<int64_t>(blocks) * " << root.rows << " * " << root.cols << ";\n"
           << "  const bool vec = (n % 8 == 0)" << align.str() << " && tsm100::ops::aligned16(args[" << store_arg << "]);\n"
           << "  int sms = 0;\n  st = tsm100::ops::sm_count(&msg, &sms);\n"
           << "  if (st == TSM100_OK && n > 0) {\n"
           << "    cudaStream_t s = static_cast<cudaStream_t>(stream);\n"
           << "    const int64_t items = vec ? n / 8 : n;\n"
           << "    const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((items + 255) / 256, static_cast<int64_t>(sms) * 8)));\n"
           << "    if (vec) " << f.name << "_ewise_vec<<<grid, 256, 0, s>>>(" << call_args.str() << "static_cast<" << to << "*>(args[" << store_arg << "]), items);\n"
           << "    else " << f.name << "_ewise_scalar<<<grid, 256, 0, s>>>(" << call_args.str() << "static_cast<" << to << "*>(args[" << store_arg << "]), items);\n"
           << "    st = tsm100::ops::cuda_ok(&msg, cudaGetLastError(), \"" << f.name << " launch\");\n  }\n";
    }
  } else if (root.kind == Kind::Matmul || root.kind == Kind::MatmulT) {
    const Tile* prod = &root;
    bool causal_chain = false;
    // softmax(causal_mask(scale(Q K^T))) V : the decomposed causal attention
    const Tile& lhs = cx.tile_of(root.in[0]);
    if (root.kind == Kind::Matmul && lhs.kind == Kind::Softmax) {
      const Tile* t = &cx.tile_of(lhs.in[0]);
      bool masked = false;
      double scale = 1.0;
      bool scaled = false;
      for (int hop = 0; hop < 2; ++hop) {
        if (t->kind == Kind::CausalMask) { masked = true; t = &cx.tile_of(t->in[0]); }
        else if (t->kind == Kind::Scale) { scaled = true; scale = t->scalar; t = &cx.tile_of(t->in[0]); }
      }
      const Tile* qk = t;
      const Tile* qt = nullptr;
      const Tile* kt = nullptr;
      if (qk->kind == Kind::MatmulT) {
        qt = &cx.tile_of(qk->in[0]);
        kt = &cx.tile_of(qk->in[1]);
      } else if (qk->kind == Kind::Matmul && cx.tile_of(qk->in[1]).kind == Kind::Transpose) {
        qt = &cx.tile_of(qk->in[0]);
        kt = &cx.tile_of(cx.tile_of(qk->in[1]).in[0]);
      }
      if (qt && kt) {
        const Tile& vt = load_of(root.in[1], "attention V");
        if (qt->kind != Kind::Load || kt->kind != Kind::Load) reject("kernel " + f.name + ": attention Q and K must come straight from tile loads");
        const long seq = qk->m, dim = qk->k;
        if (qk->n != seq || vt.rows != seq || vt.cols != dim || root.k != seq || root.n != dim)
          reject("kernel " + f.name + ": decomposed attention with inconsistent shapes");
        const double want = 1.0 / std::sqrt(static_cast<double>(dim));
        if (!scaled || std::fabs(scale - want) > 1e-6 * want)
          reject("kernel " + f.name + ": decomposed attention must scale the scores by 1/sqrt(head_dim)");
        causal_chain = true;
        k.op = "attention";
        sum << "decomposed attention (matmul, scale" << (masked ? ", causal mask" : "") << ", softmax, matmul) fused: seq " << seq
            << ", head_dim " << dim << ", " << dt_name(qt->dtype) << ", one head per block";
        body << "  tsm100_attention_desc d;\n  d.dtype = " << dt_enum(qt->dtype) << ";\n  d.causal = " << (masked ? 1 : 0)
             << ";\n  d.batch = static_cast<int32_t>(blocks);\n  d.heads_q = 1;\n  d.heads_kv = 1;\n  d.seq = " << seq
             << ";\n  d.head_dim = " << dim << ";\n"
             << "  st = tsm100::ops::attention(&msg, &d, args[" << qt->arg << "], args[" << kt->arg << "], args[" << vt.arg
             << "], args[" << store_arg << "], status, stream);\n";
        if (out_dt != qt->dtype) reject("kernel " + f.name + ": attention input and output storage types differ");
        if (qt->dtype != Dt::F32 && dim == 128)
          inst << "template __global__ void tsm100::attn::attention_fwd_kernel<" << (qt->dtype == Dt::BF16 ? "true" : "false")
               << ">(const __grid_constant__ CUtensorMap, const __grid_constant__ CUtensorMap, const __grid_constant__ CUtensorMap, uint16_t*, const tsm100::attn::Params);\n";
        else
          inst << "template __global__ void tsm100::attn_simt::attention_simt_kernel<" << cxx_type(qt->dtype) << ">(const "
               << cxx_type(qt->dtype) << "*, const " << cxx_type(qt->dtype) << "*, const " << cxx_type(qt->dtype) << "*, "
               << cxx_type(qt->dtype) << "*, const tsm100::attn_simt::Params);\n";
      }
    }
    if (!causal_chain) {
      const Tile& a = load_of(prod->in[0], "matmul A");
      const Tile& b = load_of(prod->in[1], "matmul B");
      const bool bt = prod->kind == Kind::MatmulT;
      if (a.rows != prod->m || a.cols != prod->k || (bt ? (b.rows != prod->n || b.cols != prod->k) : (b.rows != prod->k || b.cols != prod->n)) ||
          store_rows != prod->m || store_cols != prod->n)
        reject("kernel " + f.name + ": matmul tile shapes disagree between loads, op and store");
      if (a.dtype != b.dtype) reject("kernel " + f.name + ": matmul operands have different storage types");
      if (!(out_dt == a.dtype || out_dt == Dt::F32)) reject("kernel " + f.name + ": matmul output must be the input type or f32");
      k.op = "gemm";
      sum << "__tile_matmul" << (bt ? "_transposed" : "") << " " << prod->m << " x " << prod->k << " x " << prod->n << ", "
          << dt_name(a.dtype) << " in, " << dt_name(out_dt) << " out, one problem per block";
      body << "  tsm100_gemm_desc d = {};\n  d.dtype = " << dt_enum(a.dtype) << ";\n  d.out_dtype = " << dt_enum(out_dt)
           << ";\n  d.b_transposed = " << (bt ? 1 : 0) << ";\n  d.batch = static_cast<int32_t>(blocks);\n  d.m = " << prod->m
           << ";\n  d.n = " << prod->n << ";\n  d.k = " << prod->k << ";\n"
           << "  st = tsm100::ops::gemm(&msg, &d, args[" << a.arg << "], args[" << b.arg << "], args[" << store_arg
           << "], status, stream);\n";
      const bool tma = a.dtype != Dt::F32 && prod->k % 8 == 0 && (bt || prod->n % 8 == 0) &&
                       (prod->n * (out_dt == Dt::F32 ? 4 : 2)) % 16 == 0;
      const bool tf32x3 = a.dtype == Dt::F32 && prod->k % 4 == 0 && (bt || prod->n % 4 == 0) && prod->n % 2 == 0;
      if (tf32x3)
        inst << "template __global__ void tsm100::gemm_tf32x3::gemm_tf32x3_kernel<" << (bt ? "true" : "false")
             << ">(const float*, const float*, float*, const tsm100::gemm_tf32x3::Params);\n";
      else if (tma)
        inst << "template __global__ void tsm100::gemm_tc::gemm_tc_kernel<" << cxx_type(out_dt) << ", " << (bt ? "true" : "false")
             << ", " << (a.dtype == Dt::BF16 ? "true" : "false") << ">(const __grid_constant__ CUtensorMap, const __grid_constant__ CUtensorMap, " << cxx_type(out_dt)
             << "*, const tsm100::gemm_tc::Params);\n";
      else
        inst << "template __global__ void tsm100::gemm_simt::gemm_simt_kernel<" << cxx_type(a.dtype) << ", " << cxx_type(out_dt)
             << ", 64, 64, 16, 4, 4>(const " << cxx_type(a.dtype) << "*, const " << cxx_type(a.dtype) << "*, " << cxx_type(out_dt)
             << "*, const tsm100::gemm_simt::Params);\n";
    }
  } else if (root.kind == Kind::Attention || root.kind == Kind::AttentionGqa) {
    const Tile& q = load_of(root.in[0], "attention Q");
    const Tile& kk = load_of(root.in[1], "attention K");
    const Tile& v = load_of(root.in[2], "attention V");
    const bool gqa = root.kind == Kind::AttentionGqa;
    if (q.dtype != kk.dtype || q.dtype != v.dtype || out_dt != q.dtype)
      reject("kernel " + f.name + ": attention tensors must share one storage type");
    if (gqa && (root.kv_heads <= 0 || root.heads % root.kv_heads != 0))
      reject("kernel " + f.name + ": num_heads must be a positive multiple of num_kv_heads");
    k.op = "attention";
    sum << (gqa ? "__tile_attention_gqa (causal)" : "__tile_attention") << ": heads " << root.heads << "/" << root.kv_heads << ", seq "
        << root.seq << ", head_dim " << root.dim << ", " << dt_name(q.dtype) << ", one " << (gqa ? "batch" : "head") << " per block";
    body << "  tsm100_attention_desc d;\n  d.dtype = " << dt_enum(q.dtype) << ";\n  d.causal = " << (gqa ? 1 : 0)
         << ";\n  d.batch = static_cast<int32_t>(blocks);\n  d.heads_q = " << root.heads << ";\n  d.heads_kv = " << root.kv_heads
         << ";\n  d.seq = " << root.seq << ";\n  d.head_dim = " << root.dim << ";\n"
         << "  st = tsm100::ops::attention(&msg, &d, args[" << q.arg << "], args[" << kk.arg << "], args[" << v.arg << "], args["
         << store_arg << "], status, stream);\n";
    if (q.dtype != Dt::F32 && root.dim == 128)
      inst << "template __global__ void tsm100::attn::attention_fwd_kernel<" << (q.dtype == Dt::BF16 ? "true" : "false")
           << ">(const __grid_constant__ CUtensorMap, const __grid_constant__ CUtensorMap, const __grid_constant__ CUtensorMap, uint16_t*, const tsm100::attn::Params);\n";
    else
      inst << "template __global__ void tsm100::attn_simt::attention_simt_kernel<" << cxx_type(q.dtype) << ">(const "
           << cxx_type(q.dtype) << "*, const " << cxx_type(q.dtype) << "*, const " << cxx_type(q.dtype) << "*, " << cxx_type(q.dtype)
           << "*, const tsm100::attn_simt::Params);\n";
  } else {
    reject("kernel " + f.name + ": the stored tile is not produced by an operator of the cuda_sm100 target");
  }
  k.summary = sum.str();
  k.descriptor = describe(f, cx, store_arg, store_dt, store_rows, store_cols);
  k.body = body.str();
  k.instantiation = inst.str();
  return k;
}

std::string emit_source(const std::string& mlir, std::vector<std::string>* names, std::string* descriptors = nullptr) {
  if (trim(mlir).empty()) reject("empty MLIR module");
  const std::vector<Func> funcs = parse_module(mlir);
  std::vector<Kernel> kernels;
  for (const Func& f : funcs)
    if (f.is_entry) kernels.push_back(lower(f));
  if (kernels.empty()) reject("no entry kernel (llvm.func with hacc.entry) found in the module");

  std::ostringstream o;
  o << "// Generated by the tile-rs `cuda_sm100` target. Do not edit.\n"
       "// Kernels: hand-written sm_100a (tcgen05 / TMEM / TMA) templates of libtile_sm100,\n"
       "// instantiated here for the shapes the module carries.\n"
       "// Compile: nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -O3 -lineinfo --expt-relaxed-constexpr \\\n"
       "//          -shared -Xcompiler -fPIC -I<tile_sm100>/csrc -cudart static -o <module>.so <this file>\n"
       "// Load with tsm100_module_load(); launch <kernel> with tsm100_launch(module, \"<kernel>\", blocks, args, nargs, stream).\n"
       "#include <algorithm>\n#include <cstdint>\n#include <cstdio>\n#include <string>\n\n#include \"ops.cuh\"\n\n";
  for (const Kernel& k : kernels) {
    o << "// ---- kernel " << k.name << ": " << k.summary << "\n";
    o << k.instantiation;
    o << "extern \"C\" int32_t " << k.name
      << "_launch(void** args, uint32_t nargs, uint32_t blocks, void* stream, uint32_t* status, char* err, size_t err_cap) {\n"
         "  std::string msg;\n  int32_t st = TSM100_OK;\n"
         "  if (nargs != "
      << k.nargs << "u || args == nullptr) {\n    st = TSM100_ERR_INVALID;\n    msg = \"" << k.name << " takes " << k.nargs
      << " global-memory pointers\";\n  } else {\n";
    // indent the body one more level
    std::istringstream bl(k.body);
    std::string l;
    while (std::getline(bl, l)) o << "  " << l << "\n";
    o << "  }\n  if (st != TSM100_OK && err != nullptr && err_cap > 0) snprintf(err, err_cap, \"%s\", msg.c_str());\n  return st;\n}\n\n";
    names->push_back(k.name);
  }
  if (descriptors) {
    *descriptors = "[";
    for (size_t i = 0; i < kernels.size(); ++i) *descriptors += (i ? ",\n " : "") + kernels[i].descriptor;
    *descriptors += "]";
  }
  return o.str();
}

int32_t copy_out(const std::string& s, char* buf, size_t cap, size_t* len) {
  if (len) *len = s.size();
  if (!buf || cap < s.size() + 1) return TSM100_ERR_BUFFER;
  std::memcpy(buf, s.data(), s.size());
  buf[s.size()] = '\0';
  return TSM100_OK;
}

}  // namespace

extern "C" {

const char* tsm100_target_name(void) { return "cuda_sm100"; }
const char* tsm100_target_ext(void) { return "cu"; }

int32_t tsm100_emit(const char* mlir, size_t mlir_len, char* source, size_t source_cap, size_t* source_len,
                    char* names, size_t names_cap, size_t* names_len) {
  if (!mlir && mlir_len) {
    tsm100::last_error_ref() = "null MLIR text";
    return TSM100_ERR_INVALID;
  }
  try {
    std::vector<std::string> kernel_names;
    const std::string src = emit_source(std::string(mlir ? mlir : "", mlir_len), &kernel_names);
    std::string joined;
    for (size_t i = 0; i < kernel_names.size(); ++i) joined += (i ? "\n" : "") + kernel_names[i];
    const int32_t a = copy_out(src, source, source_cap, source_len);
    const int32_t b = copy_out(joined, names, names_cap, names_len);
    if (a != TSM100_OK || b != TSM100_OK) {
      tsm100::last_error_ref() = "output buffer too small";
      return TSM100_ERR_BUFFER;
    }
    return TSM100_OK;
  } catch (const EmitFailure& e) {
    tsm100::last_error_ref() = e.msg;
    return TSM100_ERR_EMIT;
  } catch (const std::exception& e) {
    tsm100::last_error_ref() = std::string("emit failed: ") + e.what();
    return TSM100_ERR_EMIT;
  }
}

int32_t tsm100_emit_descriptors(const char* mlir, size_t mlir_len, char* json, size_t json_cap, size_t* json_len) {
  if (!mlir && mlir_len) {
    tsm100::last_error_ref() = "null MLIR text";
    return TSM100_ERR_INVALID;
  }
  try {
    std::vector<std::string> kernel_names;
    std::string desc;
    emit_source(std::string(mlir ? mlir : "", mlir_len), &kernel_names, &desc);
    if (copy_out(desc, json, json_cap, json_len) != TSM100_OK) {
      tsm100::last_error_ref() = "output buffer too small";
      return TSM100_ERR_BUFFER;
    }
    return TSM100_OK;
  } catch (const EmitFailure& e) {
    tsm100::last_error_ref() = e.msg;
    return TSM100_ERR_EMIT;
  } catch (const std::exception& e) {
    tsm100::last_error_ref() = std::string("emit failed: ") + e.what();
    return TSM100_ERR_EMIT;
  }
}

}  // extern "C"
