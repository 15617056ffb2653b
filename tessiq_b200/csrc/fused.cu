// Fused elementwise chains: the selector, the NVRTC instantiation and the launch.
//
// A fusion group arrives as a small text program (see tessiq_b200.h). The selector type-checks it,
// chooses a device sequence for every operation (the CUDA math library's function, or a
// hardware-approximation sequence in `math fast`), writes `tq_body` — one output element computed
// from one element of every operand, entirely in registers — and appends it to the hand-written
// tile loop and operand readers of fused_prelude.h. NVRTC compiles the result for sm_100a into
// four kernels: {128-bit vector, scalar} x {32-bit, 64-bit index}. The launch picks by pointer
// alignment and element count.
//
// This replaces the reference's string emitter (csrc/tessiq/codegen/cuda_emitter.cpp:212-255),
// which writes one thread per element, scalar loads and a 64-bit `%` per broadcast element.
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>

#include <cctype>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "common.h"
#include "fused_prelude.h"

namespace tq {
namespace {

// ---------------------------------------------------------------------------------------------
// NVRTC, opened at run time so that the library loads without it.

struct Nvrtc {
  using Program = void*;
  int (*create)(Program*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*compile)(Program, int, const char* const*) = nullptr;
  int (*cubin_size)(Program, size_t*) = nullptr;
  int (*cubin)(Program, char*) = nullptr;
  int (*log_size)(Program, size_t*) = nullptr;
  int (*log)(Program, char*) = nullptr;
  int (*destroy)(Program*) = nullptr;
  int (*version)(int*, int*) = nullptr;
  const char* (*error_string)(int) = nullptr;
  bool ok = false;
  std::string why;
};

const Nvrtc& nvrtc() {
  static Nvrtc api = [] {
    Nvrtc n;
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    void* handle = nullptr;
    for (const char* name : names) {
      handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (handle) break;
    }
    if (!handle) {
      n.why = std::string("cannot open libnvrtc: ") + (dlerror() ? dlerror() : "not found");
      return n;
    }
    auto bind = [&](auto& slot, const char* symbol) {
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(handle, symbol));
      return slot != nullptr;
    };
    n.ok = bind(n.create, "nvrtcCreateProgram") && bind(n.compile, "nvrtcCompileProgram") &&
           bind(n.cubin_size, "nvrtcGetCUBINSize") && bind(n.cubin, "nvrtcGetCUBIN") &&
           bind(n.log_size, "nvrtcGetProgramLogSize") && bind(n.log, "nvrtcGetProgramLog") &&
           bind(n.destroy, "nvrtcDestroyProgram") && bind(n.error_string, "nvrtcGetErrorString") &&
           bind(n.version, "nvrtcVersion");
    if (!n.ok) n.why = "libnvrtc lacks a symbol this library needs";
    return n;
  }();
  return api;
}

// ---------------------------------------------------------------------------------------------
// The program

enum class Cls { kF32, kF64, kI32, kI64, kBool };

Cls cls_of(tq_dtype d) {
  switch (d) {
    case TQ_F64: return Cls::kF64;
    case TQ_I32: return Cls::kI32;
    case TQ_I64: return Cls::kI64;
    case TQ_BOOL: return Cls::kBool;
    default: return Cls::kF32;  // f32, f16, bf16 compute in float
  }
}
const char* ctype(Cls c) {
  switch (c) {
    case Cls::kF32: return "float";
    case Cls::kF64: return "double";
    case Cls::kI32: return "int";
    case Cls::kI64: return "long long";
    default: return "bool";
  }
}
const char* storage_tag(tq_dtype d) {
  switch (d) {
    case TQ_F32: return "float";
    case TQ_F64: return "double";
    case TQ_F16: return "tq_f16_tag";
    case TQ_BF16: return "tq_bf16_tag";
    case TQ_I32: return "int";
    case TQ_I64: return "long long";
    default: return "tq_bool";
  }
}
bool is_float(Cls c) { return c == Cls::kF32 || c == Cls::kF64; }
bool is_int(Cls c) { return c == Cls::kI32 || c == Cls::kI64; }

bool parse_dtype(const std::string& text, tq_dtype* out) {
  static const std::map<std::string, tq_dtype> names = {
      {"f32", TQ_F32}, {"f64", TQ_F64}, {"f16", TQ_F16}, {"bf16", TQ_BF16},
      {"i32", TQ_I32}, {"i64", TQ_I64}, {"bool", TQ_BOOL}};
  auto it = names.find(text);
  if (it == names.end()) return false;
  *out = it->second;
  return true;
}

enum class Read { kSame, kRepeated, kCycled, kStrided };

struct Input {
  std::string name;
  tq_dtype dtype;
  Read read;
};
struct ScalarArg {
  std::string name;
  tq_dtype dtype;
};

struct Program {
  bool fast = true;
  std::vector<Input> inputs;
  std::vector<ScalarArg> scalars;
  std::string body;         // statements of tq_body
  std::string result;       // variable holding the output value
  tq_dtype result_dtype = TQ_F32;
  tq_dtype out_dtype = TQ_F32;
  int divisors = 0;
  int layouts = 0;
};

bool valid_name(const std::string& s) {
  if (s.empty() || std::isdigit(static_cast<unsigned char>(s[0])) || s[0] == '-' || s[0] == '+' || s[0] == '.') return false;
  for (char c : s) {
    if (!(std::isalnum(static_cast<unsigned char>(c)) || c == '_')) return false;
  }
  return s != "inf" && s != "nan";
}

// A literal as an expression of class `c`.
bool literal(const std::string& text, Cls c, std::string* out) {
  std::string lower;
  for (char ch : text) lower += static_cast<char>(std::tolower(static_cast<unsigned char>(ch)));
  const bool negative = !lower.empty() && lower[0] == '-';
  std::string magnitude = (negative || (!lower.empty() && lower[0] == '+')) ? lower.substr(1) : lower;
  if (magnitude == "inf" || magnitude == "infinity" || magnitude == "nan") {
    if (!is_float(c)) return false;
    const bool f = c == Cls::kF32;
    std::string base = magnitude == "nan" ? (f ? "TQ_NAN_F" : "TQ_NAN_D") : (f ? "TQ_INF_F" : "TQ_INF_D");
    *out = negative ? "(-" + base + ")" : base;
    return true;
  }
  if (lower == "true" || lower == "false") {
    *out = c == Cls::kBool ? lower : std::string("(") + ctype(c) + ")" + (lower == "true" ? "1" : "0");
    return true;
  }
  char* end = nullptr;
  const double value = std::strtod(text.c_str(), &end);
  if (end == text.c_str() || *end != '\0') return false;
  char buffer[64];
  switch (c) {
    case Cls::kF32: {
      // Nine significant digits identify a float; the suffix keeps the constant out of double.
      const float narrowed = static_cast<float>(value);
      if (std::isinf(narrowed)) { *out = narrowed < 0 ? "(-TQ_INF_F)" : "TQ_INF_F"; return true; }
      snprintf(buffer, sizeof(buffer), "%.9ef", static_cast<double>(narrowed));
      break;
    }
    case Cls::kF64: snprintf(buffer, sizeof(buffer), "%.17e", value); break;
    case Cls::kI32: snprintf(buffer, sizeof(buffer), "%d", static_cast<int>(value)); break;
    case Cls::kI64: snprintf(buffer, sizeof(buffer), "%lldLL", static_cast<long long>(value)); break;
    default: snprintf(buffer, sizeof(buffer), "%s", value != 0 ? "true" : "false"); break;
  }
  *out = std::string("(") + buffer + ")";
  return true;
}

struct Value {
  std::string variable;
  tq_dtype dtype;
  // A value known only as numerator / denominator: in `math fast` the logistic family
  // (sigmoid, silu, gelu_tanh, ...) is x / (1 + 2^t), and a product of such values needs one
  // reciprocal, not one per factor. The division is written out when something other than a
  // multiplication consumes the value.
  bool lazy = false;
  std::string numerator;
  std::string denominator;
};

tq_dtype promote(tq_dtype a, tq_dtype b) {
  if (a == b) return a;
  if (cls_of(a) == Cls::kF32 && cls_of(b) == Cls::kF32) return TQ_F32;
  return a;
}

std::string substitute(const std::string& pattern, const std::vector<std::string>& args) {
  std::string out;
  for (size_t i = 0; i < pattern.size(); ++i) {
    if (pattern[i] == '$' && i + 1 < pattern.size() && std::isdigit(static_cast<unsigned char>(pattern[i + 1]))) {
      out += args[pattern[i + 1] - '0'];
      ++i;
    } else {
      out += pattern[i];
    }
  }
  return out;
}

struct UnaryMath {
  const char* f32;
  const char* f32_fast;  // null: same as f32
  const char* f64;
};

// Float-only unary operations. Names and meanings are the reference's ops.toml rows; `round` is
// rint (half to even), `rsqrt` is 1/sqrt, `sigmoid` is 1/(1+exp(-x)), `gelu` is the erf form.
const std::map<std::string, UnaryMath>& unary_math() {
  static const std::map<std::string, UnaryMath> table = {
      {"sqrt", {"sqrtf($0)", nullptr, "sqrt($0)"}},
      {"tanh", {"tanhf($0)", nullptr, "tanh($0)"}},
      {"exp", {"expf($0)", "tq_exp_fast($0)", "exp($0)"}},
      {"expm1", {"expm1f($0)", nullptr, "expm1($0)"}},
      {"log", {"logf($0)", nullptr, "log($0)"}},
      {"log1p", {"log1pf($0)", nullptr, "log1p($0)"}},
      {"log2", {"log2f($0)", nullptr, "log2($0)"}},
      {"log10", {"log10f($0)", nullptr, "log10($0)"}},
      {"rsqrt", {"(1.0f / sqrtf($0))", nullptr, "(1.0 / sqrt($0))"}},
      {"reciprocal", {"(1.0f / $0)", nullptr, "(1.0 / $0)"}},
      {"sin", {"sinf($0)", nullptr, "sin($0)"}},
      {"cos", {"cosf($0)", nullptr, "cos($0)"}},
      {"tan", {"tanf($0)", nullptr, "tan($0)"}},
      {"asin", {"asinf($0)", nullptr, "asin($0)"}},
      {"acos", {"acosf($0)", nullptr, "acos($0)"}},
      {"atan", {"atanf($0)", nullptr, "atan($0)"}},
      {"sinh", {"sinhf($0)", nullptr, "sinh($0)"}},
      {"cosh", {"coshf($0)", nullptr, "cosh($0)"}},
      {"floor", {"floorf($0)", nullptr, "floor($0)"}},
      {"ceil", {"ceilf($0)", nullptr, "ceil($0)"}},
      {"trunc", {"truncf($0)", nullptr, "trunc($0)"}},
      {"round", {"rintf($0)", nullptr, "rint($0)"}},
      {"erf", {"erff($0)", nullptr, "erf($0)"}},
      {"erfc", {"erfcf($0)", nullptr, "erfc($0)"}},
      {"sigmoid", {"(1.0f / (1.0f + expf(-$0)))", nullptr, "(1.0 / (1.0 + exp(-$0)))"}},
      {"gelu", {"(0.5f * $0 * (1.0f + erff($0 * 0.70710678118654752440f)))", nullptr,
                "(0.5 * $0 * (1.0 + erf($0 * 0.70710678118654752440)))"}},
      {"gelu_tanh", {"tq_gelu_tanh_precise($0)", nullptr, "tq_gelu_tanh_precise($0)"}},
      {"silu", {"($0 / (1.0f + expf(-$0)))", nullptr, "($0 / (1.0 + exp(-$0)))"}},
      // csrc/custom_ops/fast_gelu/fast_gelu.cpp:23
      {"fast_gelu", {"($0 * (1.0f / (1.0f + expf(-1.702f * $0))))", nullptr,
                     "($0 * (1.0 / (1.0 + exp(-1.702 * $0))))"}},
  };
  return table;
}

// `math fast`, f32: the logistic family as numerator / denominator, the denominator being
// 1 + 2^t with t a polynomial of the argument (log2(e) folded into its constants), evaluated with
// ex2.approx.ftz. 0.5 (1 + tanh u) = 1 / (1 + exp(-2u)) turns gelu_tanh into the same form with no
// cancellation in the negative tail.
struct Quotient {
  const char* numerator;
  const char* denominator;
};
const std::map<std::string, Quotient>& fast_quotients() {
  static const std::map<std::string, Quotient> table = {
      {"sigmoid", {"1.0f", "(1.0f + tq_exp2_ftz(-1.4426950408889634f * $0))"}},
      {"silu", {"$0", "(1.0f + tq_exp2_ftz(-1.4426950408889634f * $0))"}},
      {"fast_gelu", {"$0", "(1.0f + tq_exp2_ftz(-2.4554669595930156f * $0))"}},
      // -2 sqrt(2/pi) log2(e) = -2.302208198144325
      {"gelu_tanh", {"$0", "(1.0f + tq_exp2_ftz(-2.302208198144325f * ($0 + 0.044715f * $0 * $0 * $0)))"}},
  };
  return table;
}

class Selector {
 public:
  tq_status parse(const char* text, Program* program) {
    program_ = program;
    {
      // How often each name is read: a value read once, by a multiplication, can stay a quotient.
      std::istringstream all(text);
      std::string raw_line;
      while (std::getline(all, raw_line)) {
        const size_t comment = raw_line.find('#');
        if (comment != std::string::npos) raw_line.resize(comment);
        std::istringstream words(raw_line);
        std::vector<std::string> t;
        for (std::string w; words >> w;) t.push_back(w);
        if (t.size() >= 3 && t[1] == "=") {
          for (size_t i = 3; i < t.size(); ++i) ++uses_[t[i]];
        } else if (t.size() == 3 && t[0] == "out") {
          uses_[t[1]] += 2;  // stored: must be a plain value
        }
      }
    }
    std::istringstream lines(text);
    std::string line;
    int number = 0;
    bool has_out = false;
    while (std::getline(lines, line)) {
      ++number;
      const size_t hash = line.find('#');
      if (hash != std::string::npos) line.resize(hash);
      std::istringstream words(line);
      std::vector<std::string> t;
      for (std::string w; words >> w;) t.push_back(w);
      if (t.empty()) continue;
      TQ_REQUIRE(!has_out, TQ_INVALID_ARGUMENT, "line %d: statements after `out`", number);
      tq_status status = TQ_OK;
      if (t[0] == "math") {
        TQ_REQUIRE(t.size() == 2 && (t[1] == "fast" || t[1] == "precise"), TQ_INVALID_ARGUMENT,
                   "line %d: expected `math fast` or `math precise`", number);
        program->fast = t[1] == "fast";
      } else if (t[0] == "in") {
        status = parse_in(t, number);
      } else if (t[0] == "scalar") {
        status = parse_scalar(t, number);
      } else if (t[0] == "out") {
        status = parse_out(t, number);
        has_out = true;
      } else if (t.size() >= 3 && t[1] == "=") {
        status = parse_step(t, number);
      } else {
        return fail(TQ_INVALID_ARGUMENT, "line %d: cannot parse `%s`", number, line.c_str());
      }
      if (status != TQ_OK) return status;
    }
    TQ_REQUIRE(has_out, TQ_INVALID_ARGUMENT, "the program has no `out` statement");
    return TQ_OK;
  }

 private:
  tq_status define(const std::string& name, tq_dtype dtype, int number) {
    TQ_REQUIRE(valid_name(name), TQ_INVALID_ARGUMENT, "line %d: `%s` is not a valid name", number, name.c_str());
    TQ_REQUIRE(values_.find(name) == values_.end(), TQ_INVALID_ARGUMENT, "line %d: `%s` is defined twice", number, name.c_str());
    values_[name] = Value{"v_" + name, dtype};
    return TQ_OK;
  }

  tq_status parse_in(const std::vector<std::string>& t, int number) {
    TQ_REQUIRE(t.size() == 4, TQ_INVALID_ARGUMENT, "line %d: expected `in <name> <dtype> <read>`", number);
    Input input;
    input.name = t[1];
    TQ_REQUIRE(parse_dtype(t[2], &input.dtype), TQ_INVALID_ARGUMENT, "line %d: unknown dtype `%s`", number, t[2].c_str());
    if (t[3] == "same") input.read = Read::kSame;
    else if (t[3] == "repeated") input.read = Read::kRepeated;
    else if (t[3] == "cycled") input.read = Read::kCycled;
    else if (t[3] == "strided") input.read = Read::kStrided;
    else return fail(TQ_INVALID_ARGUMENT, "line %d: unknown read kind `%s`", number, t[3].c_str());
    if (input.read == Read::kRepeated || input.read == Read::kCycled) ++program_->divisors;
    if (input.read == Read::kStrided) ++program_->layouts;
    TQ_REQUIRE(program_->inputs.size() < 16, TQ_UNSUPPORTED, "line %d: more than 16 inputs", number);
    TQ_REQUIRE(program_->layouts <= 4, TQ_UNSUPPORTED, "line %d: more than 4 strided inputs", number);
    program_->inputs.push_back(input);
    return define(input.name, input.dtype, number);
  }

  tq_status parse_scalar(const std::vector<std::string>& t, int number) {
    TQ_REQUIRE(t.size() == 3, TQ_INVALID_ARGUMENT, "line %d: expected `scalar <name> <dtype>`", number);
    ScalarArg scalar;
    scalar.name = t[1];
    TQ_REQUIRE(parse_dtype(t[2], &scalar.dtype), TQ_INVALID_ARGUMENT, "line %d: unknown dtype `%s`", number, t[2].c_str());
    TQ_REQUIRE(program_->scalars.size() < 16, TQ_UNSUPPORTED, "line %d: more than 16 scalars", number);
    program_->scalars.push_back(scalar);
    return define(scalar.name, scalar.dtype, number);
  }

  tq_status parse_out(const std::vector<std::string>& t, int number) {
    TQ_REQUIRE(t.size() == 3, TQ_INVALID_ARGUMENT, "line %d: expected `out <name> <dtype>`", number);
    auto it = values_.find(t[1]);
    TQ_REQUIRE(it != values_.end(), TQ_INVALID_ARGUMENT, "line %d: `%s` is not defined", number, t[1].c_str());
    TQ_REQUIRE(parse_dtype(t[2], &program_->out_dtype), TQ_INVALID_ARGUMENT, "line %d: unknown dtype `%s`", number, t[2].c_str());
    materialize(it->second);
    TQ_REQUIRE(cls_of(it->second.dtype) == cls_of(program_->out_dtype), TQ_INVALID_ARGUMENT,
               "line %d: a %s value cannot be stored as %s without a cast", number,
               dtype_name(it->second.dtype), dtype_name(program_->out_dtype));
    program_->result = it->second.variable;
    program_->result_dtype = it->second.dtype;
    return TQ_OK;
  }

  // Resolves the arguments of a step: values keep their class; literals take `literal_class`.
  tq_status resolve(const std::vector<std::string>& raw, int number, std::vector<std::string>* expr,
                    std::vector<tq_dtype>* dtypes, std::vector<bool>* is_value, Cls* value_class, bool* any_value) {
    *any_value = false;
    for (const std::string& a : raw) {
      auto it = values_.find(a);
      if (it != values_.end()) {
        if (!*any_value) *value_class = cls_of(it->second.dtype);
        *any_value = true;
      }
    }
    for (const std::string& a : raw) {
      auto it = values_.find(a);
      if (it != values_.end()) {
        materialize(it->second);
        expr->push_back(it->second.variable);
        dtypes->push_back(it->second.dtype);
        is_value->push_back(true);
      } else {
        TQ_REQUIRE(!valid_name(a), TQ_INVALID_ARGUMENT, "line %d: `%s` is not defined", number, a.c_str());
        expr->push_back(a);  // patched once the class is known
        dtypes->push_back(TQ_F32);
        is_value->push_back(false);
      }
    }
    return TQ_OK;
  }

  tq_status parse_step(const std::vector<std::string>& t, int number) {
    const std::string& result = t[0];
    const std::string& op = t[2];
    std::vector<std::string> raw(t.begin() + 3, t.end());

    if (op == "cast") {
      TQ_REQUIRE(raw.size() == 2, TQ_INVALID_ARGUMENT, "line %d: expected `<name> = cast <arg> <dtype>`", number);
      tq_dtype to;
      TQ_REQUIRE(parse_dtype(raw[1], &to), TQ_INVALID_ARGUMENT, "line %d: unknown dtype `%s`", number, raw[1].c_str());
      auto it = values_.find(raw[0]);
      TQ_REQUIRE(it != values_.end(), TQ_INVALID_ARGUMENT, "line %d: `%s` is not defined", number, raw[0].c_str());
      materialize(it->second);
      const Cls from = cls_of(it->second.dtype), target = cls_of(to);
      std::string e = it->second.variable;
      if (target == Cls::kBool) {
        e = from == Cls::kBool ? e : "(" + e + " != 0)";
      } else {
        e = std::string("((") + ctype(target) + ")" + e + ")";
        if (to == TQ_BF16 && it->second.dtype != TQ_BF16) e = "tq_round_bf16(" + e + ")";
        if (to == TQ_F16 && it->second.dtype != TQ_F16) e = "tq_round_f16(" + e + ")";
      }
      return emit(result, to, e, number);
    }

    if (program_->fast) {
      bool handled = false;
      if (tq_status s = fast_quotient_step(result, op, raw, number, &handled)) return s;
      if (handled) return TQ_OK;
    }

    std::vector<std::string> expr;
    std::vector<tq_dtype> dtypes;
    std::vector<bool> is_value;
    Cls cls = Cls::kF32;
    bool any_value = false;
    if (tq_status s = resolve(raw, number, &expr, &dtypes, &is_value, &cls, &any_value)) return s;
    TQ_REQUIRE(any_value, TQ_INVALID_ARGUMENT, "line %d: `%s` of constants only; fold it before the kernel", number, op.c_str());

    auto patch_literals = [&](Cls literal_class, size_t from = 0) -> tq_status {
      for (size_t i = from; i < expr.size(); ++i) {
        if (!is_value[i]) {
          std::string e;
          TQ_REQUIRE(literal(raw[i], literal_class, &e), TQ_INVALID_ARGUMENT,
                     "line %d: `%s` is not a %s constant", number, raw[i].c_str(), ctype(literal_class));
          expr[i] = e;
        } else {
          TQ_REQUIRE(cls_of(dtypes[i]) == literal_class, TQ_INVALID_ARGUMENT,
                     "line %d: `%s` mixes %s with %s operands; insert a cast", number, op.c_str(),
                     ctype(cls_of(dtypes[i])), ctype(literal_class));
        }
      }
      return TQ_OK;
    };
    auto value_dtype = [&](size_t from = 0) {
      bool first = true;
      tq_dtype d = TQ_F32;
      for (size_t i = from; i < expr.size(); ++i) {
        if (!is_value[i]) continue;
        d = first ? dtypes[i] : promote(d, dtypes[i]);
        first = false;
      }
      return d;
    };
    auto no_kernel = [&]() {
      return fail(TQ_UNSUPPORTED, "line %d: `%s` has no kernel for %s operands", number, op.c_str(), ctype(cls));
    };
    const char* zero = cls == Cls::kF32 ? "0.0f" : cls == Cls::kF64 ? "0.0" : cls == Cls::kI64 ? "0LL" : "0";

    // ---- unary ----
    if (expr.size() == 1) {
      const tq_dtype d = dtypes[0];
      auto math = unary_math().find(op);
      if (math != unary_math().end()) {
        if (!is_float(cls)) return no_kernel();
        const char* pattern = cls == Cls::kF64 ? math->second.f64
                              : (program_->fast && math->second.f32_fast) ? math->second.f32_fast
                                                                          : math->second.f32;
        return emit(result, d, substitute(pattern, expr), number);
      }
      if (op == "abs") {
        if (cls == Cls::kBool) return no_kernel();
        const char* pattern = cls == Cls::kF32 ? "fabsf($0)" : cls == Cls::kF64 ? "fabs($0)" : "($0 < 0 ? -$0 : $0)";
        return emit(result, d, substitute(pattern, expr), number);
      }
      if (op == "neg") {
        if (cls == Cls::kBool) return no_kernel();
        return emit(result, d, substitute("(-$0)", expr), number);
      }
      if (op == "relu") {
        // x < 0 ? 0 : x keeps NaN and -0.0 (ops.toml:62-68).
        if (cls == Cls::kBool) return no_kernel();
        return emit(result, d, "(" + expr[0] + " < " + zero + " ? " + zero + " : " + expr[0] + ")", number);
      }
      if (op == "logical_not") {
        return emit(result, TQ_BOOL, cls == Cls::kBool ? "(!" + expr[0] + ")" : "(" + expr[0] + " == 0)", number);
      }
      if (op == "bitwise_not") {
        if (cls == Cls::kBool) return emit(result, TQ_BOOL, "(!" + expr[0] + ")", number);
        if (is_int(cls)) return emit(result, d, "(~" + expr[0] + ")", number);
        return no_kernel();
      }
      return fail(TQ_UNSUPPORTED, "line %d: no unary operation named `%s`", number, op.c_str());
    }

    // ---- binary ----
    if (expr.size() == 2) {
      if (op == "logical_and" || op == "logical_or") {
        std::vector<std::string> truth;
        for (size_t i = 0; i < 2; ++i) {
          if (!is_value[i]) {
            std::string e;
            TQ_REQUIRE(literal(raw[i], Cls::kBool, &e), TQ_INVALID_ARGUMENT, "line %d: bad constant `%s`", number, raw[i].c_str());
            truth.push_back(e);
          } else {
            truth.push_back(cls_of(dtypes[i]) == Cls::kBool ? expr[i] : "(" + expr[i] + " != 0)");
          }
        }
        return emit(result, TQ_BOOL, "(" + truth[0] + (op == "logical_and" ? " && " : " || ") + truth[1] + ")", number);
      }
      if (tq_status s = patch_literals(cls)) return s;
      const tq_dtype d = value_dtype();
      if (op == "add" || op == "sub" || op == "mul") {
        if (cls == Cls::kBool) return no_kernel();
        const char* sign = op == "add" ? " + " : op == "sub" ? " - " : " * ";
        return emit(result, d, "(" + expr[0] + sign + expr[1] + ")", number);
      }
      if (op == "div") {
        if (!is_float(cls)) return no_kernel();
        return emit(result, d, "(" + expr[0] + " / " + expr[1] + ")", number);
      }
      if (op == "pow") {
        if (!is_float(cls)) return no_kernel();
        return emit(result, d, std::string(cls == Cls::kF32 ? "powf(" : "pow(") + expr[0] + ", " + expr[1] + ")", number);
      }
      if (op == "maximum" || op == "minimum") {
        if (cls == Cls::kBool) return no_kernel();
        if (is_float(cls)) {
          return emit(result, d, std::string(op == "maximum" ? "tq_maximum<" : "tq_minimum<") + ctype(cls) + ">(" + expr[0] + ", " + expr[1] + ")", number);
        }
        const char* compare = op == "maximum" ? " > " : " < ";
        return emit(result, d, "(" + expr[0] + compare + expr[1] + " ? " + expr[0] + " : " + expr[1] + ")", number);
      }
      static const std::map<std::string, const char*> compares = {
          {"gt", " > "}, {"ge", " >= "}, {"lt", " < "}, {"le", " <= "}, {"eq", " == "}, {"ne", " != "}};
      auto compare = compares.find(op);
      if (compare != compares.end()) {
        return emit(result, TQ_BOOL, "(" + expr[0] + compare->second + expr[1] + ")", number);
      }
      if (op == "swiglu") {
        // csrc/custom_ops/swiglu/swiglu.cpp:22
        if (!is_float(cls)) return no_kernel();
        const char* pattern = cls == Cls::kF64 ? "($0 / (1.0 + exp(-$0)) * $1)"
                                               : "($0 / (1.0f + expf(-$0)) * $1)";
        return emit(result, d, substitute(pattern, expr), number);
      }
      return fail(TQ_UNSUPPORTED, "line %d: no binary operation named `%s`", number, op.c_str());
    }

    // ---- ternary ----
    if (expr.size() == 3 && op == "where") {
      TQ_REQUIRE(is_value[0] && cls_of(dtypes[0]) == Cls::kBool, TQ_INVALID_ARGUMENT,
                 "line %d: the condition of `where` must be a bool value", number);
      TQ_REQUIRE(is_value[1] || is_value[2], TQ_INVALID_ARGUMENT, "line %d: `where` between two constants", number);
      const Cls branch = cls_of(is_value[1] ? dtypes[1] : dtypes[2]);
      if (tq_status s = patch_literals(branch, 1)) return s;
      return emit(result, value_dtype(1), "(" + expr[0] + " ? " + expr[1] + " : " + expr[2] + ")", number);
    }
    return fail(TQ_UNSUPPORTED, "line %d: no operation `%s` of %zu arguments", number, op.c_str(), expr.size());
  }

  // Writes numerator * (1 / denominator) for a value kept as a quotient, once.
  void materialize(Value& value) {
    if (!value.lazy) return;
    program_->body += "  const float " + value.variable + " = " + value.numerator + " * tq_rcp_ftz(" + value.denominator + ");\n";
    value.lazy = false;
  }

  // In `math fast`: a member of the logistic family becomes a quotient, and a multiplication with
  // a quotient operand multiplies numerators and denominators. Only f32-class values take part.
  tq_status fast_quotient_step(const std::string& result, const std::string& op, const std::vector<std::string>& raw,
                               int number, bool* handled) {
    *handled = false;
    auto float_value = [&](const std::string& name) -> Value* {
      auto it = values_.find(name);
      if (it == values_.end() || cls_of(it->second.dtype) != Cls::kF32) return nullptr;
      return &it->second;
    };
    auto quotient = fast_quotients().find(op);
    if (quotient != fast_quotients().end() && raw.size() == 1) {
      Value* x = float_value(raw[0]);
      if (x == nullptr) return TQ_OK;
      materialize(*x);
      return define_quotient(result, x->dtype, substitute(quotient->second.numerator, {x->variable}),
                             substitute(quotient->second.denominator, {x->variable}), number, handled);
    }
    if (op == "swiglu" && raw.size() == 2) {  // gate / (1 + exp(-gate)) * up
      Value* gate = float_value(raw[0]);
      Value* up = float_value(raw[1]);
      if (gate == nullptr || up == nullptr) return TQ_OK;
      materialize(*gate);
      materialize(*up);
      return define_quotient(result, promote(gate->dtype, up->dtype), "(" + gate->variable + " * " + up->variable + ")",
                             "(1.0f + tq_exp2_ftz(-1.4426950408889634f * " + gate->variable + "))", number, handled);
    }
    if (op == "mul" && raw.size() == 2) {
      Value* a = float_value(raw[0]);
      Value* b = float_value(raw[1]);
      if (a == nullptr || b == nullptr || (!a->lazy && !b->lazy)) return TQ_OK;
      const std::string numerator = "(" + (a->lazy ? a->numerator : a->variable) + " * " + (b->lazy ? b->numerator : b->variable) + ")";
      const std::string denominator = a->lazy && b->lazy ? "(" + a->denominator + " * " + b->denominator + ")"
                                      : a->lazy          ? a->denominator
                                                         : b->denominator;
      const tq_dtype dtype = promote(a->dtype, b->dtype);
      // The operands were read exactly once (that is why they are still quotients): consumed here.
      a->lazy = b->lazy = false;
      return define_quotient(result, dtype, numerator, denominator, number, handled);
    }
    return TQ_OK;
  }

  tq_status define_quotient(const std::string& name, tq_dtype dtype, const std::string& numerator,
                            const std::string& denominator, int number, bool* handled) {
    if (tq_status s = define(name, dtype, number)) return s;
    Value& value = values_[name];
    // Name both halves so that they are computed once wherever the division ends up.
    program_->body += "  const float v_" + name + "_n = " + numerator + ";\n";
    program_->body += "  const float v_" + name + "_d = " + denominator + ";\n";
    value.lazy = true;
    value.numerator = "v_" + name + "_n";
    value.denominator = "v_" + name + "_d";
    if (uses_[name] != 1) materialize(value);  // read more than once, stored, or never: a plain value
    *handled = true;
    return TQ_OK;
  }

  tq_status emit(const std::string& name, tq_dtype dtype, const std::string& expression, int number) {
    if (tq_status s = define(name, dtype, number)) return s;
    program_->body += std::string("  const ") + ctype(cls_of(dtype)) + " v_" + name + " = " + expression + ";\n";
    return TQ_OK;
  }

  Program* program_ = nullptr;
  std::map<std::string, Value> values_;
  std::map<std::string, int> uses_;
};

// ---------------------------------------------------------------------------------------------
// Source generation

int vector_width(const Program& p) {
  int smallest = dtype_size(p.out_dtype);
  for (const Input& in : p.inputs) {
    if (dtype_size(in.dtype) < smallest) smallest = dtype_size(in.dtype);
  }
  int vec = 16 / smallest;
  if (vec > 8) vec = 8;
  return vec;
}

int unroll_for(const Program& p, int vec) {
  // Registers that hold operands between the load phase and the compute phase.
  int words = 0;
  for (const Input& in : p.inputs) words += vec * (cls_of(in.dtype) == Cls::kF64 || cls_of(in.dtype) == Cls::kI64 ? 2 : 1);
  // Measured on config 1 (two 4-byte operands, 8 words): 2 tiles of loads per thread beat 4
  // (23.0 us against 24.4 us) — smaller CTAs retire and refill at a finer grain.
  // Vectors of 8 or 16 narrow elements already mean 8-16 conversions and results per load: one tile
  // per thread measured best for them at 2^28 elements (bf16 six-op chain 6.84 against 6.13 TB/s with
  // two, row broadcast 5.94 against 5.28, plain add 6.88 against 6.83).
  if (vec >= 8) return 1;
  if (words <= 4) return 4;
  if (words <= 24) return 2;
  return 1;
}

std::string generate(const Program& p) {
  const int vec = vector_width(p);
  const int unroll = unroll_for(p, vec);
  const int scalar_unroll = 4;
  std::ostringstream s;
  s << kFusedPrelude;
  s << "\n// ---- selected for this fusion group ----\n";
  s << "#define TQ_VEC " << vec << "\n#define TQ_UNROLL " << unroll << "\n#define TQ_UNROLL_SCALAR " << scalar_unroll << "\n";
  for (size_t k = 0; k < p.inputs.size(); ++k) s << "typedef " << storage_tag(p.inputs[k].dtype) << " tq_s" << k << ";\n";
  s << "typedef " << storage_tag(p.out_dtype) << " tq_so;\n";

  // tq_body
  s << "TQ_DEV void tq_body(";
  for (size_t k = 0; k < p.inputs.size(); ++k) s << "const " << ctype(cls_of(p.inputs[k].dtype)) << " v_" << p.inputs[k].name << ", ";
  for (const ScalarArg& a : p.scalars) s << "const " << ctype(cls_of(a.dtype)) << " v_" << a.name << ", ";
  s << ctype(cls_of(p.out_dtype)) << "& tq_result) {\n" << p.body << "  tq_result = " << p.result << ";\n}\n\n";

  // parameter lists
  std::ostringstream params, forward, tile_params;
  for (size_t k = 0; k < p.inputs.size(); ++k) {
    params << "const void* __restrict__ p" << k << ", ";
    tile_params << "const void* __restrict__ p" << k << ", ";
    forward << "p" << k << ", ";
  }
  params << "void* __restrict__ po, long long n";
  tile_params << "void* __restrict__ po, Index n";
  forward << "po, (Index)n";
  int divisor = 0, layout = 0;
  for (const Input& in : p.inputs) {
    if (in.read == Read::kRepeated || in.read == Read::kCycled) {
      params << ", long long d" << divisor << ", unsigned long long m" << divisor;
      tile_params << ", Index d" << divisor << ", unsigned long long m" << divisor;
      forward << ", (Index)d" << divisor << ", m" << divisor;
      ++divisor;
    }
  }
  for (const Input& in : p.inputs) {
    if (in.read == Read::kStrided) {
      params << ", const tq_layout_t l" << layout;
      tile_params << ", const tq_layout_t& l" << layout;
      forward << ", l" << layout;
      ++layout;
    }
  }
  params << ", unsigned flags";
  tile_params << ", unsigned flags";
  forward << ", flags";
  for (const ScalarArg& a : p.scalars) {
    params << ", " << ctype(cls_of(a.dtype)) << " v_" << a.name;
    tile_params << ", " << ctype(cls_of(a.dtype)) << " v_" << a.name;
    forward << ", v_" << a.name;
  }

  auto reads = [&](const char* width, const char* index, const char* target, const char* target_suffix) {
    std::ostringstream r;
    int d = 0, l = 0;
    for (size_t k = 0; k < p.inputs.size(); ++k) {
      const Input& in = p.inputs[k];
      switch (in.read) {
        case Read::kSame:
          r << "      tq_read_same<tq_s" << k << ", " << width << ", Index>(p" << k << ", " << index << ", " << target << k << target_suffix << ");\n";
          break;
        case Read::kCycled:
          r << "      tq_read_cycled<tq_s" << k << ", " << width << ", Index>(p" << k << ", " << index << ", d" << d << ", m" << d << ", (flags >> " << k << ") & 1u, " << target << k << target_suffix << ");\n";
          ++d;
          break;
        case Read::kRepeated:
          r << "      tq_read_repeated<tq_s" << k << ", " << width << ", Index>(p" << k << ", " << index << ", d" << d << ", m" << d << ", (flags >> " << k << ") & 1u, " << target << k << target_suffix << ");\n";
          ++d;
          break;
        case Read::kStrided:
          r << "      tq_read_strided<tq_s" << k << ", " << width << ", Index>(p" << k << ", " << index << ", l" << l++ << ", (flags >> " << k << ") & 1u, " << target << k << target_suffix << ");\n";
          break;
      }
    }
    return r.str();
  };
  auto body_call = [&](const char* element, const char* result) {
    std::ostringstream c;
    c << "tq_body(";
    for (size_t k = 0; k < p.inputs.size(); ++k) c << "a" << k << element << ", ";
    for (const ScalarArg& a : p.scalars) c << "v_" << a.name << ", ";
    c << result << ");";
    return c.str();
  };

  // The tile loop: every load of a tile is issued before the first use, so each thread keeps
  // UNROLL x (operands) 128-bit requests in flight.
  s << "template <typename Index, int VEC, int UNROLL>\nTQ_DEV void tq_tile(" << tile_params.str() << ") {\n";
  s << "  const Index tile = (Index)TQ_BLOCK * VEC * UNROLL;\n  const Index base = (Index)blockIdx.x * tile;\n";
  for (size_t k = 0; k < p.inputs.size(); ++k) {
    s << "  tq_storage<tq_s" << k << ">::compute a" << k << "[UNROLL][VEC];\n";
  }
  s << "  bool whole[UNROLL];\n#pragma unroll\n  for (int u = 0; u < UNROLL; ++u) {\n";
  s << "    const Index idx = base + ((Index)u * TQ_BLOCK + threadIdx.x) * VEC;\n";
  s << "    whole[u] = idx + VEC <= n;\n    if (whole[u]) {\n" << reads("VEC", "idx", "a", "[u]") << "    }\n  }\n";
  s << "#pragma unroll\n  for (int u = 0; u < UNROLL; ++u) {\n";
  s << "    const Index idx = base + ((Index)u * TQ_BLOCK + threadIdx.x) * VEC;\n";
  s << "    if (whole[u]) {\n      tq_storage<tq_so>::compute r[VEC];\n#pragma unroll\n      for (int e = 0; e < VEC; ++e) { "
    << body_call("[u][e]", "r[e]") << " }\n      tq_write<tq_so, VEC, Index>(po, idx, r);\n    }\n  }\n";
  // The ragged end: fewer than VEC elements, taken one at a time by the thread they fall to.
  s << "  if (VEC > 1) {\n#pragma unroll\n    for (int u = 0; u < UNROLL; ++u) {\n";
  s << "      const Index idx = base + ((Index)u * TQ_BLOCK + threadIdx.x) * VEC;\n";
  s << "      if (!whole[u] && idx < n) {\n        for (Index i = idx; i < n; ++i) {\n";
  for (size_t k = 0; k < p.inputs.size(); ++k) s << "          tq_storage<tq_s" << k << ">::compute b" << k << "[1];\n";
  s << reads("1", "i", "b", "");
  s << "          tq_storage<tq_so>::compute r[1];\n          ";
  {
    std::ostringstream c;
    c << "tq_body(";
    for (size_t k = 0; k < p.inputs.size(); ++k) c << "b" << k << "[0], ";
    for (const ScalarArg& a : p.scalars) c << "v_" << a.name << ", ";
    c << "r[0]);";
    s << c.str();
  }
  s << "\n          tq_write<tq_so, 1, Index>(po, i, r);\n        }\n      }\n    }\n  }\n}\n\n";

  const char* names[4] = {"tq_fused_v32", "tq_fused_v64", "tq_fused_s32", "tq_fused_s64"};
  const char* index_types[4] = {"unsigned", "long long", "unsigned", "long long"};
  const char* widths[4] = {"TQ_VEC", "TQ_VEC", "1", "1"};
  const char* unrolls[4] = {"TQ_UNROLL", "TQ_UNROLL", "TQ_UNROLL_SCALAR", "TQ_UNROLL_SCALAR"};
  for (int i = 0; i < 4; ++i) {
    s << "extern \"C\" __global__ void __launch_bounds__(TQ_BLOCK) " << names[i] << "(" << params.str() << ") {\n";
    s << "  typedef " << index_types[i] << " Index;\n";
    s << "  tq_tile<Index, " << widths[i] << ", " << unrolls[i] << ">(" << forward.str() << ");\n}\n";
  }
  return s.str();
}

// ---------------------------------------------------------------------------------------------
// Compilation and loading

struct Module {
  std::string source;
  std::string cubin;
  std::mutex mutex;
  cudaLibrary_t library = nullptr;
  cudaKernel_t kernels[4] = {nullptr, nullptr, nullptr, nullptr};
};

// ---------------------------------------------------------------------------------------------
// On-disk cubin cache, as in the reference (csrc/tessiq/codegen/cubin_cache.cpp:43-64,98-168): the
// key is FNV-1a over the source, the architecture and the NVRTC version (the source already
// contains the whole template library, so a library change changes the key); files are written to a
// temporary name and renamed; a cache that cannot be read or written is not an error.

std::atomic<long long> g_cache_hits{0}, g_cache_misses{0}, g_cache_stores{0};

std::string cache_directory() {
  if (const char* dir = std::getenv("TESSIQ_CACHE_DIR")) return dir[0] ? std::string(dir) : std::string();
  if (const char* home = std::getenv("HOME")) return std::string(home) + "/.cache/tessiq_b200";
  return std::string();
}

std::string cache_path(const std::string& source) {
  const std::string dir = cache_directory();
  if (dir.empty()) return std::string();
  int major = 0, minor = 0;
  if (nvrtc().ok) nvrtc().version(&major, &minor);
  const std::string salt = "|sm_100a|nvrtc " + std::to_string(major) + "." + std::to_string(minor);
  uint64_t hash = 1469598103934665603ull;
  auto mix = [&](const std::string& text) {
    for (unsigned char c : text) {
      hash ^= c;
      hash *= 1099511628211ull;
    }
  };
  mix(source);
  mix(salt);
  char name[32];
  snprintf(name, sizeof(name), "%016llx", static_cast<unsigned long long>(hash));
  return dir + "/" + name + ".sm_100a.cubin";
}

bool cache_load(const std::string& path, std::string* cubin) {
  if (path.empty()) return false;
  FILE* file = fopen(path.c_str(), "rb");
  if (!file) return false;
  std::string data;
  char buffer[65536];
  size_t got;
  while ((got = fread(buffer, 1, sizeof(buffer), file)) > 0) data.append(buffer, got);
  fclose(file);
  if (data.size() < 64 || data.compare(0, 4, "\x7f" "ELF") != 0) return false;  // a cubin is an ELF image
  *cubin = std::move(data);
  return true;
}

void cache_store(const std::string& path, const std::string& cubin) {
  if (path.empty()) return;
  const std::string dir = path.substr(0, path.rfind('/'));
  std::string partial;
  for (size_t i = 1; i <= dir.size(); ++i) {  // mkdir -p
    if (i == dir.size() || dir[i] == '/') {
      partial = dir.substr(0, i);
      mkdir(partial.c_str(), 0755);
    }
  }
  const std::string temporary = path + ".tmp." + std::to_string(static_cast<long long>(getpid()));
  FILE* file = fopen(temporary.c_str(), "wb");
  if (!file) return;
  const bool written = fwrite(cubin.data(), 1, cubin.size(), file) == cubin.size();
  fclose(file);
  if (written && rename(temporary.c_str(), path.c_str()) == 0) {
    ++g_cache_stores;
  } else {
    remove(temporary.c_str());
  }
}

tq_status compile(const std::string& source, std::string* cubin) {
  const Nvrtc& n = nvrtc();
  TQ_REQUIRE(n.ok, TQ_EXTERNAL, "NVRTC is not available: %s", n.why.c_str());
  const std::string cached = cache_path(source);
  if (cache_load(cached, cubin)) {
    ++g_cache_hits;
    return TQ_OK;
  }
  ++g_cache_misses;
  Nvrtc::Program program = nullptr;
  int status = n.create(&program, source.c_str(), "tq_fused.cu", 0, nullptr, nullptr);
  TQ_REQUIRE(status == 0, TQ_EXTERNAL, "nvrtcCreateProgram failed: %s", n.error_string(status));
  const char* options[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "-lineinfo"};
  status = n.compile(program, 4, options);
  if (status != 0) {
    size_t size = 0;
    n.log_size(program, &size);
    std::string log(size, '\0');
    if (size) n.log(program, log.data());
    n.destroy(&program);
    return fail(TQ_EXTERNAL, "NVRTC could not compile the fused kernel (%s):\n%.800s", n.error_string(status), log.c_str());
  }
  size_t size = 0;
  status = n.cubin_size(program, &size);
  if (status == 0 && size > 0) {
    cubin->resize(size);
    status = n.cubin(program, cubin->data());
  }
  n.destroy(&program);
  TQ_REQUIRE(status == 0 && size > 0, TQ_EXTERNAL, "NVRTC produced no cubin: %s", n.error_string(status));
  cache_store(cached, *cubin);
  return TQ_OK;
}

std::mutex g_cache_mutex;
std::map<std::string, std::shared_ptr<Module>>& module_cache() {
  static std::map<std::string, std::shared_ptr<Module>> cache;
  return cache;
}

tq_status load(Module* module) {
  std::lock_guard<std::mutex> lock(module->mutex);
  if (module->library != nullptr) return TQ_OK;
  cudaLibrary_t library = nullptr;
  TQ_CUDA(cudaLibraryLoadData(&library, module->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  const char* names[4] = {"tq_fused_v32", "tq_fused_v64", "tq_fused_s32", "tq_fused_s64"};
  for (int i = 0; i < 4; ++i) TQ_CUDA(cudaLibraryGetKernel(&module->kernels[i], library, names[i]));
  module->library = library;
  return TQ_OK;
}

}  // namespace
}  // namespace tq

struct tq_fused {
  tq::Program program;
  std::shared_ptr<tq::Module> module;
  int vec = 1;
  int unroll = 1;
};

extern "C" {

tq_status tq_fused_create(const char* program_text, tq_fused** kernel) {
  TQ_REQUIRE(program_text != nullptr && kernel != nullptr, TQ_INVALID_ARGUMENT, "null program or out-pointer");
  auto fused = std::make_unique<tq_fused>();
  tq::Selector selector;
  if (tq_status s = selector.parse(program_text, &fused->program)) return s;
  fused->vec = tq::vector_width(fused->program);
  fused->unroll = tq::unroll_for(fused->program, fused->vec);
  const std::string source = tq::generate(fused->program);
  {
    std::lock_guard<std::mutex> lock(tq::g_cache_mutex);
    auto it = tq::module_cache().find(source);
    if (it != tq::module_cache().end()) fused->module = it->second;
  }
  if (!fused->module) {
    auto module = std::make_shared<tq::Module>();
    module->source = source;
    if (tq_status s = tq::compile(source, &module->cubin)) return s;
    std::lock_guard<std::mutex> lock(tq::g_cache_mutex);
    auto inserted = tq::module_cache().emplace(source, module);
    fused->module = inserted.first->second;
  }
  *kernel = fused.release();
  return TQ_OK;
}

tq_status tq_cubin_cache_stats(int64_t* hits, int64_t* misses, int64_t* stores) {
  if (hits) *hits = tq::g_cache_hits.load();
  if (misses) *misses = tq::g_cache_misses.load();
  if (stores) *stores = tq::g_cache_stores.load();
  return TQ_OK;
}

tq_status tq_fused_destroy(tq_fused* kernel) {
  delete kernel;  // the compiled module stays cached for the life of the process
  return TQ_OK;
}

tq_status tq_fused_source(const tq_fused* kernel, char* buffer, size_t capacity, size_t* length) {
  TQ_REQUIRE(kernel != nullptr, TQ_INVALID_ARGUMENT, "null kernel");
  const std::string& source = kernel->module->source;
  if (length) *length = source.size();
  if (buffer && capacity) {
    const size_t n = source.size() < capacity - 1 ? source.size() : capacity - 1;
    std::memcpy(buffer, source.data(), n);
    buffer[n] = '\0';
  }
  return TQ_OK;
}

tq_status tq_fused_launch(const tq_fused* kernel, const void* const* inputs, void* out, int64_t elements,
                          const int64_t* divisors, const tq_layout* layouts, const double* scalars,
                          int32_t device, void* stream) {
  TQ_REQUIRE(kernel != nullptr, TQ_INVALID_ARGUMENT, "null kernel");
  TQ_REQUIRE(elements >= 0, TQ_INVALID_ARGUMENT, "negative element count %lld", (long long)elements);
  if (tq::recording()) {
    // Recorded: the argument arrays are copied, the kernel handle and the data pointers are kept.
    const tq::Program& q = kernel->program;
    TQ_REQUIRE((q.inputs.empty() || inputs != nullptr) && (q.divisors == 0 || divisors != nullptr) &&
                   (q.layouts == 0 || layouts != nullptr) && (q.scalars.empty() || scalars != nullptr),
               TQ_INVALID_ARGUMENT, "a null argument array cannot be recorded");
    std::vector<const void*> kept_inputs(inputs, inputs + q.inputs.size());
    std::vector<int64_t> kept_divisors(divisors, divisors + q.divisors);
    std::vector<tq_layout> kept_layouts(layouts, layouts + q.layouts);
    std::vector<double> kept_scalars(scalars, scalars + q.scalars.size());
    return tq::record([=](int32_t d, void* s) {
      return tq_fused_launch(kernel, kept_inputs.data(), out, elements, kept_divisors.data(), kept_layouts.data(),
                             kept_scalars.data(), d, s);
    });
  }
  if (elements == 0) return TQ_OK;
  const tq::Program& p = kernel->program;
  TQ_REQUIRE(out != nullptr && (p.inputs.empty() || inputs != nullptr), TQ_INVALID_ARGUMENT, "null input or output");
  TQ_REQUIRE(p.divisors == 0 || divisors != nullptr, TQ_INVALID_ARGUMENT, "the kernel reads broadcast operands and was given no divisors");
  TQ_REQUIRE(p.layouts == 0 || layouts != nullptr, TQ_INVALID_ARGUMENT, "the kernel reads strided operands and was given no layouts");
  TQ_REQUIRE(p.scalars.empty() || scalars != nullptr, TQ_INVALID_ARGUMENT, "the kernel takes scalars and was given none");

  const int vec = kernel->vec;
  auto vector_aligned = [&](const void* pointer, tq_dtype dtype) {
    const size_t bytes = static_cast<size_t>(vec) * tq::dtype_size(dtype);
    return tq::aligned_to(pointer, bytes > 16 ? 16 : bytes);
  };
  bool vector_path = vector_aligned(out, p.out_dtype);
  TQ_REQUIRE(tq::aligned_to(out, tq::dtype_size(p.out_dtype)), TQ_INVALID_ARGUMENT, "output pointer is not aligned to its element type");
  unsigned flags = 0;
  int divisor_index = 0, layout_index = 0;
  for (size_t k = 0; k < p.inputs.size(); ++k) {
    const tq::Input& in = p.inputs[k];
    TQ_REQUIRE(inputs[k] != nullptr, TQ_INVALID_ARGUMENT, "input %zu is null", k);
    TQ_REQUIRE(tq::aligned_to(inputs[k], tq::dtype_size(in.dtype)), TQ_INVALID_ARGUMENT,
               "input %zu is not aligned to its element type", k);
    switch (in.read) {
      case tq::Read::kSame:
        vector_path = vector_path && vector_aligned(inputs[k], in.dtype);
        break;
      case tq::Read::kCycled: {
        const int64_t d = divisors[divisor_index++];
        TQ_REQUIRE(d > 0 && d <= elements, TQ_INVALID_ARGUMENT, "divisor %lld of input %zu is not in [1, %lld]", (long long)d, k, (long long)elements);
        if (d % vec == 0 && vector_aligned(inputs[k], in.dtype)) flags |= 1u << k;
        break;
      }
      case tq::Read::kRepeated: {
        const int64_t d = divisors[divisor_index++];
        TQ_REQUIRE(d > 0 && d <= elements, TQ_INVALID_ARGUMENT, "divisor %lld of input %zu is not in [1, %lld]", (long long)d, k, (long long)elements);
        if (d % vec == 0) flags |= 1u << k;
        break;
      }
      case tq::Read::kStrided: {
        const tq_layout& l = layouts[layout_index++];
        TQ_REQUIRE(l.rank >= 1 && l.rank <= 8, TQ_INVALID_ARGUMENT, "layout of input %zu has rank %d", k, l.rank);
        long long count = 1;
        bool fast = l.strides[l.rank - 1] == 1 && l.sizes[l.rank - 1] % vec == 0 && vector_aligned(inputs[k], in.dtype);
        for (int d = 0; d < l.rank; ++d) {
          TQ_REQUIRE(l.sizes[d] > 0, TQ_INVALID_ARGUMENT, "layout of input %zu has extent %lld", k, (long long)l.sizes[d]);
          TQ_REQUIRE(l.strides[d] >= 0, TQ_UNSUPPORTED, "negative stride on input %zu has no kernel", k);
          if (d < l.rank - 1 && l.strides[d] % vec != 0) fast = false;
          count *= l.sizes[d];
        }
        TQ_REQUIRE(count == elements, TQ_INVALID_ARGUMENT, "layout of input %zu covers %lld elements, the output has %lld", k, count, (long long)elements);
        if (fast) flags |= 1u << k;
        break;
      }
    }
  }

  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  if (tq_status s = tq::load(kernel->module.get())) return s;

  const int width = vector_path ? vec : 1;
  const int unroll = vector_path ? kernel->unroll : 4;
  const long long tile = 256LL * width * unroll;
  const long long blocks = (elements + tile - 1) / tile;
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld elements are more than a grid holds", (long long)elements);
  const bool narrow = elements + tile < 0xffffffffLL;
  cudaKernel_t function = kernel->module->kernels[(vector_path ? 0 : 2) + (narrow ? 0 : 1)];

  // Argument storage must outlive cudaLaunchKernel only.
  std::vector<void*> arguments;
  std::vector<const void*> pointer_slots(p.inputs.size());
  for (size_t k = 0; k < p.inputs.size(); ++k) {
    pointer_slots[k] = inputs[k];
    arguments.push_back(&pointer_slots[k]);
  }
  void* out_slot = out;
  long long n_slot = elements;
  arguments.push_back(&out_slot);
  arguments.push_back(&n_slot);
  // Each divisor and each extent of a layout travels with floor(2^64 / d) + 1, which turns the kernels'
  // 32-bit `/` and `%` into a multiplication (tq_quotient in the prelude).
  auto magic_of = [](long long d) { return d == 1 ? ~0ull : ~0ull / static_cast<unsigned long long>(d) + 1ull; };
  std::vector<long long> divisor_slots(p.divisors);
  std::vector<unsigned long long> magic_slots(p.divisors);
  for (int j = 0; j < p.divisors; ++j) {
    divisor_slots[j] = divisors[j];
    magic_slots[j] = magic_of(divisors[j]);
    arguments.push_back(&divisor_slots[j]);
    arguments.push_back(&magic_slots[j]);
  }
  struct DeviceLayout { int rank; long long sizes[8]; long long strides[8]; unsigned long long magics[8]; };   // tq_layout_t of the prelude
  std::vector<DeviceLayout> layout_slots(p.layouts);
  for (int j = 0; j < p.layouts; ++j) {
    DeviceLayout& l = layout_slots[j];
    l = DeviceLayout{};
    l.rank = layouts[j].rank;
    for (int d = 0; d < l.rank; ++d) {
      l.sizes[d] = layouts[j].sizes[d];
      l.strides[d] = layouts[j].strides[d];
      l.magics[d] = magic_of(layouts[j].sizes[d]);
    }
    arguments.push_back(&l);
  }
  arguments.push_back(&flags);
  union Slot { float f; double d; int i; long long l; bool b; };
  std::vector<Slot> scalar_slots(p.scalars.size());
  for (size_t j = 0; j < p.scalars.size(); ++j) {
    switch (tq::cls_of(p.scalars[j].dtype)) {
      case tq::Cls::kF32: scalar_slots[j].f = static_cast<float>(scalars[j]); break;
      case tq::Cls::kF64: scalar_slots[j].d = scalars[j]; break;
      case tq::Cls::kI32: scalar_slots[j].i = static_cast<int>(static_cast<long long>(scalars[j])); break;
      case tq::Cls::kI64: scalar_slots[j].l = static_cast<long long>(scalars[j]); break;
      default: scalar_slots[j].b = scalars[j] != 0; break;
    }
    arguments.push_back(&scalar_slots[j]);
  }
  TQ_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(function), dim3(static_cast<unsigned>(blocks)), dim3(256),
                           arguments.data(), 0, static_cast<cudaStream_t>(stream)));
  return TQ_OK;
}

}  // extern "C"
