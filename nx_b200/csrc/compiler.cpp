// defn compiler: fusion planner + CUDA source generator.
//
// Replaces the Expr -> StableHLO lowering of exla/lib/exla/defn.ex:1090-1706 and
// XLA's fusion passes for the subset of ops on the hot path.  Strategy:
//
//   * values that must live in HBM ("materialised"): parameters, literals,
//     program outputs, dot operands/results, concatenate results, and reduction
//     results read by another kernel;
//   * every other elementwise / view / iota / constant node is generated inline
//     into each kernel that needs it (index maps of broadcast / transpose /
//     slice / squeeze compose into the load address, so views cost nothing);
//   * reductions over trailing axes with the same row shape, everything they
//     depend on and everything computed from their results are fused into ONE
//     "row kernel": a CTA (or a warp) owns a row, keeps it in registers, and
//     runs the dependent phases (max -> exp/sum -> normalise ...) back to back;
//   * remaining elementwise outputs become flat 128-bit-vectorised kernels.
//
// All shapes are compile-time constants of the generated source (programs are
// specialised per argument signature, as in the reference).
#include <chrono>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <set>
#include <sstream>

#include "program.h"

namespace nxb {

namespace {

// ---------------------------------------------------------------------------------
// op tables
const std::set<std::string> kUnaryMath = {"exp", "expm1", "log", "log1p", "sigmoid", "cos", "sin", "tan", "cosh",
                                          "sinh", "tanh", "acos", "asin", "atan", "acosh", "asinh", "atanh", "sqrt",
                                          "rsqrt", "cbrt", "erf", "erfc", "erf_inv"};
const std::set<std::string> kUnaryOther = {"abs", "bitwise_not", "ceil", "floor", "negate", "round", "sign",
                                           "count_leading_zeros", "population_count", "is_nan", "is_infinity",
                                           "as_type", "copy"};
const std::set<std::string> kBinary = {"add", "subtract", "multiply", "divide", "pow", "remainder", "atan2", "min",
                                       "max", "quotient", "bitwise_and", "bitwise_or", "bitwise_xor", "left_shift",
                                       "right_shift", "equal", "not_equal", "greater", "less", "greater_equal",
                                       "less_equal", "logical_and", "logical_or", "logical_xor"};
const std::set<std::string> kCompare = {"equal", "not_equal", "greater", "less", "greater_equal", "less_equal"};
const std::set<std::string> kLogical = {"logical_and", "logical_or", "logical_xor"};
const std::set<std::string> kReduce = {"sum", "product", "reduce_max", "reduce_min", "all", "any"};
const std::set<std::string> kArgReduce = {"argmax", "argmin"};
const std::set<std::string> kView = {"reshape", "squeeze", "broadcast", "transpose", "slice", "metadata"};

bool is_reduce(const Node& n) { return kReduce.count(n.op) || kArgReduce.count(n.op); }
bool is_inline(const Node& n) {   // can be generated inside a consumer's kernel
  return kUnaryMath.count(n.op) || kUnaryOther.count(n.op) || kBinary.count(n.op) || kView.count(n.op) ||
         n.op == "select" || n.op == "clip" || n.op == "constant" || n.op == "iota" || n.op == "gather" || n.op == "put_slice" || n.op == "pad" || n.op == "reverse" ||
         n.op == "window_sum" || n.op == "window_max" || n.op == "window_min" || n.op == "window_product";
}

const char* storage_type(DType t) {
  static const char* n[] = {"uint8_t", "uint16_t", "uint32_t", "uint64_t", "int8_t", "int16_t", "int32_t", "int64_t",
                            "f16_t", "bf16_t", "float", "double"};
  return n[(int)t];
}
const char* reg_type(DType t) {
  if (t == NXB_F16 || t == NXB_BF16) return "float";
  return storage_type(t);
}
const char* unsigned_of(DType t) {
  static const char* n[] = {"uint8_t", "uint16_t", "uint32_t", "uint64_t", "uint8_t", "uint16_t", "uint32_t", "uint64_t"};
  return n[(int)t];
}

std::vector<int64_t> cstrides(const std::vector<int64_t>& s) {
  std::vector<int64_t> st(s.size(), 1);
  for (int i = (int)s.size() - 2; i >= 0; --i) st[i] = st[i + 1] * s[i + 1];
  return st;
}

std::vector<int64_t> strip_units(const std::vector<int64_t>& s) {
  std::vector<int64_t> o;
  for (auto d : s) if (d != 1) o.push_back(d);
  return o;
}

struct FusionError : std::exception {
  std::string msg;
  explicit FusionError(std::string m) : msg(std::move(m)) {}
  const char* what() const noexcept override { return msg.c_str(); }
};

// ---------------------------------------------------------------------------------
// affine index expressions over the kernel's loop variables
struct Aff {
  int64_t c = 0;
  std::vector<int64_t> k;
  bool opaque = false;
  std::string expr;
  bool is_const() const {
    if (opaque) return false;
    for (auto v : k) if (v) return false;
    return true;
  }
};

Aff aff_const(int nv, int64_t c) { Aff a; a.c = c; a.k.assign(nv, 0); return a; }
Aff aff_var(int nv, int j) { Aff a; a.k.assign(nv, 0); a.k[j] = 1; return a; }

// ---------------------------------------------------------------------------------
struct Root {
  int node;
  bool is_reduce;
};

// One generated kernel.
class KernelBuilder {
 public:
  enum Mode { EW, ROW, EPI };   // EPI: body of a matrix-product epilogue (a __device__ function)
  int acc_node = -1;            // EPI: the dot node whose accumulator the function receives
  int force_v = 0;              // EPI: vector width to generate (8 or 1)
  std::vector<int> seed_args;   // EPI: argument order to reuse (so both widths see the same pointers)
  int ret_node = -1;            // EPI: generate `float f(acc, batch, row, col, ep)` returning this node's value
                                // at index (batch..., row, col) instead of a storing epilogue
  bool epi_to_regs = false;     // EPI: the one stored value is handed back in `out[v]` (the product kernel stores
                                // the tile through shared memory) instead of being written by the function
  bool epi_regs_ok = true;      // cleared when the store is not a float value at the thread's own position
  std::string idx_type() const { return idx_t(); }
  KernelBuilder(Plan& plan, Mode mode, std::vector<int64_t> F, int k, std::vector<int> perm)
      : plan_(plan), g_(plan.g), mode_(mode), F_(std::move(F)), k_(k), perm_(std::move(perm)) {
    nv_ = (int)F_.size();
    if (nv_ == 0) { F_.push_back(1); nv_ = 1; }
    numel_ = shape_numel(F_);
    C_ = 1;
    for (int j = nv_ - k_; j < nv_; ++j) C_ *= F_[j];
    R_ = C_ ? numel_ / std::max<int64_t>(C_, 1) : 0;
  }

  std::vector<int> stores;     // nodes written to their slot by this kernel
  std::vector<int> reduces;    // reductions accumulated by this kernel (ROW)
  std::set<int> produced;

  KernelSpec build(const std::string& name);

 private:
  struct Val { std::string v; bool elem; };

  Plan& plan_;
  Graph& g_;
  Mode mode_;
  std::vector<int64_t> F_;
  int k_;
  std::vector<int> perm_;    // for a lone reduce over non-trailing axes: F dim j is input dim perm_[j]
  int nv_ = 0;
  int64_t numel_ = 0, R_ = 0, C_ = 1;
public:
  int vec_width() const { return V_; }
private:
  int V_ = 1, T_ = 32, block_ = 256, rpc_ = 1, chunks_ = 1;
  bool cache_ = false, guard_ = false, big_ = false;
  // Row staging: full-row inputs of a one-CTA-per-row kernel are brought into shared memory by a
  // bulk copy issued one row ahead, so the load of row r+1 overlaps the arithmetic of row r.
  bool stage_ = false;
  struct Staged { std::string param, stype; int64_t bytes, offset; };
  std::vector<Staged> staged_;
  std::string stage_load_sec_;
  int64_t stage_bytes_ = 0;

  // code sinks
  int phase_ = 0, nphases_ = 1;
  std::vector<std::string> row_sec_, pre_sec_, lane_sec_, post_sec_;
  std::string decls_;
  std::map<std::string, std::string> row_memo_;
  std::vector<std::map<std::string, std::string>> elem_memo_;
  std::map<std::string, std::pair<std::string, int>> cached_loads_;
  std::set<int> used_vars_;
  // Register reuse across phases of a row kernel.  A transcendental value needed again in a later
  // phase (exp(x - max) for the softmax division) would be recomputed there, because the row's 32
  // registers per thread hold x.  When x itself is not needed after the producing phase, the value
  // is written over x at the end of that phase and read from there later.  A planning pass (a
  // throw-away copy of the builder) records where every cached row load is referenced and under
  // which candidate values; the real pass then follows the plan.
  std::map<int, bool> ident_loads_;      // read slot -> all loads so far were at the thread's own position
  std::set<int> ident_stores_;           // written slots stored at the thread's own position
  bool planning_ = false;
  struct Stash { std::string array; int phase; };
  std::map<std::string, Stash> stash_plan_;                       // value key -> where it is kept
  std::vector<std::string> ctx_;                                  // candidate values being generated
  std::vector<std::set<std::string>> dep_stack_;                  // cached loads each open value depends on
  std::map<std::string, std::set<std::string>> deps_;             // per phase-qualified memo key
  struct LoadRef { int phase; std::set<std::string> ctx; };
  std::map<std::string, std::vector<LoadRef>> load_refs_;         // cached load key -> references
  std::map<std::string, std::set<int>> emitted_in_;               // candidate key -> phases that computed it
  std::map<std::string, std::string> load_array_;                 // cached load key -> register array name
  std::map<std::string, DType> load_type_;
  void note_load(const std::string& key) {
    if (!planning_) return;
    LoadRef r{phase_, std::set<std::string>(ctx_.begin(), ctx_.end())};
    load_refs_[key].push_back(r);
    for (auto& d : dep_stack_) d.insert(key);
  }
  // 16-bit float values that are still held at f32 precision ("excess precision", what XLA does
  // inside a fusion by default): arithmetic consumes them as they are; comparisons, index
  // reductions, integer conversions and rounding ops first round them to their declared type.
  std::set<std::string> raw_;
  bool excess_ = getenv("NXB200_STRICT_ROUNDING") == nullptr;
  std::string exact(const Val& x, DType dt) {
    if (!raw_.count(x.v)) return x.v;
    std::string key = "exact:" + x.v;
    auto& memo = x.elem ? elem_memo_[phase_] : row_memo_;
    auto it = memo.find(key);
    if (it != memo.end()) return it->second;
    std::string v = newvar("rx");
    stmt(x.elem, "const float " + v + " = " + (dt == NXB_BF16 ? "round_bf16(" : "round_f16(") + x.v + ");");
    memo[key] = v;
    return v;
  }
  bool used_flat_ = false;
  std::vector<int> arg_slots_;
  std::map<int, int> slot_param_;
  std::map<int, std::string> red_var_;
  std::map<int, int> level_memo_;
  int tmp_ = 0;

  std::string idx_t() const { return big_ ? "long long" : "int"; }
  std::string newvar(const char* pfx = "t") { return std::string(pfx) + std::to_string(tmp_++); }
  std::string param(int slot) {
    auto it = slot_param_.find(slot);
    if (it != slot_param_.end()) return "p" + std::to_string(it->second);
    int i = (int)arg_slots_.size();
    arg_slots_.push_back(slot);
    slot_param_[slot] = i;
    return "p" + std::to_string(i);
  }
  bool col_dep(const Aff& a) const {
    if (a.opaque) return true;
    for (int j = nv_ - (mode_ == ROW ? k_ : nv_); j < nv_; ++j) if (a.k[j]) return true;
    return false;
  }
  bool any_col_dep(const std::vector<Aff>& idx) const {
    for (auto& a : idx) if (col_dep(a)) return true;
    return false;
  }
  std::string affkey(const Aff& a) const {
    if (a.opaque) return "o(" + a.expr + ")";
    std::string s = std::to_string(a.c);
    for (auto v : a.k) s += "," + std::to_string(v);
    return s;
  }
  std::string idxkey(const std::vector<Aff>& idx) const {
    std::string s;
    for (auto& a : idx) s += affkey(a) + ";";
    return s;
  }
  // Text of an affine expression.  base=true substitutes the vector's first lane
  // for the innermost variable.
  std::string affstr(const Aff& a, bool base) {
    if (a.opaque) return a.expr;
    // shortcut: the address of a same-shape contiguous operand is the flat index
    if (ret_node < 0 && !a.is_const() && a.c == 0 && a.k == cstrides(F_) && nv_ > 1) {
      used_flat_ = true;
      return base ? "flat0" : "flat";
    }
    std::string s;
    auto term = [&](const std::string& t) { s += (s.empty() ? "" : " + ") + t; };
    for (int j = 0; j < nv_; ++j) {
      if (!a.k[j] || F_[j] == 1) continue;
      used_vars_.insert(j);
      std::string v = (j == nv_ - 1 && base) ? "ib" : "i" + std::to_string(j);
      term(a.k[j] == 1 ? v : "(" + idx_t() + ")" + std::to_string(a.k[j]) + " * " + v);
    }
    if (a.c || s.empty()) term("(" + idx_t() + ")" + std::to_string(a.c));
    return "(" + s + ")";
  }

  void stmt(bool elem, const std::string& line) {
    (elem ? lane_sec_[phase_] : row_sec_[phase_]) += "        " + line + "\n";
  }

  // a node that merely renames the product's buffer (reshape / squeeze / metadata over it)
  bool aliases_acc(int n) const {
    if (acc_node < 0 || n == acc_node) return false;
    int a = n;
    while (a >= 0 && g_.nodes[a].alias >= 0) a = g_.nodes[a].alias;
    return a == acc_node;
  }
  // the value (or the value a reshape / squeeze / metadata chain renames) is computed by this kernel:
  // it must be taken from registers, its buffer is not written yet
  bool made_here(int n) const {
    for (int a = n; a >= 0; a = g_.nodes[a].alias)
      if (produced.count(a) || std::count(reduces.begin(), reduces.end(), a)) return true;
    return false;
  }
  int level(int n);
  Val value(int n, const std::vector<Aff>& idx);
  Val load(int n, const std::vector<Aff>& idx);
  Val emit_op(int n, const std::vector<Aff>& idx);
  std::string cvt(const std::string& e, DType from, DType to);
  std::string literal(double f, int64_t i, bool is_f, DType t);
  std::vector<Aff> arg_index_binary(const Node& out, const Node& arg, const std::vector<Aff>& idx);
  std::vector<Aff> full_index() {
    std::vector<Aff> v;
    for (int j = 0; j < nv_; ++j) v.push_back(F_[j] == 1 ? aff_const(nv_, 0) : aff_var(nv_, j));
    return v;
  }
  // index of a node whose shape is the kernel's full shape or its row shape
  std::vector<Aff> index_for_shape(const std::vector<int64_t>& shape, bool* full);
  void emit_store(int n);
  void configure();
};

// ---- helpers -----------------------------------------------------------------------

std::string hexf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  char b[48];
  snprintf(b, sizeof b, "__uint_as_float(0x%08xu)", u);
  return b;
}
std::string hexd(double d) {
  uint64_t u;
  memcpy(&u, &d, 8);
  char b[64];
  snprintf(b, sizeof b, "__longlong_as_double(0x%016llxLL)", (unsigned long long)u);
  return b;
}
float to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if (f != f) return f;
  u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000u;
  memcpy(&f, &u, 4);
  return f;
}

std::string KernelBuilder::literal(double f, int64_t i, bool is_f, DType t) {
  if (dtype_is_float(t)) {
    double v = is_f ? f : (double)i;
    if (t == NXB_F64) return hexd(v);
    float x = (float)v;
    if (t == NXB_BF16) x = to_bf16_rne(x);
    if (t == NXB_F16) return "round_f16(" + hexf(x) + ")";
    return hexf(x);
  }
  long long v = is_f ? (long long)f : (long long)i;
  return std::string("(") + reg_type(t) + ")" + std::to_string(v) + "LL";
}

std::string KernelBuilder::cvt(const std::string& e, DType from, DType to) {
  if (from == to) return e;
  if (dtype_is_float(to)) {
    if (to == NXB_F64) return "(double)(" + e + ")";
    std::string f = (from == NXB_F32 || from == NXB_BF16 || from == NXB_F16) ? e : "(float)(" + e + ")";
    if (to == NXB_BF16) return "round_bf16(" + f + ")";
    if (to == NXB_F16) return "round_f16(" + f + ")";
    return f;
  }
  if (dtype_is_float(from)) return std::string("f2i<") + reg_type(to) + ">((double)(" + e + "))";
  return std::string("(") + reg_type(to) + ")(" + e + ")";
}

std::vector<Aff> KernelBuilder::arg_index_binary(const Node& out, const Node& arg, const std::vector<Aff>& idx) {
  // NumPy-style right alignment (nx/lib/nx/shape.ex binary_broadcast)
  int ro = (int)out.shape.size(), ra = (int)arg.shape.size();
  std::vector<Aff> r;
  for (int j = 0; j < ra; ++j) {
    int oj = j + ro - ra;
    if (arg.shape[j] == 1 || oj < 0) r.push_back(aff_const(nv_, 0));
    else r.push_back(idx[oj]);
  }
  return r;
}

std::vector<Aff> KernelBuilder::index_for_shape(const std::vector<int64_t>& shape, bool* full) {
  // Match the non-unit dims of `shape` against the kernel's dims in order: either
  // all of them (full) or the leading, non-reduced ones (row shaped).
  std::vector<int> fdims, rdims;
  for (int j = 0; j < nv_; ++j) if (F_[j] != 1) fdims.push_back(j);
  for (int j = 0; j < nv_ - k_; ++j) if (F_[j] != 1) rdims.push_back(j);
  std::vector<int64_t> su = strip_units(shape);
  auto dims_of = [&](const std::vector<int>& d) { std::vector<int64_t> o; for (int j : d) o.push_back(F_[j]); return o; };
  const std::vector<int>* use = nullptr;
  if (su == dims_of(fdims)) { use = &fdims; *full = true; }
  else if (mode_ == ROW && su == dims_of(rdims)) { use = &rdims; *full = false; }
  else throw FusionError("shape " + shape_str(shape) + " does not fit kernel space " + shape_str(F_));
  std::vector<Aff> idx;
  size_t q = 0;
  for (auto d : shape) {
    if (d == 1) idx.push_back(aff_const(nv_, 0));
    else idx.push_back(aff_var(nv_, (*use)[q++]));
  }
  return idx;
}

int KernelBuilder::level(int n) {
  auto it = level_memo_.find(n);
  if (it != level_memo_.end()) return it->second;
  const Node& nd = g_.nodes[n];
  int l = 0;
  bool ext = (nd.slot >= 0 && !made_here(n) && !aliases_acc(n)) || n == acc_node;
  if (!ext) {
    if (is_reduce(nd)) {
      if (!std::count(reduces.begin(), reduces.end(), n)) throw FusionError("reduction outside the kernel is not materialised");
      l = level(nd.args[0]) + 1;
    } else {
      for (int a : nd.args) l = std::max(l, level(a));
    }
  }
  level_memo_[n] = l;
  return l;
}

KernelBuilder::Val KernelBuilder::load(int n, const std::vector<Aff>& idx) {
  const Node& nd = g_.nodes[n];
  auto st = cstrides(nd.shape);
  Aff addr = aff_const(nv_, 0);
  for (size_t j = 0; j < idx.size(); ++j) {
    if (nd.shape[j] == 1) continue;
    if (idx[j].opaque || addr.opaque) {
      std::string e = addr.opaque ? addr.expr : affstr(addr, false);
      addr.opaque = true;
      addr.expr = "(" + e + " + (" + idx_t() + ")" + std::to_string(st[j]) + " * " + affstr(idx[j], false) + ")";
      continue;
    }
    addr.c += idx[j].c * st[j];
    for (int v = 0; v < nv_; ++v) addr.k[v] += idx[j].k[v] * st[j];
  }
  const std::string S = storage_type(nd.dt), Rt = reg_type(nd.dt);
  std::string p = param(nd.slot);
  {
    // donation: a slot may be overwritten in place only if every load of it is at the position
    // the loading thread itself stores to (the flat index of the kernel's space)
    const bool ident = !addr.opaque && addr.c == 0 && addr.k == cstrides(F_) && shape_numel(nd.shape) == numel_;
    auto it = ident_loads_.find(nd.slot);
    if (it == ident_loads_.end()) ident_loads_[nd.slot] = ident;
    else it->second = it->second && ident;
  }
  std::string key = "L" + std::to_string(nd.slot) + ":" + affkey(addr);
  bool cdep = col_dep(addr);
  if (mode_ == ROW && !cdep) {
    auto it = row_memo_.find(key);
    if (it != row_memo_.end()) return {it->second, false};
    std::string v = newvar("lv");
    stmt(false, "const " + Rt + " " + v + " = ld1<" + S + ">(" + p + " + " + affstr(addr, false) + ");");
    row_memo_[key] = v;
    return {v, false};
  }
  int64_t kv = addr.opaque ? -1 : addr.k[nv_ - 1];
  bool aligned = !addr.opaque && addr.c % V_ == 0;
  if (aligned)
    for (int j = 0; j < nv_ - 1; ++j) if (F_[j] != 1 && addr.k[j] % V_ != 0) aligned = false;
  if (V_ > 1 && kv == 1 && aligned) {
    if (mode_ == ROW && cache_) {
      auto it = cached_loads_.find(key);
      if (it == cached_loads_.end()) {
        std::string v = newvar("lv");
        decls_ += "      " + Rt + " " + v + "[" + std::to_string(chunks_) + "][" + std::to_string(V_) + "];\n";
        const int64_t row_bytes = C_ * (int64_t)dtype_size(nd.dt);
        const bool flat_row = addr.c == 0 && addr.k == cstrides(F_) && nv_ > 1;
        if (stage_ && phase_ == 0 && flat_row && row_bytes % 16 == 0 && stage_bytes_ + row_bytes <= 200 * 1024) {
          Staged sg{p, S, row_bytes, stage_bytes_};
          stage_bytes_ += (row_bytes + 127) / 128 * 128;
          staged_.push_back(sg);
          // loaded by a loop of its own ahead of phase 0, so the buffer is free again at once
          stage_load_sec_ += "          if (use_stage) ld_vec<" + S + ", " + std::to_string(V_) + ">(reinterpret_cast<const " + S + "*>(stage_buf + " +
                             std::to_string(sg.offset) + ") + col0, " + v + "[ch]);\n          else ld_vec<" + S + ", " + std::to_string(V_) + ">(" + p +
                             " + rowbase + col0, " + v + "[ch]);\n";
        } else {
          pre_sec_[phase_] += "          ld_vec<" + S + ", " + std::to_string(V_) + ">(" + p + " + " + affstr(addr, true) + ", " + v + "[ch]);\n";
        }
        it = cached_loads_.emplace(key, std::make_pair(v, phase_)).first;
        load_array_[key] = v;
        load_type_[key] = nd.dt;
      }
      note_load(key);
      return {it->second.first + "[ch][v]", true};
    }
    auto& memo = elem_memo_[phase_];
    auto it = memo.find(key);
    if (it != memo.end()) return {it->second, true};
    std::string v = newvar("lv");
    pre_sec_[phase_] += "          " + Rt + " " + v + "[" + std::to_string(V_) + "]; ld_vec<" + S + ", " + std::to_string(V_) + ">(" + p + " + " +
                        affstr(addr, true) + ", " + v + ");\n";
    memo[key] = v + "[v]";
    return {v + "[v]", true};
  }
  auto& memo = elem_memo_[phase_];
  auto it = memo.find(key);
  if (it != memo.end()) return {it->second, true};
  std::string v = newvar("lv");
  if (V_ == 1 || kv != 0 || addr.opaque) {
    stmt(true, "const " + Rt + " " + v + " = ld1<" + S + ">(" + p + " + " + affstr(addr, false) + ");");
  } else {
    // same address for every lane of the vector: load once per vector
    pre_sec_[phase_] += "          const " + Rt + " " + v + " = ld1<" + S + ">(" + p + " + " + affstr(addr, true) + ");\n";
  }
  memo[key] = v;
  return {v, true};
}

KernelBuilder::Val KernelBuilder::value(int n, const std::vector<Aff>& idx) {
  const Node& nd = g_.nodes[n];
  if (n == acc_node) {
    // the product's own element: only legal at the position this thread's accumulator holds
    auto st = cstrides(nd.shape);
    Aff addr = aff_const(nv_, 0);
    for (size_t j = 0; j < idx.size(); ++j) {
      if (idx[j].opaque) throw FusionError("product read through a reshaped index");
      addr.c += idx[j].c * st[j];
      for (int v = 0; v < nv_; ++v) addr.k[v] += idx[j].k[v] * st[j];
    }
    auto fs = cstrides(F_);
    bool same = addr.c == 0;
    for (int j = 0; j < nv_; ++j) if (F_[j] != 1 && addr.k[j] != fs[j]) same = false;
    if (!same) throw FusionError("product consumed at a transposed or sliced position");
    std::string key = "acc";
    auto it = elem_memo_[phase_].find(key);
    if (it != elem_memo_[phase_].end()) return {it->second, true};
    std::string v = newvar();
    const bool keep_f32 = excess_ && (nd.dt == NXB_BF16 || nd.dt == NXB_F16);
    stmt(true, std::string("const ") + reg_type(nd.dt) + " " + v + " = " + (keep_f32 ? std::string("acc[v]") : cvt("acc[v]", NXB_F32, nd.dt)) + ";");
    if (keep_f32) raw_.insert(v);
    elem_memo_[phase_][key] = v;
    return {v, true};
  }
  if (nd.slot >= 0 && !made_here(n) && !aliases_acc(n)) return load(n, idx);
  if (nd.op == "constant") {
    bool isf = !nd.flts.empty();
    return {literal(isf ? nd.flts[0] : 0.0, isf ? 0 : nd.ints[0], isf, nd.dt), false};
  }
  std::string key = std::to_string(n) + ":" + idxkey(idx);
  auto rit = row_memo_.find(key);
  if (rit != row_memo_.end()) return {rit->second, false};
  auto eit = elem_memo_[phase_].find(key);
  if (eit != elem_memo_[phase_].end()) {
    if (planning_) {
      // a second consumer of a memoised value: its row loads are referenced again, in this context
      for (auto& l : deps_[std::to_string(phase_) + "/" + key]) note_load(l);
    }
    return {eit->second, true};
  }
  {
    auto sp = stash_plan_.find(key);
    if (sp != stash_plan_.end() && phase_ > sp->second.phase) return {sp->second.array + "[ch][v]", true};
  }
  const bool candidate = mode_ == ROW && cache_ && nd.dt == NXB_F32 && kUnaryMath.count(nd.op) && idxkey(idx) == idxkey(full_index());
  if (planning_) {
    dep_stack_.emplace_back();
    if (candidate) ctx_.push_back(key);
  }
  Val v = emit_op(n, idx);
  if (planning_) {
    if (candidate) { ctx_.pop_back(); if (v.elem) emitted_in_[key].insert(phase_); }
    deps_[std::to_string(phase_) + "/" + key] = dep_stack_.back();
    dep_stack_.pop_back();
  }
  if (v.elem) elem_memo_[phase_][key] = v.v;
  else row_memo_[key] = v.v;
  return v;
}

KernelBuilder::Val KernelBuilder::emit_op(int n, const std::vector<Aff>& idx) {
  const Node& nd = g_.nodes[n];
  const std::string& op = nd.op;
  const DType t = nd.dt;
  auto def = [&](bool elem, DType dt, const std::string& e) -> Val {
    std::string v = newvar();
    stmt(elem, std::string("const ") + reg_type(dt) + " " + v + " = " + e + ";");
    return {v, elem};
  };

  if (is_reduce(nd)) {
    // result of a reduction accumulated by this kernel: must be asked for at the current row
    auto it = red_var_.find(n);
    if (it == red_var_.end()) throw FusionError("reduction result used before it is complete");
    const Node& in = g_.nodes[nd.args[0]];
    // build the expected index: non-reduced dims in order -> row variables, kept dims -> 0
    std::vector<Aff> want;
    std::vector<int64_t> inshape = in.shape;
    if (inshape.empty()) inshape.push_back(1);
    bool full;
    std::vector<Aff> w = index_for_shape(nd.shape, &full);
    if (full && k_ > 0 && C_ != 1) throw FusionError("reduction result has the full shape");
    for (size_t j = 0; j < idx.size(); ++j)
      if (affkey(idx[j]) != affkey(w[j])) throw FusionError("reduction result indexed off the current row");
    return {it->second, false};
  }
  if (op == "metadata" || op == "copy") return value(nd.args[0], idx);
  if (op == "iota") {
    int ax = (int)nd.ints[0];
    Aff a;
    if (ax >= 0) a = idx[ax];
    else {
      a = aff_const(nv_, 0);
      auto st = cstrides(nd.shape);
      bool any_opaque = false;
      for (auto& i : idx) any_opaque = any_opaque || i.opaque;
      if (any_opaque) {                           // position computed from the index expressions themselves
        std::string s;
        for (size_t j = 0; j < idx.size(); ++j) {
          if (nd.shape[j] == 1) continue;
          s += (s.empty() ? "" : " + ") + std::string("(long long)") + std::to_string(st[j]) + " * (long long)" + affstr(idx[j], false);
        }
        if (s.empty()) s = "0ll";
        return def(true, t, cvt("(" + s + ")", NXB_S64, t));
      }
      for (size_t j = 0; j < idx.size(); ++j) {
        a.c += idx[j].c * st[j];
        for (int v = 0; v < nv_; ++v) a.k[v] += idx[j].k[v] * st[j];
      }
    }
    bool e = col_dep(a);
    if (a.is_const()) return {literal(0, a.c, false, t), false};
    return def(e, t, cvt("(long long)" + affstr(a, false), NXB_S64, t));
  }
  if (op == "broadcast") {
    const Node& a = g_.nodes[nd.args[0]];
    int na = (int)nd.ints[0];
    std::vector<Aff> ai;
    for (int j = 0; j < na; ++j) ai.push_back(a.shape[j] == 1 ? aff_const(nv_, 0) : idx[nd.ints[1 + j]]);
    return value(nd.args[0], ai);
  }
  if (op == "squeeze") {
    const Node& a = g_.nodes[nd.args[0]];
    std::set<int64_t> ax(nd.ints.begin() + 1, nd.ints.end());
    std::vector<Aff> ai;
    size_t q = 0;
    for (size_t j = 0; j < a.shape.size(); ++j) ai.push_back(ax.count((int64_t)j) ? aff_const(nv_, 0) : idx[q++]);
    return value(nd.args[0], ai);
  }
  if (op == "transpose") {
    std::vector<Aff> ai(idx.size(), aff_const(nv_, 0));
    for (size_t j = 0; j < idx.size(); ++j) ai[nd.ints[j]] = idx[j];
    return value(nd.args[0], ai);
  }
  if (op == "slice" && nd.args.size() > 1) {
    // dynamic starts (Nx.slice with tensor indices): a start is clamped so that the slice fits
    const Node& a = g_.nodes[nd.args[0]];
    size_t r = idx.size();
    std::vector<Aff> ai;
    for (size_t j = 0; j < r; ++j) {
      const int64_t span = nd.ints[r + j], sd = nd.ints[2 * r + j];     // window length before striding, stride
      Val sv = value(nd.args[1 + j], {});
      Val s = def(true, NXB_S64, "nx_clamp_index(" + sv.v + ", (long long)" + std::to_string(a.shape[j] - span + 1) + ")");
      Aff o;
      o.opaque = true;
      o.k.assign(nv_, 0);
      o.expr = "((" + idx_t() + ")" + s.v + " + (" + idx_t() + ")" + std::to_string(sd) + " * " + affstr(idx[j], false) + ")";
      ai.push_back(o);
    }
    return value(nd.args[0], ai);
  }
  if (op == "gather") {
    // out dims = batch dims of `indices` ++ dims of `tensor` that are not indexed; an index is
    // clamped into its axis (XLA's gather semantics, exla/lib/exla/defn.ex gather lowering)
    const Node& T = g_.nodes[nd.args[0]];
    const Node& I = g_.nodes[nd.args[1]];
    const size_t nb = I.shape.size() - 1;
    std::vector<Aff> tidx(T.shape.size(), aff_const(nv_, 0));
    std::set<int64_t> indexed(nd.ints.begin(), nd.ints.end());
    size_t q = nb;
    for (size_t j = 0; j < T.shape.size(); ++j)
      if (!indexed.count((int64_t)j)) tidx[j] = idx[q++];
    for (size_t i = 0; i < nd.ints.size(); ++i) {
      std::vector<Aff> ii(idx.begin(), idx.begin() + nb);
      ii.push_back(aff_const(nv_, (int64_t)i));
      Val iv = value(nd.args[1], ii);
      Aff o;
      o.opaque = true;
      o.k.assign(nv_, 0);
      o.expr = "(" + idx_t() + ")nx_clamp_index(" + iv.v + ", (long long)" + std::to_string(T.shape[nd.ints[i]]) + ")";
      tidx[nd.ints[i]] = o;
    }
    return value(nd.args[0], tidx);
  }
  if (op == "window_sum" || op == "window_max" || op == "window_min" || op == "window_product") {
    // ints: window dims, strides, low padding, high padding, dilations (rank entries each).  The
    // window is unrolled: each of its positions is an index expression of the output position
    // (pooling windows are small); positions in the padding contribute the operation's identity.
    const Node& a = g_.nodes[nd.args[0]];
    const size_t r = idx.size();
    int64_t vol = 1;
    for (size_t j = 0; j < r; ++j) vol *= nd.ints[j];
    if (vol > 256) fail(NXB_ERR_UNSUPPORTED, "window reductions over more than 256 positions are not implemented");
    const std::string RT = reg_type(t);
    std::string ident;
    if (op == "window_sum") ident = "(" + RT + ")0";
    else if (op == "window_product") ident = "(" + RT + ")1";
    else {
      const bool mx = op == "window_max";
      if (dtype_is_float(t)) ident = std::string(mx ? "-" : "") + (t == NXB_F64 ? "(double)NXB_INF" : "NXB_INF");
      else {
        const int bits = (int)dtype_size(t) * 8;
        const int64_t lo = dtype_is_signed(t) ? -(int64_t)((uint64_t)1 << (bits - 1)) : 0;
        const int64_t hi = dtype_is_signed(t) ? (int64_t)(((uint64_t)1 << (bits - 1)) - 1) : (bits == 64 ? -1 : (int64_t)(((uint64_t)1 << bits) - 1));
        ident = literal(0, mx ? lo : hi, false, t);
      }
    }
    std::string acc;
    bool elem = false;
    std::vector<int64_t> w(r, 0);
    for (int64_t pos = 0; pos < vol; ++pos) {
      std::vector<Aff> ai;
      std::string inside;
      for (size_t j = 0; j < r; ++j) {
        const int64_t stride = nd.ints[r + j], lo = nd.ints[2 * r + j], hi = nd.ints[3 * r + j], dil = nd.ints[4 * r + j];
        const int64_t off = w[j] * dil - lo;
        if (lo == 0 && hi == 0 && !idx[j].opaque) {
          Aff x = idx[j];
          x.c = x.c * stride + off;
          for (auto& kk : x.k) kk *= stride;
          ai.push_back(x);
          continue;
        }
        const std::string c = "((long long)(" + affstr(idx[j], false) + ") * " + std::to_string(stride) + "LL + " + std::to_string(off) + "LL)";
        if (lo != 0 || hi != 0) inside += (inside.empty() ? "" : " && ") + std::string("(") + c + " >= 0 && " + c + " < " + std::to_string(a.shape[j]) + "LL)";
        Aff o;
        o.opaque = true;
        o.k.assign(nv_, 0);
        o.expr = "(" + idx_t() + ")nx_clamp_index(" + c + ", (long long)" + std::to_string(a.shape[j]) + ")";
        ai.push_back(o);
      }
      Val x = value(nd.args[0], ai);
      elem = elem || x.elem;
      std::string term = cvt(x.v, a.dt, t);
      if (!inside.empty()) { term = "((" + inside + ") ? " + term + " : " + ident + ")"; elem = true; }
      if (acc.empty()) acc = term;
      else if (op == "window_sum") acc = "(" + acc + " + " + term + ")";
      else if (op == "window_product") acc = "(" + acc + " * " + term + ")";
      else acc = std::string(op == "window_max" ? "nx_max" : "nx_min") + "(" + acc + ", " + term + ")";
      if (pos % 8 == 7 || pos + 1 == vol) {        // keep expressions short: a statement every few terms
        Val part = def(true, t, acc);
        acc = part.v;
        elem = true;
      }
      for (int j = (int)r - 1; j >= 0; --j) { if (++w[j] < nd.ints[j]) break; w[j] = 0; }
    }
    return {acc, true};
  }
  if (op == "reverse") {
    // ints: the reversed axes.  index = dim - 1 - i along each
    const Node& a = g_.nodes[nd.args[0]];
    std::vector<Aff> ai = idx;
    for (int64_t ax : nd.ints) {
      Aff& x = ai[ax];
      if (x.opaque) x.expr = "((" + idx_t() + ")" + std::to_string(a.shape[ax] - 1) + " - " + x.expr + ")";
      else { x.c = a.shape[ax] - 1 - x.c; for (auto& kk : x.k) kk = -kk; }
    }
    return value(nd.args[0], ai);
  }
  if (op == "pad") {
    // args: tensor, scalar pad value; ints: low..., high..., interior... (Nx.pad, negative edges crop).
    // out[i] is x[(i - low) / (interior + 1)] where that position exists, else the pad value.
    const Node& a = g_.nodes[nd.args[0]];
    const size_t r = idx.size();
    std::vector<Aff> ai;
    std::string inside;
    for (size_t j = 0; j < r; ++j) {
      const int64_t lo = nd.ints[j], hi = nd.ints[r + j], in = nd.ints[2 * r + j];
      if (lo == 0 && in == 0 && hi <= 0) { ai.push_back(idx[j]); continue; }     // a cropped or untouched tail: same index
      const std::string c = "((long long)(" + affstr(idx[j], false) + ") - " + std::to_string(lo) + "LL)";
      std::string cond = "(" + c + " >= 0 && " + c + " < " + std::to_string((a.shape[j] - 1) * (in + 1) + 1) + "LL";
      if (in > 0) cond += " && " + c + " % " + std::to_string(in + 1) + "LL == 0";
      cond += ")";
      inside += (inside.empty() ? "" : " && ") + cond;
      Aff o;
      o.opaque = true;
      o.k.assign(nv_, 0);
      o.expr = "(" + idx_t() + ")nx_clamp_index(" + c + " / " + std::to_string(in + 1) + "LL, (long long)" + std::to_string(a.shape[j]) + ")";
      ai.push_back(o);
    }
    Val x = value(nd.args[0], ai);
    if (inside.empty()) return def(x.elem, t, cvt(x.v, a.dt, t));
    Val pv = value(nd.args[1], {});
    return def(true, t, "(" + inside + ") ? " + cvt(x.v, a.dt, t) + " : " + cvt(pv.v, g_.nodes[nd.args[1]].dt, t));
  }
  if (op == "put_slice") {
    // args: tensor, slice, one scalar start per axis (clamped so that the slice fits)
    const Node& T = g_.nodes[nd.args[0]];
    const Node& S = g_.nodes[nd.args[1]];
    const size_t r = idx.size();
    std::vector<Aff> sidx;
    std::string inside;
    bool elem = false;
    for (size_t j = 0; j < r; ++j) {
      if (S.shape[j] == T.shape[j]) { sidx.push_back(idx[j]); continue; }     // the slice spans the axis: start is 0
      Val sv = value(nd.args[2 + j], {});
      Val s = def(true, NXB_S64, "nx_clamp_index(" + sv.v + ", (long long)" + std::to_string(T.shape[j] - S.shape[j] + 1) + ")");
      const std::string c = "((long long)(" + affstr(idx[j], false) + ") - " + s.v + ")";
      inside += (inside.empty() ? "" : " && ") + std::string("(") + c + " >= 0 && " + c + " < " + std::to_string(S.shape[j]) + ")";
      Aff o;
      o.opaque = true;
      o.k.assign(nv_, 0);
      o.expr = "(" + idx_t() + ")nx_clamp_index(" + c + ", (long long)" + std::to_string(S.shape[j]) + ")";
      sidx.push_back(o);
      elem = true;
    }
    Val x = value(nd.args[1], sidx);
    if (inside.empty()) return def(x.elem, t, cvt(x.v, S.dt, t));           // the slice replaces everything
    Val y = value(nd.args[0], idx);
    return def(true, t, "(" + inside + ") ? " + cvt(x.v, S.dt, t) + " : " + cvt(y.v, T.dt, t));
  }
  if (op == "slice") {
    size_t r = idx.size();
    std::vector<Aff> ai;
    for (size_t j = 0; j < r; ++j) {
      Aff a = idx[j];
      int64_t st = nd.ints[j], sd = nd.ints[2 * r + j];
      if (a.opaque) a.expr = "((" + idx_t() + ")" + std::to_string(st) + " + (" + idx_t() + ")" + std::to_string(sd) + " * " + a.expr + ")";
      else { a.c = a.c * sd + st; for (auto& kk : a.k) kk *= sd; }
      ai.push_back(a);
    }
    return value(nd.args[0], ai);
  }
  if (op == "reshape") {
    const Node& a = g_.nodes[nd.args[0]];
    std::vector<Aff> ai;
    if (strip_units(a.shape) == strip_units(nd.shape)) {
      // only unit dims were added or removed
      std::vector<Aff> nonunit;
      for (size_t j = 0; j < idx.size(); ++j) if (nd.shape[j] != 1) nonunit.push_back(idx[j]);
      size_t q = 0;
      for (auto d : a.shape) ai.push_back(d == 1 ? aff_const(nv_, 0) : nonunit[q++]);
    } else {
      // general case: linear offset in the new shape, then div/mod into the old one
      auto st = cstrides(nd.shape);
      Aff lin = aff_const(nv_, 0);
      bool opq = false;
      std::string e;
      for (size_t j = 0; j < idx.size(); ++j) {
        if (idx[j].opaque) opq = true;
      }
      if (!opq) {
        for (size_t j = 0; j < idx.size(); ++j) {
          lin.c += idx[j].c * st[j];
          for (int v = 0; v < nv_; ++v) lin.k[v] += idx[j].k[v] * st[j];
        }
        e = affstr(lin, false);
      } else {
        for (size_t j = 0; j < idx.size(); ++j)
          e += (j ? " + " : "") + std::string("(") + idx_t() + ")" + std::to_string(st[j]) + " * " + affstr(idx[j], false);
        e = "(" + e + ")";
      }
      auto ast = cstrides(a.shape);
      for (size_t j = 0; j < a.shape.size(); ++j) {
        Aff o;
        o.opaque = true;
        o.k.assign(nv_, 0);
        o.expr = "((" + e + " / (" + idx_t() + ")" + std::to_string(ast[j]) + ") % (" + idx_t() + ")" + std::to_string(a.shape[j]) + ")";
        ai.push_back(a.shape[j] == 1 ? aff_const(nv_, 0) : o);
      }
    }
    return value(nd.args[0], ai);
  }

  // ---- elementwise ------------------------------------------------------------------
  if (op == "as_type") {
    const Node& a = g_.nodes[nd.args[0]];
    Val x = value(nd.args[0], idx);
    if (a.dt == t) return x;
    return def(x.elem, t, cvt(dtype_is_float(t) ? x.v : exact(x, a.dt), a.dt, t));
  }
  if (kUnaryMath.count(op) || kUnaryOther.count(op)) {
    const Node& a = g_.nodes[nd.args[0]];
    Val x = value(nd.args[0], idx);
    const bool dbl = t == NXB_F64;
    auto fn = [&](const char* base) { return std::string(base) + (dbl ? "" : "f"); };
    std::string e;
    if (op == "is_nan") {
      e = dtype_is_float(a.dt) ? "(uint8_t)(" + x.v + " != " + x.v + ")" : "(uint8_t)0";
      return def(x.elem, t, e);
    }
    if (op == "is_infinity") {
      e = dtype_is_float(a.dt) ? "(uint8_t)(" + std::string(a.dt == NXB_F64 ? "fabs" : "fabsf") + "(" + x.v + ") == NXB_INF)" : "(uint8_t)0";
      return def(x.elem, t, e);
    }
    if (op == "population_count" || op == "count_leading_zeros") {
      e = std::string(op == "population_count" ? "nx_popc<" : "nx_clz<") + reg_type(a.dt) + ">(" + x.v + ")";
      return def(x.elem, t, cvt(e, a.dt, t));
    }
    const bool exact_in = op == "floor" || op == "ceil" || op == "round" || op == "sign";
    std::string xv = cvt(exact_in ? exact(x, a.dt) : x.v, a.dt, t);     // the argument is converted to the output type first
    if (dtype_is_float(t)) {
      static const std::map<std::string, const char*> lib = {
          {"expm1", "expm1"}, {"log1p", "log1p"}, {"cos", "cos"}, {"sin", "sin"}, {"tan", "tan"}, {"cosh", "cosh"},
          {"sinh", "sinh"}, {"acos", "acos"}, {"asin", "asin"}, {"atan", "atan"}, {"acosh", "acosh"},
          {"asinh", "asinh"}, {"atanh", "atanh"}, {"sqrt", "sqrt"}, {"cbrt", "cbrt"}, {"erf", "erf"},
          {"erfc", "erfc"}, {"abs", "fabs"}, {"floor", "floor"}, {"ceil", "ceil"}};
      static const std::map<std::string, const char*> own = {
          {"exp", "nx_exp"}, {"log", "nx_log"}, {"sigmoid", "nx_sigmoid"}, {"tanh", "nx_tanh"},
          {"rsqrt", "nx_rsqrt"}, {"erf_inv", "nx_erf_inv"}, {"round", "nx_round"}, {"sign", "nx_sign"}};
      if (lib.count(op)) e = fn(lib.at(op)) + "(" + xv + ")";
      else if (own.count(op)) e = std::string(own.at(op)) + "(" + xv + ")";
      else if (op == "negate") e = "-" + xv;
      else fail(NXB_ERR_INVALID_ARGUMENT, "op " + op + " is not defined for " + dtype_name(t));
      if ((t == NXB_BF16 || t == NXB_F16) && excess_ && !exact_in) {
        Val r = def(x.elem, t, e);
        raw_.insert(r.v);
        return r;
      }
      if (t == NXB_BF16) e = "round_bf16(" + e + ")";
      if (t == NXB_F16) e = "round_f16(" + e + ")";
    } else {
      const std::string RT = reg_type(t), UT = unsigned_of(t);
      if (op == "negate") e = "(" + RT + ")((" + UT + ")0 - (" + UT + ")" + xv + ")";
      else if (op == "abs") e = dtype_is_signed(t) ? "(" + RT + ")(" + xv + " < 0 ? (" + UT + ")0 - (" + UT + ")" + xv + " : (" + UT + ")" + xv + ")" : xv;
      else if (op == "sign") e = dtype_is_signed(t) ? "nx_sign_i<" + RT + ">(" + xv + ")" : "(" + RT + ")(" + xv + " != 0)";
      else if (op == "bitwise_not") e = "(" + RT + ")~" + xv;
      else if (op == "floor" || op == "ceil" || op == "round") e = xv;
      else fail(NXB_ERR_INVALID_ARGUMENT, "op " + op + " is not defined for " + dtype_name(t));
    }
    return def(x.elem, t, e);
  }
  if (kBinary.count(op)) {
    const Node& a = g_.nodes[nd.args[0]];
    const Node& b = g_.nodes[nd.args[1]];
    Val x = value(nd.args[0], arg_index_binary(nd, a, idx));
    Val y = value(nd.args[1], arg_index_binary(nd, b, idx));
    bool elem = x.elem || y.elem;
    if (kLogical.count(op)) {
      std::string xa = "(" + exact(x, a.dt) + " != 0)", yb = "(" + exact(y, b.dt) + " != 0)";
      std::string o = op == "logical_and" ? " && " : op == "logical_or" ? " || " : " != ";
      return def(elem, t, "(uint8_t)(" + xa + o + yb + ")");
    }
    // operands are converted to the merged type first, the result to the node's type after
    // (exla/lib/exla/defn.ex:2380-2410)
    DType ct = dtype_merge(a.dt, b.dt);
    if (!kCompare.count(op)) ct = dtype_merge(ct, t);
    const bool cmp = kCompare.count(op) > 0;
    std::string xv = cvt(cmp ? exact(x, a.dt) : x.v, a.dt, ct), yv = cvt(cmp ? exact(y, b.dt) : y.v, b.dt, ct);
    std::string e;
    if (kCompare.count(op)) {
      static const std::map<std::string, const char*> sym = {{"equal", "=="}, {"not_equal", "!="}, {"greater", ">"},
                                                            {"less", "<"}, {"greater_equal", ">="}, {"less_equal", "<="}};
      return def(elem, t, "(uint8_t)(" + xv + " " + sym.at(op) + " " + yv + ")");
    }
    const bool dbl = ct == NXB_F64;
    if (dtype_is_float(ct)) {
      if (op == "add") e = xv + " + " + yv;
      else if (op == "subtract") e = xv + " - " + yv;
      else if (op == "multiply") e = xv + " * " + yv;
      else if (op == "divide") {
        if (mode_ == ROW && x.elem && !y.elem && ct != NXB_F64) {
          // dividing a row by a per-row value: one reciprocal per row, one multiply per element
          std::string rk = "rcp:" + yv;
          auto it = row_memo_.find(rk);
          std::string rv;
          if (it != row_memo_.end()) rv = it->second;
          else {
            rv = newvar("rc");
            stmt(false, "const float " + rv + " = 1.0f / " + yv + ";");
            row_memo_[rk] = rv;
          }
          e = xv + " * " + rv;
        } else {
          e = xv + " / " + yv;
        }
      }
      else if (op == "max") e = "nx_max(" + xv + ", " + yv + ")";
      else if (op == "min") e = "nx_min(" + xv + ", " + yv + ")";
      else if (op == "pow") e = std::string(dbl ? "pow" : "powf") + "(" + xv + ", " + yv + ")";
      else if (op == "remainder") e = std::string(dbl ? "fmod" : "fmodf") + "(" + xv + ", " + yv + ")";
      else if (op == "atan2") e = std::string(dbl ? "atan2" : "atan2f") + "(" + xv + ", " + yv + ")";
      else fail(NXB_ERR_INVALID_ARGUMENT, "op " + op + " is not defined for " + dtype_name(ct));
      const bool keeps = op == "add" || op == "subtract" || op == "multiply" || op == "divide" || op == "max" || op == "min";
      if ((ct == NXB_BF16 || ct == NXB_F16) && ct == t && excess_ && keeps) {
        Val r = def(elem, t, e);
        raw_.insert(r.v);
        return r;
      }
      if (ct == NXB_BF16) e = "round_bf16(" + e + ")";
      if (ct == NXB_F16) e = "round_f16(" + e + ")";
    } else {
      const std::string RT = reg_type(ct), UT = unsigned_of(ct);
      auto wrap = [&](const char* o) { return "(" + RT + ")((" + UT + ")" + xv + " " + o + " (" + UT + ")" + yv + ")"; };
      if (op == "add") e = wrap("+");
      else if (op == "subtract") e = wrap("-");
      else if (op == "multiply") e = wrap("*");
      else if (op == "bitwise_and") e = wrap("&");
      else if (op == "bitwise_or") e = wrap("|");
      else if (op == "bitwise_xor") e = wrap("^");
      else if (op == "max") e = "nx_max(" + xv + ", " + yv + ")";
      else if (op == "min") e = "nx_min(" + xv + ", " + yv + ")";
      else if (op == "quotient" || op == "divide") e = "nx_idiv<" + RT + ">(" + xv + ", " + yv + ")";
      else if (op == "remainder") e = "nx_irem<" + RT + ">(" + xv + ", " + yv + ")";
      else if (op == "pow") e = "nx_ipow<" + RT + ">(" + xv + ", " + yv + ")";
      else if (op == "left_shift") e = "nx_shl<" + RT + ">(" + xv + ", " + yv + ")";
      else if (op == "right_shift") {
        // the reference shifts logically when the RESULT type is unsigned, whatever signed type the operands
        // were merged to (a u64 tensor shifted by a number is computed in s64): exla/lib/exla/defn.ex:1328-1335
        if (!dtype_is_signed(t) && dtype_is_signed(ct)) e = "(" + RT + ")nx_shr<" + UT + ">((" + UT + ")" + xv + ", (" + UT + ")" + yv + ")";
        else e = "nx_shr<" + RT + ">(" + xv + ", " + yv + ")";
      }
      else fail(NXB_ERR_INVALID_ARGUMENT, "op " + op + " is not defined for " + dtype_name(ct));
    }
    return def(elem, t, cvt(e, ct, t));
  }
  if (op == "select") {
    const Node& p = g_.nodes[nd.args[0]];
    const Node& a = g_.nodes[nd.args[1]];
    const Node& b = g_.nodes[nd.args[2]];
    Val pv = value(nd.args[0], arg_index_binary(nd, p, idx));
    Val x = value(nd.args[1], arg_index_binary(nd, a, idx));
    Val y = value(nd.args[2], arg_index_binary(nd, b, idx));
    Val r = def(pv.elem || x.elem || y.elem, t, "(" + pv.v + " != 0) ? " + cvt(x.v, a.dt, t) + " : " + cvt(y.v, b.dt, t));
    if ((t == NXB_BF16 || t == NXB_F16) && (raw_.count(x.v) || raw_.count(y.v))) raw_.insert(r.v);
    return r;
  }
  if (op == "clip") {
    Val x = value(nd.args[0], idx);
    Val lo = value(nd.args[1], {});
    Val hi = value(nd.args[2], {});
    std::string e = "nx_min(nx_max(" + cvt(x.v, g_.nodes[nd.args[0]].dt, t) + ", " + cvt(lo.v, g_.nodes[nd.args[1]].dt, t) + "), " +
                    cvt(hi.v, g_.nodes[nd.args[2]].dt, t) + ")";
    Val r = def(x.elem || lo.elem || hi.elem, t, e);
    if ((t == NXB_BF16 || t == NXB_F16) && raw_.count(x.v)) raw_.insert(r.v);
    return r;
  }
  throw FusionError("op " + op + " cannot be generated inline");
}

void KernelBuilder::emit_store(int n) {
  const Node& nd = g_.nodes[n];
  bool full;
  std::vector<Aff> idx = index_for_shape(nd.shape, &full);
  Val v = value(n, idx);
  std::string p = param(nd.slot);
  const std::string S = storage_type(nd.dt), Rt = reg_type(nd.dt);
  // a piece of a concatenate writes into its parent's buffer with the parent's strides
  auto st = nd.out_strides.empty() ? cstrides(nd.shape) : nd.out_strides;
  Aff addr = aff_const(nv_, nd.out_offset);
  for (size_t j = 0; j < idx.size(); ++j) {
    addr.c += idx[j].c * st[j];
    for (int q = 0; q < nv_; ++q) addr.k[q] += idx[j].k[q] * st[j];
  }
  if (full && addr.c == 0 && addr.k == cstrides(F_) && shape_numel(nd.shape) == numel_ && nd.window_axes.empty()) ident_stores_.insert(nd.slot);
  std::string dyn;       // offset of a window whose position is held in scalar tensors
  bool dyn_aligned = true;
  for (size_t i = 0; i < nd.window_axes.size(); ++i) {
    Val sv = value(nd.args[1 + i], {});
    // (per element, with scalar stores: a window is small next to the tensor it lands in)
    std::string o = newvar("wo");
    stmt(true, "const " + idx_t() + " " + o + " = (" + idx_t() + ")nx_clamp_index(" + sv.v + ", (long long)" + std::to_string(nd.window_limit[i]) + ") * (" +
                   idx_t() + ")" + std::to_string(st[nd.window_axes[i]]) + ";");
    dyn += " + " + o;
    dyn_aligned = false;
  }
  if (mode_ == EPI && epi_to_regs) {
    bool ident = full && addr.c == 0 && shape_numel(nd.shape) == numel_ && nd.window_axes.empty() && nd.out_strides.empty();
    const std::vector<int64_t> fs = cstrides(F_);
    for (int q = 0; q < nv_; ++q) if (F_[q] != 1 && addr.k[q] != fs[q]) ident = false;     // extents of 1 carry no index
    if (ident && (nd.dt == NXB_BF16 || nd.dt == NXB_F16 || nd.dt == NXB_F32)) {
      lane_sec_[phase_] += "        out[v] = " + v.v + ";\n";
      return;
    }
    epi_regs_ok = false;
  }
  if (mode_ == ROW && !full) {
    // one value per row: lane 0 of the row writes it
    row_sec_[phase_] += "        if (tid == 0) st1<" + S + ">(" + p + " + " + affstr(addr, false) + ", " + v.v + ");\n";
    return;
  }
  bool aligned = addr.c % V_ == 0 && addr.k[nv_ - 1] == 1 && dyn_aligned;
  for (int j = 0; j < nv_ - 1; ++j) if (F_[j] != 1 && addr.k[j] % V_ != 0) aligned = false;
  if (V_ > 1 && aligned) {
    std::string sv = newvar("st");
    pre_sec_[phase_] += "          " + Rt + " " + sv + "[" + std::to_string(V_) + "];\n";
    lane_sec_[phase_] += "        " + sv + "[v] = " + v.v + ";\n";
    post_sec_[phase_] += "          st_vec<" + S + ", " + std::to_string(V_) + ">(" + p + " + " + affstr(addr, true) + dyn + ", " + sv + ");\n";
  } else {
    lane_sec_[phase_] += "        st1<" + S + ">(" + p + " + " + affstr(addr, false) + dyn + ", " + v.v + ");\n";
  }
}

void KernelBuilder::configure() {
  // vector width: 16 bytes of the narrowest element touched, limited by divisibility
  size_t minsz = 8;
  for (int n : stores) minsz = std::min(minsz, dtype_size(g_.nodes[n].dt));
  for (int n : reduces) minsz = std::min(minsz, dtype_size(g_.nodes[g_.nodes[n].args[0]].dt));
  std::function<void(int, std::set<int>&)> scan = [&](int n, std::set<int>& seen) {
    if (!seen.insert(n).second) return;
    const Node& nd = g_.nodes[n];
    if (n == acc_node) return;
    if (nd.slot >= 0 && !made_here(n) && !aliases_acc(n)) {
      if (strip_units(nd.shape) == strip_units(F_)) minsz = std::min(minsz, dtype_size(nd.dt));
      return;
    }
    for (int a : nd.args) scan(a, seen);
  };
  std::set<int> seen;
  for (int n : stores) scan(n, seen);
  for (int n : reduces) scan(n, seen);
  V_ = (int)std::min<size_t>(8, 16 / minsz);
  if (!perm_.empty()) V_ = 1;
  if (mode_ == EPI) V_ = force_v;
  while (V_ > 1 && F_[nv_ - 1] % V_ != 0) V_ /= 2;
  big_ = numel_ >= (int64_t(1) << 31) - 4096;
  for (int n : seen)
    if (shape_numel(g_.nodes[n].shape) >= (int64_t(1) << 31) - 4096) big_ = true;
  if (mode_ == ROW) {
    int64_t per = std::max<int64_t>(1, C_ / V_);
    int64_t want = (per + 3) / 4;        // aim for <= 4 vectors per thread
    T_ = 32;
    while (T_ < want && T_ < 1024) T_ *= 2;
    chunks_ = (int)((per + T_ - 1) / T_);
    guard_ = (per % T_) != 0;
    if (T_ >= 64) { block_ = T_; rpc_ = 1; } else { block_ = 128; rpc_ = 4; }
    cache_ = chunks_ * V_ <= 32 && chunks_ <= 16;
    // worth it when a CTA is so large that only one fits per SM (nothing else hides the load)
    stage_ = cache_ && rpc_ == 1 && !guard_ && block_ >= 512 && perm_.empty() && R_ > 148;
  } else {
    block_ = 256;
  }
}

KernelSpec KernelBuilder::build(const std::string& name) {
  if (!planning_ && mode_ == ROW && !getenv("NXB200_NO_REGISTER_REUSE")) {
    KernelBuilder probe(*this);
    probe.planning_ = true;
    probe.build(name);
    // a value computed in phase p and again later, and a row-register array of the same type that
    // nothing else reads after p: keep the value there
    std::set<std::string> taken;
    for (auto& e : probe.emitted_in_) {
      if (e.second.size() < 2) continue;
      const int p = *e.second.begin();
      for (auto& lr : probe.load_refs_) {
        const std::string& lk = lr.first;
        if (taken.count(lk) || probe.load_type_[lk] != NXB_F32) continue;
        bool ok = false, clean = true;
        for (auto& r : lr.second) {
          if (r.phase <= p) { if (r.phase == p && r.ctx.count(e.first)) ok = true; continue; }
          if (!r.ctx.count(e.first)) clean = false;       // someone else still needs the row value later
        }
        if (ok && clean) {
          stash_plan_[e.first] = Stash{probe.load_array_[lk], p};
          taken.insert(lk);
          break;
        }
      }
    }
  }
  for (int n : stores) produced.insert(n);
  for (int sl : seed_args) param(sl);
  configure();

  // phases
  std::map<int, int> red_phase;
  nphases_ = 1;
  if (mode_ == ROW) {
    for (int r : reduces) {
      red_phase[r] = level(g_.nodes[r].args[0]);
      nphases_ = std::max(nphases_, red_phase[r] + 1);
    }
    for (int s : stores) nphases_ = std::max(nphases_, level(s) + 1);
  }
  row_sec_.assign(nphases_ + 1, "");
  pre_sec_.assign(nphases_ + 1, "");
  lane_sec_.assign(nphases_ + 1, "");
  post_sec_.assign(nphases_ + 1, "");
  elem_memo_.assign(nphases_ + 1, {});
  std::vector<std::string> red_init(nphases_ + 1), red_fin(nphases_ + 1);
  struct Fin { bool arg; std::string acc, res, op, rt, out_rt, round; };
  std::vector<std::vector<Fin>> fins(nphases_ + 1);
  int scratch_slots = 2;

  std::vector<int> row_stores;
  static const bool defer_off = getenv("NXB200_NO_DEFERRED_STORES") != nullptr;
  for (phase_ = 0; phase_ < nphases_; ++phase_) {
    for (int r : reduces) {
      if (red_phase[r] != phase_) continue;
      const Node& nd = g_.nodes[r];
      const Node& in = g_.nodes[nd.args[0]];
      // index of the input element in terms of the kernel's variables
      std::vector<Aff> idx(in.shape.size(), aff_const(nv_, 0));
      if (!perm_.empty()) {
        for (int j = 0; j < nv_; ++j) if (F_[j] != 1) idx[perm_[j]] = aff_var(nv_, j);
      } else if (in.shape.empty()) {
        idx.clear();
      } else {
        bool full;
        idx = index_for_shape(in.shape, &full);
        if (!full && C_ != 1) throw FusionError("reduction input does not span the kernel space");
      }
      Val x = value(nd.args[0], idx);
      std::string acc = newvar("acc"), res = newvar("red");
      const std::string T = std::to_string(T_);
      if (kArgReduce.count(nd.op)) {
        const std::string RT = reg_type(in.dt);
        bool is_max = nd.op == "argmax", high = nd.ints[0] != 0;
        std::string tpl = std::string(is_max ? "true" : "false") + ", " + (high ? "true" : "false");
        red_init[phase_] += "      ArgPair<" + RT + "> " + acc + "; " + acc + ".v = (" + RT + ")0; " + acc + ".i = -1;\n";
        lane_sec_[phase_] += "        arg_step<" + tpl + ">(" + acc + ", " + exact(x, in.dt) + ", (long long)(col0 + v));\n";
        fins[phase_].push_back({true, acc, res, tpl, RT, reg_type(nd.dt), ""});
      } else {
        DType ot = nd.dt;
        const std::string RT = reg_type(ot);
        std::string init, opn, xv = cvt(x.v, in.dt, ot);
        if (nd.op == "sum") { init = "(" + RT + ")0"; opn = "OpSum"; }
        else if (nd.op == "product") { init = "(" + RT + ")1"; opn = "OpProd"; }
        else if (nd.op == "reduce_max") {
          opn = "OpMax";
          init = dtype_is_float(ot) ? (ot == NXB_F64 ? "-(double)NXB_INF" : "-NXB_INF")
                                    : literal(0, dtype_is_signed(ot) ? -(int64_t)((uint64_t)1 << (dtype_size(ot) * 8 - 1)) : 0, false, ot);
        } else if (nd.op == "reduce_min") {
          opn = "OpMin";
          int bits = (int)dtype_size(ot) * 8;
          int64_t mx = dtype_is_signed(ot) ? (int64_t)(((uint64_t)1 << (bits - 1)) - 1) : (bits == 64 ? -1 : (int64_t)(((uint64_t)1 << bits) - 1));
          init = dtype_is_float(ot) ? (ot == NXB_F64 ? "(double)NXB_INF" : "NXB_INF") : literal(0, mx, false, ot);
        } else if (nd.op == "all") { init = "(uint8_t)1"; opn = "OpAnd"; xv = "(uint8_t)(" + exact(x, in.dt) + " != 0)"; }
        else { init = "(uint8_t)0"; opn = "OpOr"; xv = "(uint8_t)(" + exact(x, in.dt) + " != 0)"; }
        // narrow integer accumulators are widened to 32 bits for the shuffle
        red_init[phase_] += "      " + RT + " " + acc + " = " + init + ";\n";
        lane_sec_[phase_] += "        " + acc + " = " + opn + "::apply(" + acc + ", " + xv + ");\n";
        fins[phase_].push_back({false, acc, res, opn, RT, RT, ot == NXB_BF16 ? "round_bf16" : ot == NXB_F16 ? "round_f16" : ""});
      }
      red_var_[r] = res;
    }
    for (int s : stores) {
      if (mode_ == ROW) {
        bool full;
        index_for_shape(g_.nodes[s].shape, &full);
        if (!full) { if (phase_ == 0) row_stores.push_back(s); continue; }
        // A full-size result that depends on no reduction could be stored in the first phase.  With the row
        // in registers it is stored in the second instead: the first phase then only reduces (no stores
        // queue up behind the load of the next row), and the result's arithmetic runs between the stores
        // of the second phase (measured on the fused row configuration: 0.736 -> 0.715 ms).
        int sp = level(s);
        if (sp == 0 && nphases_ > 1 && cache_ && !defer_off) sp = 1;
        if (sp != phase_) continue;
      }
      emit_store(s);
    }
    if (ret_node >= 0) {
      Val r = value(ret_node, full_index());
      lane_sec_[0] += "        result = " + cvt(r.v, g_.nodes[ret_node].dt, NXB_F32) + ";\n";
    }
    // values kept for later phases overwrite the row registers they outlive (last statement of the phase)
    for (auto& sp : stash_plan_) {
      if (sp.second.phase != phase_) continue;
      auto it = elem_memo_[phase_].find(sp.first);
      if (it == elem_memo_[phase_].end()) throw FusionError("internal: planned value was not generated in its phase");
      lane_sec_[phase_] += "        " + sp.second.array + "[ch][v] = " + it->second + ";\n";
    }
  }
  // finish the reductions of each phase together: one pair of barriers per phase
  for (int p = 0; p < nphases_; ++p) {
    if (fins[p].empty()) continue;
    const std::string T = std::to_string(T_);
    std::string& o = red_fin[p];
    int slot = 0;
    std::vector<int> slots;
    for (auto& f : fins[p]) {
      if (f.arg) o += "      ArgPair<" + f.rt + "> w_" + f.res + " = warp_arg_reduce<" + f.op + ">(" + f.acc + ");\n";
      else o += "      " + f.rt + " w_" + f.res + " = warp_reduce<" + f.op + ">(" + f.acc + ");\n";
      slots.push_back(slot);
      slot += f.arg ? 2 : 1;
    }
    scratch_slots = std::max(scratch_slots, slot);
    if (T_ > 32) {
      o += "      __syncthreads();\n      if ((threadIdx.x & 31) == 0) {\n";
      for (size_t i = 0; i < fins[p].size(); ++i) {
        auto& f = fins[p][i];
        o += std::string("        ") + (f.arg ? "park_arg_partial<" : "park_partial<") + f.rt + ">(scratch, " + std::to_string(slots[i]) + ", w_" + f.res + ");\n";
      }
      o += "      }\n      __syncthreads();\n";
      for (size_t i = 0; i < fins[p].size(); ++i) {
        auto& f = fins[p][i];
        if (f.arg) o += "      w_" + f.res + " = fold_arg_partials<" + f.op + ", " + f.rt + ", " + T + ">(scratch, " + std::to_string(slots[i]) + ");\n";
        else o += "      w_" + f.res + " = fold_partials<" + f.op + ", " + f.rt + ", " + T + ">(scratch, " + std::to_string(slots[i]) + ");\n";
      }
    }
    for (auto& f : fins[p]) {
      if (f.arg) o += "      const " + f.out_rt + " " + f.res + " = (" + f.out_rt + ")w_" + f.res + ".i;\n";
      else o += "      const " + f.out_rt + " " + f.res + " = " + (f.round.empty() ? "w_" + f.res : f.round + "(w_" + f.res + ")") + ";\n";
    }
  }
  // results of reductions that are themselves kernel outputs, and other per-row values
  phase_ = nphases_;
  for (int r : reduces) {
    const Node& nd = g_.nodes[r];
    if (nd.slot < 0) continue;
    // address of the result: its own shape indexed by the row variables
    bool full;
    std::vector<Aff> idx = index_for_shape(nd.shape, &full);
    auto st = cstrides(nd.shape);
    Aff addr = aff_const(nv_, 0);
    for (size_t j = 0; j < idx.size(); ++j) {
      addr.c += idx[j].c * st[j];
      for (int q = 0; q < nv_; ++q) addr.k[q] += idx[j].k[q] * st[j];
    }
    row_sec_[phase_] += "        if (tid == 0) st1<" + std::string(storage_type(nd.dt)) + ">(" + param(nd.slot) + " + " + affstr(addr, false) + ", " + red_var_[r] + ");\n";
  }
  for (int s : row_stores) emit_store(s);

  // ---- assemble the source ------------------------------------------------------------------
  std::ostringstream o;
  const std::string I = idx_t();
  std::vector<const Node*> argn;
  auto is_written = [&](int slot) {
    for (int s : stores) if (g_.nodes[s].slot == slot) return true;
    for (int r : reduces) if (g_.nodes[r].slot == slot) return true;
    return false;
  };
  if (mode_ == EPI && ret_node >= 0) {
    o << "__device__ __forceinline__ float " << name << "(const float accv, const long long bh, const long long qrow, const long long kcol, void* const* ep) {\n";
    o << "  const float* acc = &accv;\n  float result = 0.f;\n";
    for (size_t i = 0; i < arg_slots_.size(); ++i) {
      const Slot& sl = plan_.slots[arg_slots_[i]];
      o << "  const " << storage_type(sl.dt) << "* __restrict__ p" << i << " = (const " << storage_type(sl.dt) << "*)ep[" << i << "];\n";
    }
  } else if (mode_ == EPI) {
    o << "__device__ __forceinline__ void " << name << "(const float* acc, const " << I << " flat0, void* const* ep" << (epi_to_regs ? ", float* out" : "") << ") {\n";
    for (size_t i = 0; i < arg_slots_.size(); ++i) {
      const Slot& sl = plan_.slots[arg_slots_[i]];
      o << "  " << (is_written(arg_slots_[i]) ? "" : "const ") << storage_type(sl.dt) << "* __restrict__ p" << i << " = (" <<
          (is_written(arg_slots_[i]) ? "" : "const ") << storage_type(sl.dt) << "*)ep[" << i << "];\n";
    }
  } else {
    o << "extern \"C\" __global__ void __launch_bounds__(" << block_ << ") " << name << "(";
    for (size_t i = 0; i < arg_slots_.size(); ++i) {
      const Slot& sl = plan_.slots[arg_slots_[i]];
      o << (i ? ", " : "") << (is_written(arg_slots_[i]) ? "" : "const ") << storage_type(sl.dt) << "* __restrict__ p" << i;
    }
    o << ") {\n";
  }
  auto decomp = [&](int lo, int hi, const std::string& src, bool with_base) {
    // define index variables i<lo>..i<hi-1> from the linear index `src`
    std::string rem = src;
    for (int j = hi - 1; j >= lo; --j) {
      if (F_[j] == 1) continue;
      bool last_nonunit = true;
      for (int q = lo; q < j; ++q) if (F_[q] != 1) last_nonunit = false;
      std::string nm = (with_base && j == nv_ - 1) ? "ib" : "i" + std::to_string(j);
      if (used_vars_.count(j)) {
        o << "        const " << I << " " << nm << " = " << (last_nonunit ? rem : "(" + rem + ") % (" + I + ")" + std::to_string(F_[j])) << ";\n";
      }
      if (!last_nonunit) rem = "(" + rem + ") / (" + I + ")" + std::to_string(F_[j]);
    }
  };
  if (mode_ == EPI && ret_node >= 0) {
    // index variables: the batch dims from `bh`, then the query row and the key column
    if (nv_ > 2) decomp(0, nv_ - 2, "(" + I + ")bh", false);
    if (nv_ >= 2 && used_vars_.count(nv_ - 2)) o << "        const " << I << " i" << nv_ - 2 << " = (" << I << ")qrow;\n";
    o << "        const " << I << " ib = (" << I << ")kcol;\n";
    o << pre_sec_[0];
    o << "      { const int v = 0;\n";
    if (used_vars_.count(nv_ - 1)) o << "        const " << I << " i" << nv_ - 1 << " = ib;\n";
    o << lane_sec_[0] << "      }\n  return result;\n}\n";
  } else if (mode_ == EPI) {
    decomp(0, nv_, "flat0", true);
    o << pre_sec_[0];
    o << "#pragma unroll\n      for (int v = 0; v < " << V_ << "; ++v) {\n";
    if (used_vars_.count(nv_ - 1)) o << "        const " << I << " i" << nv_ - 1 << " = ib + v;\n";
    if (used_flat_) o << "        const " << I << " flat = flat0 + v;\n";
    o << lane_sec_[0] << "      }\n" << post_sec_[0] << "}\n";
  } else if (mode_ == EW) {
    int64_t nvec = numel_ / V_;
    o << "  const " << I << " nvec = (" << I << ")" << nvec << "LL;\n";
    o << "  for (" << I << " g = (" << I << ")blockIdx.x * " << block_ << " + threadIdx.x; g < nvec; g += (" << I << ")gridDim.x * " << block_ << ") {\n";
    o << "        const " << I << " flat0 = g * " << V_ << ";\n";
    decomp(0, nv_, "flat0", true);
    o << row_sec_[0];          // values that depend on no index (e.g. a comparison of two literals)
    o << pre_sec_[0];
    o << "#pragma unroll\n      for (int v = 0; v < " << V_ << "; ++v) {\n";
    if (used_vars_.count(nv_ - 1)) o << "        const " << I << " i" << nv_ - 1 << " = ib + v;\n";
    if (used_flat_) o << "        const " << I << " flat = flat0 + v;\n";
    o << lane_sec_[0] << "      }\n" << post_sec_[0] << "  }\n}\n";
  } else {
    o << "  __shared__ long long scratch_all[" << 32 * scratch_slots << "];\n";
    o << "  void* scratch = scratch_all;\n";
    if (rpc_ > 1) o << "  const int tid = threadIdx.x & 31;\n  const " << I << " row_in_cta = threadIdx.x >> 5;\n";
    else o << "  const int tid = threadIdx.x;\n  const " << I << " row_in_cta = 0;\n";
    const bool staging = !staged_.empty();
    std::string issue_copies;      // lane 0 posts the byte count and one bulk copy per staged input
    if (staging) {
      int64_t total = 0;
      for (auto& sg : staged_) total += sg.bytes;
      issue_copies = "stg_expect(&stage_bar, " + std::to_string(total) + "u);";
      for (auto& sg : staged_)
        issue_copies += " stg_copy(stage_buf + " + std::to_string(sg.offset) + ", " + sg.param + " + NEXT_ROW * (" + I + ")" + std::to_string(C_) + "LL, " +
                        std::to_string(sg.bytes) + "u, &stage_bar);";
      o << "  extern __shared__ __align__(1024) unsigned char stage_buf[];\n";
      o << "  __shared__ unsigned long long stage_bar;\n  __shared__ int stage_off;\n";
      o << "  if (threadIdx.x == 0) { stg_bar_init(&stage_bar); stage_off = 0; }\n  __syncthreads();\n";
      o << "  unsigned stage_parity = 0;\n";
      std::string first = issue_copies;
      for (size_t pos; (pos = first.find("NEXT_ROW")) != std::string::npos;) first.replace(pos, 8, "((" + I + ")blockIdx.x)");
      o << "  if (threadIdx.x == 0 && (" << I << ")blockIdx.x < (" << I << ")" << R_ << "LL) { " << first << " }\n";
    }
    o << "  for (" << I << " row = (" << I << ")blockIdx.x * " << rpc_ << " + row_in_cta; row < (" << I << ")" << R_ << "LL; row += (" << I << ")gridDim.x * " << rpc_ << ") {\n";
    o << "        const " << I << " rowbase = row * (" << I << ")" << C_ << "LL;\n";
    if (staging) {
      o << "        bool use_stage = stage_off == 0;\n";
      o << "        if (use_stage) { if (!stg_wait(&stage_bar, stage_parity)) { stage_off = 1; use_stage = false; } stage_parity ^= 1u; }\n";
    }
    decomp(0, nv_ - k_, "row", false);
    o << decls_;
    if (staging) {
      std::string next = issue_copies;
      for (size_t pos; (pos = next.find("NEXT_ROW")) != std::string::npos;) next.replace(pos, 8, "(row + (" + I + ")gridDim.x)");
      o << "#pragma unroll\n      for (int ch = 0; ch < " << chunks_ << "; ++ch) {\n";
      o << "        const " << I << " col0 = ((" << I << ")ch * " << T_ << " + tid) * " << V_ << ";\n" << stage_load_sec_ << "      }\n";
      // every thread has its part of the row in registers: the buffer can take the next row
      o << "      __syncthreads();\n";
      o << "      if (threadIdx.x == 0 && stage_off == 0 && row + (" << I << ")gridDim.x < (" << I << ")" << R_ << "LL) { " << next << " }\n";
    }
    for (int p = 0; p < nphases_; ++p) {
      o << row_sec_[p] << red_init[p];
      bool has_loop = !pre_sec_[p].empty() || !lane_sec_[p].empty() || !post_sec_[p].empty();
      if (has_loop) {
        o << (cache_ || chunks_ <= 16 ? "#pragma unroll\n" : "#pragma unroll 2\n");
        o << "      for (int ch = 0; ch < " << chunks_ << "; ++ch) {\n";
        o << "        const " << I << " col0 = ((" << I << ")ch * " << T_ << " + tid) * " << V_ << ";\n";
        if (guard_) o << "        if (col0 < (" << I << ")" << C_ << "LL) {\n";
        o << "        const " << I << " flat0 = rowbase + col0;\n";
        // column variables
        {
          std::string rem = "col0";
          for (int j = nv_ - 1; j >= nv_ - k_; --j) {
            if (F_[j] == 1) continue;
            bool last_nonunit = true;
            for (int q = nv_ - k_; q < j; ++q) if (F_[q] != 1) last_nonunit = false;
            std::string nm = (j == nv_ - 1) ? "ib" : "i" + std::to_string(j);
            if (used_vars_.count(j))
              o << "        const " << I << " " << nm << " = " << (last_nonunit ? rem : "(" + rem + ") % (" + I + ")" + std::to_string(F_[j])) << ";\n";
            if (!last_nonunit) rem = "(" + rem + ") / (" + I + ")" + std::to_string(F_[j]);
          }
        }
        o << pre_sec_[p];
        o << "#pragma unroll\n        for (int v = 0; v < " << V_ << "; ++v) {\n";
        if (used_vars_.count(nv_ - 1)) o << "        const " << I << " i" << nv_ - 1 << " = ib + v;\n";
        if (used_flat_) o << "        const " << I << " flat = flat0 + v;\n";
        o << lane_sec_[p] << "        }\n" << post_sec_[p];
        if (guard_) o << "        }\n";
        o << "      }\n";
      }
      o << red_fin[p];
    }
    o << row_sec_[nphases_];
    o << "  }\n}\n";
  }

  KernelSpec ks;
  ks.name = name;
  ks.source = o.str();
  ks.block = (unsigned)block_;
  ks.arg_slots = arg_slots_;
  ks.arg_offsets.assign(arg_slots_.size(), 0);
  for (int sl : arg_slots_) if (is_written(sl)) ks.written_slots.push_back(sl);
  if (mode_ == EW || (mode_ == ROW && cache_)) {
    // (a row kernel that re-reads its input in later phases would see its own results)
    for (auto& kv : ident_loads_) if (kv.second) ks.inplace_ok.push_back(kv.first);
    for (int sl : ident_stores_) ks.inplace_ok.push_back(-1 - sl);      // negative: written at the thread's own position
  }
  int64_t nblocks;
  if (mode_ == EW) nblocks = (numel_ / V_ + block_ - 1) / block_;
  else nblocks = (R_ + rpc_ - 1) / rpc_;
  if (!staged_.empty()) {
    nblocks = std::min<int64_t>(nblocks, 148);      // persistent: one CTA per SM walks the rows
    ks.smem = (unsigned)stage_bytes_;
  }
  ks.grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(nblocks, 0x7fffffff));
  std::ostringstream d;
  d << name << (mode_ == EW ? " elementwise" : " row") << " space=" << shape_str(F_);
  if (mode_ == ROW) d << " rows=" << R_ << " cols=" << C_ << " threads/row=" << T_ << " phases=" << nphases_ << (cache_ ? " row-in-registers" : " streaming")
                      << (staged_.empty() ? "" : " next-row-staged-in-smem");
  d << " vec=" << V_ << " grid=" << ks.grid << " block=" << ks.block << " stores=[";
  for (size_t i = 0; i < stores.size(); ++i) d << (i ? "," : "") << g_.nodes[stores[i]].op << "#" << stores[i];
  d << "] reduces=[";
  for (size_t i = 0; i < reduces.size(); ++i) d << (i ? "," : "") << g_.nodes[reduces[i]].op << "#" << reduces[i];
  d << "]";
  ks.desc = d.str();
  return ks;
}

}  // namespace

// =====================================================================================
// planner
// =====================================================================================

namespace {

struct Unit {           // one launch-to-be
  enum Kind { ROW, EW, GEMM, ALLREDUCE, ATTN } kind = EW;
  bool fused_epilogue = false;   // GEMM whose epilogue computes `stores`
  std::vector<int64_t> F;
  int k = 0;
  std::vector<int> perm;
  std::vector<int> reduces, stores;
  int gemm_node = -1;
  std::set<int> reads, writes;   // slots
};

struct Planner {
  Plan& plan;
  Graph& g;
  std::vector<char> mat;            // value must live in a slot
  explicit Planner(Plan& p) : plan(p), g(p.g) {}

  int new_slot(Slot::Kind kind, int node, int index) {
    Slot s;
    s.kind = kind;
    s.node = node;
    s.index = index;
    s.dt = g.nodes[node].dt;
    s.shape = g.nodes[node].shape;
    s.nbytes = (size_t)shape_numel(s.shape) * dtype_size(s.dt);
    plan.slots.push_back(s);
    return (int)plan.slots.size() - 1;
  }

  // reductions whose axes are the trailing ones: signature = (input shape, k)
  bool trailing_reduce(const Node& nd, std::vector<int64_t>* F, int* k, std::vector<int>* perm) {
    const Node& in = g.nodes[nd.args[0]];
    int r = (int)in.shape.size();
    std::vector<int> axes;
    if (kArgReduce.count(nd.op)) {
      if (nd.ints[1] < 0) for (int j = 0; j < r; ++j) axes.push_back(j);
      else axes.push_back((int)nd.ints[1]);
    } else {
      for (int j = 0; j < nd.ints[1]; ++j) axes.push_back((int)nd.ints[2 + j]);
    }
    std::sort(axes.begin(), axes.end());
    bool trailing = true;
    for (size_t j = 0; j < axes.size(); ++j) if (axes[j] != r - (int)axes.size() + (int)j) trailing = false;
    *k = (int)axes.size();
    perm->clear();
    if (trailing) { *F = in.shape; return true; }
    // move the reduced axes last
    F->clear();
    for (int j = 0; j < r; ++j) if (!std::count(axes.begin(), axes.end(), j)) { F->push_back(in.shape[j]); perm->push_back(j); }
    for (int a : axes) { F->push_back(in.shape[a]); perm->push_back(a); }
    return false;
  }

  // Number of buffer boundaries (dot, concatenate) on the longest path from the inputs.
  // Members of one fused kernel must share it: then no path between two members can
  // leave the kernel through a boundary and come back, i.e. no dependency cycle.
  std::vector<int> depth_memo;
  std::vector<char> table;     // elementwise values materialised as tables (see build_plan)
  int depth(int n) {
    if (depth_memo.size() != g.nodes.size()) depth_memo.assign(g.nodes.size(), -1);
    if (depth_memo[n] >= 0) return depth_memo[n];
    int d = 0;
    for (int a : g.nodes[n].args) {
      const std::string& op = g.nodes[a].op;
      d = std::max(d, depth(a) + ((op == "dot" || op == "concatenate" || op == "all_reduce" || op == "attention" || op == "sort" || op == "argsort" || op == "indexed_add" || op == "indexed_put") ? 1 : 0));
    }
    return depth_memo[n] = d;
  }

  bool is_leaf(int n) const {
    const std::string& op = g.nodes[n].op;
    return op == "parameter" || op == "tensor" || op == "dot" || op == "concatenate" || op == "all_reduce" || op == "attention" || op == "sort" || op == "argsort" ||
           op == "indexed_add" || op == "indexed_put";
  }

  // Nodes reachable backwards through everything a kernel can generate inline
  // (elementwise, views, reductions); `leaves` collects the buffers it ends at.
  void cone(int n, std::set<int>& seen, std::set<int>& leaves, std::set<int>& reds, bool root) {
    if (is_leaf(n)) { leaves.insert(n); return; }
    const Node& nd = g.nodes[n];
    // an elementwise value that is a buffer anyway (a table computed once) ends the cone like a parameter
    if (!root && table[n]) { leaves.insert(n); return; }
    if (!seen.insert(n).second) return;
    if (is_reduce(nd) && !root) reds.insert(n);
    for (int a : nd.args) cone(a, seen, leaves, reds, false);
  }
};

}  // namespace

std::string Plan::describe() const {
  std::ostringstream o;
  for (auto& st : steps) {
    if (st.kind == Step::KERNEL) o << kernels[st.index].desc << "\n";
    else if (st.kind == Step::GEMM) o << gemms[st.index].desc << "\n";
    else if (st.kind == Step::ATTENTION) o << attentions[st.index].desc << "\n";
    else if (st.kind == Step::SORT) o << sorts[st.index].desc << "\n";
    else if (st.kind == Step::SCATTER) o << scatters[st.index].desc << "\n";
    else o << collectives[st.index].desc << "\n";
  }
  for (auto& a : aliases)
    o << "donation: argument " << a.param << " -> result " << a.output << (a.in_place ? " (written in place)" : " (own buffer; the argument is released after the run)") << "\n";
  return o.str();
}

// implemented in gemm_plan.cpp
bool plan_dot(Plan& plan, int node, std::vector<int>& need_materialised, GemmSpec* out);
bool sort_rows_supported(int64_t len);   // sort_rows.cu
void canonicalize_dots(Graph& g);
void share_shifted_exp_sums(Graph& g);
void rewrite_quantised_linears(Graph& g);
void rewrite_attention(Graph& g);
int attn_smem_bytes();
int tc_pick_bn(int64_t m, int64_t n, int64_t batch, int sm_count);
int tc_smem_bytes(int bn);
int tc_block_threads(int64_t k);

static std::unique_ptr<Plan> build_plan_from(const uint8_t* bytes, size_t nbytes, int first_level);

std::unique_ptr<Plan> build_plan(const uint8_t* bytes, size_t nbytes) {
  try {
    return build_plan_from(bytes, nbytes, 2);
  } catch (const Error& first) {
    // A fused row kernel that the runtime compiler rejects (a value the generator placed in a section the
    // kernel does not have): plan again with one kernel per materialised value.  Graphs whose fused plan
    // compiles never come here.
    if (first.status != NXB_ERR_RUNTIME || first.msg.find("failed to compile") == std::string::npos) throw;
    if (getenv("NXB200_NO_REPLAN")) throw;    // diagnostics: show the rejected kernel instead
    try {
      return build_plan_from(bytes, nbytes, 1);
    } catch (const Error&) {
      throw first;
    }
  }
}

// first_level 2: fused row kernels, falling back to level 1 when the units depend on each other;
// first_level 1: one kernel per materialised value from the start
static std::unique_ptr<Plan> build_plan_from(const uint8_t* bytes, size_t nbytes, int first_level) {
  const auto t_start = std::chrono::steady_clock::now();
  auto plan = std::make_unique<Plan>();
  plan->g = parse_graph(bytes, nbytes);
  Graph& g = plan->g;
  // common-subexpression elimination: the tracer gives every call a fresh node, so
  // e.g. two reduce_max over the same tensor arrive as two nodes
  {
    std::map<std::string, int> seen;
    std::vector<int> remap(g.nodes.size());
    for (size_t n = 0; n < g.nodes.size(); ++n) {
      Node& nd = g.nodes[n];
      for (int& a : nd.args) a = remap[a];
      remap[n] = (int)n;
      if (nd.op == "parameter") continue;
      std::string key = nd.op + "|" + std::to_string((int)nd.dt) + "|" + shape_str(nd.shape) + "|";
      for (int a : nd.args) key += std::to_string(a) + ",";
      key += "|";
      for (auto v : nd.ints) key += std::to_string(v) + ",";
      key += "|";
      for (auto v : nd.flts) { char b[32]; uint64_t u; memcpy(&u, &v, 8); snprintf(b, sizeof b, "%llx,", (unsigned long long)u); key += b; }
      key += "|" + nd.blob;
      auto it = seen.find(key);
      if (it != seen.end()) remap[n] = it->second;
      else seen.emplace(std::move(key), (int)n);
    }
    for (int& o : g.outputs) o = remap[o];
  }
  if (!getenv("NXB200_NO_SIMPLIFY")) share_shifted_exp_sums(g);
  rewrite_quantised_linears(g);
  rewrite_attention(g);
  canonicalize_dots(g);
  Planner P(*plan);

  // outputs that are leaves, aliases of leaves, or repeated get an identity node so that
  // every result is a fresh buffer (exla/lib/exla/defn.ex:387-393)
  {
    std::set<int> seen_out;
    for (auto& o : g.outputs) {
      const Node& nd = g.nodes[o];
      bool leafish = nd.op == "parameter" || nd.op == "tensor" || nd.op == "metadata" || nd.op == "reshape" ||
                     nd.op == "squeeze" || !seen_out.insert(o).second;
      if (leafish) {
        Node c;
        c.op = "copy";
        c.dt = nd.dt;
        c.shape = nd.shape;
        c.args = {o};
        g.nodes.push_back(c);
        o = (int)g.nodes.size() - 1;
        seen_out.insert(o);
      }
    }
  }
  // put_slice into a donated argument that nothing else reads: only the window is written, the
  // rest of the result is the argument's own memory (an update of a KV cache costs O(slice))
  std::set<int> window_outputs;
  if (!getenv("NXB200_NO_WINDOW_UPDATE")) {
    std::vector<int> uses(g.nodes.size(), 0);
    for (auto& nd : g.nodes) for (int a : nd.args) uses[a]++;
    for (int o : g.outputs) uses[o]++;
    for (auto& al : g.aliases) {
      const int o = g.outputs[al.second];
      Node& nd = g.nodes[o];
      if (nd.op != "put_slice") continue;
      const int p = nd.args[0];
      if (g.nodes[p].op != "parameter" || g.nodes[p].ints.at(0) != al.first || g.nodes[p].dt != nd.dt) continue;
      const int piece = nd.args[1];
      // Readers of the result are fine (they run after the window was written, on the same memory).
      // The argument itself may only be read by this put_slice and by slices of exactly the window
      // it writes (same start operands, the piece's shape, unit strides): the kernel that writes a
      // window element then reads the old value of that very element, before it stores.
      {
        int others = 0;
        const size_t r = nd.shape.size();
        for (size_t u = 0; u < g.nodes.size(); ++u) {
          const Node& un = g.nodes[u];
          const int reads = (int)std::count(un.args.begin(), un.args.end(), p);
          if (!reads) continue;
          if ((int)u == o && reads == 1) continue;
          bool window_read = un.op == "slice" && reads == 1 && un.args.size() == 1 + r && un.args[0] == p && un.shape == g.nodes[piece].shape &&
                             un.ints.size() == 3 * r;
          for (size_t j = 0; window_read && j < r; ++j)
            if (un.args[1 + j] != nd.args[2 + j] || un.ints[2 * r + j] != 1) window_read = false;
          if (!window_read) ++others;
        }
        if (std::count(g.outputs.begin(), g.outputs.end(), p)) ++others;
        if (others) continue;
      }
      Node w;
      w.op = g.nodes[piece].dt == nd.dt ? "copy" : "as_type";
      w.dt = nd.dt;
      w.shape = g.nodes[piece].shape;
      w.args = {piece};
      w.piece_of = o;
      w.out_strides = cstrides(nd.shape);
      w.out_offset = 0;
      for (size_t j = 0; j < nd.shape.size(); ++j) {
        if (w.shape[j] == nd.shape[j]) continue;           // the piece spans the axis: start is 0
        w.window_axes.push_back((int)j);
        w.window_limit.push_back(nd.shape[j] - w.shape[j] + 1);
        w.args.push_back(nd.args[2 + j]);
      }
      g.nodes.push_back(w);
      Node& out = g.nodes[o];
      out.op = "concatenate";
      out.ints = {0};
      out.args = {(int)g.nodes.size() - 1};
      window_outputs.insert(al.second);
    }
  }
  // concatenate: every input becomes a "piece" node that is written straight into its
  // slice of the result (inputs converted to the result type, exla/lib/exla/defn.ex:1659-1668)
  {
    size_t n0 = g.nodes.size();
    for (size_t n = 0; n < n0; ++n) {
      if (g.nodes[n].op != "concatenate") continue;
      if (g.nodes[n].args.size() == 1 && g.nodes[g.nodes[n].args[0]].piece_of == (int)n) continue;    // a window update (above)
      const int axis = (int)g.nodes[n].ints.at(0);
      const std::vector<int64_t> pst = cstrides(g.nodes[n].shape);
      int64_t off = 0;
      std::vector<int> pieces;
      for (int a : std::vector<int>(g.nodes[n].args)) {
        Node c;
        c.op = g.nodes[a].dt == g.nodes[n].dt ? "copy" : "as_type";
        c.dt = g.nodes[n].dt;
        c.shape = g.nodes[a].shape;
        c.args = {a};
        c.piece_of = (int)n;
        c.out_strides = pst;
        c.out_offset = off * pst[axis];
        off += g.nodes[a].shape[axis];
        g.nodes.push_back(c);
        pieces.push_back((int)g.nodes.size() - 1);
      }
      g.nodes[n].args = pieces;
    }
  }
  const int N = (int)g.nodes.size();

  // liveness + op support
  {
    std::vector<int> stack(g.outputs.begin(), g.outputs.end());
    while (!stack.empty()) {
      int n = stack.back();
      stack.pop_back();
      if (g.nodes[n].live) continue;
      g.nodes[n].live = true;
      for (int a : g.nodes[n].args) stack.push_back(a);
    }
    for (int n = 0; n < N; ++n) {
      const Node& nd = g.nodes[n];
      if (!nd.live) continue;
      bool ok = is_inline(nd) || is_reduce(nd) || nd.op == "parameter" || nd.op == "tensor" || nd.op == "dot" || nd.op == "concatenate" ||
                nd.op == "all_reduce" || nd.op == "attention" || nd.op == "sort" || nd.op == "argsort" || nd.op == "indexed_add" || nd.op == "indexed_put";
      if (!ok) fail(NXB_ERR_UNSUPPORTED, "Nx op :" + nd.op + " is not implemented by the B200 compiler");
      if (nd.op == "slice" && nd.args.size() != 1 && nd.args.size() != 1 + nd.shape.size())
        fail(NXB_ERR_INVALID_ARGUMENT, "slice with dynamic start indices takes one start per axis");
      if (nd.op == "gather") {
        if (nd.args.size() != 2 || nd.ints.empty()) fail(NXB_ERR_INVALID_ARGUMENT, "gather takes (tensor, indices) and its indexed axes");
        const Node& ix = g.nodes[nd.args[1]];
        if (dtype_is_float(ix.dt) || ix.shape.empty() || ix.shape.back() != (int64_t)nd.ints.size())
          fail(NXB_ERR_INVALID_ARGUMENT, "gather indices must be integers with one column per indexed axis");
      }
      if (nd.op == "put_slice" && nd.args.size() != 2 + nd.shape.size())
        fail(NXB_ERR_INVALID_ARGUMENT, "put_slice takes (tensor, slice, one start per axis)");
      if (nd.op == "indexed_add" || nd.op == "indexed_put") {
        if (nd.args.size() != 3 || nd.ints.empty()) fail(NXB_ERR_INVALID_ARGUMENT, nd.op + " takes (tensor, indices, updates) and its indexed axes");
        const Node &tg = g.nodes[nd.args[0]], &ix = g.nodes[nd.args[1]], &up = g.nodes[nd.args[2]];
        if ((ix.dt != NXB_S32 && ix.dt != NXB_S64) || ix.shape.size() != 2 || ix.shape[1] != (int64_t)nd.ints.size())
          fail(NXB_ERR_INVALID_ARGUMENT, nd.op + ": indices must be s32 or s64 {n, indexed axes}");
        if (tg.dt != nd.dt || up.dt != nd.dt || tg.shape != nd.shape || up.shape.empty() || up.shape[0] != ix.shape[0] ||
            up.shape.size() - 1 + nd.ints.size() != nd.shape.size())
          fail(NXB_ERR_INVALID_ARGUMENT, nd.op + ": target and updates must have the result's type, updates {n, slice...}");
        for (size_t k = 0; k < nd.ints.size(); ++k)
          if (nd.ints[k] < 0 || nd.ints[k] >= (int64_t)nd.shape.size() || (k && nd.ints[k] <= nd.ints[k - 1]))
            fail(NXB_ERR_INVALID_ARGUMENT, nd.op + ": axes must be ascending axes of the target");
      }
    }
  }

  // slots for leaves
  plan->param_slots.assign(g.n_params, -1);
  P.mat.assign(N, 0);
  P.table.assign(N, 0);
  for (int n = 0; n < N; ++n) {
    Node& nd = g.nodes[n];
    if (!nd.live) continue;
    if (nd.op == "parameter") {
      int pi = (int)nd.ints[0];
      if (plan->param_slots[pi] < 0) plan->param_slots[pi] = P.new_slot(Slot::PARAM, n, pi);
      nd.slot = plan->param_slots[pi];
    } else if (nd.op == "tensor") {
      nd.slot = P.new_slot(Slot::LITERAL, n, n);
    }
  }
  // what must be materialised regardless of fusion
  for (int o : g.outputs) P.mat[o] = 1;
  std::vector<int> dots, concats, allreduces, attns;
  for (int n = 0; n < N; ++n) {
    const Node& nd = g.nodes[n];
    if (!nd.live) continue;
    if (nd.op == "dot") { P.mat[n] = 1; dots.push_back(n); }
    if (nd.op == "concatenate") { P.mat[n] = 1; concats.push_back(n); }
    if (nd.piece_of >= 0) P.mat[n] = 1;
    if (nd.op == "attention") {
      P.mat[n] = 1;
      attns.push_back(n);
      for (int k = 0; k < 3; ++k) {
        const std::string& aop = g.nodes[nd.args[k]].op;
        if (aop != "parameter" && aop != "tensor") P.mat[nd.args[k]] = 1;
      }
    }
    if (nd.op == "gather") {
      // rows are fetched by computed addresses: the table has to be a buffer
      const std::string& aop = g.nodes[nd.args[0]].op;
      if (aop != "parameter" && aop != "tensor") P.mat[nd.args[0]] = 1;
    }
    if (nd.op == "sort" || nd.op == "argsort") {
      // a library step like the all-reduce: one buffer in, one out (ints: descending[, stable])
      if (nd.args.size() != 1 || nd.shape.empty() || !sort_rows_supported(nd.shape.back()))
        fail(NXB_ERR_UNSUPPORTED, "sort is implemented along a last axis of at most 16384 elements");
    }
    if (nd.op == "all_reduce" || nd.op == "sort" || nd.op == "argsort" || nd.op == "indexed_add" || nd.op == "indexed_put") {
      // library steps: buffers in, one buffer out
      P.mat[n] = 1;
      allreduces.push_back(n);
      for (int a : nd.args) {
        const std::string& aop = g.nodes[a].op;
        if (aop != "parameter" && aop != "tensor") P.mat[a] = 1;
      }
    }
  }
  // A value with transcendental functions in it that a much larger consumer broadcasts (the cos / sin
  // table of a rotary embedding under {batch, head, position, dim}) is computed once into a buffer: inline,
  // every element of the consumer would evaluate it again (256 times per table entry in the decoder
  // block, with the full-range cosf / sinf).  Only where it pays: a consumer of at least a million
  // elements, sixteen of them per table entry, and nothing in the value that needs a kernel of its own.
  if (!getenv("NXB200_NO_TABLES")) {
    std::function<int(int)> expensive_ops = [&](int a) -> int {     // -1: not a plain elementwise value
      const Node& nd = g.nodes[a];
      if (nd.op == "parameter" || nd.op == "tensor" || nd.op == "constant" || nd.op == "iota" || P.mat[a]) return 0;
      if (!is_inline(nd) || nd.op == "gather" || nd.op == "put_slice") return -1;
      int total = kUnaryMath.count(nd.op) || nd.op == "pow" || nd.op == "atan2" ? 1 : 0;
      for (int x : nd.args) {
        const int sub = expensive_ops(x);
        if (sub < 0) return -1;
        total += sub;
      }
      return total;
    };
    for (int n = 0; n < N; ++n) {
      const Node& nd = g.nodes[n];
      if (!nd.live || !is_inline(nd)) continue;
      const int64_t big = shape_numel(nd.shape);
      if (big < (1 << 20)) continue;
      for (int a : nd.args) {
        const Node& an = g.nodes[a];
        const int64_t small = shape_numel(an.shape);
        if (P.mat[a] || small < 256 || small * 16 > big || an.op == "parameter" || an.op == "tensor") continue;
        if (expensive_ops(a) > 0) { P.mat[a] = 1; P.table[a] = 1; }
      }
    }
  }
  // dot operands: decided by the GEMM planner (it may accept a transposed view directly)
  std::map<int, GemmSpec> gemm_of;
  for (int n : dots) {
    std::vector<int> need;
    GemmSpec gs;
    plan_dot(*plan, n, need, &gs);
    for (int m : need) P.mat[m] = 1;
  }
  // a reshape / squeeze / metadata chain over a parameter, a literal or a value that is a buffer anyway
  // (a product, an attention, ...) is that buffer under another shape: nothing to compute (results
  // still get memory of their own)
  {
    std::set<int> outs(g.outputs.begin(), g.outputs.end());
    for (int n = 0; n < N; ++n) {
      if (!g.nodes[n].live || !P.mat[n] || outs.count(n)) continue;
      int a = n;
      while ((g.nodes[a].op == "reshape" || g.nodes[a].op == "squeeze" || g.nodes[a].op == "metadata") && !g.nodes[a].args.empty()) a = g.nodes[a].args[0];
      if (a != n && (g.nodes[a].op == "parameter" || g.nodes[a].op == "tensor" || P.mat[a])) P.mat[n] = 0;
    }
  }
  // contiguous reshapes / metadata over materialised values share the buffer
  auto propagate_alias = [&]() {
    for (int n = 0; n < N; ++n) {
      Node& nd = g.nodes[n];
      if (!nd.live || nd.slot >= 0) continue;
      if ((nd.op == "metadata" || nd.op == "reshape" || nd.op == "squeeze") && !nd.args.empty()) {
        const Node& a = g.nodes[nd.args[0]];
        if (a.slot >= 0 && !P.mat[n]) { nd.slot = a.slot; nd.alias = nd.args[0]; }
      }
    }
  };

  // ---- fusion: decide units ----------------------------------------------------------------
  // `level 2` = fused row kernels; `level 1` = one kernel per materialised value (always valid)
  if (first_level < 2)
    for (int n = 0; n < N; ++n) if (g.nodes[n].live && is_reduce(g.nodes[n])) P.mat[n] = 1;
  for (int fusion = first_level; fusion >= 1; --fusion) {
    try {
      // reset planner state that depends on the fusion attempt
      Plan& pl = *plan;
      pl.steps.clear();
      pl.kernels.clear();
      pl.gemms.clear();
      pl.slots.resize(0);
      for (auto& nd : g.nodes) { nd.slot = -1; nd.alias = -1; }
      pl.param_slots.assign(g.n_params, -1);
      for (int n = 0; n < N; ++n) {
        Node& nd = g.nodes[n];
        if (!nd.live) continue;
        if (nd.op == "parameter") {
          int pi = (int)nd.ints[0];
          if (pl.param_slots[pi] < 0) pl.param_slots[pi] = P.new_slot(Slot::PARAM, n, pi);
          nd.slot = pl.param_slots[pi];
        } else if (nd.op == "tensor") {
          nd.slot = P.new_slot(Slot::LITERAL, n, n);
        }
      }
      // Fixpoint: reductions read from outside their kernel become materialised.
      std::vector<Unit> units;
      for (int iter = 0; iter < 64; ++iter) {
        bool changed = false;
        units.clear();
        // (1) reduction groups
        struct RInfo { int node; std::vector<int64_t> F; int k; std::vector<int> perm; std::set<int> cone, leaves, reds; };
        std::vector<RInfo> rs;
        for (int n = 0; n < N; ++n) {
          const Node& nd = g.nodes[n];
          if (!nd.live || !is_reduce(nd)) continue;
          RInfo ri;
          ri.node = n;
          P.trailing_reduce(nd, &ri.F, &ri.k, &ri.perm);
          P.cone(n, ri.cone, ri.leaves, ri.reds, true);
          rs.push_back(std::move(ri));
        }
        std::vector<int> grp(rs.size());
        for (size_t i = 0; i < rs.size(); ++i) grp[i] = (int)i;
        std::function<int(int)> find = [&](int x) { return grp[x] == x ? x : grp[x] = find(grp[x]); };
        std::map<int, int> ridx;
        for (size_t i = 0; i < rs.size(); ++i) ridx[rs[i].node] = (int)i;
        if (fusion >= 2) {
          for (size_t i = 0; i < rs.size(); ++i)
            for (size_t j = 0; j < i; ++j) {
              if (!rs[i].perm.empty() || !rs[j].perm.empty()) continue;
              if (rs[i].F != rs[j].F || rs[i].k != rs[j].k) continue;
              if (P.depth(rs[i].node) != P.depth(rs[j].node)) continue;
              bool share = rs[i].reds.count(rs[j].node) || rs[j].reds.count(rs[i].node);
              if (!share)
                for (int l : rs[i].leaves) if (rs[j].leaves.count(l) && strip_units(g.nodes[l].shape) == strip_units(rs[i].F)) { share = true; break; }
              if (share) grp[find((int)i)] = find((int)j);
            }
        }
        // a reduction that depends on a reduction of another group reads it from memory
        for (size_t i = 0; i < rs.size(); ++i)
          for (int r : rs[i].reds)
            if (find(ridx[r]) != find((int)i) && !P.mat[r]) { P.mat[r] = 1; changed = true; }
        if (changed) continue;
        std::map<int, int> unit_of_group;
        for (size_t i = 0; i < rs.size(); ++i) {
          int gi = find((int)i);
          if (!unit_of_group.count(gi)) {
            Unit u;
            u.kind = Unit::ROW;
            u.F = rs[i].F;
            u.k = rs[i].k;
            u.perm = rs[i].perm;
            unit_of_group[gi] = (int)units.size();
            units.push_back(u);
          }
          units[unit_of_group[gi]].reduces.push_back(rs[i].node);
        }
        // (2) store roots
        std::vector<int> roots;
        for (int n = 0; n < N; ++n) {
          const Node& nd = g.nodes[n];
          if (!nd.live || !P.mat[n]) continue;
          if (nd.op == "parameter" || nd.op == "tensor" || nd.op == "dot" || nd.op == "concatenate" || nd.op == "all_reduce" || nd.op == "attention" || nd.op == "sort" || nd.op == "argsort" || nd.op == "indexed_add" || nd.op == "indexed_put" || is_reduce(nd)) continue;
          roots.push_back(n);
        }
        for (int n : roots) {
          std::set<int> seen, leaves, reds;
          P.cone(n, seen, leaves, reds, true);
          const Node& nd = g.nodes[n];
          int target = -1;
          bool conflict = false;
          for (int r : reds) {
            int u = unit_of_group[find(ridx[r])];
            if (target < 0) target = u;
            else if (target != u) conflict = true;
          }
          auto fits = [&](const Unit& u) {
            if (!u.perm.empty()) return false;
            if (P.depth(u.reduces[0]) != P.depth(n)) return false;
            std::vector<int64_t> su = strip_units(nd.shape), fu = strip_units(u.F);
            std::vector<int64_t> ru(u.F.begin(), u.F.end() - u.k);
            ru = strip_units(ru);
            return su == fu || su == ru;
          };
          if (target >= 0 && (conflict || fusion < 2 || nd.piece_of >= 0 || !fits(units[target]))) {
            // cannot ride in the reductions' kernel: read their results from memory instead
            bool marked = false;
            for (int r : reds) if (!P.mat[r]) { P.mat[r] = 1; marked = true; }
            if (marked) { changed = true; continue; }
            target = -1;
            conflict = true;
          }
          if (target < 0 && fusion >= 2 && !conflict && nd.piece_of < 0) {
            // no reduction involved: ride along with a row kernel that already reads the same data
            for (size_t ui = 0; ui < units.size() && target < 0; ++ui) {
              Unit& u = units[ui];
              if (u.kind != Unit::ROW || !u.perm.empty() || strip_units(nd.shape) != strip_units(u.F)) continue;
              if (P.depth(u.reduces[0]) != P.depth(n)) continue;
              std::set<int> uleaves;
              for (int r : u.reduces) { auto& ri = rs[ridx[r]]; uleaves.insert(ri.leaves.begin(), ri.leaves.end()); }
              bool sub = !leaves.empty();
              for (int l : leaves) if (!uleaves.count(l) && g.nodes[l].op != "constant") sub = false;
              if (sub) target = (int)ui;
            }
          }
          if (target >= 0) units[target].stores.push_back(n);
          else {
            // elementwise kernel; merge with an existing one of the same shape that shares an input
            int merged = -1;
            for (size_t ui = 0; ui < units.size() && merged < 0 && fusion >= 2 && nd.piece_of < 0; ++ui) {
              Unit& u = units[ui];
              if (u.kind != Unit::EW || u.F != nd.shape || g.nodes[u.stores[0]].piece_of >= 0) continue;
              if (P.depth(u.stores[0]) != P.depth(n)) continue;
              for (int s : u.stores) {
                std::set<int> s2, l2, r2;
                P.cone(s, s2, l2, r2, true);
                // merging is only safe if neither root depends on the other
                if (s2.count(n) || seen.count(s)) { merged = -2; break; }
                for (int l : leaves) if (l2.count(l)) merged = (int)ui;
                // two values computed from indices and constants alone (the cos and sin tables of one angle)
                if (leaves.empty() && l2.empty()) merged = (int)ui;
              }
              if (merged == -2) merged = -1;
            }
            if (merged >= 0) units[merged].stores.push_back(n);
            else {
              Unit u;
              u.kind = Unit::EW;
              u.F = nd.shape;
              u.stores.push_back(n);
              units.push_back(u);
            }
          }
        }
        if (!changed) break;
      }

      // ---- slots for everything materialised ------------------------------------------------
      std::map<int, int> out_index;
      for (size_t i = 0; i < g.outputs.size(); ++i) out_index[g.outputs[i]] = (int)i;
      pl.output_slots.assign(g.outputs.size(), -1);
      for (int n = 0; n < N; ++n) {
        Node& nd = g.nodes[n];
        if (!nd.live || !P.mat[n] || nd.slot >= 0) continue;
        if (nd.piece_of >= 0) { nd.slot = g.nodes[nd.piece_of].slot; continue; }
        if (out_index.count(n)) {
          nd.slot = P.new_slot(Slot::OUTPUT, n, out_index[n]);
          pl.output_slots[out_index[n]] = nd.slot;
        } else {
          nd.slot = P.new_slot(Slot::TEMP, n, n);
        }
      }
      propagate_alias();

      // ---- a matrix product absorbs the elementwise kernel that consumes it ---------------------
      std::set<int> fused_dots;
      if (fusion >= 2) {
        std::vector<std::vector<int>> consumers(N);
        for (int n = 0; n < N; ++n)
          if (g.nodes[n].live) for (int a : g.nodes[n].args) consumers[a].push_back(n);
        std::set<int> outs(g.outputs.begin(), g.outputs.end());
        for (auto& u : units) {
          if (u.kind != Unit::EW || g.nodes[u.stores[0]].piece_of >= 0) continue;
          std::set<int> seen, leaves, reds;
          for (int st : u.stores) P.cone(st, seen, leaves, reds, true);
          if (!reds.empty()) continue;
          // the product that runs last takes the epilogue; earlier products in the cone are
          // ordinary buffers the epilogue reads
          // (products of equal depth cannot depend on one another: the later node takes it)
          int D = -1;
          for (int l : leaves) {
            if (g.nodes[l].op != "dot") continue;
            if (D < 0 || P.depth(l) > P.depth(D) || (P.depth(l) == P.depth(D) && l > D)) D = l;
          }
          if (D < 0 || outs.count(D) || fused_dots.count(D)) continue;
          // a buffer produced after D (it may depend on D) cannot be read by D's epilogue
          bool later = false;
          for (int l : leaves) {
            const std::string& lop = g.nodes[l].op;
            if (l != D && (lop == "concatenate" || lop == "all_reduce" || lop == "attention" || lop == "sort" || lop == "argsort" || lop == "indexed_add" || lop == "indexed_put") && P.depth(l) > P.depth(D)) later = true;
          }
          if (later) continue;
          const Node& dn = g.nodes[D];
          const DType ta = g.nodes[dn.args[0]].dt, tb = g.nodes[dn.args[1]].dt;
          if (!(ta == tb && (ta == NXB_BF16 || ta == NXB_F16) && (dn.dt == ta || dn.dt == NXB_F32))) continue;
          if (shape_numel(dn.shape) != shape_numel(u.F) || shape_numel(u.F) == 0) continue;
          bool inside = true;
          for (int c : consumers[D]) if (!seen.count(c)) inside = false;
          if (!inside) continue;
          std::vector<int> need;
          GemmSpec gs;
          plan_dot(pl, D, need, &gs);
          if (gs.k % 8 != 0 || gs.batch > 65535) continue;
          try {
            KernelBuilder dry(pl, KernelBuilder::EPI, u.F, 0, {});
            dry.stores = u.stores;
            dry.acc_node = D;
            dry.force_v = 1;
            dry.build("dry");
          } catch (const FusionError&) {
            continue;
          }
          u.kind = Unit::GEMM;
          u.fused_epilogue = true;
          u.gemm_node = D;
          fused_dots.insert(D);
        }
      }
      // gemm + concatenate units
      for (int n : dots) {
        if (fused_dots.count(n)) continue;
        Unit u;
        u.kind = Unit::GEMM;
        u.gemm_node = n;
        units.push_back(u);
      }

      for (int n : attns) {
        Unit u;
        u.kind = Unit::ATTN;
        u.gemm_node = n;
        units.push_back(u);
      }
      for (int n : allreduces) {
        Unit u;
        u.kind = Unit::ALLREDUCE;
        u.gemm_node = n;
        units.push_back(u);
      }

      // ---- order units by data dependence ---------------------------------------------------------
      auto unit_io = [&](Unit& u) {
        u.reads.clear();
        u.writes.clear();
        if (u.kind == Unit::ALLREDUCE) {
          const Node& nd = g.nodes[u.gemm_node];
          u.writes.insert(nd.slot);
          for (int a : nd.args) u.reads.insert(g.nodes[a].slot);
          return;
        }
        if (u.kind == Unit::ATTN) {
          const Node& nd = g.nodes[u.gemm_node];
          u.writes.insert(nd.slot);
          for (int a : nd.args) u.reads.insert(g.nodes[a].slot);
          return;
        }
        if (u.kind == Unit::GEMM) {
          const Node& nd = g.nodes[u.gemm_node];
          std::vector<int> need;
          GemmSpec gs;
          plan_dot(pl, u.gemm_node, need, &gs);
          u.reads.insert(gs.a.slot);
          u.reads.insert(gs.b.slot);
          if (gs.scale_slot >= 0) u.reads.insert(gs.scale_slot);
          if (!u.fused_epilogue) { u.writes.insert(nd.slot); return; }
        }
        std::set<int> seen, leaves, reds;
        for (int s : u.stores) { u.writes.insert(g.nodes[s].slot); }
        for (int r : u.reduces) if (g.nodes[r].slot >= 0) u.writes.insert(g.nodes[r].slot);
        std::set<int> own(u.stores.begin(), u.stores.end());
        own.insert(u.reduces.begin(), u.reduces.end());
        std::function<void(int)> walk = [&](int n) {
          if (!seen.insert(n).second) return;
          if (u.fused_epilogue && n == u.gemm_node) return;
          const Node& nd = g.nodes[n];
          if (u.fused_epilogue && nd.alias >= 0) {
            int a = n;
            while (a >= 0 && g.nodes[a].alias >= 0) a = g.nodes[a].alias;
            if (a == u.gemm_node) { for (int x : nd.args) walk(x); return; }
          }
          if (nd.slot >= 0 && !own.count(n)) { u.reads.insert(nd.slot); return; }
          for (int a : nd.args) walk(a);
        };
        for (int s : u.stores) walk(s);
        for (int r : u.reduces) walk(r);
      };
      for (auto& u : units) unit_io(u);
      std::vector<int> order;
      {
        size_t U = units.size();
        std::vector<char> done(U, 0);
        std::set<int> ready;   // slots whose every writer has been scheduled
        std::map<int, int> writers;
        for (auto& u : units) for (int w : u.writes) writers[w]++;
        for (auto& sl : pl.slots) if (sl.kind == Slot::PARAM || sl.kind == Slot::LITERAL) ready.insert((int)(&sl - &pl.slots[0]));
        for (size_t round = 0; round < U; ++round) {
          bool progress = false;
          for (size_t i = 0; i < U; ++i) {
            if (done[i]) continue;
            bool ok = true;
            for (int r : units[i].reads) if (!ready.count(r) && !units[i].writes.count(r)) ok = false;
            if (!ok) continue;
            done[i] = 1;
            order.push_back((int)i);
            for (int w : units[i].writes) if (--writers[w] == 0) ready.insert(w);
            progress = true;
          }
          if (!progress) break;
        }
        if (order.size() != U) {
          if (getenv("NXB200_DEBUG")) {
            for (size_t i = 0; i < U; ++i) {
              if (done[i]) continue;
              fprintf(stderr, "[nxb200] stuck unit kind=%d gemm=%d stores=", (int)units[i].kind, units[i].gemm_node);
              for (int st : units[i].stores) fprintf(stderr, "%s#%d ", g.nodes[st].op.c_str(), st);
              fprintf(stderr, " waits for slots:");
              for (int r : units[i].reads) if (!ready.count(r) && !units[i].writes.count(r)) fprintf(stderr, " %d(node %d %s)", r, pl.slots[r].node, g.nodes[pl.slots[r].node].op.c_str());
              fprintf(stderr, "\n");
            }
          }
          throw FusionError("fused kernels depend on each other");
        }
      }

      // ---- generate -------------------------------------------------------------------------------
      int kid = 0;
      for (int ui : order) {
        Unit& u = units[ui];
        int step_index = (int)pl.steps.size();
        if (u.kind == Unit::ATTN) {
          const Node& nd = g.nodes[u.gemm_node];
          const int xnode = (int)nd.ints[0], d1 = (int)nd.ints[1];
          const std::string kname = "nxb_k" + std::to_string(kid++) + "_attn";
          // the score transform: value of X at (batch..., query row, key column) given the raw score
          KernelBuilder kx(pl, KernelBuilder::EPI, g.nodes[d1].shape, 0, {});
          kx.acc_node = d1;
          kx.force_v = 1;
          kx.ret_node = xnode;
          KernelSpec fx = kx.build(kname + "_xform");
          std::ostringstream o;
          o << fx.source;
          // With a proven causal mask  X = select(row >= col, Y, -inf)  the kernel reads Y directly in the
          // key blocks that lie entirely below the diagonal (same buffers, same order, as the full transform).
          bool has_plain = false;
          if (nd.ints[2] && g.nodes[xnode].op == "select" && g.nodes[xnode].args.size() == 3) {
            KernelBuilder kp(pl, KernelBuilder::EPI, g.nodes[d1].shape, 0, {});
            kp.acc_node = d1;
            kp.force_v = 1;
            kp.ret_node = g.nodes[xnode].args[1];
            kp.seed_args = fx.arg_slots;
            KernelSpec fp = kp.build(kname + "_plain");
            if (fp.arg_slots == fx.arg_slots) { o << fp.source; has_plain = true; }
          }
          // The unmasked transform  Y = c * scores  with a positive constant c (the usual 1/sqrt(d)): the kernel
          // then folds c into the exponent's multiply-add and takes maxima of the raw scores.  Only with
          // intermediate values kept in f32 (the default); with strict rounding Y is rounded to bf16 first.
          bool scale_only = false, plain_always = false;
          float scale_value = 1.f;
          {
            const int y = has_plain ? g.nodes[xnode].args[1] : xnode;
            const Node& Y = g.nodes[y];
            auto scalar_constant = [&](int n, float* out) {
              while (g.nodes[n].op == "broadcast" || g.nodes[n].op == "metadata" || g.nodes[n].op == "reshape") n = g.nodes[n].args[0];
              const Node& c = g.nodes[n];
              if (c.op != "constant" || c.flts.empty() || !dtype_is_float(c.dt) || c.dt == NXB_F64) return false;
              float v = (float)c.flts[0];
              if (c.dt == NXB_BF16) v = to_bf16_rne(v);
              if (c.dt == NXB_F16) return false;
              *out = v;
              return true;
            };
            if (getenv("NXB200_STRICT_ROUNDING") == nullptr && Y.op == "multiply" && Y.args.size() == 2 && fx.arg_slots.empty()) {
              const int other = Y.args[0] == d1 ? Y.args[1] : Y.args[1] == d1 ? Y.args[0] : -1;
              float c = 0.f;
              if (other >= 0 && other != d1 && scalar_constant(other, &c) && c > 0.f && c < 1e30f) {
                scale_only = true;
                scale_value = c;
                plain_always = !has_plain && y == xnode;
              }
            }
          }
          uint32_t scale_bits;
          memcpy(&scale_bits, &scale_value, 4);
          o << "struct AttnXform {\n  static constexpr bool kHasPlain = " << (has_plain ? "true" : "false") << ";\n"
            << "  static constexpr bool kScaleOnly = " << (scale_only ? "true" : "false") << ";\n"
            << "  static constexpr bool kPlainAlways = " << (plain_always ? "true" : "false") << ";\n"
            << "  static __device__ __forceinline__ float scale() { return __uint_as_float(0x" << std::hex << scale_bits << std::dec << "u); }\n"
            << "  static __device__ __forceinline__ float apply(float s, long long bh, long long qi, long long kj, void* const* ep) { return "
            << kname << "_xform(s, bh, qi, kj, ep); }\n"
            << "  static __device__ __forceinline__ float plain(float s, long long bh, long long qi, long long kj, void* const* ep) { return "
            << kname << (has_plain ? "_plain" : "_xform") << "(s, bh, qi, kj, ep); }\n};\n";
          o << "extern \"C\" __global__ void __launch_bounds__(320, 1) " << kname
            << "(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const nxb_attn::AttnParams p) {\n"
            << "  nxb_attn::attn_body<AttnXform>(map_q, map_k, map_v, p);\n}\n";
          KernelSpec ks;
          ks.name = kname;
          ks.source = o.str();
          ks.block = 320;
          ks.smem = (unsigned)attn_smem_bytes();
          ks.arg_slots = fx.arg_slots;
          ks.arg_offsets.assign(ks.arg_slots.size(), 0);
          ks.tensor_core = true;
          ks.attention = true;
          AttentionSpec as;
          as.q_slot = g.nodes[nd.args[0]].slot;
          as.k_slot = g.nodes[nd.args[1]].slot;
          as.v_slot = g.nodes[nd.args[2]].slot;
          as.out_slot = nd.slot;
          as.sq = nd.ints[3];
          as.sk = nd.ints[4];
          as.causal = (int)nd.ints[2];
          as.batch_heads = shape_numel(nd.shape) / (as.sq * 128);
          as.heads = nd.ints.size() > 5 ? nd.ints[5] : 1;
          as.v_bshd = nd.ints.size() > 6 && nd.ints[6] != 0;
          as.out_bshd = nd.ints.size() > 7 && nd.ints[7] != 0;
          std::ostringstream d;
          d << "attention#" << u.gemm_node << " fused QK^T -> transform(" << g.nodes[xnode].op << "#" << xnode << ") -> softmax -> PV, batch*heads=" << as.batch_heads
            << " Sq=" << as.sq << " Sk=" << as.sk << " head_dim=128 bf16" << (as.causal ? " causal (key blocks above the diagonal skipped)" : "")
            << (as.v_bshd ? " v read as {batch,key,head,dim}" : "") << (as.out_bshd ? " result written as {batch,row,head,dim}" : "") << " (" << kname << ")";
          as.desc = d.str();
          ks.desc = as.desc;
          pl.kernels.push_back(std::move(ks));
          as.jit_kernel = (int)pl.kernels.size() - 1;
          pl.attentions.push_back(as);
          pl.steps.push_back({Step::ATTENTION, (int)pl.attentions.size() - 1});
        } else if (u.kind == Unit::ALLREDUCE && (g.nodes[u.gemm_node].op == "sort" || g.nodes[u.gemm_node].op == "argsort")) {
          const Node& nd = g.nodes[u.gemm_node];
          const Node& in = g.nodes[nd.args[0]];
          SortSpec ss;
          ss.in_slot = in.slot;
          ss.out_slot = nd.slot;
          ss.len = nd.shape.back();
          ss.rows = shape_numel(nd.shape) / std::max<int64_t>(ss.len, 1);
          ss.dt = in.dt;
          ss.out_dt = nd.dt;
          ss.descending = !nd.ints.empty() && nd.ints[0] != 0;
          ss.indices = nd.op == "argsort";
          ss.desc = nd.op + "#" + std::to_string(u.gemm_node) + " " + dtype_name(in.dt) + shape_str(in.shape) + " along the last axis, " +
                    (ss.descending ? "descending" : "ascending") + " (bitonic network over (key, position) pairs in shared memory)";
          pl.sorts.push_back(ss);
          pl.steps.push_back({Step::SORT, (int)pl.sorts.size() - 1});
        } else if (u.kind == Unit::ALLREDUCE && (g.nodes[u.gemm_node].op == "indexed_add" || g.nodes[u.gemm_node].op == "indexed_put")) {
          const Node& nd = g.nodes[u.gemm_node];
          ScatterSpec sc;
          sc.target_slot = g.nodes[nd.args[0]].slot;
          sc.indices_slot = g.nodes[nd.args[1]].slot;
          sc.updates_slot = g.nodes[nd.args[2]].slot;
          sc.out_slot = nd.slot;
          sc.dt = nd.dt;
          sc.index_dt = g.nodes[nd.args[1]].dt;
          sc.add = nd.op == "indexed_add";
          sc.target_shape = nd.shape;
          sc.update_shape = g.nodes[nd.args[2]].shape;
          for (auto a : nd.ints) sc.axes.push_back((int)a);
          sc.desc = nd.op + "#" + std::to_string(u.gemm_node) + " " + dtype_name(nd.dt) + shape_str(nd.shape) + " <- " + std::to_string(sc.update_shape[0]) +
                    " slices " + shape_str(sc.update_shape) + (sc.add ? " (copy of the target, then atomic adds)" : " (copy of the target, then stores)");
          pl.scatters.push_back(sc);
          pl.steps.push_back({Step::SCATTER, (int)pl.scatters.size() - 1});
        } else if (u.kind == Unit::ALLREDUCE) {
          const Node& nd = g.nodes[u.gemm_node];
          CollectiveSpec cs;
          cs.in_slot = g.nodes[nd.args[0]].slot;
          cs.out_slot = nd.slot;
          cs.count = shape_numel(nd.shape);
          cs.dt = nd.dt;
          cs.desc = "all_reduce#" + std::to_string(u.gemm_node) + " sum " + dtype_name(nd.dt) + shape_str(nd.shape) + " over the tensor-parallel group (NCCL)";
          pl.collectives.push_back(cs);
          pl.steps.push_back({Step::ALLREDUCE, (int)pl.collectives.size() - 1});
        } else if (u.kind == Unit::GEMM && u.fused_epilogue) {
          std::vector<int> need;
          GemmSpec gs;
          plan_dot(pl, u.gemm_node, need, &gs);
          gs.bn = tc_pick_bn(gs.m, gs.n, gs.batch, 148);
          const std::string kname = "nxb_k" + std::to_string(kid++) + "_gemm";
          // the epilogue in two widths: whole 16-byte vectors, and single elements for ragged edges
          KernelBuilder ks1(pl, KernelBuilder::EPI, u.F, 0, {});
          ks1.stores = u.stores; ks1.acc_node = u.gemm_node; ks1.force_v = 1;
          KernelSpec f1 = ks1.build(kname + "_epi1");
          KernelBuilder ksv(pl, KernelBuilder::EPI, u.F, 0, {});
          ksv.stores = u.stores; ksv.acc_node = u.gemm_node; ksv.force_v = (gs.n % 8 == 0) ? 8 : 1; ksv.seed_args = f1.arg_slots;
          KernelSpec fv = ksv.build(kname + "_epiv");
          if (fv.arg_slots.size() != f1.arg_slots.size()) {
            KernelBuilder again(pl, KernelBuilder::EPI, u.F, 0, {});
            again.stores = u.stores; again.acc_node = u.gemm_node; again.force_v = 1; again.seed_args = fv.arg_slots;
            f1 = again.build(kname + "_epi1");
          }
          if (fv.arg_slots != f1.arg_slots) throw FusionError("epilogue variants disagree on their arguments");
          const int V = ksv.vec_width();
          const std::string I = ksv.idx_type();
          const DType ta = g.nodes[g.nodes[u.gemm_node].args[0]].dt;
          std::ostringstream o;
          o << fv.source << f1.source;
          // One float result at the product's own position: the generated functions hand the value back and
          // the tile leaves through shared memory and TMA stores (full lines instead of 16 bytes per lane).
          bool to_regs = false;
          int staged_arg = -1;
          if (u.stores.size() == 1) {
            const Node& sn = g.nodes[u.stores[0]];
            const int64_t es = (int64_t)dtype_size(sn.dt);
            if ((sn.dt == NXB_BF16 || sn.dt == NXB_F16 || sn.dt == NXB_F32) && (gs.n * es) % 16 == 0) {
              KernelBuilder kr1(pl, KernelBuilder::EPI, u.F, 0, {});
              kr1.stores = u.stores; kr1.acc_node = u.gemm_node; kr1.force_v = 1; kr1.seed_args = fv.arg_slots; kr1.epi_to_regs = true;
              KernelSpec r1 = kr1.build(kname + "_reg1");
              KernelBuilder krv(pl, KernelBuilder::EPI, u.F, 0, {});
              krv.stores = u.stores; krv.acc_node = u.gemm_node; krv.force_v = ksv.vec_width(); krv.seed_args = fv.arg_slots; krv.epi_to_regs = true;
              KernelSpec rv = krv.build(kname + "_regv");
              if (kr1.epi_regs_ok && krv.epi_regs_ok && r1.arg_slots == fv.arg_slots && rv.arg_slots == fv.arg_slots) {
                for (size_t i = 0; i < fv.arg_slots.size(); ++i) if (fv.arg_slots[i] == sn.slot) staged_arg = (int)i;
                if (staged_arg >= 0) {
                  to_regs = true;
                  o << rv.source << r1.source;
                  gs.staged_arg = staged_arg;
                  gs.staged_dt = sn.dt;
                }
              }
            }
          }
          o << "struct EpiGen {\n  static constexpr bool kStaged = " << (to_regs ? "true" : "false") << ";\n  static constexpr bool kTransform = " << (to_regs ? "true" : "false") << ";\n";
          o << "  static __device__ __forceinline__ void transform(const nxb_gemm::TcParams& p, float (&f)[32], long long b, long long m, long long n0) {\n";
          if (to_regs) {
            o << "    const " << I << " flat0 = (" << I << ")((b * p.m + m) * p.n + n0);\n";
            o << "    if (n0 + 32 <= p.n) {\n#pragma unroll\n      for (int j = 0; j < 32; j += " << V << ") " << kname << "_regv(f + j, flat0 + j, p.ep, f + j);\n    } else {\n";
            o << "      for (int j = 0; j < 32 && n0 + j < p.n; ++j) " << kname << "_reg1(f + j, flat0 + j, p.ep, f + j);\n    }\n";
          }
          o << "  }\n";
          o << "  static __device__ __forceinline__ void store(const nxb_gemm::TcParams& p, float (&f)[32], const uint32_t (&raw)[32], long long b, long long m, long long n0) {\n";
          o << "    const " << I << " flat0 = (" << I << ")((b * p.m + m) * p.n + n0);\n";
          o << "    if (n0 + 32 <= p.n) {\n#pragma unroll\n      for (int j = 0; j < 32; j += " << V << ") " << kname << "_epiv(f + j, flat0 + j, p.ep);\n    } else {\n";
          o << "      for (int j = 0; j < 32 && n0 + j < p.n; ++j) " << kname << "_epi1(f + j, flat0 + j, p.ep);\n    }\n  }\n};\n";
          o << "extern \"C\" __global__ void __launch_bounds__(320, 1) " << kname
            << "(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c, const nxb_gemm::TcParams p) {\n"
            << "  nxb_gemm::tc_gemm_body<" << (ta == NXB_BF16 ? "nxb_gemm::KIND_BF16" : "nxb_gemm::KIND_F16") << ", " << gs.bn << ", EpiGen>(map_a, map_b, map_c, p);\n}\n";
          KernelSpec ks;
          ks.name = kname;
          ks.source = o.str();
          ks.block = (unsigned)tc_block_threads(gs.k);
          ks.smem = (unsigned)tc_smem_bytes(gs.bn);
          ks.arg_slots = fv.arg_slots;
          ks.arg_offsets.assign(ks.arg_slots.size(), 0);
          ks.tensor_core = true;
          std::ostringstream d;
          d << gs.desc << " tile=128x" << gs.bn << " fused epilogue -> stores=[";
          for (size_t i = 0; i < u.stores.size(); ++i) d << (i ? "," : "") << g.nodes[u.stores[i]].op << "#" << u.stores[i];
          d << "]" << (to_regs ? " staged TMA store" : "") << " (" << kname << ")";
          ks.desc = d.str();
          gs.desc = ks.desc;
          pl.kernels.push_back(std::move(ks));
          gs.jit_kernel = (int)pl.kernels.size() - 1;
          pl.gemms.push_back(gs);
          pl.steps.push_back({Step::GEMM, (int)pl.gemms.size() - 1});
        } else if (u.kind == Unit::GEMM) {
          std::vector<int> need;
          GemmSpec gs;
          plan_dot(pl, u.gemm_node, need, &gs);
          pl.gemms.push_back(gs);
          pl.steps.push_back({Step::GEMM, (int)pl.gemms.size() - 1});
        } else {
          KernelBuilder kb(pl, u.kind == Unit::ROW ? KernelBuilder::ROW : KernelBuilder::EW, u.F, u.kind == Unit::ROW ? u.k : 0, u.perm);
          kb.stores = u.stores;
          kb.reduces = u.reduces;
          // reductions nobody outside reads and that are not outputs need no slot; fine as is
          KernelSpec ks = kb.build("nxb_k" + std::to_string(kid++) + (u.kind == Unit::ROW ? "_row" : "_ew"));
          pl.kernels.push_back(std::move(ks));
          pl.steps.push_back({Step::KERNEL, (int)pl.kernels.size() - 1});
        }
        for (int s : u.reads) { Slot& sl = pl.slots[s]; if (sl.first_step < 0) sl.first_step = step_index; sl.last_step = step_index; }
        for (int s : u.writes) { Slot& sl = pl.slots[s]; if (sl.first_step < 0) sl.first_step = step_index; sl.last_step = step_index; }
      }
      break;   // success
    } catch (const FusionError& e) {
      if (fusion == 1) fail(NXB_ERR_UNSUPPORTED, std::string("cannot compile this graph: ") + e.what());
      if (getenv("NXB200_DEBUG")) fprintf(stderr, "[nxb200] fused plan rejected: %s\n", e.what());
      // retry without cross-reduction fusion
      for (int n = 0; n < N; ++n) if (g.nodes[n].live && is_reduce(g.nodes[n])) P.mat[n] = 1;
    }
  }

  // ---- buffer donation: which results may be written straight into their donated argument ----
  Plan& pl = *plan;
  for (auto& al : pl.g.aliases) {
    Plan::Alias a{al.first, al.second, false};
    if (window_outputs.count(al.second)) {
      a.in_place = a.window = true;
      pl.aliases.push_back(a);
      continue;
    }
    const int sp = pl.param_slots[a.param], so = pl.output_slots[a.output];
    if (sp >= 0 && so >= 0 && sp != so && pl.slots[so].kind == Slot::OUTPUT) {
      // every reader of the argument, and the writer of the result
      int readers = 0, writer = -1;
      bool other = false;
      for (size_t st = 0; st < pl.steps.size(); ++st) {
        const Step& step = pl.steps[st];
        if (step.kind == Step::KERNEL) {
          const KernelSpec& ks = pl.kernels[step.index];
          const bool reads = std::count(ks.arg_slots.begin(), ks.arg_slots.end(), sp) > 0;
          const bool writes = std::count(ks.written_slots.begin(), ks.written_slots.end(), so) > 0;
          if (reads) ++readers;
          if (writes) writer = (int)st;
          if (reads && !writes) other = true;
        } else if (step.kind == Step::GEMM) {
          const GemmSpec& gs = pl.gemms[step.index];
          if (gs.a.slot == sp || gs.b.slot == sp || gs.scale_slot == sp || gs.out_slot == so) other = true;
          if (gs.jit_kernel >= 0) {
            const KernelSpec& ks = pl.kernels[gs.jit_kernel];
            if (std::count(ks.arg_slots.begin(), ks.arg_slots.end(), sp) || std::count(ks.arg_slots.begin(), ks.arg_slots.end(), so)) other = true;
          }
        } else if (step.kind == Step::ATTENTION) {
          const AttentionSpec& as = pl.attentions[step.index];
          const KernelSpec& ks = pl.kernels[as.jit_kernel];
          if (as.q_slot == sp || as.k_slot == sp || as.v_slot == sp || as.out_slot == so || std::count(ks.arg_slots.begin(), ks.arg_slots.end(), sp)) other = true;
        } else if (step.kind == Step::SORT) {
          const SortSpec& ss = pl.sorts[step.index];
          if (ss.in_slot == sp || ss.out_slot == so) other = true;
        } else if (step.kind == Step::SCATTER) {
          const ScatterSpec& sc = pl.scatters[step.index];
          if (sc.target_slot == sp || sc.indices_slot == sp || sc.updates_slot == sp || sc.out_slot == so) other = true;
        } else {
          const CollectiveSpec& cs = pl.collectives[step.index];
          if (cs.in_slot == sp || cs.out_slot == so) other = true;
        }
      }
      if (!other && readers == 1 && writer >= 0) {
        const KernelSpec& ks = pl.kernels[pl.steps[writer].index];
        const bool rd = std::count(ks.inplace_ok.begin(), ks.inplace_ok.end(), sp) > 0;
        const bool wr = std::count(ks.inplace_ok.begin(), ks.inplace_ok.end(), -1 - so) > 0;
        a.in_place = rd && wr && pl.slots[sp].nbytes == pl.slots[so].nbytes;
      }
    }
    pl.aliases.push_back(a);
  }

  const auto t_planned = std::chrono::steady_clock::now();
  // A generated kernel that writes more than two L2 capacities' worth of results stores them with the
  // streaming hint (evict first): nothing reads them back from the cache, and they no longer push the
  // kernel's own input out of it (fused row configuration, 3 GiB of results per launch: 0.720 -> 0.710 ms).
  // Smaller results keep the default: the next kernel usually finds them in L2.
  for (auto& ks : plan->kernels) {
    if (ks.tensor_core || ks.attention || getenv("NXB200_NO_STREAMING_STORES")) continue;
    size_t written = 0;
    for (int sl : ks.written_slots) written += plan->slots[sl].nbytes;
    if (written >= ((size_t)256 << 20)) { ks.prologue = "#define NXB_STREAMING_STORES 1\n"; ks.desc += " streaming-stores"; }
  }
  for (auto& ks : plan->kernels) ks.cubin = compile_to_cubin(ks.source, ks.name, ks.tensor_core, ks.attention, ks.prologue);
  const auto t_done = std::chrono::steady_clock::now();
  plan->plan_seconds = std::chrono::duration<double>(t_planned - t_start).count();
  plan->codegen_seconds = std::chrono::duration<double>(t_done - t_planned).count();
  return plan;
}

}  // namespace nxb
