// TEST INFRASTRUCTURE ONLY — CPU oracle for the B200 Accelerate backend.
//
// A sequential, tree-walking restatement of the reference interpreter
// (src/Data/Array/Accelerate/Interpreter.hs) over the S-expression program
// text that the B200 backend also consumes.  Nothing in the product path may
// link, import or execute this file; only the test-suite, the smoke check and
// the benchmark's CPU-baseline leg do.
//
// Parity status: the reference is Haskell and no Haskell toolchain exists in
// the build environment, so this restatement cannot be compared with the
// reference running; it is pinned against the known-answer vectors transcribed
// from the reference's own tests and haddock examples (tests/golden/).
// stencil2 has no results test in the reference: parity unpinned for that node.
//
// Each function cites the reference lines it follows (paths relative to the
// reference project root; "Interp" = src/Data/Array/Accelerate/Interpreter.hs,
// "Shape" = src/Data/Array/Accelerate/Representation/Shape.hs).
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fPIC -shared interp.cpp -o _build/liboracle.so

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

// ----------------------------------------------------------------------------
// S-expressions
// ----------------------------------------------------------------------------
struct Sx {
  bool atom = false;
  std::string s;
  std::vector<Sx> k;
  const Sx& operator[](size_t i) const {
    if (i >= k.size()) throw std::runtime_error("sexp: missing operand in (" + head() + " ...)");
    return k[i];
  }
  std::string head() const { return (!atom && !k.empty() && k[0].atom) ? k[0].s : std::string(); }
  size_t size() const { return k.size(); }
};

struct SxParser {
  const char* p;
  const char* e;
  void ws() {
    while (p < e) {
      if (*p == ';') { while (p < e && *p != '\n') ++p; }
      else if (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r') ++p;
      else break;
    }
  }
  Sx parse() {
    ws();
    if (p >= e) throw std::runtime_error("sexp: unexpected end of input");
    Sx r;
    if (*p == '(') {
      ++p;
      for (;;) {
        ws();
        if (p >= e) throw std::runtime_error("sexp: unbalanced '('");
        if (*p == ')') { ++p; break; }
        r.k.push_back(parse());
      }
    } else if (*p == ')') {
      throw std::runtime_error("sexp: unexpected ')'");
    } else {
      r.atom = true;
      const char* b = p;
      while (p < e && *p != '(' && *p != ')' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;
      r.s.assign(b, p);
    }
    return r;
  }
};

// ----------------------------------------------------------------------------
// Scalar types and values
// ----------------------------------------------------------------------------
enum Ty : uint8_t { I8, I16, I32, I64, U8, U16, U32, U64, F32, F64, F16, NTY };
const char* ty_name[] = {"i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f32", "f64", "f16"};
const int ty_bytes[] = {1, 2, 4, 8, 1, 2, 4, 8, 4, 8, 2};
inline bool ty_signed(Ty t) { return t <= I64; }
inline bool ty_int(Ty t) { return t <= U64; }
inline int ty_bits(Ty t) { return ty_bytes[t] * 8; }

Ty parse_ty(const std::string& s) {
  if (s == "bool") return U8;
  if (s == "int") return I64;
  if (s == "word") return U64;
  for (int i = 0; i < NTY; ++i)
    if (s == ty_name[i]) return (Ty)i;
  throw std::runtime_error("unknown scalar type '" + s + "'");
}

// A scalar: integers are kept sign-/zero-extended to 64 bits in .i.
struct Scalar {
  Ty ty = I64;
  union {
    int64_t i;
    float f;
    double d;
  };
  Scalar() : i(0) {}
};

inline int64_t wrap_int(Ty t, uint64_t v) {
  switch (t) {
    case I8: return (int8_t)v;
    case I16: return (int16_t)v;
    case I32: return (int32_t)v;
    case I64: return (int64_t)v;
    case U8: return (int64_t)(uint8_t)v;
    case U16: return (int64_t)(uint16_t)v;
    case U32: return (int64_t)(uint32_t)v;
    default: return (int64_t)v;
  }
}
inline Scalar mk_int(Ty t, uint64_t v) { Scalar s; s.ty = t; s.i = wrap_int(t, v); return s; }
inline Scalar mk_f32(float v) { Scalar s; s.ty = F32; s.i = 0; s.f = v; return s; }
inline Scalar mk_f64(double v) { Scalar s; s.ty = F64; s.d = v; return s; }
// Half (Type.hs:127): the value is kept in .f, always one a binary16 can hold.  The package behind it
// (half >= 0.3, accelerate.cabal:335; not in the tree) computes every operation in Float and converts
// back, rounding to nearest even; the compiler's _Float16 conversion does that rounding here.
inline Scalar mk_f16(float v) { Scalar s; s.ty = F16; s.i = 0; s.f = (float)(_Float16)v; return s; }
// (NaNs keep their payload and their signalling bit on the way in and out, as a bit pattern stored in an
// array does in the reference: a conversion instruction would quieten them)
inline uint16_t f16_bits(float v) {
  if (v != v) {
    uint32_t x; memcpy(&x, &v, 4);
    uint16_t m = (uint16_t)((x >> 13) & 0x3ffu);
    return (uint16_t)(((x >> 16) & 0x8000u) | 0x7c00u | (m ? m : 0x200u));
  }
  _Float16 h = (_Float16)v; uint16_t b; memcpy(&b, &h, 2); return b;
}
inline float f16_value(uint16_t b) {
  if ((b & 0x7c00u) == 0x7c00u && (b & 0x3ffu)) {
    uint32_t x = ((uint32_t)(b & 0x8000u) << 16) | 0x7f800000u | ((uint32_t)(b & 0x3ffu) << 13);
    float f; memcpy(&f, &x, 4); return f;
  }
  _Float16 h; memcpy(&h, &b, 2); return (float)h;
}
inline Scalar mk_bool(bool b) { return mk_int(U8, b ? 1 : 0); }

// Values are tuple trees of scalars (the reference's nested-pair EltR, flattened
// one level: an n-ary tuple node holds n children).
struct Value {
  bool tuple = false;
  Scalar s;
  std::vector<Value> e;
  static Value scalar(const Scalar& x) { Value v; v.s = x; return v; }
  static Value tup(std::vector<Value> xs) { Value v; v.tuple = true; v.e = std::move(xs); return v; }
};

// Element type trees
struct EltTy {
  bool tuple = false;
  Ty ty = I64;
  std::vector<EltTy> e;
};
EltTy parse_elt(const Sx& x) {
  EltTy t;
  if (x.atom) { t.ty = parse_ty(x.s); return t; }
  t.tuple = true;
  if (x.size() == 3 && x.k[0].atom && x.k[0].s == "vec") {
    // Vec n t (Type.hs:140-152): a value is its n components; evalVecPack/evalVecUnpack
    // (Interp:951-952) convert between the two views of the same scalars
    for (int i = 0, n = atoi(x.k[1].s.c_str()); i < n; ++i) t.e.push_back(parse_elt(x.k[2]));
    return t;
  }
  size_t b = (x.size() && x.k[0].atom && x.k[0].s == "tup") ? 1 : 0;
  for (size_t i = b; i < x.size(); ++i) t.e.push_back(parse_elt(x.k[i]));
  return t;
}
void flatten_elt(const EltTy& t, std::vector<Ty>& out) {
  if (!t.tuple) { out.push_back(t.ty); return; }
  for (auto& c : t.e) flatten_elt(c, out);
}

// ----------------------------------------------------------------------------
// Arrays: struct-of-arrays, row-major, innermost dimension last
// (Representation/Array.hs:43-46, Array/Data.hs:95-98)
// ----------------------------------------------------------------------------
struct Array {
  EltTy elt;
  std::vector<Ty> leaf_ty;
  std::vector<int64_t> sh;
  std::vector<std::vector<uint8_t>> leaf;  // one buffer per scalar leaf
  int64_t n = 0;
};
typedef std::shared_ptr<Array> ArrayP;

// Shape.hs:67-71
int64_t shape_size(const std::vector<int64_t>& sh) {
  int64_t n = 1;
  for (int64_t d : sh) { if (d <= 0) return 0; n *= d; }
  return n;
}

// how `atrace` prints an array, e.g. "Vector (Z :. 3) [1,2,3]" (tuples in parentheses)
std::string trace_render(const Array& a) {
  const size_t rank = a.sh.size();
  std::string out = rank == 0 ? "Scalar" : rank == 1 ? "Vector" : rank == 2 ? "Matrix" : "Array";
  out += rank ? " (Z" : " Z";
  for (int64_t d : a.sh) out += " :. " + std::to_string(d);
  out += rank ? ") [" : " [";
  char buf[64];
  for (int64_t i = 0; i < a.n; ++i) {
    if (i) out += ",";
    if (a.leaf.size() > 1) out += "(";
    for (size_t l = 0; l < a.leaf.size(); ++l) {
      if (l) out += ",";
      const uint8_t* q = a.leaf[l].data() + (size_t)i * ty_bytes[a.leaf_ty[l]];
      switch (a.leaf_ty[l]) {
        case I8: snprintf(buf, sizeof buf, "%d", (int)*(const int8_t*)q); break;
        case I16: { int16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%d", (int)v); break; }
        case I32: { int32_t v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%d", v); break; }
        case I64: { int64_t v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%lld", (long long)v); break; }
        case U8: snprintf(buf, sizeof buf, "%u", (unsigned)*q); break;
        case U16: { uint16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%u", (unsigned)v); break; }
        case U32: { uint32_t v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%u", v); break; }
        case U64: { uint64_t v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%llu", (unsigned long long)v); break; }
        case F32: { float v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%.9g", (double)v); break; }
        case F16: { uint16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%.5g", (double)f16_value(v)); break; }
        default: { double v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%.17g", v); break; }
      }
      out += buf;
    }
    if (a.leaf.size() > 1) out += ")";
  }
  return out + "]";
}

ArrayP new_array(const EltTy& elt, const std::vector<int64_t>& sh) {
  auto a = std::make_shared<Array>();
  a->elt = elt;
  flatten_elt(elt, a->leaf_ty);
  a->sh = sh;
  a->n = shape_size(sh);
  for (Ty t : a->leaf_ty) a->leaf.emplace_back((size_t)a->n * ty_bytes[t]);
  return a;
}

inline Scalar read_leaf(const Array& a, size_t l, int64_t i) {
  Ty t = a.leaf_ty[l];
  const uint8_t* p = a.leaf[l].data() + (size_t)i * ty_bytes[t];
  Scalar s;
  s.ty = t;
  s.i = 0;
  switch (t) {
    case I8: s.i = *(const int8_t*)p; break;
    case I16: { int16_t v; memcpy(&v, p, 2); s.i = v; break; }
    case I32: { int32_t v; memcpy(&v, p, 4); s.i = v; break; }
    case I64: { int64_t v; memcpy(&v, p, 8); s.i = v; break; }
    case U8: s.i = *(const uint8_t*)p; break;
    case U16: { uint16_t v; memcpy(&v, p, 2); s.i = v; break; }
    case U32: { uint32_t v; memcpy(&v, p, 4); s.i = v; break; }
    case U64: { uint64_t v; memcpy(&v, p, 8); s.i = (int64_t)v; break; }
    case F32: memcpy(&s.f, p, 4); break;
    case F64: memcpy(&s.d, p, 8); break;
    case F16: { uint16_t v; memcpy(&v, p, 2); s.f = f16_value(v); break; }
    default: break;
  }
  return s;
}
inline void write_leaf(Array& a, size_t l, int64_t i, const Scalar& s) {
  Ty t = a.leaf_ty[l];
  uint8_t* p = a.leaf[l].data() + (size_t)i * ty_bytes[t];
  switch (t) {
    case F32: memcpy(p, &s.f, 4); break;
    case F64: memcpy(p, &s.d, 8); break;
    case F16: { uint16_t v = f16_bits(s.f); memcpy(p, &v, 2); break; }
    default: memcpy(p, &s.i, ty_bytes[t]); break;  // little endian: low bytes
  }
}
void read_value_rec(const Array& a, const EltTy& t, size_t& l, int64_t i, Value& out) {
  if (!t.tuple) { out.tuple = false; out.s = read_leaf(a, l++, i); return; }
  out.tuple = true;
  out.e.resize(t.e.size());
  for (size_t c = 0; c < t.e.size(); ++c) read_value_rec(a, t.e[c], l, i, out.e[c]);
}
Value read_value(const Array& a, int64_t i) {
  if (i < 0 || i >= a.n) throw std::runtime_error("index out of bounds");  // Error.hs:61 indexCheck
  Value v; size_t l = 0;
  read_value_rec(a, a.elt, l, i, v);
  return v;
}
void write_value_rec(Array& a, size_t& l, int64_t i, const Value& v) {
  if (!v.tuple) {
    if (l >= a.leaf_ty.size()) throw std::runtime_error("value has more leaves than the array element type");
    write_leaf(a, l++, i, v.s);
    return;
  }
  for (auto& c : v.e) write_value_rec(a, l, i, c);
}
void write_value(Array& a, int64_t i, const Value& v) {
  size_t l = 0;
  write_value_rec(a, l, i, v);
  if (l != a.leaf_ty.size()) throw std::runtime_error("value has fewer leaves than the array element type");
}

// Shape.hs:102-106 toIndex (with indexCheck); Shape.hs:110-120 fromIndex
int64_t to_index(const std::vector<int64_t>& sh, const std::vector<int64_t>& ix) {
  int64_t r = 0;
  for (size_t d = 0; d < sh.size(); ++d) {
    if (ix[d] < 0 || ix[d] >= sh[d]) throw std::runtime_error("index out of bounds");
    r = r * sh[d] + ix[d];
  }
  return r;
}
std::vector<int64_t> from_index(const std::vector<int64_t>& sh, int64_t i) {
  std::vector<int64_t> ix(sh.size());
  for (size_t d = sh.size(); d-- > 0;) {
    if (d == 0) {
      // outermost: no remainder taken, but the bounds check applies (Shape.hs:117-119)
      if (i < 0 || i >= sh[d]) throw std::runtime_error("index out of bounds");
      ix[d] = i;
    } else {
      if (sh[d] == 0) throw std::runtime_error("divide by zero");
      ix[d] = i % sh[d];
      i = i / sh[d];
    }
  }
  return ix;
}

Value shape_value(const std::vector<int64_t>& sh) {
  std::vector<Value> e;
  for (int64_t d : sh) e.push_back(Value::scalar(mk_int(I64, (uint64_t)d)));
  return Value::tup(std::move(e));
}
std::vector<int64_t> value_shape(const Value& v) {
  std::vector<int64_t> sh;
  if (!v.tuple) { sh.push_back(v.s.i); return sh; }
  for (auto& c : v.e) {
    if (c.tuple) throw std::runtime_error("shape value must be a flat tuple of Int");
    sh.push_back(c.s.i);
  }
  return sh;
}

// ----------------------------------------------------------------------------
// Scalar expression trees (AST.hs:524-645 OpenExp), variables resolved to slots
// ----------------------------------------------------------------------------
enum Op {
  O_ADD, O_SUB, O_MUL, O_NEG, O_ABS, O_SIG, O_QUOT, O_REM, O_QUOTREM, O_IDIV, O_MOD, O_DIVMOD,
  O_BAND, O_BOR, O_BXOR, O_BNOT, O_SHL, O_SHR, O_ROTL, O_ROTR, O_POPCNT, O_CLZ, O_CTZ,
  O_FDIV, O_RECIP, O_SIN, O_COS, O_TAN, O_ASIN, O_ACOS, O_ATAN, O_SINH, O_COSH, O_TANH,
  O_ASINH, O_ACOSH, O_ATANH, O_EXP, O_SQRT, O_LOG, O_FPOW, O_LOGBASE, O_ATAN2,
  O_TRUNCATE, O_ROUND, O_FLOOR, O_CEILING, O_ISNAN, O_ISINF,
  O_LT, O_GT, O_LE, O_GE, O_EQ, O_NE, O_MAX, O_MIN, O_LAND, O_LOR, O_LNOT,
  O_FROMINTEGRAL, O_TOFLOATING, O_NOPS
};
const char* op_name[] = {
  "add", "sub", "mul", "neg", "abs", "sig", "quot", "rem", "quotrem", "idiv", "mod", "divmod",
  "band", "bor", "bxor", "bnot", "shl", "shr", "rotl", "rotr", "popcount", "clz", "ctz",
  "fdiv", "recip", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh",
  "asinh", "acosh", "atanh", "exp", "sqrt", "log", "fpow", "logbase", "atan2",
  "truncate", "round", "floor", "ceiling", "isnan", "isinf",
  "lt", "gt", "le", "ge", "eq", "ne", "max", "min", "land", "lor", "lnot",
  "fromintegral", "tofloating"};

enum EKind {
  E_CONST, E_VAR, E_LET, E_TUP, E_PRJ, E_COND, E_WHILE, E_PRIM, E_INDEX, E_LINDEX, E_SHAPE,
  E_SHAPESIZE, E_TOINDEX, E_FROMINDEX, E_COERCE, E_UNDEF, E_APP, E_CASE, E_SNOC, E_INIT
};

struct Fun;
struct Exp {
  EKind kind;
  Scalar c;                  // E_CONST
  int slot = -1;             // E_VAR: env slot, E_LET: bound slot; E_PRJ: component
  int arr = -1;              // array variable slot (E_INDEX/E_LINDEX/E_SHAPE)
  Op op = O_ADD;             // E_PRIM
  Ty t1 = I64, t2 = I64;     // E_PRIM operand type / conversion target; E_COERCE
  EltTy ety;                 // E_UNDEF
  std::vector<std::unique_ptr<Exp>> a;
  std::vector<std::unique_ptr<Fun>> f;  // E_WHILE: cond, body; E_APP: fun
  std::vector<int64_t> tags;            // E_CASE
  bool has_default = false;
};
struct Fun {
  std::vector<int> params;  // env slots
  std::unique_ptr<Exp> body;
};

struct Scope {
  std::vector<std::pair<std::string, int>> names;  // scalar variable -> slot
  int next_slot = 0;
  int max_slot = 0;
  const std::map<std::string, int>* arrays = nullptr;
  int lookup(const std::string& n) const {
    for (size_t i = names.size(); i-- > 0;)
      if (names[i].first == n) return names[i].second;
    throw std::runtime_error("unbound scalar variable '" + n + "'");
  }
  int bind(const std::string& n) {
    int s = next_slot++;
    if (next_slot > max_slot) max_slot = next_slot;
    names.emplace_back(n, s);
    return s;
  }
  int array(const std::string& n) const {
    auto it = arrays->find(n);
    if (it == arrays->end()) throw std::runtime_error("unbound array variable '" + n + "'");
    return it->second;
  }
};

Scalar parse_const(Ty t, const std::string& lit) {
  if (t == F32 || t == F64 || t == F16) {
    double d;
    if (lit == "inf") d = INFINITY;
    else if (lit == "-inf") d = -INFINITY;
    else if (lit == "nan") d = NAN;
    else d = strtod(lit.c_str(), nullptr);  // accepts C99 hex floats
    if (t == F16) return mk_f16((float)d);
    return t == F32 ? mk_f32((float)d) : mk_f64(d);
  }
  if (ty_signed(t)) return mk_int(t, (uint64_t)strtoll(lit.c_str(), nullptr, 10));
  return mk_int(t, strtoull(lit.c_str(), nullptr, 10));
}

std::unique_ptr<Exp> parse_exp(const Sx& x, Scope& sc);

std::unique_ptr<Fun> parse_fun(const Sx& x, Scope& sc) {
  if (x.head() != "lam") throw std::runtime_error("expected (lam (params) body)");
  auto f = std::make_unique<Fun>();
  size_t mark = sc.names.size();
  int slot_mark = sc.next_slot;
  for (auto& p : x[1].k) {
    const std::string& nm = p.atom ? p.s : p[0].s;  // (name type) or bare name
    f->params.push_back(sc.bind(nm));
  }
  f->body = parse_exp(x[2], sc);
  sc.names.resize(mark);
  sc.next_slot = slot_mark;
  return f;
}

std::unique_ptr<Exp> parse_exp(const Sx& x, Scope& sc) {
  auto e = std::make_unique<Exp>();
  if (x.atom) throw std::runtime_error("expression must be a list, got atom '" + x.s + "'");
  std::string h = x.head();
  auto sub = [&](size_t i) { e->a.push_back(parse_exp(x[i], sc)); };
  if (h == "vecpack" || h == "vecunpack") return parse_exp(x[3], sc);  // (vecpack N T e): same scalars
  if (h == "const") {
    e->kind = E_CONST;
    e->c = parse_const(parse_ty(x[1].s), x[2].s);
  } else if (h == "minbound" || h == "maxbound") {
    e->kind = E_CONST;
    Ty t = parse_ty(x[1].s);
    if (!ty_int(t)) throw std::runtime_error("minbound/maxbound need an integral type");
    int b = ty_bits(t);
    if (h == "minbound") e->c = mk_int(t, ty_signed(t) ? (uint64_t)1 << (b - 1) : 0);
    else e->c = mk_int(t, ty_signed(t) ? (((uint64_t)1 << (b - 1)) - 1) : ~(uint64_t)0);
  } else if (h == "pi") {
    e->kind = E_CONST;
    Ty t = parse_ty(x[1].s);
    e->c = t == F16 ? mk_f16((float)M_PI) : ((t == F32) ? mk_f32((float)M_PI) : mk_f64(M_PI));
  } else if (h == "var") {
    e->kind = E_VAR;
    e->slot = sc.lookup(x[1].s);
  } else if (h == "let") {
    e->kind = E_LET;
    e->a.push_back(parse_exp(x[2], sc));
    size_t mark = sc.names.size();
    int slot_mark = sc.next_slot;
    e->slot = sc.bind(x[1].s);
    e->a.push_back(parse_exp(x[3], sc));
    sc.names.resize(mark);
    sc.next_slot = slot_mark;
  } else if (h == "tup") {
    e->kind = E_TUP;
    for (size_t i = 1; i < x.size(); ++i) sub(i);
  } else if (h == "snoc") {   // Pair on snoc-list tuples (AST.hs:536-540): append one component
    e->kind = E_SNOC;
    sub(1); sub(2);
  } else if (h == "last") {   // the final component
    e->kind = E_PRJ;
    e->slot = -1;
    sub(1);
  } else if (h == "init") {   // all components but the last
    e->kind = E_INIT;
    sub(1);
  } else if (h == "prj") {
    e->kind = E_PRJ;
    e->slot = atoi(x[1].s.c_str());
    sub(2);
  } else if (h == "cond") {
    e->kind = E_COND;
    sub(1); sub(2); sub(3);
  } else if (h == "while") {
    e->kind = E_WHILE;
    e->f.push_back(parse_fun(x[1], sc));
    e->f.push_back(parse_fun(x[2], sc));
    sub(3);
  } else if (h == "prim") {
    e->kind = E_PRIM;
    int o = -1;
    for (int i = 0; i < O_NOPS; ++i)
      if (x[1].s == op_name[i]) { o = i; break; }
    if (o < 0) throw std::runtime_error("unknown primitive '" + x[1].s + "'");
    e->op = (Op)o;
    size_t argi = 3;
    bool two_types = (o == O_TRUNCATE || o == O_ROUND || o == O_FLOOR || o == O_CEILING ||
                      o == O_FROMINTEGRAL || o == O_TOFLOATING);
    if (o == O_LAND || o == O_LOR || o == O_LNOT) {
      e->t1 = U8;
      argi = (x.size() > 2 && x[2].atom) ? 3 : 2;  // type is optional for logical prims
    } else {
      e->t1 = parse_ty(x[2].s);
    }
    if (two_types) { e->t2 = parse_ty(x[3].s); argi = 4; }
    for (size_t i = argi; i < x.size(); ++i) sub(i);
  } else if (h == "index" || h == "lindex") {
    e->kind = h == "index" ? E_INDEX : E_LINDEX;
    e->arr = sc.array(x[1].s);
    sub(2);
  } else if (h == "shape") {
    e->kind = E_SHAPE;
    e->arr = sc.array(x[1].s);
  } else if (h == "shapesize") {
    e->kind = E_SHAPESIZE;
    sub(1);
  } else if (h == "toindex") {
    e->kind = E_TOINDEX;
    sub(1); sub(2);
  } else if (h == "fromindex") {
    e->kind = E_FROMINDEX;
    sub(1); sub(2);
  } else if (h == "coerce") {
    e->kind = E_COERCE;
    e->t1 = parse_ty(x[1].s);
    e->t2 = parse_ty(x[2].s);
    sub(3);
  } else if (h == "undef") {
    e->kind = E_UNDEF;
    e->ety = parse_elt(x[1]);
  } else if (h == "app") {
    e->kind = E_APP;
    e->f.push_back(parse_fun(x[1], sc));
    for (size_t i = 2; i < x.size(); ++i) sub(i);
  } else if (h == "case") {
    // (case scrutinee ((tag rhs) ...) [default])
    e->kind = E_CASE;
    sub(1);
    for (auto& alt : x[2].k) {
      e->tags.push_back(strtoll(alt[0].s.c_str(), nullptr, 10));
      e->a.push_back(parse_exp(alt[1], sc));
    }
    if (x.size() > 3) { e->has_default = true; sub(3); }
  } else {
    throw std::runtime_error("unknown expression form '" + h + "'");
  }
  return e;
}

// ----------------------------------------------------------------------------
// Primitive functions (Interp:1086-1416; arithmetic itself is GHC base:
// two's-complement wrap, IEEE-754 round-to-nearest-even, floor div/mod)
// ----------------------------------------------------------------------------
inline double as_double(const Scalar& s) { return s.ty == F32 || s.ty == F16 ? (double)s.f : s.d; }

#define FUN1(NAME)                                                        \
  do {                                                                    \
    if (t == F32) return Value::scalar(mk_f32(NAME##f(x.f)));             \
    return Value::scalar(mk_f64(NAME(x.d)));                              \
  } while (0)

int64_t floor_div(int64_t a, int64_t b) {
  int64_t q = a / b, r = a % b;
  if (r != 0 && ((r < 0) != (b < 0))) --q;
  return q;
}
int64_t floor_mod(int64_t a, int64_t b) {
  int64_t r = a % b;
  if (r != 0 && ((r < 0) != (b < 0))) r += b;
  return r;
}

template <class F>
bool cmp_scalar(Ty t, const Scalar& a, const Scalar& b, F f) {
  if (t == F32 || t == F16) return f(a.f, b.f);
  if (t == F64) return f(a.d, b.d);
  if (ty_signed(t)) return f(a.i, b.i);
  return f((uint64_t)a.i, (uint64_t)b.i);
}

Scalar convert_to(Ty from, Ty to, const Scalar& x, Op how) {
  // fromIntegral / toFloating (Interp:1170-1191), truncate/round/floor/ceiling (:1266-1288)
  if (ty_int(from)) {
    if (ty_int(to)) return mk_int(to, (uint64_t)x.i);
    if (ty_signed(from)) return to == F32 ? mk_f32((float)x.i) : mk_f64((double)x.i);
    return to == F32 ? mk_f32((float)(uint64_t)x.i) : mk_f64((double)(uint64_t)x.i);
  }
  double d = as_double(x);
  if (!ty_int(to)) {
    if (to == F32) return mk_f32(from == F32 ? x.f : (float)x.d);
    return mk_f64(d);
  }
  double r;
  switch (how) {
    case O_TRUNCATE: r = std::trunc(d); break;
    case O_ROUND: r = std::nearbyint(d); break;  // half-to-even, as GHC's round
    case O_FLOOR: r = std::floor(d); break;
    case O_CEILING: r = std::ceil(d); break;
    default: r = d; break;
  }
  if (!ty_signed(to) && r >= 9223372036854775808.0) return mk_int(to, (uint64_t)r);
  return mk_int(to, (uint64_t)(int64_t)r);
}

Value eval_prim_at(Op op, Ty t1, Ty t2, const std::vector<Value>& arg) {
  Ty t = t1;
  const Scalar& x = arg[0].s;
  const Scalar* yp = arg.size() > 1 ? &arg[1].s : nullptr;
  auto ibin = [&](uint64_t v) { return Value::scalar(mk_int(t, v)); };
  switch (op) {
    case O_ADD:
      if (t == F32) return Value::scalar(mk_f32(x.f + yp->f));
      if (t == F64) return Value::scalar(mk_f64(x.d + yp->d));
      return ibin((uint64_t)x.i + (uint64_t)yp->i);
    case O_SUB:
      if (t == F32) return Value::scalar(mk_f32(x.f - yp->f));
      if (t == F64) return Value::scalar(mk_f64(x.d - yp->d));
      return ibin((uint64_t)x.i - (uint64_t)yp->i);
    case O_MUL:
      if (t == F32) return Value::scalar(mk_f32(x.f * yp->f));
      if (t == F64) return Value::scalar(mk_f64(x.d * yp->d));
      return ibin((uint64_t)x.i * (uint64_t)yp->i);
    case O_NEG:
      if (t == F32) return Value::scalar(mk_f32(-x.f));
      if (t == F64) return Value::scalar(mk_f64(-x.d));
      return ibin((uint64_t)0 - (uint64_t)x.i);
    case O_ABS:
      if (t == F32) return Value::scalar(mk_f32(std::fabs(x.f)));
      if (t == F64) return Value::scalar(mk_f64(std::fabs(x.d)));
      if (ty_signed(t) && x.i < 0) return ibin((uint64_t)0 - (uint64_t)x.i);
      return ibin((uint64_t)x.i);
    case O_SIG:
      // GHC: signum x | x > 0 = 1 | x < 0 = -1 | otherwise = x  (NaN and -0 pass through)
      if (t == F32) return Value::scalar(mk_f32(x.f > 0 ? 1.0f : (x.f < 0 ? -1.0f : x.f)));
      if (t == F64) return Value::scalar(mk_f64(x.d > 0 ? 1.0 : (x.d < 0 ? -1.0 : x.d)));
      if (ty_signed(t)) return ibin((uint64_t)(x.i > 0 ? 1 : (x.i < 0 ? -1 : 0)));
      return ibin(x.i != 0 ? 1 : 0);
    case O_QUOT: case O_REM: case O_IDIV: case O_MOD: case O_QUOTREM: case O_DIVMOD: {
      if (yp->i == 0) throw std::runtime_error("divide by zero");
      uint64_t q, r;
      if (ty_signed(t)) {
        int64_t a = x.i, b = yp->i;
        if (b == -1) { q = (uint64_t)0 - (uint64_t)a; r = 0; }  // avoids the INT64_MIN trap; wraps
        else if (op == O_QUOT || op == O_REM || op == O_QUOTREM) { q = (uint64_t)(a / b); r = (uint64_t)(a % b); }
        else { q = (uint64_t)floor_div(a, b); r = (uint64_t)floor_mod(a, b); }
      } else {
        uint64_t a = (uint64_t)x.i, b = (uint64_t)yp->i;
        q = a / b; r = a % b;
      }
      if (op == O_QUOT || op == O_IDIV) return ibin(q);
      if (op == O_REM || op == O_MOD) return ibin(r);
      return Value::tup({Value::scalar(mk_int(t, q)), Value::scalar(mk_int(t, r))});
    }
    case O_BAND: return ibin((uint64_t)x.i & (uint64_t)yp->i);
    case O_BOR: return ibin((uint64_t)x.i | (uint64_t)yp->i);
    case O_BXOR: return ibin((uint64_t)x.i ^ (uint64_t)yp->i);
    case O_BNOT: return ibin(~(uint64_t)x.i);
    case O_SHL: {
      int64_t n = yp->i;
      if (n < 0) throw std::runtime_error("arithmetic overflow");  // GHC: negative shift
      return ibin(n >= 64 ? 0 : ((uint64_t)x.i << n));
    }
    case O_SHR: {
      int64_t n = yp->i;
      if (n < 0) throw std::runtime_error("arithmetic overflow");
      if (ty_signed(t)) return ibin((uint64_t)(n >= 64 ? (x.i < 0 ? -1 : 0) : (x.i >> n)));
      return ibin(n >= 64 ? 0 : ((uint64_t)x.i >> n));
    }
    case O_ROTL: case O_ROTR: {
      int b = ty_bits(t);
      int64_t n = yp->i;
      if (op == O_ROTR) n = -n;
      int r = (int)(((n % b) + b) % b);
      uint64_t mask = b == 64 ? ~(uint64_t)0 : (((uint64_t)1 << b) - 1);
      uint64_t v = (uint64_t)x.i & mask;
      if (r == 0) return ibin(v);
      return ibin(((v << r) | (v >> (b - r))) & mask);
    }
    case O_POPCNT: case O_CLZ: case O_CTZ: {
      int b = ty_bits(t);
      uint64_t mask = b == 64 ? ~(uint64_t)0 : (((uint64_t)1 << b) - 1);
      uint64_t v = (uint64_t)x.i & mask;
      int64_t r;
      if (op == O_POPCNT) r = __builtin_popcountll(v);
      else if (op == O_CLZ) r = v == 0 ? b : (__builtin_clzll(v) - (64 - b));
      else r = v == 0 ? b : __builtin_ctzll(v);
      return Value::scalar(mk_int(I64, (uint64_t)r));
    }
    case O_FDIV:
      if (t == F32) return Value::scalar(mk_f32(x.f / yp->f));
      return Value::scalar(mk_f64(x.d / yp->d));
    case O_RECIP:
      if (t == F32) return Value::scalar(mk_f32(1.0f / x.f));
      return Value::scalar(mk_f64(1.0 / x.d));
    case O_SIN: FUN1(sin);
    case O_COS: FUN1(cos);
    case O_TAN: FUN1(tan);
    case O_ASIN: FUN1(asin);
    case O_ACOS: FUN1(acos);
    case O_ATAN: FUN1(atan);
    case O_SINH: FUN1(sinh);
    case O_COSH: FUN1(cosh);
    case O_TANH: FUN1(tanh);
    case O_ASINH: FUN1(asinh);
    case O_ACOSH: FUN1(acosh);
    case O_ATANH: FUN1(atanh);
    case O_EXP: FUN1(exp);
    case O_SQRT: FUN1(sqrt);
    case O_LOG: FUN1(log);
    case O_FPOW:
      if (t == F32) return Value::scalar(mk_f32(powf(x.f, yp->f)));
      return Value::scalar(mk_f64(pow(x.d, yp->d)));
    case O_LOGBASE:  // logBase b v = log v / log b
      if (t == F32) return Value::scalar(mk_f32(logf(yp->f) / logf(x.f)));
      return Value::scalar(mk_f64(log(yp->d) / log(x.d)));
    case O_ATAN2:
      if (t == F32) return Value::scalar(mk_f32(atan2f(x.f, yp->f)));
      return Value::scalar(mk_f64(atan2(x.d, yp->d)));
    case O_TRUNCATE: case O_ROUND: case O_FLOOR: case O_CEILING:
    case O_FROMINTEGRAL: case O_TOFLOATING:
      return Value::scalar(convert_to(t1, t2, x, op));
    case O_ISNAN: return Value::scalar(mk_bool(t == F32 ? std::isnan(x.f) : std::isnan(x.d)));
    case O_ISINF: return Value::scalar(mk_bool(t == F32 ? std::isinf(x.f) : std::isinf(x.d)));
    case O_LT: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a < b; })));
    case O_GT: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a > b; })));
    case O_LE: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a <= b; })));
    case O_GE: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a >= b; })));
    case O_EQ: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a == b; })));
    case O_NE: return Value::scalar(mk_bool(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a != b; })));
    // GHC Ord defaults: max x y = if x <= y then y else x ; min x y = if x <= y then x else y
    case O_MAX: return Value::scalar(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a <= b; }) ? *yp : x);
    case O_MIN: return Value::scalar(cmp_scalar(t, x, *yp, [](auto a, auto b) { return a <= b; }) ? x : *yp);
    case O_LAND: return Value::scalar(mk_bool(x.i != 0 && yp->i != 0));  // Interp:1162-1169
    case O_LOR: return Value::scalar(mk_bool(x.i != 0 || yp->i != 0));
    case O_LNOT: return Value::scalar(mk_bool(x.i == 0));
    default: break;
  }
  throw std::runtime_error("unhandled primitive");
}

Value eval_prim(const Exp& e, const std::vector<Value>& arg) {
  if (e.t1 != F16 && e.t2 != F16) return eval_prim_at(e.op, e.t1, e.t2, arg);
  // Numeric.Half: a + b = toHalf (fromHalf a + fromHalf b), and so on for every class method; the
  // comparisons compare the converted values.  (.f of a Half scalar already is that Float.)
  std::vector<Value> a = arg;
  if (e.t1 == F16)
    for (auto& v : a)
      if (!v.tuple && v.s.ty == F16) v.s.ty = F32;
  Value r = eval_prim_at(e.op, e.t1 == F16 ? F32 : e.t1, e.t2 == F16 ? F32 : e.t2, a);
  const bool to_float = (e.op == O_TOFLOATING || e.op == O_FROMINTEGRAL) && e.t2 == F32;
  if (!r.tuple && r.s.ty == F32 && !to_float) r.s = mk_f16(r.s.f);
  return r;
}

Value undef_value(const EltTy& t) {
  if (!t.tuple) {
    Scalar s; s.ty = t.ty; s.i = 0;
    return Value::scalar(s);
  }
  std::vector<Value> e;
  for (auto& c : t.e) e.push_back(undef_value(c));
  return Value::tup(std::move(e));
}

struct Env {
  std::vector<Value> slots;
  const std::vector<ArrayP>* arrays;
};

Value eval(const Exp& e, Env& env);

Value apply_fun(const Fun& f, Env& env, const Value* args, size_t nargs) {
  if (nargs != f.params.size()) throw std::runtime_error("function applied to wrong number of arguments");
  for (size_t i = 0; i < nargs; ++i) env.slots[f.params[i]] = args[i];
  return eval(*f.body, env);
}
Value apply1(const Fun& f, Env& env, const Value& a) { return apply_fun(f, env, &a, 1); }
Value apply2(const Fun& f, Env& env, const Value& a, const Value& b) {
  Value args[2] = {a, b};
  return apply_fun(f, env, args, 2);
}

// evalOpenExp, Interp:912-1001
Value eval(const Exp& e, Env& env) {
  switch (e.kind) {
    case E_CONST: return Value::scalar(e.c);
    case E_VAR: return env.slots[e.slot];
    case E_LET: {
      Value v = eval(*e.a[0], env);
      env.slots[e.slot] = std::move(v);
      return eval(*e.a[1], env);
    }
    case E_TUP: {
      std::vector<Value> xs;
      xs.reserve(e.a.size());
      for (auto& c : e.a) xs.push_back(eval(*c, env));
      return Value::tup(std::move(xs));
    }
    case E_SNOC: {
      Value l = eval(*e.a[0], env);
      if (!l.tuple) throw std::runtime_error("snoc: left operand is not a tuple");
      l.e.push_back(eval(*e.a[1], env));
      return l;
    }
    case E_INIT: {
      Value v = eval(*e.a[0], env);
      if (!v.tuple || v.e.empty()) throw std::runtime_error("init of a non-tuple or empty tuple");
      v.e.pop_back();
      return v;
    }
    case E_PRJ: {
      Value v = eval(*e.a[0], env);
      if (v.tuple && e.slot == -1 && !v.e.empty()) return v.e.back();
      if (!v.tuple || (size_t)e.slot >= v.e.size()) throw std::runtime_error("prj: not a tuple / index out of range");
      return v.e[e.slot];
    }
    case E_COND: {
      Value c = eval(*e.a[0], env);
      return c.s.i != 0 ? eval(*e.a[1], env) : eval(*e.a[2], env);  // toBool: non-zero is true
    }
    case E_WHILE: {
      Value x = eval(*e.a[0], env);
      for (;;) {
        Value c = apply1(*e.f[0], env, x);
        if (c.s.i == 0) break;
        x = apply1(*e.f[1], env, x);
      }
      return x;
    }
    case E_PRIM: {
      std::vector<Value> args;
      args.reserve(e.a.size());
      for (auto& c : e.a) args.push_back(eval(*c, env));
      // a primitive of two arguments may receive them as one pair
      if (args.size() == 1 && args[0].tuple) { std::vector<Value> t = args[0].e; args = t; }
      return eval_prim(e, args);
    }
    case E_INDEX: {
      const Array& a = *(*env.arrays)[e.arr];
      Value ix = eval(*e.a[0], env);
      return read_value(a, to_index(a.sh, value_shape(ix)));
    }
    case E_LINDEX: {
      const Array& a = *(*env.arrays)[e.arr];
      Value i = eval(*e.a[0], env);
      // Interp:996-998: fromIndex (bounds-checked) then (!)
      return read_value(a, i.s.i);
    }
    case E_SHAPE: return shape_value((*env.arrays)[e.arr]->sh);
    case E_SHAPESIZE: return Value::scalar(mk_int(I64, (uint64_t)shape_size(value_shape(eval(*e.a[0], env)))));
    case E_TOINDEX: {
      auto sh = value_shape(eval(*e.a[0], env));
      auto ix = value_shape(eval(*e.a[1], env));
      return Value::scalar(mk_int(I64, (uint64_t)to_index(sh, ix)));
    }
    case E_FROMINDEX: {
      auto sh = value_shape(eval(*e.a[0], env));
      Value i = eval(*e.a[1], env);
      return shape_value(from_index(sh, i.s.i));
    }
    case E_COERCE: {
      // bit reinterpretation between equal-sized scalar types (Interp:1010-1012)
      Value v = eval(*e.a[0], env);
      uint64_t bits = 0;
      if (e.t1 == F16) bits = f16_bits(v.s.f);
      else if (e.t1 == F32) memcpy(&bits, &v.s.f, 4);
      else if (e.t1 == F64) memcpy(&bits, &v.s.d, 8);
      else bits = (uint64_t)v.s.i;
      if (e.t2 == F16) { Scalar h; h.ty = F16; h.i = 0; h.f = f16_value((uint16_t)bits); return Value::scalar(h); }
      if (e.t2 == F32) { float f; uint32_t b = (uint32_t)bits; memcpy(&f, &b, 4); return Value::scalar(mk_f32(f)); }
      if (e.t2 == F64) { double d; memcpy(&d, &bits, 8); return Value::scalar(mk_f64(d)); }
      return Value::scalar(mk_int(e.t2, bits));
    }
    case E_UNDEF: return undef_value(e.ety);
    case E_APP: {
      std::vector<Value> args;
      for (auto& c : e.a) args.push_back(eval(*c, env));
      return apply_fun(*e.f[0], env, args.data(), args.size());
    }
    case E_CASE: {
      Value tag = eval(*e.a[0], env);
      for (size_t i = 0; i < e.tags.size(); ++i)
        if (e.tags[i] == tag.s.i) return eval(*e.a[1 + i], env);
      if (e.has_default) return eval(*e.a.back(), env);
      throw std::runtime_error("unmatched case");
    }
  }
  throw std::runtime_error("unhandled expression kind");
}

// ----------------------------------------------------------------------------
// Array-level nodes (AST.hs:230-460 PreOpenAcc; Interp:175-259 evalOpenAcc)
// ----------------------------------------------------------------------------

// Delayed array: extent + index function (Interp:188-192); a manifest operand
// becomes the obvious closure over the array.
struct Delayed {
  bool manifest = false;
  int arr = -1;
  std::unique_ptr<Exp> extent;
  std::unique_ptr<Fun> index;
};

struct Node;
// An array-level function (Awhile's condition and step, Apply's function) or a branch of Acond.
struct Body {
  std::vector<int> params;
  std::vector<Node> nodes;
  std::vector<int> outs;
};

struct Node {
  std::string kind;
  std::vector<int> outs;  // array slots defined
  std::vector<Body> body;              // acond: then, else; awhile: condition, step; apply: function
  std::vector<int> args;               // awhile: initial state; apply: arguments; atrace: the arrays handed on
  std::vector<int> shown;              // atrace: the arrays to print
  std::string message;                 // atrace
  ArrayP use_val;                      // use: the embedded array
  std::vector<std::unique_ptr<Fun>> f;
  std::vector<std::unique_ptr<Exp>> x;
  std::vector<Delayed> d;
  std::vector<EltTy> elt;              // result element type(s)
  bool right = false, seeded = false;  // scans / folds
  int arr = -1;                        // permute defaults, reshape source
  std::vector<std::vector<int>> stencil_extent;     // per input, per dim
  std::vector<std::string> bnd_kind;                // per stencil input
  std::vector<std::unique_ptr<Exp>> bnd_const;
  std::vector<std::unique_ptr<Fun>> bnd_fun;
};

struct Program {
  std::map<std::string, int> arrays;
  std::vector<std::string> array_names;
  std::vector<int> inputs;
  std::vector<EltTy> input_elt;
  std::vector<int> input_rank;
  std::vector<Node> nodes;
  std::vector<int> outputs;
  int max_slot = 0;
  // run state
  std::vector<ArrayP> vals;
  std::string error;
};

int def_array(Program& p, const std::string& name) {
  int s = (int)p.array_names.size();
  p.array_names.push_back(name);
  p.arrays[name] = s;  // shadowing allowed
  return s;
}

Delayed parse_delayed(const Sx& x, Scope& sc) {
  Delayed d;
  if (x.head() == "manifest") {
    d.manifest = true;
    d.arr = sc.array(x[1].s);
  } else if (x.head() == "delayed") {
    d.extent = parse_exp(x[1], sc);
    d.index = parse_fun(x[2], sc);
  } else {
    throw std::runtime_error("expected (manifest a) or (delayed sh fun)");
  }
  return d;
}

void parse_boundary(const Sx& x, Scope& sc, Node& n) {
  if (x.atom) {
    if (x.s != "clamp" && x.s != "mirror" && x.s != "wrap") throw std::runtime_error("unknown boundary '" + x.s + "'");
    n.bnd_kind.push_back(x.s);
    n.bnd_const.emplace_back();
    n.bnd_fun.emplace_back();
  } else if (x.head() == "constant") {
    n.bnd_kind.push_back("constant");
    n.bnd_const.push_back(parse_exp(x[1], sc));
    n.bnd_fun.emplace_back();
  } else if (x.head() == "function") {
    n.bnd_kind.push_back("function");
    n.bnd_const.emplace_back();
    n.bnd_fun.push_back(parse_fun(x[1], sc));
  } else {
    throw std::runtime_error("bad boundary");
  }
}

std::vector<int> parse_stencilr(const Sx& x) {
  if (x.head() != "stencilr") throw std::runtime_error("expected (stencilr e0 e1 ..)");
  std::vector<int> r;
  for (size_t i = 1; i < x.size(); ++i) {
    int v = atoi(x.k[i].s.c_str());
    if (v != 3 && v != 5 && v != 7 && v != 9) throw std::runtime_error("stencil extent must be 3, 5, 7 or 9");
    r.push_back(v);
  }
  return r;
}

// Node grammar (element types are written explicitly so that empty results can
// still be typed):
//   (generate ELT sh fun)
//   (fold ELT fun [seed] D)            fold / fold1
//   (foldseg ELT fun [seed] D Dseg)    segment operand holds OFFSETS (Interp:390-424)
//   (scanl|scanr ELT fun [seed] D)     scanl/scanl1/scanr/scanr1
//   (scanl'|scanr' ELT fun seed D)     two results
//   (permute ELT fun defaults ixfun D)
//   (stencil ELT stencilr fun bnd D)
//   (stencil2 ELT stencilr1 stencilr2 fun bnd1 D1 bnd2 D2)
//   (reshape sh a)
void parse_node(Program& p, std::vector<Node>& into, const Sx& bind, Scope& sc);

// (afun ((p (array R T)) ...) (let ..)* (out ..))  |  (branch (let ..)* (out ..))
Body parse_body(Program& p, const Sx& x, Scope& sc, bool with_params) {
  if (x.head() != (with_params ? "afun" : "branch")) throw std::runtime_error("expected an array function");
  Body b;
  size_t i = 1;
  if (with_params) {
    for (auto& q : x[1].k) b.params.push_back(def_array(p, q[0].s));
    i = 2;
  }
  for (; i < x.size(); ++i) {
    const Sx& f = x.k[i];
    if (f.head() == "let") parse_node(p, b.nodes, f, sc);
    else if (f.head() == "out") for (size_t j = 1; j < f.size(); ++j) b.outs.push_back(sc.array(f.k[j].s));
    else throw std::runtime_error("unknown form in an array function");
  }
  if (b.outs.empty()) throw std::runtime_error("array function has no (out ...)");
  return b;
}

int hex_val(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  throw std::runtime_error("bad hexadecimal digit");
}

void parse_node(Program& p, std::vector<Node>& into, const Sx& bind, Scope& sc) {
  const Sx& lhs = bind[1];
  const Sx& x = bind[2];
  Node n;
  n.kind = x.head();
  const std::string& k = n.kind;
  size_t i = 1;
  auto is_fun = [&](const Sx& s) { return s.head() == "lam"; };
  auto is_delayed = [&](const Sx& s) { return s.head() == "manifest" || s.head() == "delayed"; };
  if (k == "generate") {
    n.elt.push_back(parse_elt(x[1]));
    n.x.push_back(parse_exp(x[2], sc));
    n.f.push_back(parse_fun(x[3], sc));
  } else if (k == "fold" || k == "foldseg" || k == "scanl" || k == "scanr" || k == "scanl'" || k == "scanr'") {
    n.elt.push_back(parse_elt(x[1]));
    n.f.push_back(parse_fun(x[2], sc));
    i = 3;
    if (!is_delayed(x[i])) { n.seeded = true; n.x.push_back(parse_exp(x[i], sc)); ++i; }
    n.d.push_back(parse_delayed(x[i++], sc));
    if (k == "foldseg") n.d.push_back(parse_delayed(x[i++], sc));
    n.right = (k == "scanr" || k == "scanr'");
    if ((k == "scanl'" || k == "scanr'") && !n.seeded) throw std::runtime_error(k + " needs a seed");
  } else if (k == "permute") {
    n.elt.push_back(parse_elt(x[1]));
    n.f.push_back(parse_fun(x[2], sc));
    n.arr = sc.array(x[3].s);
    n.f.push_back(parse_fun(x[4], sc));
    n.d.push_back(parse_delayed(x[5], sc));
  } else if (k == "stencil") {
    n.elt.push_back(parse_elt(x[1]));
    n.stencil_extent.push_back(parse_stencilr(x[2]));
    n.f.push_back(parse_fun(x[3], sc));
    parse_boundary(x[4], sc, n);
    n.d.push_back(parse_delayed(x[5], sc));
  } else if (k == "stencil2") {
    n.elt.push_back(parse_elt(x[1]));
    n.stencil_extent.push_back(parse_stencilr(x[2]));
    n.stencil_extent.push_back(parse_stencilr(x[3]));
    n.f.push_back(parse_fun(x[4], sc));
    parse_boundary(x[5], sc, n);
    n.d.push_back(parse_delayed(x[6], sc));
    parse_boundary(x[7], sc, n);
    n.d.push_back(parse_delayed(x[8], sc));
  } else if (k == "reshape") {
    n.x.push_back(parse_exp(x[1], sc));
    n.arr = sc.array(x[2].s);
  } else if (k == "use") {
    // (use (array R ELT) (shape d..) (hex LEAF)...): Use, Interp:231
    EltTy elt = parse_elt(x[1][2]);
    std::vector<int64_t> sh;
    for (size_t d = 1; d < x[2].size(); ++d) sh.push_back(atoll(x[2].k[d].s.c_str()));
    n.use_val = new_array(elt, sh);
    if (x.size() != 3 + n.use_val->leaf.size()) throw std::runtime_error("use: one (hex ...) per leaf expected");
    for (size_t l = 0; l < n.use_val->leaf.size(); ++l) {
      const std::string digits = x[3 + l].size() > 1 ? x[3 + l][1].s : std::string();
      auto& buf = n.use_val->leaf[l];
      if (digits.size() != 2 * buf.size()) throw std::runtime_error("use: payload size mismatch");
      for (size_t b = 0; b < buf.size(); ++b) buf[b] = (unsigned char)(hex_val(digits[2 * b]) * 16 + hex_val(digits[2 * b + 1]));
    }
  } else if (k == "acond") {
    n.x.push_back(parse_exp(x[1], sc));
    n.body.push_back(parse_body(p, x[2], sc, false));
    n.body.push_back(parse_body(p, x[3], sc, false));
  } else if (k == "awhile") {
    n.body.push_back(parse_body(p, x[1], sc, true));
    n.body.push_back(parse_body(p, x[2], sc, true));
    for (size_t j = 1; j < x[3].size(); ++j) n.args.push_back(sc.array(x[3].k[j].s));
  } else if (k == "apply") {
    n.body.push_back(parse_body(p, x[1], sc, true));
    for (size_t j = 1; j < x[2].size(); ++j) n.args.push_back(sc.array(x[2].k[j].s));
  } else if (k == "atrace") {
    // (atrace (hex MESSAGE) (show a..) (args b..))
    const std::string digits = x[1].size() > 1 ? x[1].k[1].s : std::string();
    auto hv = [](char ch) { return ch <= '9' ? ch - '0' : (ch | 32) - 'a' + 10; };
    for (size_t i = 0; i + 1 < digits.size(); i += 2) n.message.push_back((char)(hv(digits[i]) * 16 + hv(digits[i + 1])));
    for (size_t j = 1; j < x[2].size(); ++j) n.shown.push_back(sc.array(x[2].k[j].s));
    for (size_t j = 1; j < x[3].size(); ++j) n.args.push_back(sc.array(x[3].k[j].s));
  } else {
    throw std::runtime_error("unknown array node '" + k + "'");
  }
  (void)is_fun;
  // define outputs after parsing operands (no recursive bindings)
  if (lhs.atom) n.outs.push_back(def_array(p, lhs.s));
  else for (auto& nm : lhs.k) n.outs.push_back(def_array(p, nm.s));
  into.push_back(std::move(n));
}

Program* parse_program(const std::string& text) {
  SxParser sp{text.data(), text.data() + text.size()};
  Sx top = sp.parse();
  if (top.head() != "program") throw std::runtime_error("expected (program ...)");
  auto p = std::make_unique<Program>();
  Scope sc;
  sc.arrays = &p->arrays;
  for (size_t i = 1; i < top.size(); ++i) {
    const Sx& f = top.k[i];
    std::string h = f.head();
    if (h == "in") {
      // (in name (array RANK ELT))
      int s = def_array(*p, f[1].s);
      p->inputs.push_back(s);
      p->input_rank.push_back(atoi(f[2][1].s.c_str()));
      p->input_elt.push_back(parse_elt(f[2][2]));
    } else if (h == "let") {
      parse_node(*p, p->nodes, f, sc);
    } else if (h == "out") {
      for (size_t j = 1; j < f.size(); ++j) p->outputs.push_back(sc.array(f.k[j].s));
    } else {
      throw std::runtime_error("unknown program form '" + h + "'");
    }
  }
  p->max_slot = sc.max_slot + 4;
  return p.release();
}

// The closure a delayed operand denotes
struct DelayedFn {
  std::vector<int64_t> sh;
  const Delayed* d;
  Env* env;
  const Array* arr = nullptr;
  Value at(const std::vector<int64_t>& ix) const {
    if (d->manifest) return read_value(*arr, to_index(arr->sh, ix));
    return apply1(*d->index, *env, shape_value(ix));
  }
};
DelayedFn force_delayed(const Delayed& d, Env& env) {
  DelayedFn f;
  f.d = &d;
  f.env = &env;
  if (d.manifest) {
    f.arr = (*env.arrays)[d.arr].get();
    f.sh = f.arr->sh;
  } else {
    f.sh = value_shape(eval(*d.extent, env));
  }
  return f;
}

// iterate an index space in row-major order (Shape.hs:127-132 with (>>))
template <class F>
void for_each_index(const std::vector<int64_t>& sh, F f) {
  int64_t n = shape_size(sh);
  std::vector<int64_t> ix(sh.size(), 0);
  for (int64_t i = 0; i < n; ++i) {
    f(ix, i);
    for (size_t d = sh.size(); d-- > 0;) {
      if (++ix[d] < sh[d]) break;
      ix[d] = 0;
    }
  }
}

std::vector<int64_t> with_inner(const std::vector<int64_t>& outer, int64_t i) {
  std::vector<int64_t> r = outer;
  r.push_back(i);
  return r;
}

// foldOp Interp:371-377 (iter: strict left fold from the seed, Shape.hs:127-132)
// fold1Op Interp:380-387 (iter1: right-nested, Shape.hs:136-142)
Value fold_range(const Fun& f, Env& env, const Value* seed, int64_t n, const std::vector<int64_t>& outer,
                 int64_t start, const DelayedFn& arr) {
  if (seed) {
    Value r = *seed;
    for (int64_t i = 0; i < n; ++i) r = apply2(f, env, r, arr.at(with_inner(outer, start + i)));
    return r;
  }
  Value r = arr.at(with_inner(outer, start + n - 1));
  for (int64_t i = n - 2; i >= 0; --i) r = apply2(f, env, arr.at(with_inner(outer, start + i)), r);
  return r;
}

void run_node(Program& p, const Node& n, Env& env);

// Evaluate an array-level function on the given arrays (evalOpenAfun, Interp:144-156)
std::vector<ArrayP> call_body(Program& p, const Body& b, const std::vector<ArrayP>& args, Env& env) {
  if (args.size() != b.params.size()) throw std::runtime_error("array function: wrong number of arguments");
  for (size_t k = 0; k < args.size(); ++k) p.vals[b.params[k]] = args[k];
  for (auto& m : b.nodes) run_node(p, m, env);
  std::vector<ArrayP> r;
  for (int o : b.outs) r.push_back(p.vals[o]);
  return r;
}

void run_node(Program& p, const Node& n, Env& env) {
  const std::string& k = n.kind;
  auto& vals = p.vals;
  if (k == "use") {
    vals[n.outs[0]] = n.use_val;                                   // Interp:231
  } else if (k == "acond") {
    // Interp:217-219
    const bool yes = eval(*n.x[0], env).s.i != 0;
    std::vector<ArrayP> r = call_body(p, n.body[yes ? 0 : 1], {}, env);
    for (size_t i = 0; i < n.outs.size(); ++i) vals[n.outs[i]] = r[i];
  } else if (k == "awhile") {
    // Interp:221-229: go a = if cond a `linearIndex` 0 then go (body a) else a
    std::vector<ArrayP> st;
    for (int a : n.args) st.push_back(vals[a]);
    for (;;) {
      std::vector<ArrayP> c = call_body(p, n.body[0], st, env);
      if (read_value(*c[0], 0).s.i == 0) break;
      st = call_body(p, n.body[1], st, env);
    }
    for (size_t i = 0; i < n.outs.size(); ++i) vals[n.outs[i]] = st[i];
  } else if (k == "apply") {
    // Interp:215
    std::vector<ArrayP> as;
    for (int a : n.args) as.push_back(vals[a]);
    std::vector<ArrayP> r = call_body(p, n.body[0], as, env);
    for (size_t i = 0; i < n.outs.size(); ++i) vals[n.outs[i]] = r[i];
  } else if (k == "atrace") {
    // Interp:215 and atraceOp (Interp:873-880): the message, ": " and the arrays when there are any, on standard
    // error; the arrays behind it are handed on.  (Rendering: constructor by rank, shape, elements in row-major order.)
    std::string line = n.message;
    for (size_t j = 0; j < n.shown.size(); ++j) line += (j ? ", " : ": ") + trace_render(*vals[n.shown[j]]);
    fprintf(stderr, "%s\n", line.c_str());
    fflush(stderr);
    for (size_t i = 0; i < n.outs.size(); ++i) vals[n.outs[i]] = vals[n.args[i]];
  } else if (k == "generate") {
    // generateOp Interp:269-275 via fromFunctionM (Representation/Array.hs:109-122)
    auto sh = value_shape(eval(*n.x[0], env));
    ArrayP out = new_array(n.elt[0], sh);
    for_each_index(sh, [&](const std::vector<int64_t>& ix, int64_t i) {
      write_value(*out, i, apply1(*n.f[0], env, shape_value(ix)));
    });
    vals[n.outs[0]] = out;
  } else if (k == "fold") {
    DelayedFn arr = force_delayed(n.d[0], env);
    if (arr.sh.empty()) throw std::runtime_error("fold: rank-0 input");
    std::vector<int64_t> osh(arr.sh.begin(), arr.sh.end() - 1);
    int64_t m = arr.sh.back();
    if (!n.seeded && m <= 0) throw std::runtime_error("empty array");  // Interp:386
    Value seed;
    if (n.seeded) seed = eval(*n.x[0], env);
    ArrayP out = new_array(n.elt[0], osh);
    for_each_index(osh, [&](const std::vector<int64_t>& ix, int64_t i) {
      write_value(*out, i, fold_range(*n.f[0], env, n.seeded ? &seed : nullptr, m < 0 ? 0 : m, ix, 0, arr));
    });
    vals[n.outs[0]] = out;
  } else if (k == "foldseg") {
    // foldSegOp Interp:390-406, fold1SegOp Interp:409-424
    DelayedFn arr = force_delayed(n.d[0], env);
    DelayedFn seg = force_delayed(n.d[1], env);
    int64_t ns = seg.sh.at(0);
    if (ns <= 0) throw std::runtime_error("empty segment descriptor");
    std::vector<int64_t> osh(arr.sh.begin(), arr.sh.end() - 1);
    osh.push_back(ns - 1);
    Value seed;
    if (n.seeded) seed = eval(*n.x[0], env);
    ArrayP out = new_array(n.elt[0], osh);
    for_each_index(osh, [&](const std::vector<int64_t>& ix, int64_t i) {
      std::vector<int64_t> sz(ix.begin(), ix.end() - 1);
      int64_t j = ix.back();
      Value a = seg.at({j}), b = seg.at({j + 1});
      int64_t start = a.s.ty >= U8 && a.s.ty <= U64 ? (int64_t)(uint64_t)a.s.i : a.s.i;
      int64_t end = b.s.i;
      if (n.seeded ? !(end >= start) : !(end > start)) throw std::runtime_error("empty segment");
      write_value(*out, i, fold_range(*n.f[0], env, n.seeded ? &seed : nullptr, end - start, sz, start, arr));
    });
    vals[n.outs[0]] = out;
  } else if (k == "scanl" || k == "scanr") {
    // scanl1Op :427-448, scanlOp :451-474, scanrOp :506-529, scanr1Op :532-552
    DelayedFn ain = force_delayed(n.d[0], env);
    std::vector<int64_t> outer(ain.sh.begin(), ain.sh.end() - 1);
    int64_t m = ain.sh.back() < 0 ? 0 : ain.sh.back();
    int64_t mo = n.seeded ? m + 1 : m;
    ArrayP out = new_array(n.elt[0], with_inner(outer, mo));
    Value seed;
    if (n.seeded) seed = eval(*n.x[0], env);
    for_each_index(outer, [&](const std::vector<int64_t>& sz, int64_t row) {
      int64_t base = row * mo;
      Value acc;
      if (!n.right) {
        for (int64_t i = 0; i < mo; ++i) {
          if (i == 0) acc = n.seeded ? seed : ain.at(with_inner(sz, 0));
          else acc = apply2(*n.f[0], env, acc, ain.at(with_inner(sz, n.seeded ? i - 1 : i)));
          write_value(*out, base + i, acc);
        }
      } else {
        for (int64_t i = 0; i < mo; ++i) {
          // position written: seeded n-i (of n+1), unseeded n-i-1
          if (i == 0) acc = n.seeded ? seed : ain.at(with_inner(sz, m - 1));
          else acc = apply2(*n.f[0], env, ain.at(with_inner(sz, n.seeded ? m - i : m - i - 1)), acc);
          write_value(*out, base + (mo - 1 - i), acc);
        }
      }
    });
    vals[n.outs[0]] = out;
  } else if (k == "scanl'" || k == "scanr'") {
    // scanl'Op :477-503, scanr'Op :555-582
    DelayedFn ain = force_delayed(n.d[0], env);
    std::vector<int64_t> outer(ain.sh.begin(), ain.sh.end() - 1);
    int64_t m = ain.sh.back() < 0 ? 0 : ain.sh.back();
    ArrayP out = new_array(n.elt[0], with_inner(outer, m));
    ArrayP sums = new_array(n.elt[0], outer);
    Value seed = eval(*n.x[0], env);
    for_each_index(outer, [&](const std::vector<int64_t>& sz, int64_t row) {
      Value acc = seed;
      for (int64_t i = 0; i <= m; ++i) {
        if (i > 0) {
          if (!n.right) acc = apply2(*n.f[0], env, acc, ain.at(with_inner(sz, i - 1)));
          else acc = apply2(*n.f[0], env, ain.at(with_inner(sz, m - i)), acc);
        }
        if (i == m) write_value(*sums, row, acc);
        else write_value(*out, row * m + (n.right ? m - 1 - i : i), acc);
      }
    });
    vals[n.outs[0]] = out;
    vals[n.outs[1]] = sums;
  } else if (k == "permute") {
    // permuteOp Interp:585-624: copy defaults, then update in row-major source
    // order with f applied as (f new old).
    const Array& def = *vals[n.arr];
    DelayedFn ain = force_delayed(n.d[0], env);
    ArrayP out = new_array(n.elt[0], def.sh);
    for (size_t l = 0; l < def.leaf.size(); ++l) out->leaf[l] = def.leaf[l];
    for_each_index(ain.sh, [&](const std::vector<int64_t>& src, int64_t) {
      Value m = apply1(*n.f[1], env, shape_value(src));  // PrimMaybe sh' = (tag, ix)  (AST.hs:201-202)
      if (!m.tuple || m.e.size() != 2) throw std::runtime_error("permute: index function must return (tag ix)");
      int64_t tag = m.e[0].s.i;
      if (tag == 0) return;
      if (tag != 1) throw std::runtime_error("unexpected tag");
      int64_t j = to_index(def.sh, value_shape(m.e[1]));
      Value x = ain.at(src);
      Value y = read_value(*out, j);
      write_value(*out, j, apply2(*n.f[0], env, x, y));
    });
    vals[n.outs[0]] = out;
  } else if (k == "stencil" || k == "stencil2") {
    // stencilOp :637-649, stencil2Op :652-668, stencilAccess :670-794, bounded :797-839
    size_t nin = n.d.size();
    std::vector<DelayedFn> in;
    for (size_t a = 0; a < nin; ++a) in.push_back(force_delayed(n.d[a], env));
    std::vector<int64_t> sh = in[0].sh;
    if (nin == 2)
      for (size_t d = 0; d < sh.size(); ++d) sh[d] = std::min(sh[d], in[1].sh[d]);  // intersect, Shape.hs:81-91
    std::vector<Value> bconst(nin);
    for (size_t a = 0; a < nin; ++a)
      if (n.bnd_kind[a] == "constant") bconst[a] = eval(*n.bnd_const[a], env);
    auto bounded = [&](size_t a, const std::vector<int64_t>& ix) -> Value {
      const auto& ash = in[a].sh;
      bool inside = true;
      for (size_t d = 0; d < ash.size(); ++d) inside = inside && ix[d] >= 0 && ix[d] < ash[d];
      if (inside) return in[a].at(ix);
      const std::string& b = n.bnd_kind[a];
      if (b == "function") return apply1(*n.bnd_fun[a], env, shape_value(ix));
      if (b == "constant") return bconst[a];
      std::vector<int64_t> jx = ix;
      for (size_t d = 0; d < ash.size(); ++d) {
        int64_t iz = ix[d], sz = ash[d];
        if (iz < 0) jx[d] = b == "clamp" ? 0 : (b == "mirror" ? -iz : sz + iz);
        else if (iz >= sz) jx[d] = b == "clamp" ? sz - 1 : (b == "mirror" ? sz - (iz - sz + 2) : iz - sz);
      }
      return in[a].at(jx);
    };
    // neighbourhood tuple: outermost dimension is the outermost tuple level,
    // offsets run -r..+r at every level (Interp:670-794)
    std::vector<int64_t> cur;
    std::function<Value(size_t, size_t, const std::vector<int64_t>&)> access;
    access = [&](size_t a, size_t d, const std::vector<int64_t>& ix) -> Value {
      if (d == ix.size()) return bounded(a, cur);
      int ext = n.stencil_extent[a][d], r = ext / 2;
      std::vector<Value> e;
      for (int o = -r; o <= r; ++o) {
        cur[d] = ix[d] + o;
        e.push_back(access(a, d + 1, ix));
      }
      cur[d] = ix[d];
      return Value::tup(std::move(e));
    };
    ArrayP out = new_array(n.elt[0], sh);
    for_each_index(sh, [&](const std::vector<int64_t>& ix, int64_t i) {
      cur = ix;
      std::vector<Value> args;
      for (size_t a = 0; a < nin; ++a) args.push_back(access(a, 0, ix));
      write_value(*out, i, apply_fun(*n.f[0], env, args.data(), args.size()));
    });
    vals[n.outs[0]] = out;
  } else if (k == "reshape") {
    // reshapeOp Interp:293-303: sizes must agree
    auto sh = value_shape(eval(*n.x[0], env));
    const ArrayP& src = vals[n.arr];
    if (shape_size(sh) != src->n) throw std::runtime_error("shape mismatch");
    auto out = std::make_shared<Array>(*src);
    out->sh = sh;
    vals[n.outs[0]] = out;
  }
}

}  // namespace

// ----------------------------------------------------------------------------
// C interface for the test harness
// ----------------------------------------------------------------------------
extern "C" {

void* orc_parse(const char* text, char* err, int errlen) {
  try {
    return parse_program(text);
  } catch (std::exception& e) {
    snprintf(err, errlen, "%s", e.what());
    return nullptr;
  }
}

void orc_free(void* h) { delete (Program*)h; }

int orc_num_inputs(void* h) { return (int)((Program*)h)->inputs.size(); }

// Bind input k: shape and one pointer per scalar leaf (copied).
int orc_set_input(void* h, int k, int rank, const int64_t* shape, int nleaves, const void* const* leaves) {
  Program* p = (Program*)h;
  try {
    if (p->vals.size() != p->array_names.size()) p->vals.assign(p->array_names.size(), nullptr);
    if (rank != p->input_rank[k]) throw std::runtime_error("input rank mismatch");
    ArrayP a = new_array(p->input_elt[k], std::vector<int64_t>(shape, shape + rank));
    if ((size_t)nleaves != a->leaf.size()) throw std::runtime_error("input leaf count mismatch");
    for (int l = 0; l < nleaves; ++l)
      if (!a->leaf[l].empty()) memcpy(a->leaf[l].data(), leaves[l], a->leaf[l].size());
    p->vals[p->inputs[k]] = a;
    return 0;
  } catch (std::exception& e) {
    p->error = e.what();
    return 1;
  }
}

int orc_run(void* h) {
  Program* p = (Program*)h;
  try {
    if (p->vals.size() != p->array_names.size()) p->vals.assign(p->array_names.size(), nullptr);
    Env env;
    env.slots.resize(p->max_slot + 64);
    env.arrays = &p->vals;
    for (auto& n : p->nodes) run_node(*p, n, env);
    return 0;
  } catch (std::exception& e) {
    p->error = e.what();
    return 1;
  }
}

const char* orc_error(void* h) { return ((Program*)h)->error.c_str(); }
int orc_num_outputs(void* h) { return (int)((Program*)h)->outputs.size(); }
int orc_out_rank(void* h, int k) { Program* p = (Program*)h; return (int)p->vals[p->outputs[k]]->sh.size(); }
void orc_out_shape(void* h, int k, int64_t* sh) {
  Program* p = (Program*)h;
  auto& s = p->vals[p->outputs[k]]->sh;
  for (size_t i = 0; i < s.size(); ++i) sh[i] = s[i];
}
int orc_out_nleaves(void* h, int k) { Program* p = (Program*)h; return (int)p->vals[p->outputs[k]]->leaf.size(); }
const char* orc_out_leaf_type(void* h, int k, int l) {
  Program* p = (Program*)h;
  return ty_name[p->vals[p->outputs[k]]->leaf_ty[l]];
}
void orc_out_leaf_copy(void* h, int k, int l, void* dst) {
  Program* p = (Program*)h;
  auto& b = p->vals[p->outputs[k]]->leaf[l];
  if (!b.empty()) memcpy(dst, b.data(), b.size());
}

}  // extern "C"
