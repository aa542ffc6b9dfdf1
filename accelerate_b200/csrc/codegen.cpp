// Scalar code generator: OpenExp trees -> CUDA statements over struct-of-scalars
// values, with the primitive semantics of the reference interpreter
// (Interpreter.hs:1086-1416): fixed-width integers wrap, `div`/`mod` floor,
// `quot`/`rem` truncate, shifts by >= the bit width are defined, `round` is
// half-to-even, `max x y = if x <= y then y else x`, Bool is a Word8 where any
// non-zero value is true, and no floating-point contraction (the kernels are
// compiled with --fmad=false).
#include "codegen.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <sstream>

namespace accb200 {

namespace {

struct CVal {
  Type ty;
  std::vector<std::string> leaf;  // one C expression per scalar leaf
};

std::string struct_name(const Type& t) {
  std::vector<Ty> l = t.leaves();
  if (l.empty()) return "E_unit";
  std::string s = "E";
  for (Ty x : l) s += std::string("_") + ty_name[x];
  return s;
}

// (a Half travels through the kernels as its 16 bits; only the primitives look inside)
std::string cty(Ty t) { return t == F16 ? "u16" : ty_name[t]; }

struct ParamSet {
  std::vector<std::string> arrays;             // arrays referenced, first-use order
  std::vector<std::string> named;              // named fields, first-use order
  const std::map<std::string, ArrayInfo>* info;
  std::set<std::string> structs;               // element structs already emitted
  std::string struct_code;
  void use_array(const std::string& a) {
    for (auto& x : arrays) if (x == a) return;
    arrays.push_back(a);
  }
  void use_named(const std::string& n) {
    for (auto& x : named) if (x == n) return;
    named.push_back(n);
  }
  const ArrayInfo& array(const std::string& a) const { return info->at(a); }
  // declare the struct for an element type (plus its warp-shuffle helpers)
  std::string need_struct(const Type& t) {
    std::string nm = struct_name(t);
    if (structs.insert(nm).second) {
      std::vector<Ty> l = t.leaves();
      std::ostringstream o;
      o << "struct " << nm << " {";
      for (size_t i = 0; i < l.size(); ++i) o << " " << cty(l[i]) << " l" << i << ";";
      o << " };\n";
      const char* sh[3] = {"down", "up", "idx"};
      for (int k = 0; k < 3; ++k) {
        o << "__device__ __forceinline__ " << nm << " acc_shfl_" << sh[k] << "(const " << nm << "& v, int d) { " << nm << " r;";
        for (size_t i = 0; i < l.size(); ++i) o << " r.l" << i << " = acc_shfl1_" << sh[k] << "(v.l" << i << ", d);";
        o << " return r; }\n";
      }
      struct_code += o.str();
    }
    return nm;
  }
};

std::string uty(Ty t) {
  switch (ty_bytes[t]) { case 1: return "u8"; case 2: return "u16"; case 4: return "u32"; default: return "u64"; }
}

std::string float_literal(Ty t, const std::string& lit) {
  double d;
  if (lit == "inf") d = INFINITY;
  else if (lit == "-inf") d = -INFINITY;
  else if (lit == "nan") d = NAN;
  else d = strtod(lit.c_str(), nullptr);
  char buf[96];
  if (t == F16) {
    snprintf(buf, sizeof buf, "((u16)0x%04xu)", (unsigned)half_from_float((float)d));
  } else if (t == F32) {
    float f = (float)d;
    uint32_t b;
    memcpy(&b, &f, 4);
    snprintf(buf, sizeof buf, "__uint_as_float(0x%08xu)", b);
  } else {
    uint64_t b;
    memcpy(&b, &d, 8);
    snprintf(buf, sizeof buf, "__longlong_as_double((long long)0x%016llxull)", (unsigned long long)b);
  }
  return buf;
}

std::string int_literal(Ty t, const std::string& lit) {
  if (ty_is_signed(t)) {
    long long v = strtoll(lit.c_str(), nullptr, 10);
    if (v == (-9223372036854775807LL - 1)) return "((i64)(-9223372036854775807LL - 1))";
    return "((" + cty(t) + ")" + std::to_string(v) + "LL)";
  }
  unsigned long long v = strtoull(lit.c_str(), nullptr, 10);
  return "((" + cty(t) + ")" + std::to_string(v) + "ULL)";
}

class Gen {
 public:
  ParamSet& ps;
  std::ostringstream out;
  int& tmp;
  std::vector<std::pair<std::string, CVal>> env;
  // stream detection: (index A ix) where ix evaluates to exactly the loop index becomes a
  // function parameter supplied by the skeleton
  std::vector<std::string> loop_ix;
  std::vector<std::string>* streams = nullptr;
  std::string ind = "  ";

  Gen(ParamSet& p, int& counter) : ps(p), tmp(counter) {}

  std::string fresh() { return "t" + std::to_string(tmp++); }

  std::string def(Ty t, const std::string& expr) {
    std::string v = fresh();
    out << ind << "const " << cty(t) << " " << v << " = " << expr << ";\n";
    return v;
  }
  CVal declare(const Type& t) {
    CVal r;
    r.ty = t;
    for (Ty l : t.leaves()) {
      std::string v = fresh();
      out << ind << cty(l) << " " << v << ";\n";
      r.leaf.push_back(v);
    }
    return r;
  }
  void assign(const CVal& dst, const CVal& src) {
    for (size_t i = 0; i < dst.leaf.size(); ++i) out << ind << dst.leaf[i] << " = " << src.leaf[i] << ";\n";
  }
  const CVal& lookup(const std::string& n) {
    for (size_t i = env.size(); i-- > 0;)
      if (env[i].first == n) return env[i].second;
    throw Error(B200_ERR_TYPE, "code generator: unbound variable '" + n + "'");
  }

  std::string to_index(const std::vector<std::string>& sh, const std::vector<std::string>& ix) {
    if (sh.empty()) return "((i64)0)";
    std::string r = ix[0];
    for (size_t d = 1; d < sh.size(); ++d) r = "(" + r + " * " + sh[d] + " + " + ix[d] + ")";
    return r;
  }
  std::vector<std::string> shape_of(const std::string& arr) {
    ps.use_array(arr);
    std::vector<std::string> r;
    for (int d = 0; d < ps.array(arr).rank; ++d) r.push_back("p." + arr + "_d" + std::to_string(d));
    return r;
  }
  CVal load(const std::string& arr, const std::string& lin) {
    ps.use_array(arr);
    const ArrayInfo& ai = ps.array(arr);
    CVal r;
    r.ty = ai.elt;
    std::vector<Ty> l = ai.elt.leaves();
    std::string a = def(I64, lin);
    for (size_t i = 0; i < l.size(); ++i) r.leaf.push_back(def(l[i], "__ldg(p." + arr + "_l" + std::to_string(i) + " + " + a + ")"));
    return r;
  }

  CVal apply(const Fun& f, const std::vector<CVal>& args) {
    size_t mark = env.size();
    for (size_t i = 0; i < args.size(); ++i) env.emplace_back(f.params[i], args[i]);
    CVal r = gen(*f.body);
    env.resize(mark);
    return r;
  }

  CVal gen(const Expr& e) {
    CVal r;
    r.ty = e.ty;
    switch (e.kind) {
      case X_CONST: {
        Ty t = e.ty.s;
        r.leaf.push_back(ty_is_float(t) ? float_literal(t, e.lit) : int_literal(t, e.lit));
        return r;
      }
      case X_VAR: return lookup(e.name);
      case X_LET: {
        CVal v = gen(*e.a[0]);
        env.emplace_back(e.name, v);
        r = gen(*e.a[1]);
        env.pop_back();
        return r;
      }
      case X_TUP:
        for (auto& c : e.a) {
          CVal v = gen(*c);
          r.leaf.insert(r.leaf.end(), v.leaf.begin(), v.leaf.end());
        }
        return r;
      case X_SNOC:
        for (auto& c : e.a) {
          CVal v = gen(*c);
          r.leaf.insert(r.leaf.end(), v.leaf.begin(), v.leaf.end());
        }
        return r;
      case X_INIT: {
        CVal v = gen(*e.a[0]);
        r.leaf.assign(v.leaf.begin(), v.leaf.end() - v.ty.e.back().nleaves());
        return r;
      }
      case X_PRJ: {
        CVal v = gen(*e.a[0]);
        size_t off = 0;
        for (int i = 0; i < e.n; ++i) off += v.ty.e[i].nleaves();
        size_t cnt = v.ty.e[e.n].nleaves();
        r.leaf.assign(v.leaf.begin() + off, v.leaf.begin() + off + cnt);
        return r;
      }
      case X_COND: {
        CVal c = gen(*e.a[0]);
        r = declare(e.ty);
        out << ind << "if (" << c.leaf[0] << " != 0) {\n";
        std::string save = ind;
        ind += "  ";
        assign(r, gen(*e.a[1]));
        ind = save;
        out << ind << "} else {\n";
        ind += "  ";
        assign(r, gen(*e.a[2]));
        ind = save;
        out << ind << "}\n";
        return r;
      }
      case X_WHILE: {
        CVal s = gen(*e.a[0]);
        r = declare(e.ty);
        assign(r, s);
        out << ind << "for (;;) {\n";
        std::string save = ind;
        ind += "  ";
        CVal c = apply(*e.f[0], {r});
        out << ind << "if (" << c.leaf[0] << " == 0) break;\n";
        CVal nx = apply(*e.f[1], {r});
        assign(r, nx);
        ind = save;
        out << ind << "}\n";
        return r;
      }
      case X_PRIM: return gen_prim(e);
      case X_INDEX: {
        const Expr& ix = *e.a[0];
        CVal iv = gen(ix);
        if (streams && iv.leaf == loop_ix) {
          // element at exactly the loop index: supplied by the skeleton
          size_t k = 0;
          for (; k < streams->size(); ++k)
            if ((*streams)[k] == e.name) break;
          if (k == streams->size()) streams->push_back(e.name);
          ps.use_array(e.name);
          size_t nl = e.ty.nleaves();
          for (size_t i = 0; i < nl; ++i) r.leaf.push_back("s" + std::to_string(k) + "_l" + std::to_string(i));
          return r;
        }
        return load(e.name, to_index(shape_of(e.name), iv.leaf));
      }
      case X_LINDEX: {
        CVal iv = gen(*e.a[0]);
        return load(e.name, iv.leaf[0]);
      }
      case X_SHAPE:
        r.leaf = shape_of(e.name);
        return r;
      case X_SHAPESIZE: {
        CVal sh = gen(*e.a[0]);
        std::string s = "((i64)1)";
        for (auto& d : sh.leaf) s = "(" + s + " * (" + d + " <= 0 ? (i64)0 : " + d + "))";
        r.leaf.push_back(def(I64, s));
        return r;
      }
      case X_TOINDEX: {
        CVal sh = gen(*e.a[0]);
        CVal ix = gen(*e.a[1]);
        r.leaf.push_back(def(I64, to_index(sh.leaf, ix.leaf)));
        return r;
      }
      case X_FROMINDEX: {
        CVal sh = gen(*e.a[0]);
        CVal i = gen(*e.a[1]);
        size_t n = sh.leaf.size();
        r.leaf.resize(n);
        std::string cur = i.leaf[0];
        for (size_t d = n; d-- > 0;) {
          if (d == 0) { r.leaf[0] = cur; break; }
          r.leaf[d] = def(I64, cur + " % " + sh.leaf[d]);
          cur = def(I64, cur + " / " + sh.leaf[d]);
        }
        return r;
      }
      case X_COERCE: {
        CVal v = gen(*e.a[0]);
        const std::string& x = v.leaf[0];
        std::string s;
        if (e.t1 == F32 && e.t2 != F32) s = "(" + cty(e.t2) + ")__float_as_uint(" + x + ")";
        else if (e.t1 == F64 && e.t2 != F64) s = "(" + cty(e.t2) + ")__double_as_longlong(" + x + ")";
        else if (e.t2 == F32 && e.t1 != F32) s = "__uint_as_float((u32)" + x + ")";
        else if (e.t2 == F64 && e.t1 != F64) s = "__longlong_as_double((long long)" + x + ")";
        else s = "(" + cty(e.t2) + ")" + x;
        r.leaf.push_back(def(e.t2, s));
        return r;
      }
      case X_UNDEF:
        for (Ty l : e.ty.leaves()) r.leaf.push_back("((" + cty(l) + ")0)");
        return r;
      case X_APP: {
        std::vector<CVal> args;
        for (auto& c : e.a) args.push_back(gen(*c));
        return apply(*e.f[0], args);
      }
      case X_CASE: {
        CVal tag = gen(*e.a[0]);
        r = declare(e.ty);
        std::string save = ind;
        size_t nalt = e.tags.size();
        for (size_t i = 0; i < nalt; ++i) {
          out << ind << (i ? "} else if (" : "if (") << tag.leaf[0] << " == " << e.tags[i] << ") {\n";
          ind = save + "  ";
          assign(r, gen(*e.a[1 + i]));
          ind = save;
        }
        if (e.has_default) {
          out << ind << "} else {\n";
          ind = save + "  ";
          assign(r, gen(*e.a.back()));
          ind = save;
        }
        out << ind << "}\n";
        return r;
      }
    }
    throw Error(B200_ERR_UNSUPPORTED, "code generator: unhandled expression");
  }

  CVal gen_prim(const Expr& e) {
    std::vector<std::string> x;
    for (auto& c : e.a) {
      CVal v = gen(*c);
      x.insert(x.end(), v.leaf.begin(), v.leaf.end());
    }
    // Half: the Float primitive on the converted operands, rounded back (Numeric.Half's instances)
    const bool half = e.t1 == F16;
    const Ty t = half ? F32 : e.t1;
    if (half)
      for (auto& s : x) s = "acc_h2f(" + s + ")";
    const std::string T = cty(t), U = uty(t);
    const bool fl = ty_is_float(t), sg = ty_is_signed(t);
    const int bits = ty_bits(t);
    const std::string sfx = (t == F32) ? "f" : "";
    CVal r;
    r.ty = e.ty;
    auto one = [&](Ty rt, const std::string& s) {
      if (half && rt == F32) r.leaf.push_back(def(F16, "acc_f2h(" + s + ")"));
      else r.leaf.push_back(def(rt, s));
      return r;
    };
    auto wrap2 = [&](const char* op) {  // integer arithmetic in the unsigned type, then narrowed
      const std::string W = bits < 32 ? "u32" : U;
      return "(" + T + ")((" + W + ")" + x[0] + " " + op + " (" + W + ")" + x[1] + ")";
    };
    auto fun1 = [&](const char* name) { return one(t, std::string(name) + sfx + "(" + x[0] + ")"); };
    switch (e.op) {
      case P_ADD: return one(t, fl ? x[0] + " + " + x[1] : wrap2("+"));
      case P_SUB: return one(t, fl ? x[0] + " - " + x[1] : wrap2("-"));
      case P_MUL: return one(t, fl ? x[0] + " * " + x[1] : wrap2("*"));
      case P_NEG: return one(t, fl ? "-" + x[0] : "(" + T + ")((" + (bits < 32 ? std::string("u32") : U) + ")0 - (" + (bits < 32 ? std::string("u32") : U) + ")" + x[0] + ")");
      case P_ABS:
        if (fl) return one(t, "fabs" + sfx + "(" + x[0] + ")");
        if (!sg) return one(t, x[0]);
        return one(t, x[0] + " < 0 ? (" + T + ")((" + (bits < 32 ? std::string("u32") : U) + ")0 - (" + (bits < 32 ? std::string("u32") : U) + ")" + x[0] + ") : " + x[0]);
      case P_SIG:
        if (fl) return one(t, x[0] + " > 0 ? (" + T + ")1 : (" + x[0] + " < 0 ? (" + T + ")-1 : " + x[0] + ")");
        if (sg) return one(t, "(" + T + ")((" + x[0] + " > 0) - (" + x[0] + " < 0))");
        return one(t, "(" + T + ")(" + x[0] + " != 0)");
      case P_QUOT: return one(t, "acc_quot<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_REM: return one(t, "acc_rem<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_IDIV: return one(t, "acc_div<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_MOD: return one(t, "acc_mod<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_QUOTREM:
        r.leaf.push_back(def(t, "acc_quot<" + T + ">(" + x[0] + ", " + x[1] + ")"));
        r.leaf.push_back(def(t, "acc_rem<" + T + ">(" + x[0] + ", " + x[1] + ")"));
        return r;
      case P_DIVMOD:
        r.leaf.push_back(def(t, "acc_div<" + T + ">(" + x[0] + ", " + x[1] + ")"));
        r.leaf.push_back(def(t, "acc_mod<" + T + ">(" + x[0] + ", " + x[1] + ")"));
        return r;
      case P_BAND: return one(t, "(" + T + ")(" + x[0] + " & " + x[1] + ")");
      case P_BOR: return one(t, "(" + T + ")(" + x[0] + " | " + x[1] + ")");
      case P_BXOR: return one(t, "(" + T + ")(" + x[0] + " ^ " + x[1] + ")");
      case P_BNOT: return one(t, "(" + T + ")(~" + x[0] + ")");
      case P_SHL: return one(t, "acc_shl<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_SHR: return one(t, "acc_shr<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_ROTL: return one(t, "acc_rotl<" + T + ">(" + x[0] + ", " + x[1] + ")");
      case P_ROTR: return one(t, "acc_rotl<" + T + ">(" + x[0] + ", -(" + x[1] + "))");
      case P_POPCNT: return one(I64, "acc_popcount<" + T + ">(" + x[0] + ")");
      case P_CLZ: return one(I64, "acc_clz<" + T + ">(" + x[0] + ")");
      case P_CTZ: return one(I64, "acc_ctz<" + T + ">(" + x[0] + ")");
      case P_FDIV: return one(t, x[0] + " / " + x[1]);
      case P_RECIP: return one(t, "(" + T + ")1 / " + x[0]);
      case P_SIN: return fun1("sin");
      case P_COS: return fun1("cos");
      case P_TAN: return fun1("tan");
      case P_ASIN: return fun1("asin");
      case P_ACOS: return fun1("acos");
      case P_ATAN: return fun1("atan");
      case P_SINH: return fun1("sinh");
      case P_COSH: return fun1("cosh");
      case P_TANH: return fun1("tanh");
      case P_ASINH: return fun1("asinh");
      case P_ACOSH: return fun1("acosh");
      case P_ATANH: return fun1("atanh");
      case P_EXP: return fun1("exp");
      case P_SQRT: return fun1("sqrt");
      case P_LOG: return fun1("log");
      case P_FPOW: return one(t, "pow" + sfx + "(" + x[0] + ", " + x[1] + ")");
      case P_LOGBASE: return one(t, "log" + sfx + "(" + x[1] + ") / log" + sfx + "(" + x[0] + ")");
      case P_ATAN2: return one(t, "atan2" + sfx + "(" + x[0] + ", " + x[1] + ")");
      case P_TRUNCATE: return one(e.t2, "(" + cty(e.t2) + ")acc_f2i<" + T + ">(trunc" + sfx + "(" + x[0] + "))");
      case P_ROUND: return one(e.t2, "(" + cty(e.t2) + ")acc_f2i<" + T + ">(rint" + sfx + "(" + x[0] + "))");
      case P_FLOOR: return one(e.t2, "(" + cty(e.t2) + ")acc_f2i<" + T + ">(floor" + sfx + "(" + x[0] + "))");
      case P_CEILING: return one(e.t2, "(" + cty(e.t2) + ")acc_f2i<" + T + ">(ceil" + sfx + "(" + x[0] + "))");
      case P_FROMINTEGRAL: case P_TOFLOATING:
        if (e.t2 == F16) { r.leaf.push_back(def(F16, "acc_f2h((f32)" + x[0] + ")")); return r; }
        if (half) { r.leaf.push_back(def(e.t2, "(" + cty(e.t2) + ")" + x[0])); return r; }
        return one(e.t2, "(" + cty(e.t2) + ")" + x[0]);
      case P_ISNAN: return one(U8, "(u8)(" + x[0] + " != " + x[0] + ")");
      case P_ISINF: return one(U8, "(u8)(isinf(" + x[0] + ") != 0)");
      case P_LT: return one(U8, "(u8)(" + x[0] + " < " + x[1] + ")");
      case P_GT: return one(U8, "(u8)(" + x[0] + " > " + x[1] + ")");
      case P_LE: return one(U8, "(u8)(" + x[0] + " <= " + x[1] + ")");
      case P_GE: return one(U8, "(u8)(" + x[0] + " >= " + x[1] + ")");
      case P_EQ: return one(U8, "(u8)(" + x[0] + " == " + x[1] + ")");
      case P_NE: return one(U8, "(u8)(" + x[0] + " != " + x[1] + ")");
      case P_MAX: return one(t, "(" + x[0] + " <= " + x[1] + ") ? " + x[1] + " : " + x[0]);
      case P_MIN: return one(t, "(" + x[0] + " <= " + x[1] + ") ? " + x[0] + " : " + x[1]);
      case P_LAND: return one(U8, "(u8)((" + x[0] + " != 0) && (" + x[1] + " != 0))");
      case P_LOR: return one(U8, "(u8)((" + x[0] + " != 0) || (" + x[1] + " != 0))");
      case P_LNOT: return one(U8, "(u8)(" + x[0] + " == 0)");
      default: break;
    }
    throw Error(B200_ERR_UNSUPPORTED, "code generator: unhandled primitive");
  }
};

// ---------------------------------------------------------------------------
struct GlueBuilder {
  ParamSet ps;
  std::ostringstream fns;
  int tmp = 0;
  Glue glue;

  std::string ret_struct(const std::string& S, const CVal& v, const std::string& ind = "  ") {
    std::ostringstream o;
    o << ind << S << " r_;";
    for (size_t i = 0; i < v.leaf.size(); ++i) o << " r_.l" << i << " = " << v.leaf[i] << ";";
    o << " return r_;\n";
    return o.str();
  }
  CVal from_struct(const Type& t, const std::string& var) {
    CVal v;
    v.ty = t;
    size_t n = t.nleaves();
    for (size_t i = 0; i < n; ++i) v.leaf.push_back(var + ".l" + std::to_string(i));
    return v;
  }
  CVal index_val(int rank, const std::string& prefix) {
    CVal v;
    v.ty = Type::shape(rank);
    for (int d = 0; d < rank; ++d) v.leaf.push_back(prefix + std::to_string(d));
    return v;
  }
  std::string ix_params(int rank, const std::string& prefix = "ix") {
    std::string s;
    for (int d = 0; d < rank; ++d) s += ", i64 " + prefix + std::to_string(d);
    return s;
  }
  std::string ix_args(int rank, const std::string& prefix = "ix") {
    std::string s;
    for (int d = 0; d < rank; ++d) s += ", " + prefix + std::to_string(d);
    return s;
  }

  // E NAME(const Params& p, const E& a, const E& b)
  void binary_fun(const std::string& name, const Fun& f, const Type& elt) {
    std::string S = ps.need_struct(elt);
    Gen g(ps, tmp);
    g.env.emplace_back(f.params[0], from_struct(elt, "a"));
    g.env.emplace_back(f.params[1], from_struct(elt, "b"));
    CVal r = g.gen(*f.body);
    fns << "__device__ __forceinline__ " << S << " " << name << "(const Params& p, const " << S << "& a, const " << S << "& b) {\n"
        << g.out.str() << ret_struct(S, r) << "}\n";
  }
  // E NAME(const Params& p)
  void nullary_fun(const std::string& name, const Expr& e) {
    std::string S = ps.need_struct(e.ty);
    Gen g(ps, tmp);
    CVal r = g.gen(e);
    fns << "__device__ __forceinline__ " << S << " " << name << "(const Params& p) {\n" << g.out.str() << ret_struct(S, r) << "}\n";
  }

  // The access functions of a delayed operand (see codegen.hpp: streams).
  void delayed(const std::string& D, const Fun& index, int rank, const Type& elt) {
    delayed_custom(D, rank, elt, [&](Gen& g, const CVal& ix) { return g.apply(index, {ix}); });
  }
  // `body` produces the element at loop index `ix` (leaves ix0, ix1, ...)
  void delayed_custom(const std::string& D, int rank, const Type& elt, const std::function<CVal(Gen&, const CVal&)>& body) {
    std::string S = ps.need_struct(elt);
    std::vector<std::string> streams;
    Gen g(ps, tmp);
    g.loop_ix = index_val(rank, "ix").leaf;
    g.streams = &streams;
    CVal r = body(g, index_val(rank, "ix"));
    // stream value parameters
    std::string sparams, sargs_generic, sargs_lin, decl4, sargs4;
    std::ostringstream gen_loads, lin_loads, vec_loads;
    for (size_t k = 0; k < streams.size(); ++k) {
      const ArrayInfo& ai = ps.array(streams[k]);
      std::vector<Ty> l = ai.elt.leaves();
      std::vector<std::string> sh, ix;
      for (int d = 0; d < ai.rank; ++d) { sh.push_back("p." + streams[k] + "_d" + std::to_string(d)); ix.push_back("ix" + std::to_string(d)); }
      Gen tmpg(ps, tmp);
      gen_loads << "  const i64 a" << k << " = " << tmpg.to_index(sh, ix) << ";\n";
      for (size_t i = 0; i < l.size(); ++i) {
        std::string sv = "s" + std::to_string(k) + "_l" + std::to_string(i);
        std::string ptr = "p." + streams[k] + "_l" + std::to_string(i);
        sparams += ", " + cty(l[i]) + " " + sv;
        sargs_generic += ", __ldg(" + ptr + " + a" + std::to_string(k) + ")";
        sargs_lin += ", __ldg(" + ptr + " + lin)";
        vec_loads << "  " << cty(l[i]) << " " << sv << "[4]; acc_ld4(" << ptr << " + lin, " << sv << ");\n";
        sargs4 += ", " + sv + "[k]";
      }
    }
    glue.streams.push_back(streams);
    const std::string ixp = ix_params(rank), ixa = ix_args(rank);
    fns << "__device__ __forceinline__ " << S << " " << D << "_body(const Params& p" << ixp << sparams << ") {\n"
        << g.out.str() << ret_struct(S, r) << "}\n";
    // arbitrary index
    fns << "__device__ __forceinline__ " << S << " " << D << "_at_ix(const Params& p" << ixp << ") {\n"
        << gen_loads.str() << "  return " << D << "_body(p" << ixa << sargs_generic << ");\n}\n";
    // (row, j): row = linear index over the outer dimensions of the extent, j = innermost index
    std::ostringstream decomp;
    for (int d = 0; d < rank; ++d) ps.use_named(D + "_e" + std::to_string(d));
    ps.use_named(D + "_fast");
    if (rank >= 1) decomp << "  const i64 ix" << (rank - 1) << " = j;\n";
    if (rank == 2) decomp << "  const i64 ix0 = row;\n";
    if (rank >= 3) {
      decomp << "  i64 r_ = row;\n";
      for (int d = rank - 2; d >= 1; --d) decomp << "  const i64 ix" << d << " = r_ % p." << D << "_e" << d << "; r_ /= p." << D << "_e" << d << ";\n";
      decomp << "  const i64 ix0 = r_;\n";
    }
    const std::string inner = rank >= 1 ? "p." + D + "_e" + std::to_string(rank - 1) : "(i64)1";
    fns << "__device__ __forceinline__ " << S << " " << D << "_get(const Params& p, i64 row, i64 j) {\n" << decomp.str();
    if (!streams.empty()) {
      fns << "  if (p." << D << "_fast) {\n    const i64 lin = row * " << inner << " + j;\n    return " << D << "_body(p" << ixa << sargs_lin << ");\n  }\n";
    }
    fns << "  return " << D << "_at_ix(p" << ixa << ");\n}\n";
    // four consecutive innermost positions j..j+3 (needs the fast layout and 4-element alignment)
    std::string ixa4;
    for (int d = 0; d < rank; ++d) ixa4 += d == rank - 1 ? ", j + k" : ", ix" + std::to_string(d);
    fns << "__device__ __forceinline__ void " << D << "_get4(const Params& p, i64 row, i64 j, " << S << " (&o)[4]) {\n" << decomp.str()
        << "  const i64 lin = row * " << inner << " + j; (void)lin;\n" << vec_loads.str()
        << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) o[k] = " << D << "_body(p" << ixa4 << sargs4 << ");\n}\n";
    // the same from shared-memory copies of the streams' tiles (one pointer per stream leaf)
    if (!streams.empty()) {
      std::string sm_params, sm_loads, call_ptrs, bulk;
      size_t off = 0;   // in units of tile elements times bytes: offsets are (off * SCAN_TILE)
      for (size_t k = 0; k < streams.size(); ++k) {
        const ArrayInfo& ai = ps.array(streams[k]);
        std::vector<Ty> l = ai.elt.leaves();
        for (size_t i = 0; i < l.size(); ++i) {
          const std::string sv = "s" + std::to_string(k) + "_l" + std::to_string(i);
          sm_params += ", const " + cty(l[i]) + "* sm_" + sv;
          sm_loads += "  " + cty(l[i]) + " " + sv + "[4]; acc_lds4(sm_" + sv + ", " + sv + ");\n";
          call_ptrs += ", reinterpret_cast<const " + cty(l[i]) + "*>((BASE) + " + std::to_string(off) + " * SCAN_TILE) + (E)";
          bulk += "acc_bulk_g2s((BASE) + " + std::to_string(off) + " * SCAN_TILE, p." + streams[k] + "_l" + std::to_string(i) + " + (SRC), SCAN_TILE * " +
                  std::to_string(ty_bytes[l[i]]) + ", BAR); ";
          off += ty_bytes[l[i]];
        }
      }
      fns << "__device__ __forceinline__ void " << D << "_get4_sm_impl(const Params& p, i64 row, i64 j" << sm_params << ", " << S << " (&o)[4]) {\n"
          << decomp.str() << sm_loads << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) o[k] = " << D << "_body(p" << ixa4 << sargs4 << ");\n}\n";
      glue.defines[D + "_get4_sm(P, ROW, J, BASE, E, O)"] = D + "_get4_sm_impl(P, ROW, J" + call_ptrs + ", O)";
      glue.defines[D + "_BULK_ISSUE(BASE, BAR, SRC)"] = bulk;
      glue.defines[D + "_STAGE_BYTES"] = "(" + std::to_string(off) + " * SCAN_TILE)";
      glue.defines[D + "_STREAM_BYTES"] = std::to_string(off);
      size_t nleaves = 0;
      for (auto& sn : streams) nleaves += ps.array(sn).elt.nleaves();
      glue.defines[D + "_STREAM_NLEAVES"] = std::to_string(nleaves);
    }
    // same with the linear address of the first element supplied by the caller
    fns << "__device__ __forceinline__ void " << D << "_get4_lin(const Params& p, i64 lin, i64 row, i64 j, " << S << " (&o)[4]) {\n" << decomp.str()
        << "  (void)lin;\n" << vec_loads.str()
        << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) o[k] = " << D << "_body(p" << ixa4 << sargs4 << ");\n}\n";
    glue.defines[D + "_NSTREAMS"] = std::to_string(streams.size());
    glue.defines[D + "_INNER"] = rank >= 1 ? "(p." + D + "_e" + std::to_string(rank - 1) + ")" : "((i64)1)";
  }

  // void OUTk_store(p, lin, v) / OUTk_store4(p, lin, v[4])
  void output(int k, const Type& elt) {
    std::string S = ps.need_struct(elt);
    std::vector<Ty> l = elt.leaves();
    std::string O = "OUT" + std::to_string(k);
    fns << "__device__ __forceinline__ void " << O << "_store(const Params& p, i64 lin, const " << S << "& v) {\n";
    for (size_t i = 0; i < l.size(); ++i) fns << "  p.out" << k << "_l" << i << "[lin] = v.l" << i << ";\n";
    fns << "}\n";
    fns << "__device__ __forceinline__ void " << O << "_store4(const Params& p, i64 lin, const " << S << " (&v)[4]) {\n";
    for (size_t i = 0; i < l.size(); ++i) {
      fns << "  { " << cty(l[i]) << " w_[4] = {v[0].l" << i << ", v[1].l" << i << ", v[2].l" << i << ", v[3].l" << i << "}; acc_st4(p.out" << k
          << "_l" << i << " + lin, w_); }\n";
    }
    fns << "}\n";
    fns << "__device__ __forceinline__ " << S << " " << O << "_load(const Params& p, i64 lin) {\n  " << S << " r_;";
    for (size_t i = 0; i < l.size(); ++i) fns << " r_.l" << i << " = __ldcg(p.out" << k << "_l" << i << " + lin);";
    fns << " return r_;\n}\n";
    out_elts.push_back(elt);
  }
  std::vector<Type> out_elts;

  Glue finish() {
    std::ostringstream o;
    // parameter block: every field is 8 bytes wide
    std::ostringstream pb;
    pb << "struct Params {\n";
    for (auto& a : ps.arrays) {
      const ArrayInfo& ai = ps.array(a);
      std::vector<Ty> l = ai.elt.leaves();
      for (size_t i = 0; i < l.size(); ++i) {
        pb << "  const " << cty(l[i]) << "* __restrict__ " << a << "_l" << i << ";\n";
        glue.slots.push_back({Slot::ARR_LEAF, a, (int)i});
      }
      for (int d = 0; d < ai.rank; ++d) {
        pb << "  i64 " << a << "_d" << d << ";\n";
        glue.slots.push_back({Slot::ARR_DIM, a, d});
      }
    }
    for (size_t k = 0; k < out_elts.size(); ++k) {
      std::vector<Ty> l = out_elts[k].leaves();
      for (size_t i = 0; i < l.size(); ++i) {
        pb << "  " << cty(l[i]) << "* __restrict__ out" << k << "_l" << i << ";\n";
        glue.slots.push_back({Slot::OUT_LEAF, "", (int)(k * 64 + i)});
      }
    }
    // Names that start with '?' are wanted by some variants of the node's kernels only: they come last
    // (the host always passes them) and are declared when the variant defines ACC_OPT_PARAMS.  A kernel
    // that does not use them keeps the parameter block, and with it the code the compiler generates,
    // unchanged when such a field is added.
    bool opt = false;
    for (auto& n : ps.named) {
      const bool o = !n.empty() && n[0] == '?';
      if (opt && !o) throw Error(B200_ERR_ARG, "optional kernel parameters must come last");
      if (o && !opt) pb << "#if defined(ACC_OPT_PARAMS) && ACC_OPT_PARAMS\n";
      opt = opt || o;
      const std::string field = o ? n.substr(1) : n;
      pb << "  i64 " << field << ";\n";
      glue.slots.push_back({Slot::NAMED, field, 0});
    }
    if (opt) pb << "#endif\n";
    pb << "};\n";
    // element structs do not depend on Params; functions do
    glue.code = ps.struct_code + pb.str() + fns.str();
    // conversions of Half, only in programs that compute with it (cvt.rn: round to nearest even)
    if (glue.code.find("acc_h2f(") != std::string::npos || glue.code.find("acc_f2h(") != std::string::npos)
      glue.code =
          "__device__ __forceinline__ f32 acc_h2f(u16 h) { f32 f; asm(\"{ .reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t; }\" : \"=f\"(f) : \"h\"(h)); return f; }\n"
          "__device__ __forceinline__ u16 acc_f2h(f32 f) { u16 h; asm(\"{ .reg .b16 t; cvt.rn.f16.f32 t, %1; mov.b16 %0, t; }\" : \"=h\"(h) : \"f\"(f)); return h; }\n" +
          glue.code;
    return glue;
  }
};

bool var_is(const Expr& e, const std::string& n) { return e.kind == X_VAR && e.name == n; }

}  // namespace

bool is_simple_prim(const Fun& f, Prim* op, Ty* ty) {
  if (f.params.size() != 2) return false;
  const Expr& b = *f.body;
  if (b.kind != X_PRIM || b.a.size() != 2) return false;
  bool ab = var_is(*b.a[0], f.params[0]) && var_is(*b.a[1], f.params[1]);
  bool ba = var_is(*b.a[0], f.params[1]) && var_is(*b.a[1], f.params[0]);
  if (!ab && !ba) return false;
  switch (b.op) {
    case P_ADD: case P_MUL: case P_MIN: case P_MAX: case P_BAND: case P_BOR: case P_BXOR: case P_LAND: case P_LOR:
      *op = b.op;
      *ty = b.t1;
      return true;
    default: return false;
  }
}

Glue build_glue(const Node& n, const std::map<std::string, ArrayInfo>& arrays) {
  GlueBuilder b;
  b.ps.info = &arrays;
  auto& def = b.glue.defines;
  const std::string E = b.ps.need_struct(n.elt);
  std::vector<std::string> named;
  Prim op;
  Ty opty;
  switch (n.kind) {
    case N_GENERATE: {
      b.delayed("D0", *n.f, (int)n.extent->ty.e.size(), n.elt);
      b.output(0, n.elt);
      break;
    }
    case N_FOLD: case N_FOLDSEG: case N_SCAN: case N_SCAN2: {
      b.delayed("D0", *n.d[0].index, n.d[0].rank, n.elt);
      if (n.kind == N_FOLDSEG) b.delayed("D1", *n.d[1].index, 1, n.d[1].elt);
      b.binary_fun("F_combine", *n.f, n.elt);
      if (n.seed) b.nullary_fun("F_seed", *n.seed);
      def["ACC_SEEDED"] = n.seed ? "1" : "0";
      def["ACC_COMMUTATIVE"] = is_simple_prim(*n.f, &op, &opty) ? "1" : "0";
      if (n.kind == N_FOLD && is_simple_prim(*n.f, &op, &opty) && (opty == I32 || opty == U32) && !n.elt.tuple) {
        // a whole warp's 32-bit integers combine in one redux.sync (add, min, max, and, or, xor)
        const char* r = nullptr;
        switch (op) {
          case P_ADD: r = "add"; break;
          case P_MIN: r = "min"; break;
          case P_MAX: r = "max"; break;
          case P_BAND: r = "and"; break;
          case P_BOR: r = "or"; break;
          case P_BXOR: r = "xor"; break;
          default: break;
        }
        if (r) {
          const bool bits = op == P_BAND || op == P_BOR || op == P_BXOR;
          def["FOLD_REDUX"] = std::string("\"redux.sync.") + r + (bits ? ".b32" : (opty == I32 ? ".s32" : ".u32")) + " %0, %1, 0xffffffff;\"";
          def["FOLD_REDUX_IDENTITY"] = op == P_ADD || op == P_BOR || op == P_BXOR ? "0u"
                                       : op == P_BAND ? "0xffffffffu"
                                       : op == P_MIN ? (opty == I32 ? "0x7fffffffu" : "0xffffffffu")
                                                     : (opty == I32 ? "0x80000000u" : "0u");
        }
      }
      b.output(0, n.elt);
      if (n.kind == N_SCAN2) b.output(1, n.elt);
      if (n.kind == N_FOLDSEG) def["seg_t"] = b.ps.need_struct(n.d[1].elt);
      if (n.kind == N_SCAN || n.kind == N_SCAN2) {
        def["ACC_RIGHT"] = n.right ? "1" : "0";
        def["ACC_SCAN2"] = n.kind == N_SCAN2 ? "1" : "0";
        std::vector<Ty> sl = n.elt.leaves();
        if (sl.size() == 1) {
          def["SCAN_PACKED"] = "1";
          def["SCAN_T"] = cty(sl[0]);
          def["SCAN_T_BYTES"] = std::to_string(ty_bytes[sl[0]]);
        } else {
          def["SCAN_PACKED"] = "0";
        }
      }
      break;
    }
    case N_PERMUTE: {
      b.binary_fun("F_combine", *n.f, n.elt);
      b.output(0, n.elt);
      // One function per source element: \ix -> (tag, toIndex (shape out) target, source ! ix).
      // Index function and source share the loop index, so every array either of them reads at
      // exactly that index is loaded once, vectorised.
      {
        const int rank = n.d[0].rank;
        const int orank = arrays.at(n.arr).rank;
        const Type pelemT = Type::tup({Type::scalar(U8), Type::scalar(I64), n.elt});
        std::vector<std::string> outsh;
        for (int d = 0; d < orank; ++d) { outsh.push_back("p.out_d" + std::to_string(d)); b.ps.use_named("out_d" + std::to_string(d)); }
        b.delayed_custom("P", rank, pelemT, [&](Gen& g, const CVal& ix) {
          CVal m = g.apply(*n.g, {ix});            // (tag, target index)
          CVal v = g.apply(*n.d[0].index, {ix});   // source value
          CVal r;
          r.ty = pelemT;
          r.leaf.push_back(m.leaf[0]);
          // linear target, or -1 when any component lies outside its dimension.  (A rank-1 target is its own
          // linear index and the kernel compares every linear index with the target's size: nothing to add.)
          std::vector<std::string> tix(m.leaf.begin() + 1, m.leaf.end());
          if (tix.size() == 1) {
            r.leaf.push_back(tix[0]);
          } else {
            std::string inside = "true";
            for (size_t d = 0; d < tix.size(); ++d) inside += " && (u64)(" + tix[d] + ") < (u64)(" + outsh[d] + ")";
            r.leaf.push_back(g.def(I64, "(" + inside + ") ? " + g.to_index(outsh, tix) + " : (i64)-1"));
          }
          r.leaf.insert(r.leaf.end(), v.leaf.begin(), v.leaf.end());
          return r;
        });
        std::string S = b.ps.need_struct(pelemT);
        size_t nl = n.elt.nleaves();
        b.fns << "typedef " << S << " pelem_t;\n__device__ __forceinline__ " << E << " P_value(const pelem_t& e) { " << E << " r_;";
        for (size_t i = 0; i < nl; ++i) b.fns << " r_.l" << i << " = e.l" << (i + 2) << ";";
        b.fns << " return r_; }\n";
      }
      // how the update is applied
      std::vector<Ty> l = n.elt.leaves();
      std::string mode = "PERMUTE_LOCK";
      bool single = l.size() == 1;
      if (single && is_simple_prim(*n.f, &op, &opty)) {
        Ty t = l[0];
        bool w32 = ty_bytes[t] == 4, w64 = ty_bytes[t] == 8;
        if (op == P_ADD && (w32 || w64)) mode = "PERMUTE_ATOMIC_ADD";
        else if ((op == P_MIN || op == P_MAX) && ty_is_int(t) && (w32 || w64)) mode = op == P_MIN ? "PERMUTE_ATOMIC_MIN" : "PERMUTE_ATOMIC_MAX";
        else if ((op == P_BAND || op == P_BOR || op == P_BXOR) && (w32 || w64))
          mode = op == P_BAND ? "PERMUTE_ATOMIC_AND" : (op == P_BOR ? "PERMUTE_ATOMIC_OR" : "PERMUTE_ATOMIC_XOR");
        else if (w32 || w64) mode = "PERMUTE_CAS";
      } else if (single && (ty_bytes[l[0]] == 4 || ty_bytes[l[0]] == 8)) {
        // `permute const`: the new value replaces the old one
        const Expr& body = *n.f->body;
        if (var_is(body, n.f->params[0])) mode = "PERMUTE_STORE";
        else mode = "PERMUTE_CAS";
      } else {
        const Expr& body = *n.f->body;
        if (var_is(body, n.f->params[0])) mode = "PERMUTE_STORE";
      }
      def["PERMUTE_MODE"] = mode;
      if (single) {
        def["PERMUTE_T"] = cty(l[0]);
        def["PERMUTE_BYTES"] = std::to_string(ty_bytes[l[0]]);
        def["PERMUTE_SIGNED"] = ty_is_signed(l[0]) ? "1" : "0";
        def["PERMUTE_FLOAT"] = ty_is_float(l[0]) ? "1" : "0";
      }
      break;
    }
    case N_STENCIL: case N_STENCIL2: {
      size_t nin = n.d.size();
      int rank = n.d[0].rank;
      if (rank < 1 || rank > 3) throw Error(B200_ERR_UNSUPPORTED, "stencil: only rank 1 to 3 arrays are supported");
      def["ST_NIN"] = std::to_string(nin);
      def["ST_RANK"] = std::to_string(rank);
      std::ostringstream smem, fill;
      for (size_t a = 0; a < nin; ++a) {
        const std::string A = std::to_string(a);
        b.delayed("D" + A, *n.d[a].index, rank, n.d[a].elt);
        std::string S = b.ps.need_struct(n.d[a].elt);
        // radii, padded to three dimensions (outermost first)
        for (int d = 0; d < 3; ++d) {
          int src = d - (3 - rank);
          def["ST_R" + A + "_" + std::to_string(d)] = std::to_string(src >= 0 ? n.st_extent[a][src] / 2 : 0);
        }
        // bounded access (Interpreter.hs:797-839): g0..g2 are padded coordinates
        std::ostringstream f;
        const int off = 3 - rank;
        std::string dims[3], gs[3];
        for (int d = 0; d < rank; ++d) {
          dims[d] = "p.D" + A + "_e" + std::to_string(d);
          gs[d] = "g" + std::to_string(d + off);
        }
        f << "__device__ __forceinline__ " << S << " ST_bounded" << A << "(const Params& p, i64 g0, i64 g1, i64 g2) {\n  (void)g0; (void)g1; (void)g2;\n";
        f << "  bool inside = true;\n";
        for (int d = 0; d < rank; ++d) f << "  inside = inside && " << gs[d] << " >= 0 && " << gs[d] << " < " << dims[d] << ";\n";
        std::string args;
        for (int d = 0; d < rank; ++d) args += ", " + gs[d];
        f << "  if (inside) return D" << A << "_at_ix(p" << args << ");\n";
        const BoundarySpec& bs = n.bnd[a];
        if (bs.kind == BND_CONSTANT) {
          Gen g(b.ps, b.tmp);
          CVal v = g.gen(*bs.value);
          f << g.out.str() << b.ret_struct(S, v);
        } else if (bs.kind == BND_FUNCTION) {
          Gen g(b.ps, b.tmp);
          CVal ixv;
          ixv.ty = Type::shape(rank);
          for (int d = 0; d < rank; ++d) ixv.leaf.push_back(gs[d]);
          g.env.emplace_back(bs.fun->params[0], ixv);
          CVal v = g.gen(*bs.fun->body);
          f << g.out.str() << b.ret_struct(S, v);
        } else {
          std::string bargs;
          for (int d = 0; d < rank; ++d) {
            const std::string& i = gs[d];
            const std::string& sz = dims[d];
            std::string lo, hi;
            if (bs.kind == BND_CLAMP) { lo = "(i64)0"; hi = sz + " - 1"; }
            else if (bs.kind == BND_MIRROR) { lo = "-" + i; hi = sz + " - (" + i + " - " + sz + " + 2)"; }
            else { lo = sz + " + " + i; hi = i + " - " + sz; }
            // the final min/max only matters when the extent is smaller than the halo (the reference
            // raises an index error there); it keeps the access inside the array
            f << "  i64 b" << d << " = " << i << " < 0 ? " << lo << " : (" << i << " >= " << sz << " ? " << hi << " : " << i << ");\n"
              << "  b" << d << " = b" << d << " < 0 ? (i64)0 : (b" << d << " >= " << sz << " ? " << sz << " - 1 : b" << d << ");\n";
            bargs += ", b" + std::to_string(d);
          }
          f << "  return D" << A << "_at_ix(p" << bargs << ");\n";
        }
        f << "}\n";
        b.fns << f.str();
        std::vector<Ty> l = n.d[a].elt.leaves();
        for (size_t i = 0; i < l.size(); ++i) smem << "__shared__ " << cty(l[i]) << " sm" << A << "_l" << i << "[ST_TILE_ELEMS" << A << "];\n";
        fill << "__device__ __forceinline__ void ST_fill" << A << "(const Params& p, int pos, i64 g0, i64 g1, i64 g2) {\n  const " << S
             << " v = ST_bounded" << A << "(p, g0, g1, g2);\n";
        for (size_t i = 0; i < l.size(); ++i) fill << "  sm" << A << "_l" << i << "[pos] = v.l" << i << ";\n";
        fill << "}\n";
      }
      // The stencil function over taps named ST_TAP(input, leaf, d0, d1, d2); the skeleton decides
      // where taps live (a shared-memory tile, or per-thread register windows for rank 2).
      {
        Gen g(b.ps, b.tmp);
        for (size_t a = 0; a < nin; ++a) {
          CVal taps;
          taps.ty = n.f->param_ty[a];
          size_t nl = n.d[a].elt.nleaves();
          const auto& ext = n.st_extent[a];
          // enumerate offsets in tuple order: outermost dimension outermost, -r..+r
          std::vector<int> idx(rank, 0);
          for (;;) {
            int off3[3] = {0, 0, 0};
            for (int d = 0; d < rank; ++d) off3[d + 3 - rank] = idx[d] - ext[d] / 2;
            for (size_t i = 0; i < nl; ++i) {
              std::ostringstream t;
              t << "ST_TAP(" << a << ", " << i << ", " << off3[0] << ", " << off3[1] << ", " << off3[2] << ")";
              taps.leaf.push_back(t.str());
            }
            int d = rank - 1;
            while (d >= 0 && ++idx[d] == ext[d]) { idx[d] = 0; --d; }
            if (d < 0) break;
          }
          g.env.emplace_back(n.f->params[a], taps);
        }
        CVal r = g.gen(*n.f->body);
        b.fns << "#if ST_REG\n";
        if (rank == 2) {
          // register-window variant: each thread owns four neighbouring columns and keeps ST_H rows
          int rymax = 0;
          for (size_t a = 0; a < nin; ++a) rymax = std::max(rymax, n.st_extent[a][0] / 2);
          def["ST_RYMAX"] = std::to_string(rymax);
          def["ST_H"] = std::to_string(2 * rymax + 1);
          std::string win_decl, win_params, win_args, issue_all, commit_all, lane_fast, issue_fast, all_fast, min_e0;
          // shared-memory staging of input rows (acc_stencil2d_bulk): every input must be read through streams
          // whose leaves are at least 4 bytes wide (a row segment then starts on a 16-byte boundary)
          std::string take_all, bulk_all, stage_off = "0";
          bool bulk_ok = true;
          for (size_t a = 0; a < nin; ++a) {
            const std::string A = std::to_string(a);
            const int rx = n.st_extent[a][1] / 2;
            def["ST_W" + A] = std::to_string(4 + 2 * rx);
            const std::string S = b.ps.need_struct(n.d[a].elt);
            std::vector<Ty> l = n.d[a].elt.leaves();
            std::string wp, wa;
            for (size_t i = 0; i < l.size(); ++i) {
              const std::string w = "w" + A + "_l" + std::to_string(i);
              win_decl += cty(l[i]) + " " + w + "[ST_HW][ST_W" + A + "]; ";
              win_params += std::string(win_params.empty() ? "" : ", ") + "const " + cty(l[i]) + " (&" + w + ")[ST_HW][ST_W" + A + "]";
              win_args += std::string(win_args.empty() ? "" : ", ") + w;
              wp += ", " + cty(l[i]) + " (&" + w + ")[ST_HW][ST_W" + A + "]";
              wa += ", " + w;
            }
            issue_all += "ST2_issue" + A + "<SLOT>(p, GY, gx0, lf" + A + wa + "); ";
            issue_fast += "ST2_issue_fast" + A + "<SLOT>(p, GY, gx0" + wa + "); ";
            all_fast += std::string(all_fast.empty() ? "" : " && ") + "lf" + A;
            min_e0 = min_e0.empty() ? "(int)p.D" + A + "_e0" : "min(" + min_e0 + ", (int)p.D" + A + "_e0)";
            lane_fast += "const bool lf" + A + " = p.D" + A + "_fast != 0 && (p.D" + A + "_e1 & 3) == 0 && gx0 >= 0 && gx0 + 4 <= (int)p.D" + A + "_e1; ";
            commit_all += "ST2_commit" + A + "<SLOT>(lane" + wa + "); ";
            // which input row supplies global row gy (or -1: evaluate element by element)
            const std::string e0 = "p.D" + A + "_e0", e1 = "p.D" + A + "_e1";
            std::string rowmap;   // in terms of the 32-bit locals gy, e0
            switch (n.bnd[a].kind) {
              case BND_CLAMP: rowmap = "gy < 0 ? 0 : (gy >= e0 ? e0 - 1 : gy)"; break;
              case BND_MIRROR: rowmap = "gy < 0 ? -gy : (gy >= e0 ? e0 - (gy - e0 + 2) : gy)"; break;
              case BND_WRAP: rowmap = "gy < 0 ? e0 + gy : (gy >= e0 ? gy - e0 : gy)"; break;
              default: rowmap = "(gy >= 0 && gy < e0) ? gy : -1"; break;
            }
            // Request a row straight into window slot SLOT (the thread's own four columns).  The
            // commit step, run just before the row is first used, takes the rx columns to either
            // side from the neighbouring lanes.
            b.fns << "template <int SLOT> __device__ __forceinline__ void ST2_issue" << A << "(const Params& p, int gy, int gx0, bool lane_fast" << wp << ") {\n"
                  << "  " << S << " own[4];\n"
                  << "  const int e0 = (int)" << e0 << ", e1 = (int)" << e1 << ";\n"
                  << "  int my = " << rowmap << ";\n  if (my >= e0) my = -1;\n"
                  << "  if (lane_fast && my >= 0) D" << A << "_get4_lin(p, (i64)my * (i64)e1 + (i64)gx0, my, gx0, own);\n"
                  << "  else { _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) own[k] = ST_bounded" << A << "(p, 0, gy, gx0 + k); }\n";
            for (size_t i = 0; i < l.size(); ++i)
              b.fns << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) w" << A << "_l" << i << "[SLOT][" << rx << " + k] = own[k].l" << i << ";\n";
            b.fns << "}\n";
            // the same for a row known to be inside the array, read by a lane on the vector path
            b.fns << "template <int SLOT> __device__ __forceinline__ void ST2_issue_fast" << A << "(const Params& p, int gy, int gx0" << wp << ") {\n"
                  << "  " << S << " own[4];\n"
                  << "  D" << A << "_get4_lin(p, (i64)gy * (i64)(int)" << e1 << " + (i64)gx0, gy, gx0, own);\n";
            for (size_t i = 0; i < l.size(); ++i)
              b.fns << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) w" << A << "_l" << i << "[SLOT][" << rx << " + k] = own[k].l" << i << ";\n";
            b.fns << "}\n";
            size_t min_leaf = 16;
            for (auto& sn : b.glue.streams[a])
              for (Ty t : b.ps.array(sn).elt.leaves()) min_leaf = std::min(min_leaf, (size_t)ty_bytes[t]);
            if (def.count("D" + A + "_STREAM_NLEAVES") && min_leaf >= 4) {
              // the same row out of its staged copy: `seg` points at this input's part of the row slot
              b.fns << "#if defined(ST2_BULK) && ST2_BULK\n"
                    << "template <int SLOT> __device__ __forceinline__ void ST2_take" << A << "(const Params& p, const unsigned char* seg, int gy, int gx0, int lane" << wp << ") {\n"
                    << "  " << S << " own[4];\n"
                    << "  D" << A << "_get4_sm(p, gy, gx0, seg, lane * 4, own);\n";
              for (size_t i = 0; i < l.size(); ++i)
                b.fns << "  _Pragma(\"unroll\") for (int k = 0; k < 4; ++k) w" << A << "_l" << i << "[SLOT][" << rx << " + k] = own[k].l" << i << ";\n";
              b.fns << "}\n#endif\n";
              take_all += "ST2_take" + A + "<SLOT>(p, (ROWBASE) + (" + stage_off + "), GY, gx0, lane" + wa + "); ";
              bulk_all += "D" + A + "_BULK_ISSUE((ROWBASE) + (" + stage_off + "), BAR, (i64)(GY) * (i64)(int)" + e1 + " + (i64)(GX0)) ";
              stage_off += " + D" + A + "_STAGE_BYTES";
            } else {
              bulk_ok = false;
            }
            b.fns << "template <int SLOT> __device__ __forceinline__ void ST2_commit" << A << "(int lane" << wp << ") {\n  (void)lane;\n";
            for (int j = 1; j <= rx; ++j) {
              for (size_t i = 0; i < l.size(); ++i) {
                const std::string w = "w" + A + "_l" + std::to_string(i);
                b.fns << "  " << w << "[SLOT][" << (rx - j) << "] = acc_shfl1_up(" << w << "[SLOT][" << (rx + 4 - j) << "], 1);\n"
                      << "  " << w << "[SLOT][" << (rx + 3 + j) << "] = acc_shfl1_down(" << w << "[SLOT][" << (rx + j - 1) << "], 1);\n";
              }
            }
            b.fns << "}\n";
          }
          def["ST2_WIN_DECL"] = win_decl;
          def["ST2_WIN_PARAMS"] = win_params;
          def["ST2_WIN_ARGS"] = win_args;
          def["ST2_ISSUE_ALL(SLOT, GY)"] = issue_all;
          def["ST2_COMMIT_ALL(SLOT)"] = commit_all;
          def["ST2_LANE_FAST_DECL"] = lane_fast;
          def["ST2_ISSUE_ALL_FAST(SLOT, GY)"] = issue_fast;
          def["ST2_ALL_LANE_FAST"] = "(" + all_fast + ")";
          def["ST2_MIN_E0"] = "(" + min_e0 + ")";
          def["ST2_BULK_OK"] = bulk_ok ? "1" : "0";
          if (bulk_ok) {
            def["ST2_TAKE_ALL(SLOT, ROWBASE, GY)"] = take_all;
            def["ST2_BULK_ISSUE_ALL(ROWBASE, BAR, GY, GX0)"] = bulk_all;
            def["ST2_STAGE_BYTES"] = "(" + stage_off + ")";
          }
          b.fns << "template <int K, int PH> __device__ __forceinline__ " << E << " ST2_apply(const Params& p, ST2_WIN_PARAMS) {\n" << g.out.str()
                << b.ret_struct(E, r) << "}\n";
        }
        b.fns << "#else\n" << smem.str() << fill.str();
        b.fns << "__device__ __forceinline__ " << E << " ST_apply(const Params& p, int l0, int l1, int l2) {\n" << g.out.str()
              << b.ret_struct(E, r) << "}\n#endif\n";
      }
      b.output(0, n.elt);
      break;
    }
    default:
      throw Error(B200_ERR_UNSUPPORTED, "this node has no kernel");      // reshape and the host-evaluated nodes
  }
  def["elt_t"] = E;
  switch (n.kind) {
    case N_GENERATE: named = {"n", "vec"}; break;
    case N_FOLD: named = {"n", "rows", "row", "vec", "scratch", "flags", "counter"}; break;
    case N_FOLDSEG: named = {"segs", "rows", "vec", "err"}; break;
    case N_SCAN: case N_SCAN2:
      named = {"n", "rows", "tiles_per_row", "total_tiles", "batches_per_row", "total_batches", "in_vec", "out_vec", "status", "agg", "incl", "gstatus", "groups_per_row", "counter", "epoch", "err", "spin_limit"};
      break;
    case N_PERMUTE: named = {"n", "vec", "out_n", "priv", "priv16", "choice", "locks", "err", "spin_limit"}; break;
    case N_STENCIL: case N_STENCIL2: named = {"o0", "o1", "o2", "row0", "row1", "tiles1", "tiles2", "vec", "?fr_strips", "?fr_r0", "?fr_r1", "?strip0", "?err", "?spin_limit", "?row2", "?row3"}; break;
    default: break;
  }
  for (auto& nm : named) b.ps.use_named(nm);
  Glue g = b.finish();
  return g;
}

}  // namespace accb200
