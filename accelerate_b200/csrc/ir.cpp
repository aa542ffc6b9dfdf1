// Parser and type checker for the backend's program text (see ir.hpp).
#include "ir.hpp"

#include <cstdlib>
#include <functional>
#include <cstring>

namespace accb200 {

const char* const ty_name[NTY] = {"i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f32", "f64", "f16"};
const int ty_bytes[NTY] = {1, 2, 4, 8, 1, 2, 4, 8, 4, 8, 2};
const char* const prim_name[P_NPRIMS] = {
    "add", "sub", "mul", "neg", "abs", "sig", "quot", "rem", "quotrem", "idiv", "mod", "divmod",
    "band", "bor", "bxor", "bnot", "shl", "shr", "rotl", "rotr", "popcount", "clz", "ctz",
    "fdiv", "recip", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh",
    "asinh", "acosh", "atanh", "exp", "sqrt", "log", "fpow", "logbase", "atan2",
    "truncate", "round", "floor", "ceiling", "isnan", "isinf",
    "lt", "gt", "le", "ge", "eq", "ne", "max", "min", "land", "lor", "lnot",
    "fromintegral", "tofloating"};

// ---- S-expression reader ------------------------------------------------------
namespace {
struct Reader {
  const char* p;
  const char* e;
  void skip() {
    for (;;) {
      while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
      if (p < e && *p == ';') { while (p < e && *p != '\n') ++p; continue; }
      break;
    }
  }
  Sx read() {
    skip();
    if (p >= e) throw Error(B200_ERR_PARSE, "program text ends inside a form");
    Sx r;
    if (*p == '(') {
      ++p;
      for (;;) {
        skip();
        if (p >= e) throw Error(B200_ERR_PARSE, "program text: unbalanced '('");
        if (*p == ')') { ++p; return r; }
        r.k.push_back(read());
      }
    }
    if (*p == ')') throw Error(B200_ERR_PARSE, "program text: stray ')'");
    r.atom = true;
    const char* b = p;
    while (p < e && !strchr("() \n\t\r", *p)) ++p;
    r.s.assign(b, p);
    return r;
  }
};
}  // namespace

Sx parse_sexp(const char* text, size_t len) {
  Reader r{text, text + len};
  Sx x = r.read();
  r.skip();
  if (r.p != r.e) throw Error(B200_ERR_PARSE, "program text: trailing input after the top-level form");
  return x;
}

// ---- types ---------------------------------------------------------------------
Ty parse_ty(const std::string& s) {
  if (s == "bool") return U8;
  if (s == "int") return I64;
  if (s == "word") return U64;
  for (int i = 0; i < NTY; ++i)
    if (s == ty_name[i]) return (Ty)i;
  throw Error(B200_ERR_TYPE, "unknown scalar type '" + s + "'");
}
bool Type::operator==(const Type& o) const {
  if (tuple != o.tuple) return false;
  if (!tuple) return s == o.s;
  if (e.size() != o.e.size()) return false;
  for (size_t i = 0; i < e.size(); ++i)
    if (!(e[i] == o.e[i])) return false;
  return true;
}
void Type::flatten(std::vector<Ty>& out) const {
  if (!tuple) { out.push_back(s); return; }
  for (auto& c : e) c.flatten(out);
}
std::string Type::str() const {
  if (!tuple) return ty_name[s];
  if (vec && !e.empty()) return "(vec " + std::to_string(e.size()) + " " + e[0].str() + ")";
  std::string r = "(tup";
  for (auto& c : e) r += " " + c.str();
  return r + ")";
}
bool Type::is_shape() const {
  if (!tuple) return false;
  for (auto& c : e)
    if (c.tuple || c.s != I64) return false;
  return true;
}
Type parse_type(const Sx& x) {
  if (x.atom) return Type::scalar(parse_ty(x.s));
  if (x.head() == "vec") {
    // (vec N T), N in 2, 3, 4, 8, 16 (Type.hs:140-152; VecElt instances, Sugar/Vec.hs)
    const int n = atoi(x.at(1).s.c_str());
    if (!x.at(2).atom || !(n == 2 || n == 3 || n == 4 || n == 8 || n == 16)) throw Error(B200_ERR_TYPE, "expected (vec 2|3|4|8|16 scalar)");
    Type r = Type::tup(std::vector<Type>((size_t)n, Type::scalar(parse_ty(x.at(2).s))));
    r.vec = true;
    return r;
  }
  std::vector<Type> xs;
  size_t b = x.head() == "tup" ? 1 : 0;
  for (size_t i = b; i < x.size(); ++i) xs.push_back(parse_type(x.k[i]));
  return Type::tup(std::move(xs));
}

// ---- expressions -----------------------------------------------------------------
namespace {

struct TEnv {
  std::vector<std::pair<std::string, Type>> vars;
  const std::map<std::string, ArrayInfo>* arrays;
  const Type& lookup(const std::string& n) const {
    for (size_t i = vars.size(); i-- > 0;)
      if (vars[i].first == n) return vars[i].second;
    throw Error(B200_ERR_TYPE, "unbound scalar variable '" + n + "'");
  }
  const ArrayInfo& array(const std::string& n) const {
    auto it = arrays->find(n);
    if (it == arrays->end()) throw Error(B200_ERR_TYPE, "unbound array variable '" + n + "'");
    return it->second;
  }
};

std::unique_ptr<Expr> parse_expr(const Sx& x, TEnv& env);

std::unique_ptr<Fun> parse_fun(const Sx& x, TEnv& env) {
  if (x.head() != "lam") throw Error(B200_ERR_PARSE, "expected (lam ((name type) ...) body)");
  auto f = std::make_unique<Fun>();
  size_t mark = env.vars.size();
  for (auto& p : x.at(1).k) {
    if (p.atom || p.size() != 2) throw Error(B200_ERR_PARSE, "lambda parameters must be written (name type)");
    f->params.push_back(p.k[0].s);
    f->param_ty.push_back(parse_type(p.k[1]));
    env.vars.emplace_back(f->params.back(), f->param_ty.back());
  }
  f->body = parse_expr(x.at(2), env);
  env.vars.resize(mark);
  return f;
}

void want_scalar(const Expr& e, Ty t, const char* what) {
  if (e.ty.tuple || e.ty.s != t)
    throw Error(B200_ERR_TYPE, std::string(what) + ": expected " + ty_name[t] + ", found " + e.ty.str());
}

Type prim_result(Prim op, Ty t1, Ty t2) {
  switch (op) {
    case P_QUOTREM: case P_DIVMOD: return Type::tup({Type::scalar(t1), Type::scalar(t1)});
    case P_POPCNT: case P_CLZ: case P_CTZ: return Type::scalar(I64);
    case P_TRUNCATE: case P_ROUND: case P_FLOOR: case P_CEILING: case P_FROMINTEGRAL: case P_TOFLOATING:
      return Type::scalar(t2);
    case P_ISNAN: case P_ISINF: case P_LT: case P_GT: case P_LE: case P_GE: case P_EQ: case P_NE:
    case P_LAND: case P_LOR: case P_LNOT:
      return Type::scalar(U8);
    default: return Type::scalar(t1);
  }
}
int prim_arity(Prim op) {
  switch (op) {
    case P_NEG: case P_ABS: case P_SIG: case P_BNOT: case P_POPCNT: case P_CLZ: case P_CTZ: case P_RECIP:
    case P_SIN: case P_COS: case P_TAN: case P_ASIN: case P_ACOS: case P_ATAN: case P_SINH: case P_COSH:
    case P_TANH: case P_ASINH: case P_ACOSH: case P_ATANH: case P_EXP: case P_SQRT: case P_LOG:
    case P_TRUNCATE: case P_ROUND: case P_FLOOR: case P_CEILING: case P_ISNAN: case P_ISINF: case P_LNOT:
    case P_FROMINTEGRAL: case P_TOFLOATING:
      return 1;
    default: return 2;
  }
}

std::unique_ptr<Expr> parse_expr(const Sx& x, TEnv& env) {
  if (x.atom) throw Error(B200_ERR_PARSE, "expression must be a list, found atom '" + x.s + "'");
  auto e = std::make_unique<Expr>();
  const std::string h = x.head();
  auto sub = [&](size_t i) -> Expr& {
    e->a.push_back(parse_expr(x.at(i), env));
    return *e->a.back();
  };
  if (h == "vecpack" || h == "vecunpack") {
    // VecPack / VecUnpack (AST.hs:566-573; Interpreter.hs:951-952): (vecpack N T e) takes the tuple of N
    // components to the vector, (vecunpack N T e) back.  Both are the identity on what the kernels hold.
    Sx vt;
    vt.k.resize(3);
    vt.k[0].atom = true;
    vt.k[0].s = "vec";
    vt.k[1] = x.at(1);
    vt.k[2] = x.at(2);
    const Type v = parse_type(vt);
    e = parse_expr(x.at(3), env);
    if (e->ty != v) throw Error(B200_ERR_TYPE, h + ": operand is " + e->ty.str() + ", expected the components of " + v.str());
    e->ty.vec = h == "vecpack";
    return e;
  }
  if (h == "const") {
    e->kind = X_CONST;
    e->ty = Type::scalar(parse_ty(x.at(1).s));
    e->lit = x.at(2).s;
  } else if (h == "minbound" || h == "maxbound" || h == "pi") {
    // PrimConst (AST.hs:649-658) folded to a literal
    e->kind = X_CONST;
    Ty t = parse_ty(x.at(1).s);
    e->ty = Type::scalar(t);
    if (h == "pi") {
      if (!ty_is_float(t)) throw Error(B200_ERR_TYPE, "pi needs a floating type");
      e->lit = t == F16 ? "0x1.92p+1" : (t == F32 ? "0x1.921fb6p+1" : "0x1.921fb54442d18p+1");
    } else {
      if (!ty_is_int(t)) throw Error(B200_ERR_TYPE, h + " needs an integral type");
      int b = ty_bits(t);
      if (h == "minbound") e->lit = ty_is_signed(t) ? std::to_string(-(long long)(((unsigned long long)1 << (b - 1)) - 1) - 1) : "0";
      else e->lit = ty_is_signed(t) ? std::to_string((((unsigned long long)1 << (b - 1)) - 1))
                                    : std::to_string(b == 64 ? ~0ull : (((unsigned long long)1 << b) - 1));
    }
  } else if (h == "var") {
    e->kind = X_VAR;
    e->name = x.at(1).s;
    e->ty = env.lookup(e->name);
  } else if (h == "let") {
    e->kind = X_LET;
    e->name = x.at(1).s;
    Expr& v = sub(2);
    env.vars.emplace_back(e->name, v.ty);
    e->ty = sub(3).ty;
    env.vars.pop_back();
  } else if (h == "tup") {
    e->kind = X_TUP;
    std::vector<Type> ts;
    for (size_t i = 1; i < x.size(); ++i) ts.push_back(sub(i).ty);
    e->ty = Type::tup(std::move(ts));
  } else if (h == "snoc") {
    // Pair as the reference builds tuples (snoc lists, AST.hs:536-540): (snoc l r) appends r as one
    // more component to the tuple l; (tup) is Nil.  (((), a), b) thus becomes the flat tuple (a, b).
    e->kind = X_SNOC;
    Expr& l = sub(1);
    Expr& r = sub(2);
    if (!l.ty.tuple) throw Error(B200_ERR_TYPE, "snoc: left operand is not a tuple");
    std::vector<Type> ts = l.ty.e;
    ts.push_back(r.ty);
    e->ty = Type::tup(std::move(ts));
  } else if (h == "last") {
    // the final component of a tuple (the right part of a pair pattern)
    e->kind = X_PRJ;
    Expr& v = sub(1);
    if (!v.ty.tuple || v.ty.e.empty()) throw Error(B200_ERR_TYPE, "last of a non-tuple or empty tuple");
    e->n = (int)v.ty.e.size() - 1;
    e->ty = v.ty.e.back();
  } else if (h == "init") {
    // all components but the last (the left part of a pair pattern)
    e->kind = X_INIT;
    Expr& v = sub(1);
    if (!v.ty.tuple || v.ty.e.empty()) throw Error(B200_ERR_TYPE, "init of a non-tuple or empty tuple");
    e->ty = Type::tup(std::vector<Type>(v.ty.e.begin(), v.ty.e.end() - 1));
  } else if (h == "prj") {
    e->kind = X_PRJ;
    e->n = atoi(x.at(1).s.c_str());
    Expr& v = sub(2);
    if (!v.ty.tuple || e->n < 0 || (size_t)e->n >= v.ty.e.size())
      throw Error(B200_ERR_TYPE, "prj " + std::to_string(e->n) + " of " + v.ty.str());
    e->ty = v.ty.e[e->n];
  } else if (h == "cond") {
    e->kind = X_COND;
    want_scalar(sub(1), U8, "cond predicate");
    Expr& t = sub(2);
    Expr& f = sub(3);
    if (t.ty != f.ty) throw Error(B200_ERR_TYPE, "cond branches differ: " + t.ty.str() + " vs " + f.ty.str());
    e->ty = t.ty;
  } else if (h == "while") {
    e->kind = X_WHILE;
    e->f.push_back(parse_fun(x.at(1), env));
    e->f.push_back(parse_fun(x.at(2), env));
    Expr& s = sub(3);
    if (e->f[0]->param_ty.size() != 1 || e->f[0]->param_ty[0] != s.ty || e->f[1]->param_ty.size() != 1 ||
        e->f[1]->param_ty[0] != s.ty || e->f[1]->result() != s.ty)
      throw Error(B200_ERR_TYPE, "while: predicate/body/seed types disagree");
    want_scalar(*e->f[0]->body, U8, "while predicate");
    e->ty = s.ty;
  } else if (h == "prim") {
    e->kind = X_PRIM;
    int o = -1;
    for (int i = 0; i < P_NPRIMS; ++i)
      if (x.at(1).s == prim_name[i]) { o = i; break; }
    if (o < 0) throw Error(B200_ERR_TYPE, "unknown primitive '" + x.at(1).s + "'");
    e->op = (Prim)o;
    size_t argi = 3;
    bool two = (o == P_TRUNCATE || o == P_ROUND || o == P_FLOOR || o == P_CEILING || o == P_FROMINTEGRAL || o == P_TOFLOATING);
    if (o == P_LAND || o == P_LOR || o == P_LNOT) {
      e->t1 = U8;
      argi = (x.size() > 2 && x.k[2].atom) ? 3 : 2;
    } else {
      e->t1 = parse_ty(x.at(2).s);
    }
    if (two) { e->t2 = parse_ty(x.at(3).s); argi = 4; }
    for (size_t i = argi; i < x.size(); ++i) sub(i);
    // a binary primitive may be applied to one pair (PrimApp f (Pair a b), AST.hs:560)
    int ar = prim_arity(e->op);
    if (ar == 2 && e->a.size() == 1 && e->a[0]->ty.tuple && e->a[0]->ty.e.size() == 2) {
      /* accepted; code generation projects the components */
    } else if ((int)e->a.size() != ar) {
      throw Error(B200_ERR_TYPE, std::string("primitive ") + prim_name[o] + ": wrong number of arguments");
    } else {
      for (int i = 0; i < ar; ++i) {
        Ty want = e->t1;
        if (i == 1 && (o == P_SHL || o == P_SHR || o == P_ROTL || o == P_ROTR)) want = I64;
        want_scalar(*e->a[i], want, prim_name[o]);
      }
    }
    e->ty = prim_result(e->op, e->t1, e->t2);
  } else if (h == "index" || h == "lindex") {
    e->kind = h == "index" ? X_INDEX : X_LINDEX;
    e->name = x.at(1).s;
    const ArrayInfo& ai = env.array(e->name);
    Expr& ix = sub(2);
    if (e->kind == X_INDEX) {
      if (!ix.ty.is_shape() || (int)ix.ty.e.size() != ai.rank)
        throw Error(B200_ERR_TYPE, "index into rank-" + std::to_string(ai.rank) + " array '" + e->name + "' with " + ix.ty.str());
    } else {
      want_scalar(ix, I64, "linear index");
    }
    e->ty = ai.elt;
  } else if (h == "shape") {
    e->kind = X_SHAPE;
    e->name = x.at(1).s;
    e->ty = Type::shape(env.array(e->name).rank);
  } else if (h == "shapesize") {
    e->kind = X_SHAPESIZE;
    if (!sub(1).ty.is_shape()) throw Error(B200_ERR_TYPE, "shapesize of a non-shape");
    e->ty = Type::scalar(I64);
  } else if (h == "toindex") {
    e->kind = X_TOINDEX;
    Expr& sh = sub(1);
    Expr& ix = sub(2);
    if (!sh.ty.is_shape() || sh.ty != ix.ty) throw Error(B200_ERR_TYPE, "toindex: shape/index mismatch");
    e->ty = Type::scalar(I64);
  } else if (h == "fromindex") {
    e->kind = X_FROMINDEX;
    Expr& sh = sub(1);
    if (!sh.ty.is_shape()) throw Error(B200_ERR_TYPE, "fromindex of a non-shape");
    want_scalar(sub(2), I64, "fromindex");
    e->ty = sh.ty;
  } else if (h == "coerce") {
    e->kind = X_COERCE;
    e->t1 = parse_ty(x.at(1).s);
    e->t2 = parse_ty(x.at(2).s);
    if (ty_bytes[e->t1] != ty_bytes[e->t2]) throw Error(B200_ERR_TYPE, "coerce between types of different size");
    want_scalar(sub(3), e->t1, "coerce");
    e->ty = Type::scalar(e->t2);
  } else if (h == "undef") {
    e->kind = X_UNDEF;
    e->ty = parse_type(x.at(1));
  } else if (h == "app") {
    e->kind = X_APP;
    e->f.push_back(parse_fun(x.at(1), env));
    for (size_t i = 2; i < x.size(); ++i) sub(i);
    if (e->a.size() != e->f[0]->params.size()) throw Error(B200_ERR_TYPE, "app: wrong number of arguments");
    for (size_t i = 0; i < e->a.size(); ++i)
      if (e->a[i]->ty != e->f[0]->param_ty[i]) throw Error(B200_ERR_TYPE, "app: argument type mismatch");
    e->ty = e->f[0]->result();
  } else if (h == "case") {
    e->kind = X_CASE;
    want_scalar(sub(1), U8, "case scrutinee");
    for (auto& alt : x.at(2).k) {
      e->tags.push_back(strtoll(alt.at(0).s.c_str(), nullptr, 10));
      e->a.push_back(parse_expr(alt.at(1), env));
    }
    if (x.size() > 3) { e->has_default = true; sub(3); }
    if (e->a.size() < 2) throw Error(B200_ERR_TYPE, "case without alternatives");
    e->ty = e->a[1]->ty;
    for (size_t i = 2; i < e->a.size(); ++i)
      if (e->a[i]->ty != e->ty) throw Error(B200_ERR_TYPE, "case alternatives differ in type");
  } else {
    throw Error(B200_ERR_PARSE, "unknown expression form '" + h + "'");
  }
  return e;
}

std::unique_ptr<Expr> make_var(const std::string& n, const Type& t) {
  auto e = std::make_unique<Expr>();
  e->kind = X_VAR;
  e->name = n;
  e->ty = t;
  return e;
}

DelayedOp parse_delayed(const Sx& x, TEnv& env) {
  DelayedOp d;
  if (x.head() == "manifest") {
    d.manifest = true;
    d.arr = x.at(1).s;
    const ArrayInfo& ai = env.array(d.arr);
    d.rank = ai.rank;
    d.elt = ai.elt;
    // a manifest operand is the delayed array (shape a, \ix -> a ! ix)  (Interp:183-192)
    d.extent = std::make_unique<Expr>();
    d.extent->kind = X_SHAPE;
    d.extent->name = d.arr;
    d.extent->ty = Type::shape(ai.rank);
    d.index = std::make_unique<Fun>();
    d.index->params.push_back("%ix");
    d.index->param_ty.push_back(Type::shape(ai.rank));
    auto body = std::make_unique<Expr>();
    body->kind = X_INDEX;
    body->name = d.arr;
    body->ty = ai.elt;
    body->a.push_back(make_var("%ix", Type::shape(ai.rank)));
    d.index->body = std::move(body);
  } else if (x.head() == "delayed") {
    d.extent = parse_expr(x.at(1), env);
    if (!d.extent->ty.is_shape()) throw Error(B200_ERR_TYPE, "delayed extent is not a shape");
    d.rank = (int)d.extent->ty.e.size();
    d.index = parse_fun(x.at(2), env);
    if (d.index->param_ty.size() != 1 || d.index->param_ty[0] != d.extent->ty)
      throw Error(B200_ERR_TYPE, "delayed index function does not take an index of the extent's rank");
    d.elt = d.index->result();
  } else {
    throw Error(B200_ERR_PARSE, "expected (manifest a) or (delayed extent fun)");
  }
  return d;
}

BoundarySpec parse_boundary(const Sx& x, TEnv& env, const DelayedOp& d) {
  BoundarySpec b;
  if (x.atom) {
    if (x.s == "clamp") b.kind = BND_CLAMP;
    else if (x.s == "mirror") b.kind = BND_MIRROR;
    else if (x.s == "wrap") b.kind = BND_WRAP;
    else throw Error(B200_ERR_PARSE, "unknown boundary '" + x.s + "'");
  } else if (x.head() == "constant") {
    b.kind = BND_CONSTANT;
    b.value = parse_expr(x.at(1), env);
    if (b.value->ty != d.elt) throw Error(B200_ERR_TYPE, "constant boundary has the wrong element type");
  } else if (x.head() == "function") {
    b.kind = BND_FUNCTION;
    b.fun = parse_fun(x.at(1), env);
    if (b.fun->param_ty.size() != 1 || b.fun->param_ty[0] != Type::shape(d.rank) || b.fun->result() != d.elt)
      throw Error(B200_ERR_TYPE, "boundary function has the wrong type");
  } else {
    throw Error(B200_ERR_PARSE, "malformed boundary");
  }
  return b;
}

std::vector<int> parse_stencilr(const Sx& x, int rank) {
  if (x.head() != "stencilr") throw Error(B200_ERR_PARSE, "expected (stencilr e0 e1 ...)");
  std::vector<int> r;
  for (size_t i = 1; i < x.size(); ++i) {
    int v = atoi(x.k[i].s.c_str());
    if (v != 3 && v != 5 && v != 7 && v != 9) throw Error(B200_ERR_TYPE, "stencil extents are 3, 5, 7 or 9 (Representation/Stencil.hs:34-70)");
    r.push_back(v);
  }
  if ((int)r.size() != rank) throw Error(B200_ERR_TYPE, "stencil pattern rank differs from the array's");
  return r;
}

Type stencil_arg_type(const std::vector<int>& ext, const Type& elt) {
  Type t = elt;
  for (size_t d = ext.size(); d-- > 0;) t = Type::tup(std::vector<Type>(ext[d], t));
  return t;
}

void check_binary(const Fun& f, const Type& elt, const char* what) {
  if (f.param_ty.size() != 2 || f.param_ty[0] != elt || f.param_ty[1] != elt || f.result() != elt)
    throw Error(B200_ERR_TYPE, std::string(what) + ": combination function is not elt -> elt -> elt for elt = " + elt.str());
}

std::string sx_text(const Sx& x) {
  if (x.atom) return x.s;
  std::string r = "(";
  for (size_t i = 0; i < x.size(); ++i) {
    if (i) r += " ";
    r += sx_text(x.k[i]);
  }
  return r + ")";
}

void parse_node(ProgramIR& p, std::vector<Node>& into, const Sx& bind, TEnv& env);

void define_array(ProgramIR& p, const std::string& name, const ArrayInfo& ai) {
  if (p.arrays.count(name)) throw Error(B200_ERR_PARSE, "array variable '" + name + "' is defined twice");
  p.arrays[name] = ai;
}

// (afun ((p (array R T)) ...) (let ..)* (out n ...))   or   (branch (let ..)* (out n ...))
Body parse_body(ProgramIR& p, const Sx& x, TEnv& env, bool with_params) {
  if (x.head() != (with_params ? "afun" : "branch")) throw Error(B200_ERR_PARSE, std::string("expected (") + (with_params ? "afun" : "branch") + " ...)");
  Body b;
  size_t i = 1;
  if (with_params) {
    const Sx& ps = x.at(1);
    for (auto& q : ps.k) {
      const Sx& at = q.at(1);
      if (at.head() != "array") throw Error(B200_ERR_PARSE, "expected (name (array rank elt)) in an array function");
      ArrayInfo ai;
      ai.rank = atoi(at.at(1).s.c_str());
      ai.elt = parse_type(at.at(2));
      define_array(p, q.at(0).s, ai);
      b.params.push_back(q.at(0).s);
      b.param_info.push_back(ai);
    }
    i = 2;
  }
  bool seen_out = false;
  for (; i < x.size(); ++i) {
    const Sx& f = x.k[i];
    if (f.head() == "let") {
      parse_node(p, b.nodes, f, env);
    } else if (f.head() == "out") {
      for (size_t j = 1; j < f.size(); ++j) {
        env.array(f.k[j].s);
        b.outs.push_back(f.k[j].s);
      }
      seen_out = true;
    } else {
      throw Error(B200_ERR_PARSE, "unknown form '" + f.head() + "' in an array function");
    }
  }
  if (!seen_out || b.outs.empty()) throw Error(B200_ERR_PARSE, "array function has no (out ...)");
  return b;
}

std::vector<ArrayInfo> body_result(const ProgramIR& p, const Body& b) {
  std::vector<ArrayInfo> r;
  for (auto& o : b.outs) r.push_back(p.arrays.at(o));
  return r;
}
bool same_arrays(const std::vector<ArrayInfo>& a, const std::vector<ArrayInfo>& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].rank != b[i].rank || a[i].elt != b[i].elt) return false;
  return true;
}

int hex_digit(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  throw Error(B200_ERR_PARSE, "bad hexadecimal digit in (use ...)");
}

void parse_node(ProgramIR& p, std::vector<Node>& into, const Sx& bind, TEnv& env) {
  const Sx& lhs = bind.at(1);
  const Sx& x = bind.at(2);
  Node n;
  n.id = p.n_nodes++;
  const std::string k = x.head();
  // (control nodes are not hashed into any kernel: their text, which may embed whole arrays, is not kept)
  if (k != "use" && k != "acond" && k != "awhile" && k != "apply" && k != "atrace") n.text = sx_text(x);
  auto is_operand = [](const Sx& s) { return s.head() == "manifest" || s.head() == "delayed"; };
  std::vector<ArrayInfo> outs;
  if (k == "generate") {
    n.kind = N_GENERATE;
    n.elt = parse_type(x.at(1));
    n.extent = parse_expr(x.at(2), env);
    if (!n.extent->ty.is_shape()) throw Error(B200_ERR_TYPE, "generate: extent is not a shape");
    n.f = parse_fun(x.at(3), env);
    if (n.f->param_ty.size() != 1 || n.f->param_ty[0] != n.extent->ty || n.f->result() != n.elt)
      throw Error(B200_ERR_TYPE, "generate: function type does not match extent/element type");
    outs.push_back({(int)n.extent->ty.e.size(), n.elt});
  } else if (k == "fold" || k == "foldseg" || k == "scanl" || k == "scanr" || k == "scanl'" || k == "scanr'") {
    n.elt = parse_type(x.at(1));
    n.f = parse_fun(x.at(2), env);
    check_binary(*n.f, n.elt, k.c_str());
    size_t i = 3;
    if (!is_operand(x.at(i))) {
      n.seed = parse_expr(x.at(i++), env);
      if (n.seed->ty != n.elt) throw Error(B200_ERR_TYPE, k + ": seed type differs from the element type");
    }
    n.d.push_back(parse_delayed(x.at(i++), env));
    if (n.d[0].elt != n.elt) throw Error(B200_ERR_TYPE, k + ": operand element type differs");
    if (n.d[0].rank < 1) throw Error(B200_ERR_TYPE, k + ": operand must have rank >= 1");
    int r = n.d[0].rank;
    if (k == "fold") {
      n.kind = N_FOLD;
      outs.push_back({r - 1, n.elt});
    } else if (k == "foldseg") {
      n.kind = N_FOLDSEG;
      n.d.push_back(parse_delayed(x.at(i++), env));
      if (n.d[1].rank != 1 || n.d[1].elt.tuple || !ty_is_int(n.d[1].elt.s))
        throw Error(B200_ERR_TYPE, "foldseg: segment descriptor must be a vector of an integral type");
      outs.push_back({r, n.elt});
    } else if (k == "scanl" || k == "scanr") {
      n.kind = N_SCAN;
      n.right = k == "scanr";
      outs.push_back({r, n.elt});
    } else {
      n.kind = N_SCAN2;
      n.right = k == "scanr'";
      if (!n.seed) throw Error(B200_ERR_TYPE, k + " needs a seed");
      outs.push_back({r, n.elt});
      outs.push_back({r - 1, n.elt});
    }
  } else if (k == "permute") {
    n.kind = N_PERMUTE;
    n.elt = parse_type(x.at(1));
    n.f = parse_fun(x.at(2), env);
    check_binary(*n.f, n.elt, "permute");
    n.arr = x.at(3).s;
    const ArrayInfo& def = env.array(n.arr);
    if (def.elt != n.elt) throw Error(B200_ERR_TYPE, "permute: defaults have a different element type");
    n.g = parse_fun(x.at(4), env);
    n.d.push_back(parse_delayed(x.at(5), env));
    if (n.d[0].elt != n.elt) throw Error(B200_ERR_TYPE, "permute: source element type differs");
    Type maybe = Type::tup({Type::scalar(U8), Type::shape(def.rank)});
    if (n.g->param_ty.size() != 1 || n.g->param_ty[0] != Type::shape(n.d[0].rank) || n.g->result() != maybe)
      throw Error(B200_ERR_TYPE, "permute: index function must map a source index to (tag, target index)");
    outs.push_back({def.rank, n.elt});
  } else if (k == "stencil") {
    n.kind = N_STENCIL;
    n.elt = parse_type(x.at(1));
    n.d.push_back(parse_delayed(x.at(5), env));
    n.st_extent.push_back(parse_stencilr(x.at(2), n.d[0].rank));
    n.f = parse_fun(x.at(3), env);
    n.bnd.push_back(parse_boundary(x.at(4), env, n.d[0]));
    if (n.f->param_ty.size() != 1 || n.f->param_ty[0] != stencil_arg_type(n.st_extent[0], n.d[0].elt) || n.f->result() != n.elt)
      throw Error(B200_ERR_TYPE, "stencil: function type does not match the pattern");
    outs.push_back({n.d[0].rank, n.elt});
  } else if (k == "stencil2") {
    n.kind = N_STENCIL2;
    n.elt = parse_type(x.at(1));
    n.d.push_back(parse_delayed(x.at(6), env));
    n.d.push_back(parse_delayed(x.at(8), env));
    if (n.d[0].rank != n.d[1].rank) throw Error(B200_ERR_TYPE, "stencil2: operand ranks differ");
    n.st_extent.push_back(parse_stencilr(x.at(2), n.d[0].rank));
    n.st_extent.push_back(parse_stencilr(x.at(3), n.d[1].rank));
    n.f = parse_fun(x.at(4), env);
    n.bnd.push_back(parse_boundary(x.at(5), env, n.d[0]));
    n.bnd.push_back(parse_boundary(x.at(7), env, n.d[1]));
    if (n.f->param_ty.size() != 2 || n.f->param_ty[0] != stencil_arg_type(n.st_extent[0], n.d[0].elt) ||
        n.f->param_ty[1] != stencil_arg_type(n.st_extent[1], n.d[1].elt) || n.f->result() != n.elt)
      throw Error(B200_ERR_TYPE, "stencil2: function type does not match the patterns");
    outs.push_back({n.d[0].rank, n.elt});
  } else if (k == "use") {
    // (use (array R ELT) (shape d0 ..) (hex LEAF0) (hex LEAF1) ...): Use, Interpreter.hs:231
    n.kind = N_USE;
    const Sx& at = x.at(1);
    if (at.head() != "array" || x.at(2).head() != "shape") throw Error(B200_ERR_PARSE, "expected (use (array rank elt) (shape ...) (hex ...)...)");
    const int rank = atoi(at.at(1).s.c_str());
    n.elt = parse_type(at.at(2));
    if ((int)x.at(2).size() - 1 != rank) throw Error(B200_ERR_TYPE, "use: shape does not have the declared rank");
    int64_t count = 1;
    for (int d = 0; d < rank; ++d) {
      n.use_shape.push_back(atoll(x.at(2).at(1 + d).s.c_str()));
      count = n.use_shape.back() <= 0 ? 0 : count * n.use_shape.back();
    }
    for (int64_t d : n.use_shape) if (d <= 0) count = 0;
    std::vector<Ty> leaves = n.elt.leaves();
    if (x.size() != 3 + leaves.size()) throw Error(B200_ERR_TYPE, "use: one (hex ...) per scalar leaf expected");
    for (size_t l = 0; l < leaves.size(); ++l) {
      const Sx& h = x.at(3 + l);
      if (h.head() != "hex") throw Error(B200_ERR_PARSE, "expected (hex DIGITS)");
      const std::string digits = h.size() > 1 ? h.at(1).s : std::string();
      const size_t bytes = (size_t)count * ty_bytes[leaves[l]];
      if (digits.size() != 2 * bytes) throw Error(B200_ERR_TYPE, "use: payload size does not match shape and element type");
      std::string raw(bytes, '\0');
      for (size_t i = 0; i < bytes; ++i) raw[i] = (char)(hex_digit(digits[2 * i]) * 16 + hex_digit(digits[2 * i + 1]));
      n.use_data.push_back(std::move(raw));
    }
    outs.push_back({rank, n.elt});
  } else if (k == "acond") {
    // (acond EXP (branch ...) (branch ...)): Acond, Interpreter.hs:217-219
    n.kind = N_ACOND;
    n.pred = parse_expr(x.at(1), env);
    if (n.pred->ty.tuple || n.pred->ty.s != U8) throw Error(B200_ERR_TYPE, "acond: the predicate is not a Bool");
    n.body.push_back(parse_body(p, x.at(2), env, false));
    n.body.push_back(parse_body(p, x.at(3), env, false));
    outs = body_result(p, n.body[0]);
    if (!same_arrays(outs, body_result(p, n.body[1]))) throw Error(B200_ERR_TYPE, "acond: the branches yield different arrays");
  } else if (k == "awhile") {
    // (awhile (afun (s..) .. (out c)) (afun (s..) .. (out s'..)) (args a..)): Awhile, Interpreter.hs:221-229
    n.kind = N_AWHILE;
    n.body.push_back(parse_body(p, x.at(1), env, true));
    n.body.push_back(parse_body(p, x.at(2), env, true));
    const Sx& as = x.at(3);
    if (as.head() != "args") throw Error(B200_ERR_PARSE, "expected (args ...)");
    for (size_t j = 1; j < as.size(); ++j) {
      n.args.push_back(as.k[j].s);
      outs.push_back(env.array(as.k[j].s));
    }
    std::vector<ArrayInfo> c = body_result(p, n.body[0]);
    if (c.size() != 1 || c[0].rank != 0 || c[0].elt.tuple || c[0].elt.s != U8) throw Error(B200_ERR_TYPE, "awhile: the condition must yield a Scalar Bool");
    if (!same_arrays(outs, n.body[0].param_info) || !same_arrays(outs, n.body[1].param_info) || !same_arrays(outs, body_result(p, n.body[1])))
      throw Error(B200_ERR_TYPE, "awhile: condition, step and initial value disagree on the type of the state");
  } else if (k == "apply") {
    // (apply (afun (x..) .. (out r..)) (args a..)): Apply, Interpreter.hs:215
    n.kind = N_APPLY;
    n.body.push_back(parse_body(p, x.at(1), env, true));
    const Sx& as = x.at(2);
    if (as.head() != "args") throw Error(B200_ERR_PARSE, "expected (args ...)");
    std::vector<ArrayInfo> given;
    for (size_t j = 1; j < as.size(); ++j) {
      n.args.push_back(as.k[j].s);
      given.push_back(env.array(as.k[j].s));
    }
    if (!same_arrays(given, n.body[0].param_info)) throw Error(B200_ERR_TYPE, "apply: arguments do not match the function's parameters");
    outs = body_result(p, n.body[0]);
  } else if (k == "atrace") {
    // (atrace (hex MESSAGE) (show a..) (args b..)): Atrace, Interpreter.hs:215 -- print the message and the
    // arrays a.., hand the arrays b.. on unchanged
    n.kind = N_ATRACE;
    const Sx& h = x.at(1);
    if (h.head() != "hex" || x.at(2).head() != "show" || x.at(3).head() != "args") throw Error(B200_ERR_PARSE, "expected (atrace (hex ..) (show ..) (args ..))");
    const std::string digits = h.size() > 1 ? h.at(1).s : std::string();
    if (digits.size() % 2) throw Error(B200_ERR_PARSE, "atrace: odd number of hex digits");
    for (size_t i = 0; i + 1 < digits.size(); i += 2) n.message.push_back((char)(hex_digit(digits[i]) * 16 + hex_digit(digits[i + 1])));
    for (size_t j = 1; j < x.at(2).size(); ++j) {
      n.shown.push_back(x.at(2).k[j].s);
      env.array(n.shown.back());
    }
    for (size_t j = 1; j < x.at(3).size(); ++j) {
      n.args.push_back(x.at(3).k[j].s);
      outs.push_back(env.array(n.args.back()));
    }
  } else if (k == "reshape") {
    n.kind = N_RESHAPE;
    n.extent = parse_expr(x.at(1), env);
    if (!n.extent->ty.is_shape()) throw Error(B200_ERR_TYPE, "reshape: not a shape");
    n.arr = x.at(2).s;
    n.elt = env.array(n.arr).elt;
    outs.push_back({(int)n.extent->ty.e.size(), n.elt});
  } else {
    throw Error(B200_ERR_PARSE, "unknown array node '" + k + "'");
  }
  std::vector<std::string> names;
  if (lhs.atom) names.push_back(lhs.s);
  else for (auto& nm : lhs.k) names.push_back(nm.s);
  if (names.size() != outs.size()) throw Error(B200_ERR_PARSE, "node '" + k + "' defines " + std::to_string(outs.size()) + " array(s)");
  n.outs = names;
  n.out_info = outs;
  for (size_t i = 0; i < names.size(); ++i) define_array(p, names[i], outs[i]);
  into.push_back(std::move(n));
}

void collect_arrays(const Expr& e, std::vector<std::string>& out) {
  if (e.kind == X_INDEX || e.kind == X_LINDEX || e.kind == X_SHAPE) {
    bool seen = false;
    for (auto& n : out) seen = seen || n == e.name;
    if (!seen) out.push_back(e.name);
  }
  for (auto& c : e.a) collect_arrays(*c, out);
  for (auto& f : e.f) collect_arrays(*f->body, out);
}

}  // namespace

void free_arrays(const Expr& e, std::vector<std::string>& out) { collect_arrays(e, out); }
void free_arrays(const Fun& f, std::vector<std::string>& out) { collect_arrays(*f.body, out); }

void node_arrays(const Node& n, std::vector<std::string>& used) {
  if (n.f) free_arrays(*n.f, used);
  if (n.g) free_arrays(*n.g, used);
  if (n.seed) free_arrays(*n.seed, used);
  if (n.extent) free_arrays(*n.extent, used);
  if (n.pred) free_arrays(*n.pred, used);
  for (auto& d : n.d) {
    if (d.extent) free_arrays(*d.extent, used);
    if (d.index) free_arrays(*d.index, used);
  }
  for (auto& b : n.bnd) {
    if (b.value) free_arrays(*b.value, used);
    if (b.fun) free_arrays(*b.fun, used);
  }
  if (!n.arr.empty()) used.push_back(n.arr);
  for (auto& a : n.args) used.push_back(a);
  for (auto& a : n.shown) used.push_back(a);
  for (auto& b : n.body) {
    for (auto& m : b.nodes) node_arrays(m, used);
    for (auto& o : b.outs) used.push_back(o);
  }
}

// ---- arrays of SIMD vectors at the program's boundary ------------------------------------------------
// The reference stores an `Array sh (Vec n t)` as n components side by side per element
// (Array/Data.hs:108-119), which is byte for byte an `Array (sh :. n) t`.  A program's inputs, embedded
// arrays and results of that type are therefore declared to the outside as rank+1 arrays of t, and the
// program gains one `generate` per such array that regroups it: components into a tuple on the way in,
// the tuple's components along the new innermost dimension on the way out.
namespace {

Sx atom(const std::string& s) { Sx x; x.atom = true; x.s = s; return x; }
Sx list(std::vector<Sx> k) { Sx x; x.k = std::move(k); return x; }
Sx i64c(int64_t v) { return list({atom("const"), atom("i64"), atom(std::to_string(v))}); }
Sx prj(int k, Sx v) { return list({atom("prj"), atom(std::to_string(k)), std::move(v)}); }
Sx shape_ty(int rank) {
  std::vector<Sx> k{atom("tup")};
  for (int d = 0; d < rank; ++d) k.push_back(atom("i64"));
  return list(std::move(k));
}
bool vec_array_type(const Sx& at, int* rank, int* n, std::string* t) {
  if (at.head() != "array" || at.size() != 3 || at.k[2].head() != "vec" || at.k[2].size() != 3) return false;
  *rank = atoi(at.k[1].s.c_str());
  *n = atoi(at.k[2].k[1].s.c_str());
  *t = at.k[2].k[2].s;
  return true;
}
// (let NAME (generate (vec n t) (init (shape RAW)) (lam ((v ix)) (tup (index RAW (ix.., 0)) ..))))
Sx regroup_in(const std::string& name, const std::string& raw, int rank, int n, const std::string& t) {
  std::vector<Sx> comps{atom("tup")};
  for (int k = 0; k < n; ++k) {
    std::vector<Sx> ix{atom("tup")};
    for (int d = 0; d < rank; ++d) ix.push_back(prj(d, list({atom("var"), atom("vx")})));
    ix.push_back(i64c(k));
    comps.push_back(list({atom("index"), atom(raw), list(std::move(ix))}));
  }
  Sx lam = list({atom("lam"), list({list({atom("vx"), shape_ty(rank)})}), list(std::move(comps))});
  Sx gen = list({atom("generate"), list({atom("vec"), atom(std::to_string(n)), atom(t)}),
                 list({atom("init"), list({atom("shape"), atom(raw)})}), std::move(lam)});
  return list({atom("let"), atom(name), std::move(gen)});
}
// (let AOS (generate t (snoc (shape NAME) n) (lam ((v ix')) (let e (index NAME (init ix')) (cond (k == 0) e.0 ..)))))
Sx regroup_out(const std::string& aos, const std::string& name, int rank, int n, const std::string& t) {
  Sx sel = prj(n - 1, list({atom("var"), atom("ve")}));
  for (int k = n - 2; k >= 0; --k)
    sel = list({atom("cond"), list({atom("prim"), atom("eq"), atom("i64"), prj(rank, list({atom("var"), atom("vx")})), i64c(k)}),
                prj(k, list({atom("var"), atom("ve")})), std::move(sel)});
  Sx body = list({atom("let"), atom("ve"), list({atom("index"), atom(name), list({atom("init"), list({atom("var"), atom("vx")})})}), std::move(sel)});
  Sx lam = list({atom("lam"), list({list({atom("vx"), shape_ty(rank + 1)})}), std::move(body)});
  Sx gen = list({atom("generate"), atom(t), list({atom("snoc"), list({atom("shape"), atom(name)}), i64c(n)}), std::move(lam)});
  return list({atom("let"), atom(aos), std::move(gen)});
}
// inputs and embedded arrays, wherever they are bound
void lower_vectors_in(Sx& x) {
  if (x.atom) return;
  std::vector<Sx> out;
  for (Sx& c : x.k) {
    int rank, n;
    std::string t;
    if (c.head() == "in" && c.size() == 3 && vec_array_type(c.k[2], &rank, &n, &t)) {
      const std::string name = c.k[1].s, raw = name + "_aos";
      out.push_back(list({atom("in"), atom(raw), list({atom("array"), atom(std::to_string(rank + 1)), atom(t)})}));
      out.push_back(regroup_in(name, raw, rank, n, t));
    } else if (c.head() == "let" && c.size() == 3 && c.k[2].head() == "use" && c.k[2].size() >= 3 && vec_array_type(c.k[2].k[1], &rank, &n, &t)) {
      const std::string name = c.k[1].s, raw = name + "_aos";
      Sx use = c.k[2];
      use.k[1] = list({atom("array"), atom(std::to_string(rank + 1)), atom(t)});
      use.k[2].k.push_back(atom(std::to_string(n)));      // (shape d.. n)
      out.push_back(list({atom("let"), atom(raw), std::move(use)}));
      out.push_back(regroup_in(name, raw, rank, n, t));
    } else {
      lower_vectors_in(c);
      out.push_back(std::move(c));
    }
  }
  x.k = std::move(out);
}
std::unique_ptr<ProgramIR> parse_program_sx(const Sx& top);
}  // namespace

Sx lower_vectors(Sx top) {
  std::function<bool(const Sx&)> mentions = [&](const Sx& x) {
    if (x.atom) return false;
    if (x.head() == "vec") return true;
    for (const Sx& c : x.k)
      if (mentions(c)) return true;
    return false;
  };
  if (!mentions(top)) return top;
  // (inputs are declared before the nodes that read them, so the regrouping nodes land in front of those)
  lower_vectors_in(top);
  // results: their types are known once the program has been read
  std::unique_ptr<ProgramIR> p = parse_program_sx(top);
  std::vector<Sx> lets;
  for (Sx& f : top.k) {
    if (f.head() != "out") continue;
    for (size_t j = 1; j < f.k.size(); ++j) {
      const ArrayInfo& ai = p->arrays.at(f.k[j].s);
      if (!ai.elt.vec) {
        std::function<bool(const Type&)> nested = [&](const Type& t) { if (t.vec) return true; for (auto& c : t.e) if (nested(c)) return true; return false; };
        if (nested(ai.elt)) throw Error(B200_ERR_UNSUPPORTED, "result '" + f.k[j].s + "': SIMD vectors inside a tuple cannot leave the program");
        continue;
      }
      const std::string aos = f.k[j].s + "_aos";
      lets.push_back(regroup_out(aos, f.k[j].s, ai.rank, (int)ai.elt.e.size(), ty_name[ai.elt.e[0].s]));
      f.k[j] = atom(aos);
    }
  }
  if (!lets.empty()) {
    std::vector<Sx> k;
    for (Sx& f : top.k) {
      if (f.head() == "out") { for (Sx& l : lets) k.push_back(l); lets.clear(); }
      k.push_back(std::move(f));
    }
    top.k = std::move(k);
  }
  return top;
}

std::unique_ptr<ProgramIR> parse_program(const char* text, size_t len) {
  return parse_program_sx(lower_vectors(parse_sexp(text, len)));   // (the tree is moved, not copied)
}
std::string program_text_lowered(const char* text, size_t len) { return sx_text(lower_vectors(parse_sexp(text, len))); }

namespace {
std::unique_ptr<ProgramIR> parse_program_sx(const Sx& top) {
  if (top.head() != "program") throw Error(B200_ERR_PARSE, "expected (program ...)");
  auto p = std::make_unique<ProgramIR>();
  TEnv env;
  env.arrays = &p->arrays;
  for (size_t i = 1; i < top.size(); ++i) {
    const Sx& f = top.k[i];
    const std::string h = f.head();
    if (h == "in") {
      const Sx& at = f.at(2);
      if (at.head() != "array") throw Error(B200_ERR_PARSE, "expected (in name (array rank elt))");
      ArrayInfo ai;
      ai.rank = atoi(at.at(1).s.c_str());
      ai.elt = parse_type(at.at(2));
      p->arrays[f.at(1).s] = ai;
      p->inputs.push_back(f.at(1).s);
    } else if (h == "let") {
      parse_node(*p, p->nodes, f, env);
    } else if (h == "out") {
      for (size_t j = 1; j < f.size(); ++j) {
        env.array(f.k[j].s);
        p->outputs.push_back(f.k[j].s);
      }
    } else {
      throw Error(B200_ERR_PARSE, "unknown program form '" + h + "'");
    }
  }
  if (p->outputs.empty()) throw Error(B200_ERR_PARSE, "program has no (out ...)");
  return p;
}
}  // namespace

}  // namespace accb200
