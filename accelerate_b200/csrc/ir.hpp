// Typed in-memory form of the program text handed to the backend.
//
// The text is a serialisation of the fused delayed AST that the reference's
// transformation pipeline hands to a backend (Trafo/Delayed.hs:51-60 over
// AST.hs:230-460 PreOpenAcc and AST.hs:524-645 OpenExp), restricted to the
// nodes Trafo/Fusion.hs:161-216 lets reach a backend.
#pragma once

#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/accelerate_b200.h"  // status codes

namespace accb200 {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// ---- S-expressions ---------------------------------------------------------
struct Sx {
  bool atom = false;
  std::string s;
  std::vector<Sx> k;
  size_t size() const { return k.size(); }
  std::string head() const { return (!atom && !k.empty() && k[0].atom) ? k[0].s : std::string(); }
  const Sx& at(size_t i) const {
    if (i >= k.size()) throw Error(B200_ERR_PARSE, "program text: (" + head() + " ...) is missing operand " + std::to_string(i));
    return k[i];
  }
};
Sx parse_sexp(const char* text, size_t len);

// ---- scalar and element types (Type.hs:112-152; Int = 64 bit, Bool = Word8) --
enum Ty : uint8_t { I8, I16, I32, I64, U8, U16, U32, U64, F32, F64, F16, NTY };
extern const char* const ty_name[NTY];
extern const int ty_bytes[NTY];
inline bool ty_is_int(Ty t) { return t <= U64; }
inline bool ty_is_signed(Ty t) { return t <= I64; }
inline bool ty_is_float(Ty t) { return t == F32 || t == F64 || t == F16; }
inline int ty_bits(Ty t) { return ty_bytes[t] * 8; }
Ty parse_ty(const std::string& s);

// Half (Type.hs:127, Numeric.Half): IEEE-754 binary16 kept as its 16 bits.  Every operation on it is the
// Float operation on the converted operands, rounded back to nearest-even, as the Num/Fractional/Floating
// instances of Numeric.Half define it (toHalf (fromHalf a + fromHalf b), ...).
inline uint16_t half_from_float(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u, ax = x & 0x7fffffffu;
  if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);  // NaN
  if (ax >= 0x38800000u) {                                   // at least 2^-14: a normal half, or infinity
    uint32_t h = (((ax >> 23) - 112) << 10) | ((ax & 0x7fffffu) >> 13);
    const uint32_t rem = ax & 0x1fffu;
    if (ax >= 0x47800000u) h = 0x7c00u;
    else if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;  // a carry runs into the exponent, up to infinity
    return (uint16_t)(sign | h);
  }
  if (ax <= 0x33000000u) return (uint16_t)sign;              // at most 2^-25: rounds to zero
  const int shift = 126 - (int)(ax >> 23);                    // 14..24: units of 2^-24
  const uint32_t m = (ax & 0x7fffffu) | 0x800000u, rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
  uint32_t h = m >> shift;
  if (rem > mid || (rem == mid && (h & 1))) ++h;
  return (uint16_t)(sign | h);
}
inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 0x3ffu;
  uint32_t x;
  if (e == 31) x = sign | 0x7f800000u | (m << 13);
  else if (e != 0) x = sign | ((e + 112) << 23) | (m << 13);
  else {
    float v = (float)m * 5.9604644775390625e-08f;  // m * 2^-24, exact
    memcpy(&x, &v, 4);
    x |= sign;
  }
  float f;
  memcpy(&f, &x, 4);
  return f;
}

struct Type {
  bool tuple = false;
  // `Vec n t` (Type.hs:140-152): inside a program a SIMD vector is the tuple of its n components (one
  // buffer per component like any tuple); the mark only says which arrays cross the program's boundary
  // in the reference's layout, n components side by side per element (see lower_vectors in ir.cpp).
  // Equality ignores it.
  bool vec = false;
  Ty s = I64;
  std::vector<Type> e;
  static Type scalar(Ty t) { Type r; r.s = t; return r; }
  static Type tup(std::vector<Type> xs) { Type r; r.tuple = true; r.e = std::move(xs); return r; }
  static Type shape(int rank) { return tup(std::vector<Type>(rank, scalar(I64))); }
  bool operator==(const Type& o) const;
  bool operator!=(const Type& o) const { return !(*this == o); }
  void flatten(std::vector<Ty>& out) const;
  std::vector<Ty> leaves() const { std::vector<Ty> v; flatten(v); return v; }
  size_t nleaves() const { return leaves().size(); }
  std::string str() const;
  bool is_shape() const;  // flat tuple of Int
};
Type parse_type(const Sx& x);

// ---- scalar expressions ------------------------------------------------------
enum Prim {
  P_ADD, P_SUB, P_MUL, P_NEG, P_ABS, P_SIG, P_QUOT, P_REM, P_QUOTREM, P_IDIV, P_MOD, P_DIVMOD,
  P_BAND, P_BOR, P_BXOR, P_BNOT, P_SHL, P_SHR, P_ROTL, P_ROTR, P_POPCNT, P_CLZ, P_CTZ,
  P_FDIV, P_RECIP, P_SIN, P_COS, P_TAN, P_ASIN, P_ACOS, P_ATAN, P_SINH, P_COSH, P_TANH,
  P_ASINH, P_ACOSH, P_ATANH, P_EXP, P_SQRT, P_LOG, P_FPOW, P_LOGBASE, P_ATAN2,
  P_TRUNCATE, P_ROUND, P_FLOOR, P_CEILING, P_ISNAN, P_ISINF,
  P_LT, P_GT, P_LE, P_GE, P_EQ, P_NE, P_MAX, P_MIN, P_LAND, P_LOR, P_LNOT,
  P_FROMINTEGRAL, P_TOFLOATING, P_NPRIMS
};
extern const char* const prim_name[P_NPRIMS];

enum ExprKind {
  X_CONST, X_VAR, X_LET, X_TUP, X_PRJ, X_COND, X_WHILE, X_PRIM, X_INDEX, X_LINDEX, X_SHAPE,
  X_SHAPESIZE, X_TOINDEX, X_FROMINDEX, X_COERCE, X_UNDEF, X_APP, X_CASE, X_SNOC, X_INIT
};

struct Fun;
struct Expr {
  ExprKind kind = X_CONST;
  Type ty;                      // result type
  std::string name;             // X_VAR / X_LET: scalar variable; X_INDEX/X_LINDEX/X_SHAPE: array variable
  std::string lit;              // X_CONST: literal text as written
  int n = 0;                    // X_PRJ component
  Prim op = P_ADD;              // X_PRIM
  Ty t1 = I64, t2 = I64;        // X_PRIM operand/target type; X_COERCE from/to
  std::vector<std::unique_ptr<Expr>> a;
  std::vector<std::unique_ptr<Fun>> f;   // X_WHILE (cond, body), X_APP
  std::vector<long long> tags;           // X_CASE
  bool has_default = false;
};
struct Fun {
  std::vector<std::string> params;
  std::vector<Type> param_ty;
  std::unique_ptr<Expr> body;
  const Type& result() const { return body->ty; }
};

// ---- array-level nodes -------------------------------------------------------
struct ArrayInfo {
  int rank = 0;
  Type elt;
};

struct DelayedOp {
  bool manifest = false;
  std::string arr;                 // manifest: the array variable
  std::unique_ptr<Expr> extent;    // delayed: extent expression (closed over array variables)
  std::unique_ptr<Fun> index;      // delayed: index -> element (manifest operands get \ix -> arr ! ix)
  int rank = 0;
  Type elt;
};

enum BoundaryKind { BND_CLAMP, BND_MIRROR, BND_WRAP, BND_CONSTANT, BND_FUNCTION };
struct BoundarySpec {
  BoundaryKind kind = BND_CLAMP;
  std::unique_ptr<Expr> value;
  std::unique_ptr<Fun> fun;
};

// Kernel nodes, and the nodes the reference evaluates on the host (Interpreter.hs:215-231):
// Use (a constant array embedded in the program), Acond, Awhile and Apply, whose operands are
// array-level functions (`Body`).
enum NodeKind { N_GENERATE, N_FOLD, N_FOLDSEG, N_SCAN, N_SCAN2, N_PERMUTE, N_STENCIL, N_STENCIL2, N_RESHAPE,
                N_USE, N_ACOND, N_AWHILE, N_APPLY, N_ATRACE };
struct Node;
// An array-level function or a branch: parameters (none for branches), nodes, results.
struct Body {
  std::vector<std::string> params;
  std::vector<ArrayInfo> param_info;
  std::vector<Node> nodes;
  std::vector<std::string> outs;
};
struct Node {
  NodeKind kind = N_GENERATE;
  int id = -1;                            // position in Program::nodes (unique over all bodies)
  std::vector<Body> body;                 // acond: then, else; awhile: condition, step; apply: the function
  std::vector<std::string> args;          // awhile: initial state; apply: arguments; atrace: the arrays handed on
  std::vector<std::string> shown;         // atrace: the arrays to print
  std::string message;                    // atrace
  std::unique_ptr<Expr> pred;             // acond
  std::vector<int64_t> use_shape;         // use
  std::vector<std::string> use_data;      // use: raw bytes of every scalar leaf
  std::string text;                       // the node's own text (hashed into kernel-cache keys)
  std::vector<std::string> outs;          // array variables defined
  std::vector<ArrayInfo> out_info;
  Type elt;
  std::unique_ptr<Fun> f;                 // generate body / combine / stencil function
  std::unique_ptr<Fun> g;                 // permute index function
  std::unique_ptr<Expr> seed;             // folds/scans (null = fold1/scanl1...)
  std::unique_ptr<Expr> extent;           // generate / reshape
  std::vector<DelayedOp> d;
  bool right = false;                     // scanr*
  std::string arr;                        // permute defaults, reshape source
  std::vector<std::vector<int>> st_extent;
  std::vector<BoundarySpec> bnd;
};

struct ProgramIR {
  int n_nodes = 0;                         // nodes of all bodies
  std::map<std::string, ArrayInfo> arrays;
  std::vector<std::string> inputs;
  std::vector<Node> nodes;
  std::vector<std::string> outputs;
};

// Parse and type-check; throws Error.
std::unique_ptr<ProgramIR> parse_program(const char* text, size_t len);
// The program with its arrays of SIMD vectors regrouped at the boundary (the identity without them).
Sx lower_vectors(Sx program);
std::string program_text_lowered(const char* text, size_t len);

// Free array variables of an expression / function (names, in first-use order).
void free_arrays(const Expr& e, std::vector<std::string>& out);
void free_arrays(const Fun& f, std::vector<std::string>& out);
// Every array variable a node mentions, the bodies of control nodes included.
void node_arrays(const Node& n, std::vector<std::string>& out);

}  // namespace accb200
