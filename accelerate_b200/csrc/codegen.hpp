// Lowering of scalar functions (OpenFun/OpenExp, AST.hs:493-645) to CUDA device
// functions, and assembly of one kernel source per array node from the
// hand-written skeletons.
#pragma once

#include <map>
#include <set>
#include <string>
#include <vector>

#include "ir.hpp"

namespace accb200 {

// One 8-byte slot of the kernel parameter block.
struct Slot {
  enum Kind { ARR_LEAF, ARR_DIM, OUT_LEAF, NAMED } kind;
  std::string name;  // array variable (ARR_*), or the named field
  int idx = 0;       // leaf / dimension / (OUT_LEAF: output number * 64 + leaf)
};

// The generated part of a kernel source: parameter block, element structs and
// device functions the skeleton calls.  `defines` describe properties the
// skeleton specialises on.
struct Glue {
  std::string code;
  std::vector<Slot> slots;
  std::map<std::string, std::string> defines;
  // per delayed operand: arrays that are read at exactly the loop index
  // ("streams"; they take the vectorised path when their shape equals the extent)
  std::vector<std::vector<std::string>> streams;
};

// Build the glue for one node.  `arrays` gives rank/element type of every array
// variable in scope.
Glue build_glue(const Node& n, const std::map<std::string, ArrayInfo>& arrays);

// Text of the common prelude and of a skeleton ("elementwise", "fold", "foldseg",
// "scan", "permute", "stencil").
const char* prelude_source();
const char* skeleton_source(const std::string& name);

// Whether a binary function is syntactically `\a b -> prim a b` for a primitive
// that commutes; `op` receives the primitive.
bool is_simple_prim(const Fun& f, Prim* op, Ty* ty);

}  // namespace accb200
