// Cluster-level program of a kernel and the plans made from it: the data model shared
// by source.cpp (reads a `.ph` declaration and classifies its tensor accesses) and
// planner.cpp (turns program + problem sizes + node count into per-node instruction
// lists).  Mirrors the shapes of phobos-cluster/src/ir.rs:5-103 and
// phobos-sched/src/lib.rs:34-62; nothing here touches a GPU.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../../include/phobos_leaf.h"

namespace ph {
namespace plan {

struct Dim {               // a tensor extent: symbolic (M, Nk) or literal
  bool sym = false;
  std::string name;
  int64_t value = 0;
};

struct AttrArg {           // phobos-lang/src/ast.rs:44-56
  enum Kind { SEARCH, KEYVALUE, POSITIONAL } kind = POSITIONAL;
  std::string name;                 // SEARCH: dimension; KEYVALUE: key
  std::vector<int64_t> declared;    // SEARCH: the values as written
  std::string literal;              // KEYVALUE / POSITIONAL: the literal's text
  bool literal_is_int = false;
  int64_t int_value = 0;
};
struct Attribute {
  std::string name;
  std::vector<AttrArg> args;
};
struct Param {
  std::string name;
  bool is_tensor = false;
  int dtype = PH_F32;
  std::vector<Dim> dims;
};
struct Token {
  enum Kind { IDENT, INT, FLOAT, PUNCT, NEWLINE, END } kind = END;
  std::string text;
  int line = 0;
};
struct KernelDecl {
  std::vector<Attribute> attrs;
  std::string name;
  std::vector<Param> params;
  std::vector<Token> body;          // tokens between the kernel's braces
};

// `[lo, hi]` with hi > lo > 0 means lo, 2lo, 4lo, ... capped by hi; longer lists are explicit
std::vector<int64_t> search_choices(const std::vector<int64_t>& declared);

// ---- cluster program -------------------------------------------------------------------------
struct SearchDim {
  std::string name;
  std::vector<int64_t> choices;
};
struct TensorDecl {
  std::string name;
  int dtype = PH_F32;
  std::vector<Dim> dims;
  std::vector<std::string> super_syms;   // per axis: the supertile symbol, or the dim's own name when not tiled
  int mode = PH_READ;
};
struct ScalarDecl {
  std::string name;
  int dtype = PH_F32;
  int param_pos = 0;
};
struct GridAxis {
  int pid = 0;
  Dim dim;
  std::string super_sym;
};
struct Leaf {
  std::string entry;                     // PTX entry name the executor resolves
  uint32_t cta_threads = 256;
  std::map<std::string, int64_t> device_tile;   // first @autotune choice per search dimension
  std::vector<int> modes;
};
struct Coord {
  enum Kind { GRID, LOOP, FULL } kind = FULL;
  int grid = 0;
  std::string loop;
  bool operator==(const Coord& o) const { return kind == o.kind && grid == o.grid && loop == o.loop; }
};
struct SuperTile {
  int tensor = 0;
  std::vector<Coord> coords;
};
struct Stmt {
  bool is_loop = false;
  // compute
  int leaf = 0;
  std::vector<std::pair<SuperTile, int>> args;
  std::vector<int> scalars;
  // loop
  std::string var;
  Dim dim;
  std::string super_sym;
  std::vector<Stmt> body;
};
struct Program {
  std::string name;
  std::vector<SearchDim> super_dims;
  std::vector<TensorDecl> tensors;
  std::vector<ScalarDecl> scalars;
  std::vector<Leaf> leaves;
  std::vector<GridAxis> grid;
  std::vector<Stmt> body;
};

// Both return false and set *err on failure.
bool parse_kernels(const std::string& text, std::vector<KernelDecl>* out, std::string* err);
bool compile_program(const KernelDecl& k, Program* out, std::string* err);
std::string describe(const Program& p);

// ---- plans -------------------------------------------------------------------------------------
struct OwnedInstr {        // a PhInstr whose pointer members point into the vectors beside it
  PhInstr in{};
  std::vector<uint64_t> deps;
  std::vector<PhTileArg> args;
  std::vector<PhScalar> scalars;
};
struct Segment {
  uint64_t id = 0;
  std::vector<OwnedInstr> instrs;
  std::vector<PhInstr> flat;   // the same instructions as one array, built by finish()
  uint64_t peak = 0, incremental = 0;
};
struct StoreRec {
  uint64_t iid;
  uint32_t node;
  uint32_t tensor;
  uint64_t lin;
};
struct Plan {
  std::vector<std::vector<Segment>> node_segments;
  std::vector<std::vector<uint64_t>> super_shapes, super_grids;
  std::vector<std::vector<std::pair<uint64_t, uint32_t>>> fetches;   // per node: (tile, from)
  uint64_t fetch_bytes = 0, peak_resident = 0;
  std::vector<StoreRec> stores;
  std::map<std::pair<uint32_t, uint64_t>, uint32_t> output_owner;
  uint64_t max_iid = 0;
};
struct PlanRequest {
  std::map<std::string, int64_t> dims, supers;
  std::map<std::string, PhScalar> scalars;     // by name; .pos is filled in from the declaration
  uint32_t nodes = 1;                           // plan(): live nodes 0..nodes-1.  recover(): cluster width
  uint64_t budget = UINT64_MAX;
  int policy = 0;                               // 0 DirectLoad, 1 HomeLoadPeerFetch
  // recovery only
  bool recover = false;
  std::vector<uint32_t> dead;
  std::vector<std::pair<uint32_t, uint64_t>> durable;
  uint16_t version = 0;
  uint64_t iid_base = 0;
};
bool make_plan(const Program& p, const PlanRequest& rq, Plan* out, std::string* err);
bool validate_plan(const Plan& pl, std::string* err);
std::map<std::string, int64_t> default_supers(const Program& p);

struct Fingerprint {       // phobos-sched/src/autotune.rs:11-28
  uint32_t nodes = 1;
  uint64_t vram_bytes = 16ull << 30;
  double link_bytes_per_sec = 10e9;
  double leaf_flops_per_sec = 10e12;
};
struct RankedConfig {
  std::map<std::string, int64_t> supers;
  double makespan_sec = 0, compute_sec = 0, comm_sec = 0;
  uint64_t peak_resident = 0, fetch_bytes = 0;
};
bool autotune(const Program& p, const std::map<std::string, int64_t>& dims, const Fingerprint& fp,
              std::vector<RankedConfig>* out, std::string* err);

}  // namespace plan
}  // namespace ph
