// Supertile planner: cluster program + problem sizes + node count -> per-node
// instruction lists for the executor (ALLOC / LOAD / FETCH / COMPUTE / STORE / FREE).
//
// Behaviour follows phobos-sched/src/lib.rs: the body is unrolled once per point of the
// supertile grid (instantiate, lib.rs:298-457), every compute is placed on the node that
// owns its output supertile (linear index modulo the live nodes, lib.rs:591-600), tiles
// are materialised at first use and stored / freed at their last use on that node
// (lib.rs:653-842), inputs come from storage (DirectLoad) or, for a tile several nodes
// read, from the lowest-numbered consumer over the interconnect (HomeLoadPeerFetch,
// lib.rs:615-620), and each node's list is cut into segments whose newly allocated bytes
// fit a budget (lib.rs:854-934).  recover = the same lowering restricted to the output
// supertiles of failed nodes, placed over the survivors (lib.rs:191-234).  The cost model
// that ranks supertile sizes is phobos-sched/src/autotune.rs:98-192 with the link and leaf
// rates supplied by the caller (NVLink and the measured kernel rates on this hardware).
#include <algorithm>
#include <array>
#include <cctype>
#include <cstdlib>
#include <set>
#include <sstream>

#include "plan.h"

namespace ph {
namespace plan {
namespace {

size_t dtype_bytes(int dt) { return phobos_dtype_bytes(dt); }

struct CompInst {
  int leaf;
  struct Arg { int tensor; std::vector<uint64_t> coords; int mode; };
  std::vector<Arg> args;
  std::vector<int> scalars;
};

struct Inst {
  std::vector<CompInst> computes;
  std::vector<std::vector<uint64_t>> super_shapes, super_grids;
  std::vector<std::array<uint32_t, 3>> leaf_grids, leaf_ctas;
  uint64_t lin(int tensor, const std::vector<uint64_t>& coords) const {
    uint64_t l = 0;
    for (size_t i = 0; i < coords.size(); i++) l = l * super_grids[tensor][i] + coords[i];
    return l;
  }
};

bool fail(std::string* err, const std::string& m) {
  *err = m;
  return false;
}
std::string dim_text(const Dim& d) { return d.sym ? d.name : std::to_string(d.value); }

bool unroll(const std::vector<Stmt>& stmts, const std::vector<uint64_t>& gpt, std::map<std::string, uint64_t>& loops,
            const PlanRequest& rq, std::vector<CompInst>* out, std::string* err) {
  for (const Stmt& s : stmts) {
    if (!s.is_loop) {
      CompInst c;
      c.leaf = s.leaf;
      c.scalars = s.scalars;
      for (const auto& a : s.args) {
        CompInst::Arg ca;
        ca.tensor = a.first.tensor;
        ca.mode = a.second;
        for (const Coord& co : a.first.coords)
          ca.coords.push_back(co.kind == Coord::GRID ? gpt[co.grid] : co.kind == Coord::LOOP ? loops[co.loop] : 0);
        c.args.push_back(std::move(ca));
      }
      out->push_back(std::move(c));
    } else {
      uint64_t d;
      if (s.dim.sym) {
        auto it = rq.dims.find(s.dim.name);
        if (it == rq.dims.end()) return fail(err, "loop dim '" + s.dim.name + "' is unbound");
        d = static_cast<uint64_t>(it->second);
      } else {
        d = static_cast<uint64_t>(s.dim.value);
      }
      auto st = rq.supers.find(s.super_sym);
      if (st == rq.supers.end()) return fail(err, "supertile dim '" + s.super_sym + "' is unbound");
      const uint64_t sv = static_cast<uint64_t>(st->second);
      if (sv == 0 || d % sv != 0)
        return fail(err, "loop bound " + std::to_string(d) + " is not a multiple of supertile dim " + s.super_sym + " = " +
                             std::to_string(sv));
      for (uint64_t i = 0; i < d / sv; i++) {
        loops[s.var] = i;
        if (!unroll(s.body, gpt, loops, rq, out, err)) return false;
      }
      loops.erase(s.var);
    }
  }
  return true;
}

bool instantiate(const Program& p, const PlanRequest& rq, Inst* inst, std::string* err) {
  if (p.tensors.size() >= (1u << 12)) return fail(err, "too many tensors for TileId encoding");
  auto dim_val = [&](const Dim& d, uint64_t* v) {
    if (!d.sym) {
      *v = static_cast<uint64_t>(d.value);
      return true;
    }
    auto it = rq.dims.find(d.name);
    if (it == rq.dims.end()) return fail(err, "problem dim '" + d.name + "' is unbound");
    if (it->second <= 0) return fail(err, "problem dim '" + d.name + "' must be positive, got " + std::to_string(it->second));
    *v = static_cast<uint64_t>(it->second);
    return true;
  };
  auto super_val = [&](const std::string& s, uint64_t* v) {
    int64_t x;
    auto it = rq.supers.find(s);
    if (it != rq.supers.end()) {
      x = it->second;
    } else if ((it = rq.dims.find(s)) != rq.dims.end()) {
      x = it->second;           // an axis that is not tiled: the supertile spans the whole dim
    } else if (!s.empty() && isdigit((unsigned char)s[0])) {
      x = strtoll(s.c_str(), nullptr, 10);   // literal extent
    } else {
      return fail(err, "supertile dim '" + s + "' is unbound");
    }
    if (x <= 0) return fail(err, "supertile dim '" + s + "' must be positive, got " + std::to_string(x));
    *v = static_cast<uint64_t>(x);
    return true;
  };

  std::vector<uint64_t> grid_ext;
  for (const GridAxis& ax : p.grid) {
    uint64_t d, s;
    if (!dim_val(ax.dim, &d) || !super_val(ax.super_sym, &s)) return false;
    if (d % s != 0)
      return fail(err, "dim " + dim_text(ax.dim) + " = " + std::to_string(d) + " is not a multiple of supertile dim " +
                           ax.super_sym + " = " + std::to_string(s));
    grid_ext.push_back(d / s);
  }
  for (const TensorDecl& t : p.tensors) {
    std::vector<uint64_t> shape, grid;
    uint64_t count = 1;
    for (size_t i = 0; i < t.dims.size(); i++) {
      uint64_t d, s;
      if (!dim_val(t.dims[i], &d) || !super_val(t.super_syms[i], &s)) return false;
      if (d % s != 0)
        return fail(err, "tensor '" + t.name + "' dim " + dim_text(t.dims[i]) + " = " + std::to_string(d) +
                             " is not a multiple of supertile dim " + t.super_syms[i] + " = " + std::to_string(s));
      shape.push_back(s);
      grid.push_back(d / s);
      count *= d / s;
    }
    if (count >= (1ull << 36)) return fail(err, "tensor '" + t.name + "' has too many supertiles for TileId encoding");
    inst->super_shapes.push_back(shape);
    inst->super_grids.push_back(grid);
  }
  // launch grid of a leaf: supertile extent / the leaf's device tile (first @autotune choice)
  for (const Leaf& leaf : p.leaves) {
    inst->leaf_ctas.push_back({leaf.cta_threads, 1u, 1u});
    std::array<uint32_t, 3> g{1u, 1u, 1u};
    for (size_t i = 0; i < p.grid.size(); i++) {
      if (i >= 3) return fail(err, "more than 3 grid axes");
      uint64_t sup;
      if (!super_val(p.grid[i].super_sym, &sup)) return false;
      auto dt = leaf.device_tile.find(p.grid[i].super_sym);
      if (dt == leaf.device_tile.end())
        return fail(err, "leaf '" + leaf.entry + "' has no @autotune default for '" + p.grid[i].super_sym + "'");
      if (dt->second <= 0 || sup % static_cast<uint64_t>(dt->second) != 0)
        return fail(err, "supertile dim " + p.grid[i].super_sym + " = " + std::to_string(sup) + " is not a multiple of leaf '" +
                             leaf.entry + "' device tile " + std::to_string(dt->second));
      g[i] = static_cast<uint32_t>(sup / static_cast<uint64_t>(dt->second));
    }
    inst->leaf_grids.push_back(g);
  }
  // one execution of the body per point of the supertile grid, last axis fastest
  std::vector<uint64_t> gpt(grid_ext.size(), 0);
  while (true) {
    std::map<std::string, uint64_t> loops;
    if (!unroll(p.body, gpt, loops, rq, &inst->computes, err)) return false;
    int ax = static_cast<int>(gpt.size()) - 1;
    for (; ax >= 0; ax--) {
      if (++gpt[ax] < grid_ext[ax]) break;
      gpt[ax] = 0;
    }
    if (ax < 0) break;
  }
  return true;
}

bool output_key(const Inst& inst, const CompInst& c, std::pair<uint32_t, uint64_t>* key, std::string* err) {
  int n = 0;
  for (const auto& a : c.args)
    if (a.mode == PH_WRITE || a.mode == PH_RMW) {
      if (n++ == 0) *key = {static_cast<uint32_t>(a.tensor), inst.lin(a.tensor, a.coords)};
    }
  if (n == 0) return fail(err, "compute writes no supertile");
  if (n > 1) return fail(err, "compute writes more than one supertile (unsupported)");
  return true;
}

struct Slot {
  uint64_t tile, alloc;
  bool have_write = false;
  uint64_t last_write = 0;
  std::vector<uint64_t> consumers;
};

PhRegion storage_region(int tensor, const std::vector<uint64_t>& coords, const Inst& inst) {
  PhRegion r{};
  r.rank = static_cast<int32_t>(coords.size());
  for (size_t i = 0; i < coords.size() && i < 2; i++) {
    r.offset[i] = coords[i] * inst.super_shapes[tensor][i];
    r.shape[i] = inst.super_shapes[tensor][i];
  }
  return r;
}

void finish_segment(Segment* s) {
  s->flat.clear();
  for (OwnedInstr& oi : s->instrs) {
    oi.in.deps = oi.deps.data();
    oi.in.n_deps = static_cast<int32_t>(oi.deps.size());
    oi.in.args = oi.args.data();
    oi.in.n_args = static_cast<int32_t>(oi.args.size());
    oi.in.scalars = oi.scalars.data();
    oi.in.n_scalars = static_cast<int32_t>(oi.scalars.size());
    s->flat.push_back(oi.in);
  }
}

// cuts one node's list before any ALLOC that would push the bytes allocated since the
// segment began over `budget`
bool cut_segments(std::vector<OwnedInstr>&& instrs, uint64_t budget, uint64_t* seg_id, std::vector<Segment>* segs,
                  uint64_t* node_peak, std::string* err) {
  std::map<uint64_t, uint64_t> bytes_of;
  for (const OwnedInstr& oi : instrs)
    if (oi.in.op == PH_OP_ALLOC) {
      uint64_t b = dtype_bytes(oi.in.data_type);
      for (int d = 0; d < oi.in.shape_rank; d++) b *= oi.in.shape[d];
      bytes_of[oi.in.tile] = b;
    }
  uint64_t resident = 0, seg_start = 0, seg_peak = 0;
  *node_peak = 0;
  Segment cur;
  auto flush = [&]() {
    if (cur.instrs.empty()) return;
    cur.id = (*seg_id)++;
    cur.peak = seg_peak;
    cur.incremental = seg_peak > seg_start ? seg_peak - seg_start : 0;
    segs->push_back(std::move(cur));
    cur = Segment();
  };
  for (OwnedInstr& oi : instrs) {
    if (oi.in.op == PH_OP_ALLOC) {
      const uint64_t b = bytes_of[oi.in.tile];
      if (b > budget)
        return fail(err, "supertile of " + std::to_string(b) + " bytes exceeds the memory budget of " + std::to_string(budget) +
                             " bytes");
      const uint64_t after = resident + b;
      if (!cur.instrs.empty() && (after > seg_start ? after - seg_start : 0) > budget) {
        flush();
        seg_start = resident;
        seg_peak = resident;
      }
      resident += b;
    } else if (oi.in.op == PH_OP_FREE) {
      auto it = bytes_of.find(oi.in.tile);
      const uint64_t b = it == bytes_of.end() ? 0 : it->second;
      resident = resident > b ? resident - b : 0;
    }
    seg_peak = std::max(seg_peak, resident);
    *node_peak = std::max(*node_peak, resident);
    cur.instrs.push_back(std::move(oi));
  }
  flush();
  return true;
}

}  // namespace

std::map<std::string, int64_t> default_supers(const Program& p) {
  std::map<std::string, int64_t> m;
  for (const SearchDim& d : p.super_dims) m[d.name] = d.choices[0];
  return m;
}

bool make_plan(const Program& p, const PlanRequest& rq, Plan* out, std::string* err) {
  if (rq.nodes == 0) return fail(err, "cluster has no nodes");
  std::vector<uint32_t> live;
  const uint32_t width = rq.nodes;
  {
    std::set<uint32_t> dead(rq.dead.begin(), rq.dead.end());
    for (uint32_t n = 0; n < width; n++)
      if (!rq.recover || !dead.count(n)) live.push_back(n);
    if (live.empty()) return fail(err, "every node has failed; cannot recover");
  }
  Inst inst;
  if (!instantiate(p, rq, &inst, err)) return false;

  // recovery: only the chains whose output a dead node owned and that are not durable yet
  bool restricted = rq.recover;
  std::set<std::pair<uint32_t, uint64_t>> lost;
  if (rq.recover) {
    std::set<uint32_t> dead(rq.dead.begin(), rq.dead.end());
    std::set<std::pair<uint32_t, uint64_t>> durable(rq.durable.begin(), rq.durable.end());
    for (const CompInst& c : inst.computes) {
      std::pair<uint32_t, uint64_t> key;
      if (!output_key(inst, c, &key, err)) return false;
      const uint32_t owner = static_cast<uint32_t>(key.second % width);
      if (dead.count(owner) && !durable.count(key)) lost.insert(key);
    }
  }

  auto resolve_scalars = [&](const std::vector<int>& idxs, std::vector<PhScalar>* dst) {
    for (int si : idxs) {
      const ScalarDecl& d = p.scalars[si];
      auto it = rq.scalars.find(d.name);
      if (it == rq.scalars.end()) return fail(err, "scalar parameter '" + d.name + "' is unbound");
      if (it->second.dtype != d.dtype)
        return fail(err, "scalar '" + d.name + "' bound as type " + std::to_string(it->second.dtype) + " but declared " +
                             std::to_string(d.dtype));
      PhScalar s = it->second;
      s.pos = static_cast<uint32_t>(d.param_pos);
      dst->push_back(s);
    }
    return true;
  };
  auto tile_bytes = [&](int t) {
    uint64_t b = dtype_bytes(p.tensors[t].dtype);
    for (uint64_t s : inst.super_shapes[t]) b *= s;
    return b;
  };

  const size_t nc = inst.computes.size();
  std::vector<uint32_t> placement(nc, 0);
  std::vector<size_t> active;
  for (size_t ci = 0; ci < nc; ci++) {
    std::pair<uint32_t, uint64_t> key;
    if (!output_key(inst, inst.computes[ci], &key, err)) return false;
    placement[ci] = live[key.second % live.size()];
    if (!restricted || lost.count(key)) {
      active.push_back(ci);
      out->output_owner[key] = placement[ci];
    }
  }
  // which nodes read each input supertile
  std::map<std::pair<int, uint64_t>, std::set<uint32_t>> consumers_of;
  for (size_t ci : active)
    for (const auto& a : inst.computes[ci].args)
      if (p.tensors[a.tensor].mode == PH_READ && a.mode == PH_READ)
        consumers_of[{a.tensor, inst.lin(a.tensor, a.coords)}].insert(placement[ci]);
  auto home = [&](const std::pair<int, uint64_t>& key) { return *consumers_of[key].begin(); };

  std::vector<std::vector<size_t>> node_computes(width);
  for (size_t ci : active) node_computes[placement[ci]].push_back(ci);

  uint64_t iid = rq.iid_base;
  std::vector<std::vector<OwnedInstr>> node_lists(width);
  out->fetches.assign(width, {});
  for (uint32_t node = 0; node < width; node++) {
    // position of the last compute on this node that touches each tile
    std::map<std::pair<int, uint64_t>, size_t> last_use;
    for (size_t pos = 0; pos < node_computes[node].size(); pos++)
      for (const auto& a : inst.computes[node_computes[node][pos]].args) last_use[{a.tensor, inst.lin(a.tensor, a.coords)}] = pos;
    std::map<std::pair<int, uint64_t>, Slot> slots;
    std::vector<OwnedInstr>& instrs = node_lists[node];
    auto emit = [&](int op) -> OwnedInstr& {
      instrs.emplace_back();
      OwnedInstr& oi = instrs.back();
      oi.in.iid = ++iid;
      oi.in.op = op;
      return oi;
    };
    for (size_t pos = 0; pos < node_computes[node].size(); pos++) {
      const CompInst& c = inst.computes[node_computes[node][pos]];
      std::vector<uint64_t> deps;
      std::vector<PhTileArg> iargs;
      for (const auto& a : c.args) {
        const std::pair<int, uint64_t> key{a.tensor, inst.lin(a.tensor, a.coords)};
        if (!slots.count(key)) {
          Slot s;
          s.tile = phobos_tile_id(static_cast<uint32_t>(a.tensor), rq.version, key.second);
          {
            OwnedInstr& al = emit(PH_OP_ALLOC);
            al.in.tile = s.tile;
            al.in.data_type = p.tensors[a.tensor].dtype;
            al.in.shape_rank = static_cast<int32_t>(inst.super_shapes[a.tensor].size());
            for (size_t d = 0; d < inst.super_shapes[a.tensor].size() && d < 2; d++) al.in.shape[d] = inst.super_shapes[a.tensor][d];
            s.alloc = al.in.iid;
          }
          const int tmode = p.tensors[a.tensor].mode;
          if (tmode == PH_RMW || tmode == PH_READ) {
            const bool fetch = tmode == PH_READ && rq.policy == 1 && node != home(key);
            OwnedInstr& in = emit(fetch ? PH_OP_FETCH : PH_OP_LOAD);
            in.in.tile = s.tile;
            in.deps.push_back(s.alloc);
            if (fetch) {
              in.in.from_node = home(key);
              out->fetches[node].push_back({s.tile, home(key)});
              out->fetch_bytes += tile_bytes(a.tensor);
            } else {
              in.in.tensor = static_cast<uint32_t>(a.tensor);
              in.in.region = storage_region(a.tensor, a.coords, inst);
            }
            s.have_write = true;
            s.last_write = in.in.iid;
          }
          slots[key] = s;
        }
        const Slot& s = slots[key];
        if (a.mode == PH_READ || a.mode == PH_RMW) {
          if (!s.have_write) return fail(err, "supertile of '" + p.tensors[a.tensor].name + "' is read before it is produced");
          deps.push_back(s.last_write);
        } else {
          deps.push_back(s.alloc);
        }
        iargs.push_back({s.tile, a.mode});
      }
      std::sort(deps.begin(), deps.end());
      deps.erase(std::unique(deps.begin(), deps.end()), deps.end());
      uint64_t ciid;
      {
        OwnedInstr& co = emit(PH_OP_COMPUTE);
        ciid = co.in.iid;
        co.deps = deps;
        co.in.kernel = static_cast<uint32_t>(c.leaf);
        co.args = iargs;
        if (!resolve_scalars(c.scalars, &co.scalars)) return false;
        for (int d = 0; d < 3; d++) {
          co.in.grid[d] = inst.leaf_grids[c.leaf][d];
          co.in.cta[d] = inst.leaf_ctas[c.leaf][d];
        }
      }
      for (const auto& a : c.args) {
        Slot& s = slots[{a.tensor, inst.lin(a.tensor, a.coords)}];
        if (a.mode == PH_WRITE || a.mode == PH_RMW) {
          s.have_write = true;
          s.last_write = ciid;
        } else {
          s.consumers.push_back(ciid);
        }
      }
      // a tile whose last use on this node was this compute is stored (outputs) and freed now
      for (const auto& a : c.args) {
        const std::pair<int, uint64_t> key{a.tensor, inst.lin(a.tensor, a.coords)};
        if (last_use[key] != pos) continue;
        const Slot& s = slots[key];
        const int tmode = p.tensors[a.tensor].mode;
        if (tmode == PH_WRITE || tmode == PH_RMW) {
          if (!s.have_write) return fail(err, "output supertile of '" + p.tensors[a.tensor].name + "' never produced");
          uint64_t st_iid;
          {
            OwnedInstr& st = emit(PH_OP_STORE);
            st_iid = st.in.iid;
            st.in.tile = s.tile;
            st.deps.push_back(s.last_write);
            st.in.tensor = static_cast<uint32_t>(a.tensor);
            st.in.region = storage_region(a.tensor, a.coords, inst);
          }
          out->stores.push_back({st_iid, node, static_cast<uint32_t>(a.tensor), key.second});
          OwnedInstr& fr = emit(PH_OP_FREE);
          fr.in.tile = s.tile;
          fr.deps.push_back(st_iid);
        } else {
          OwnedInstr& fr = emit(PH_OP_FREE);
          fr.in.tile = s.tile;
          fr.deps = s.consumers;
          if (rq.policy == 1 && node == home(key)) fr.in.expected_serves = static_cast<uint32_t>(consumers_of[key].size() - 1);
        }
      }
    }
  }
  out->max_iid = iid;

  uint64_t seg_id = 0;
  out->node_segments.assign(width, {});
  for (uint32_t node = 0; node < width; node++) {
    uint64_t node_peak = 0;
    if (!cut_segments(std::move(node_lists[node]), rq.budget, &seg_id, &out->node_segments[node], &node_peak, err)) return false;
    out->peak_resident = std::max(out->peak_resident, node_peak);
    for (Segment& s : out->node_segments[node]) finish_segment(&s);
  }
  out->super_shapes = inst.super_shapes;
  out->super_grids = inst.super_grids;
  return true;
}

bool validate_plan(const Plan& pl, std::string* err) {
  for (size_t node = 0; node < pl.node_segments.size(); node++) {
    std::set<uint64_t> seen;
    for (const Segment& s : pl.node_segments[node])
      for (const OwnedInstr& oi : s.instrs) {
        for (uint64_t d : oi.deps)
          if (!seen.count(d))
            return fail(err, "instr " + std::to_string(oi.in.iid) + " on node " + std::to_string(node) + " depends on " +
                                 std::to_string(d) + " which is not an earlier instruction in the node's dispatch order");
        seen.insert(oi.in.iid);
      }
  }
  return true;
}

// ---- cost model --------------------------------------------------------------------------------
bool autotune(const Program& p, const std::map<std::string, int64_t>& dims, const Fingerprint& fp,
              std::vector<RankedConfig>* out, std::string* err) {
  if (fp.nodes == 0) return fail(err, "cluster has no nodes");
  // every combination of the @cluster choices
  std::vector<std::map<std::string, int64_t>> configs{{}};
  for (const SearchDim& d : p.super_dims) {
    std::vector<std::map<std::string, int64_t>> next;
    for (const auto& c : configs)
      for (int64_t v : d.choices) {
        auto m = c;
        m[d.name] = v;
        next.push_back(std::move(m));
      }
    configs.swap(next);
  }
  std::string last_err;
  for (const auto& supers : configs) {
    PlanRequest rq;
    rq.dims = dims;
    rq.supers = supers;
    rq.nodes = fp.nodes;
    for (const ScalarDecl& s : p.scalars) {
      PhScalar z{};
      z.dtype = s.dtype;
      rq.scalars[s.name] = z;   // values do not matter for the shape of the plan
    }
    Plan pl;
    std::string e;
    if (!make_plan(p, rq, &pl, &e)) {
      last_err = e;
      continue;
    }
    size_t out_t = p.tensors.size() - 1;
    for (size_t t = 0; t < p.tensors.size(); t++)
      if (p.tensors[t].mode == PH_WRITE || p.tensors[t].mode == PH_RMW) {
        out_t = t;
        break;
      }
    uint64_t parallelism = 1;
    for (uint64_t g : pl.super_grids[out_t]) parallelism *= g;
    if (parallelism < fp.nodes) continue;             // some node would have nothing to do
    if (pl.peak_resident > fp.vram_bytes) continue;   // does not fit
    // busiest node: 2 * product of the distinct supertile axes of each compute
    uint64_t max_flops = 0, max_bytes = 0;
    for (const auto& segs : pl.node_segments) {
      uint64_t flops = 0;
      for (const Segment& s : segs)
        for (const OwnedInstr& oi : s.instrs) {
          if (oi.in.op != PH_OP_COMPUTE) continue;
          std::map<std::string, uint64_t> axes;
          for (const PhTileArg& a : oi.args) {
            const uint32_t t = phobos_tile_tensor(a.tile);
            for (size_t i = 0; i < p.tensors[t].super_syms.size(); i++) axes[p.tensors[t].super_syms[i]] = pl.super_shapes[t][i];
          }
          uint64_t f = 2;
          for (const auto& kv : axes) f *= kv.second;
          flops += f;
        }
      max_flops = std::max(max_flops, flops);
    }
    for (const auto& f : pl.fetches) {
      uint64_t bytes = 0;
      for (const auto& tf : f) {
        const uint32_t t = phobos_tile_tensor(tf.first);
        uint64_t b = dtype_bytes(p.tensors[t].dtype);
        for (uint64_t s : pl.super_shapes[t]) b *= s;
        bytes += b;
      }
      max_bytes = std::max(max_bytes, bytes);
    }
    RankedConfig rc;
    rc.supers = supers;
    rc.compute_sec = static_cast<double>(max_flops) / fp.leaf_flops_per_sec;
    rc.comm_sec = static_cast<double>(max_bytes) / fp.link_bytes_per_sec;
    rc.makespan_sec = std::max(rc.compute_sec, rc.comm_sec);
    rc.peak_resident = pl.peak_resident;
    rc.fetch_bytes = pl.fetch_bytes;
    out->push_back(std::move(rc));
  }
  if (out->empty())
    return fail(err, last_err.empty() ? "no feasible cluster config (all pruned by VRAM/parallelism)"
                                      : "no feasible cluster config: last error: " + last_err);
  // shortest makespan, then smallest working set, then more fetch bytes (larger supertiles)
  std::stable_sort(out->begin(), out->end(), [](const RankedConfig& a, const RankedConfig& b) {
    if (a.makespan_sec != b.makespan_sec) return a.makespan_sec < b.makespan_sec;
    if (a.peak_resident != b.peak_resident) return a.peak_resident < b.peak_resident;
    return a.fetch_bytes > b.fetch_bytes;
  });
  return true;
}

}  // namespace plan
}  // namespace ph
