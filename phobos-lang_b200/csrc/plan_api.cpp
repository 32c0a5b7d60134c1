// C ABI of the `.ph` reader and the supertile planner (declared in include/phobos_leaf.h).
#include <cstring>
#include <fstream>
#include <sstream>

#include "host.h"
#include "plan.h"

using namespace ph;
using namespace ph::plan;

struct PhProgram {
  KernelDecl decl;
  Program prog;
  bool clustered = false;      // compile_program succeeded
  std::string cluster_error;   // why not, otherwise
  std::string text;            // describe()
};

struct PhPlan {
  Plan plan;
};

struct PhPlanRequest {
  PlanRequest rq;
};

extern "C" {

PhProgram* phobos_program_parse(const char* source_text, int32_t kernel_index) {
  clear_error();
  if (!source_text) {
    fail(PH_ERR_INVALID, "null source text");
    return nullptr;
  }
  std::vector<KernelDecl> ks;
  std::string err;
  if (!parse_kernels(source_text, &ks, &err)) {
    fail(PH_ERR_PARSE, "%s", err.c_str());
    return nullptr;
  }
  if (kernel_index < 0 || kernel_index >= static_cast<int32_t>(ks.size())) {
    fail(PH_ERR_INVALID, "source holds %zu kernel(s), index %d asked", ks.size(), kernel_index);
    return nullptr;
  }
  PhProgram* p = new PhProgram();
  p->decl = ks[kernel_index];
  p->clustered = compile_program(p->decl, &p->prog, &p->cluster_error);
  if (p->clustered) p->text = describe(p->prog);
  return p;
}

void phobos_program_free(PhProgram* p) { delete p; }

const char* phobos_program_kernel_name(const PhProgram* p) { return p ? p->decl.name.c_str() : ""; }
int32_t phobos_program_n_params(const PhProgram* p) { return p ? static_cast<int32_t>(p->decl.params.size()) : 0; }
static const Param* param_at(const PhProgram* p, int32_t i) {
  return (p && i >= 0 && i < static_cast<int32_t>(p->decl.params.size())) ? &p->decl.params[i] : nullptr;
}
const char* phobos_program_param_name(const PhProgram* p, int32_t i) {
  const Param* q = param_at(p, i);
  return q ? q->name.c_str() : "";
}
int32_t phobos_program_param_is_tensor(const PhProgram* p, int32_t i) {
  const Param* q = param_at(p, i);
  return q ? (q->is_tensor ? 1 : 0) : -1;
}
int32_t phobos_program_param_dtype(const PhProgram* p, int32_t i) {
  const Param* q = param_at(p, i);
  return q ? q->dtype : -1;
}
int32_t phobos_program_param_rank(const PhProgram* p, int32_t i) {
  const Param* q = param_at(p, i);
  return q ? static_cast<int32_t>(q->dims.size()) : -1;
}
/* symbolic dims return their name and *literal = -1; literal dims return "" and the value */
const char* phobos_program_param_dim(const PhProgram* p, int32_t i, int32_t axis, int64_t* literal) {
  const Param* q = param_at(p, i);
  if (!q || axis < 0 || axis >= static_cast<int32_t>(q->dims.size())) return "";
  if (literal) *literal = q->dims[axis].sym ? -1 : q->dims[axis].value;
  return q->dims[axis].sym ? q->dims[axis].name.c_str() : "";
}
int32_t phobos_program_n_attrs(const PhProgram* p) { return p ? static_cast<int32_t>(p->decl.attrs.size()) : 0; }
const char* phobos_program_attr_name(const PhProgram* p, int32_t i) {
  return (p && i >= 0 && i < static_cast<int32_t>(p->decl.attrs.size())) ? p->decl.attrs[i].name.c_str() : "";
}
/* The expanded choices of search dimension `dim` of attribute `attr` ("cluster", "autotune"): count, values into out. */
int32_t phobos_program_search_choices(const PhProgram* p, const char* attr, const char* dim, int64_t* out, int32_t cap) {
  if (!p || !attr || !dim) return -1;
  for (const Attribute& a : p->decl.attrs)
    if (a.name == attr)
      for (const AttrArg& g : a.args)
        if (g.kind == AttrArg::SEARCH && g.name == dim) {
          std::vector<int64_t> c = search_choices(g.declared);
          for (int32_t i = 0; i < static_cast<int32_t>(c.size()) && i < cap; i++) out[i] = c[i];
          return static_cast<int32_t>(c.size());
        }
  return -1;
}
int32_t phobos_program_has_attr(const PhProgram* p, const char* attr) {
  if (!p || !attr) return 0;
  for (const Attribute& a : p->decl.attrs)
    if (a.name == attr) return 1;
  return 0;
}
/* 1 when the kernel could be read as a cluster program; otherwise 0 and the reason as last error */
int32_t phobos_program_is_clustered(const PhProgram* p) {
  if (!p) return 0;
  if (!p->clustered) fail(PH_ERR_UNSUPPORTED, "%s", p->cluster_error.c_str());
  return p->clustered ? 1 : 0;
}
const char* phobos_program_describe(const PhProgram* p) { return (p && p->clustered) ? p->text.c_str() : ""; }
int32_t phobos_program_n_leaves(const PhProgram* p) { return (p && p->clustered) ? static_cast<int32_t>(p->prog.leaves.size()) : 0; }
const char* phobos_program_leaf_entry(const PhProgram* p, int32_t i) {
  return (p && p->clustered && i >= 0 && i < static_cast<int32_t>(p->prog.leaves.size())) ? p->prog.leaves[i].entry.c_str() : "";
}
int32_t phobos_program_n_tensors(const PhProgram* p) { return (p && p->clustered) ? static_cast<int32_t>(p->prog.tensors.size()) : 0; }
int32_t phobos_program_tensor_mode(const PhProgram* p, int32_t i) {
  return (p && p->clustered && i >= 0 && i < static_cast<int32_t>(p->prog.tensors.size())) ? p->prog.tensors[i].mode : -1;
}

/* Checks a job file's bindings against the kernel's signature: every tensor parameter
 * bound with the declared element type and rank, symbolic dims consistent with the `dim`
 * lines and across tensors, every scalar parameter bound with its type, and no tensor
 * the kernel writes bound read-only. */
int phobos_job_check(const PhJob* job, const PhProgram* p) {
  clear_error();
  if (!job || !p) return fail(PH_ERR_INVALID, "null job or program");
  std::map<std::string, int64_t> dims;
  for (int32_t i = 0; i < phobos_job_n_dims(job); i++) dims[phobos_job_dim_name(job, i)] = phobos_job_dim_value(job, i);
  int tensor_index = 0;
  for (const Param& prm : p->decl.params) {
    if (prm.is_tensor) {
      int found = -1;
      for (int32_t i = 0; i < phobos_job_n_tensors(job); i++)
        if (prm.name == phobos_job_tensor_name(job, i)) found = i;
      if (found < 0) return fail(PH_ERR_INVALID, "tensor parameter '%s' is not bound by the job", prm.name.c_str());
      if (phobos_job_tensor_dtype(job, found) != prm.dtype)
        return fail(PH_ERR_INVALID, "tensor '%s' is bound with element type %d but declared %d", prm.name.c_str(),
                    phobos_job_tensor_dtype(job, found), prm.dtype);
      if (phobos_job_tensor_rank(job, found) != static_cast<int32_t>(prm.dims.size()))
        return fail(PH_ERR_INVALID, "tensor '%s' is bound with rank %d but declared with rank %zu", prm.name.c_str(),
                    phobos_job_tensor_rank(job, found), prm.dims.size());
      for (size_t ax = 0; ax < prm.dims.size(); ax++) {
        const int64_t have = phobos_job_tensor_dim(job, found, static_cast<int32_t>(ax));
        if (prm.dims[ax].sym) {
          auto it = dims.find(prm.dims[ax].name);
          if (it == dims.end()) {
            dims[prm.dims[ax].name] = have;   // first use binds it
          } else if (it->second != have) {
            return fail(PH_ERR_INVALID, "tensor '%s' axis %zu is %lld but dim %s = %lld", prm.name.c_str(), ax,
                        static_cast<long long>(have), prm.dims[ax].name.c_str(), static_cast<long long>(it->second));
          }
        } else if (prm.dims[ax].value != have) {
          return fail(PH_ERR_INVALID, "tensor '%s' axis %zu is %lld but declared %lld", prm.name.c_str(), ax,
                      static_cast<long long>(have), static_cast<long long>(prm.dims[ax].value));
        }
      }
      if (p->clustered) {
        const int kmode = p->prog.tensors[tensor_index].mode;
        const int jmode = phobos_job_tensor_mode(job, found);
        if (kmode != PH_READ && jmode == PH_READ)
          return fail(PH_ERR_INVALID, "tensor '%s' is written by the kernel but bound read-only", prm.name.c_str());
      }
      tensor_index++;
    } else {
      int found = -1;
      for (int32_t i = 0; i < phobos_job_n_scalars(job); i++)
        if (prm.name == phobos_job_scalar_name(job, i)) found = i;
      if (found < 0) return fail(PH_ERR_INVALID, "scalar parameter '%s' is unbound", prm.name.c_str());
      if (phobos_job_scalar_dtype(job, found) != prm.dtype)
        return fail(PH_ERR_INVALID, "scalar '%s' bound as type %d but declared %d", prm.name.c_str(),
                    phobos_job_scalar_dtype(job, found), prm.dtype);
    }
  }
  return PH_OK;
}

/* ---- plan requests ----------------------------------------------------------------------------- */
PhPlanRequest* phobos_plan_request_new(uint32_t nodes, uint64_t budget, int32_t policy) {
  PhPlanRequest* r = new PhPlanRequest();
  r->rq.nodes = nodes;
  r->rq.budget = budget;
  r->rq.policy = policy;
  return r;
}
void phobos_plan_request_free(PhPlanRequest* r) { delete r; }
void phobos_plan_request_dim(PhPlanRequest* r, const char* name, int64_t v) { if (r && name) r->rq.dims[name] = v; }
void phobos_plan_request_super(PhPlanRequest* r, const char* name, int64_t v) { if (r && name) r->rq.supers[name] = v; }
void phobos_plan_request_scalar(PhPlanRequest* r, const char* name, int32_t dtype, uint64_t bits) {
  if (!r || !name) return;
  PhScalar s{};
  s.dtype = dtype;
  s.bits = bits;
  r->rq.scalars[name] = s;
}
void phobos_plan_request_default_supers(PhPlanRequest* r, const PhProgram* p) {
  if (!r || !p || !p->clustered) return;
  for (const auto& kv : default_supers(p->prog)) r->rq.supers[kv.first] = kv.second;
}
void phobos_plan_request_recover(PhPlanRequest* r, const uint32_t* dead, int32_t n_dead, const uint32_t* durable_tensor,
                                 const uint64_t* durable_lin, int32_t n_durable, uint16_t version, uint64_t iid_base) {
  if (!r) return;
  r->rq.recover = true;
  r->rq.dead.assign(dead, dead + (n_dead > 0 ? n_dead : 0));
  r->rq.durable.clear();
  for (int32_t i = 0; i < n_durable; i++) r->rq.durable.push_back({durable_tensor[i], durable_lin[i]});
  r->rq.version = version;
  r->rq.iid_base = iid_base;
}

PhPlan* phobos_plan_make(const PhProgram* p, const PhPlanRequest* r) {
  clear_error();
  if (!p || !r) {
    fail(PH_ERR_INVALID, "null program or request");
    return nullptr;
  }
  if (!p->clustered) {
    fail(PH_ERR_UNSUPPORTED, "%s", p->cluster_error.c_str());
    return nullptr;
  }
  PhPlan* pl = new PhPlan();
  std::string err;
  if (!make_plan(p->prog, r->rq, &pl->plan, &err)) {
    fail(PH_ERR_INVALID, "%s", err.c_str());
    delete pl;
    return nullptr;
  }
  return pl;
}
void phobos_plan_free(PhPlan* pl) { delete pl; }
int phobos_plan_validate(const PhPlan* pl) {
  clear_error();
  if (!pl) return fail(PH_ERR_INVALID, "null plan");
  std::string err;
  if (!validate_plan(pl->plan, &err)) return fail(PH_ERR_STATE, "%s", err.c_str());
  return PH_OK;
}
uint32_t phobos_plan_n_nodes(const PhPlan* pl) { return pl ? static_cast<uint32_t>(pl->plan.node_segments.size()) : 0; }
int32_t phobos_plan_n_segments(const PhPlan* pl, uint32_t node) {
  return (pl && node < pl->plan.node_segments.size()) ? static_cast<int32_t>(pl->plan.node_segments[node].size()) : 0;
}
static const Segment* seg_at(const PhPlan* pl, uint32_t node, int32_t s) {
  if (!pl || node >= pl->plan.node_segments.size()) return nullptr;
  const auto& v = pl->plan.node_segments[node];
  return (s >= 0 && s < static_cast<int32_t>(v.size())) ? &v[s] : nullptr;
}
uint64_t phobos_plan_segment_id(const PhPlan* pl, uint32_t node, int32_t s) {
  const Segment* g = seg_at(pl, node, s);
  return g ? g->id : 0;
}
int32_t phobos_plan_segment_n_instrs(const PhPlan* pl, uint32_t node, int32_t s) {
  const Segment* g = seg_at(pl, node, s);
  return g ? static_cast<int32_t>(g->flat.size()) : 0;
}
const PhInstr* phobos_plan_segment_instrs(const PhPlan* pl, uint32_t node, int32_t s) {
  const Segment* g = seg_at(pl, node, s);
  return (g && !g->flat.empty()) ? g->flat.data() : nullptr;
}
void phobos_plan_segment_mem(const PhPlan* pl, uint32_t node, int32_t s, uint64_t* peak, uint64_t* incremental) {
  const Segment* g = seg_at(pl, node, s);
  if (peak) *peak = g ? g->peak : 0;
  if (incremental) *incremental = g ? g->incremental : 0;
}
uint64_t phobos_plan_fetch_bytes(const PhPlan* pl) { return pl ? pl->plan.fetch_bytes : 0; }
uint64_t phobos_plan_peak_resident(const PhPlan* pl) { return pl ? pl->plan.peak_resident : 0; }
uint64_t phobos_plan_max_iid(const PhPlan* pl) { return pl ? pl->plan.max_iid : 0; }
int32_t phobos_plan_n_stores(const PhPlan* pl) { return pl ? static_cast<int32_t>(pl->plan.stores.size()) : 0; }
void phobos_plan_store(const PhPlan* pl, int32_t i, uint64_t* iid, uint32_t* node, uint32_t* tensor, uint64_t* lin) {
  if (!pl || i < 0 || i >= static_cast<int32_t>(pl->plan.stores.size())) return;
  const StoreRec& s = pl->plan.stores[i];
  if (iid) *iid = s.iid;
  if (node) *node = s.node;
  if (tensor) *tensor = s.tensor;
  if (lin) *lin = s.lin;
}
int32_t phobos_plan_super_shape(const PhPlan* pl, uint32_t tensor, uint64_t* shape, uint64_t* grid, int32_t cap) {
  if (!pl || tensor >= pl->plan.super_shapes.size()) return -1;
  const auto& s = pl->plan.super_shapes[tensor];
  for (int32_t i = 0; i < static_cast<int32_t>(s.size()) && i < cap; i++) {
    if (shape) shape[i] = s[i];
    if (grid) grid[i] = pl->plan.super_grids[tensor][i];
  }
  return static_cast<int32_t>(s.size());
}
int32_t phobos_plan_owner(const PhPlan* pl, uint32_t tensor, uint64_t lin) {
  if (!pl) return -1;
  auto it = pl->plan.output_owner.find({tensor, lin});
  return it == pl->plan.output_owner.end() ? -1 : static_cast<int32_t>(it->second);
}

/* ---- supertile autotuner (cost model) -------------------------------------------------------------- */
struct PhTuneResult {
  std::vector<RankedConfig> ranked;
};
PhTuneResult* phobos_autotune(const PhProgram* p, const PhPlanRequest* dims_from, uint32_t nodes, uint64_t vram_bytes,
                              double link_bytes_per_sec, double leaf_flops_per_sec) {
  clear_error();
  if (!p || !dims_from) {
    fail(PH_ERR_INVALID, "null program or request");
    return nullptr;
  }
  if (!p->clustered) {
    fail(PH_ERR_UNSUPPORTED, "%s", p->cluster_error.c_str());
    return nullptr;
  }
  Fingerprint fp;
  fp.nodes = nodes;
  fp.vram_bytes = vram_bytes;
  fp.link_bytes_per_sec = link_bytes_per_sec;
  fp.leaf_flops_per_sec = leaf_flops_per_sec;
  PhTuneResult* r = new PhTuneResult();
  std::string err;
  if (!autotune(p->prog, dims_from->rq.dims, fp, &r->ranked, &err)) {
    fail(PH_ERR_INVALID, "%s", err.c_str());
    delete r;
    return nullptr;
  }
  return r;
}
void phobos_autotune_free(PhTuneResult* r) { delete r; }
int32_t phobos_autotune_n(const PhTuneResult* r) { return r ? static_cast<int32_t>(r->ranked.size()) : 0; }
int64_t phobos_autotune_super(const PhTuneResult* r, int32_t i, const char* name) {
  if (!r || i < 0 || i >= static_cast<int32_t>(r->ranked.size()) || !name) return -1;
  auto it = r->ranked[i].supers.find(name);
  return it == r->ranked[i].supers.end() ? -1 : it->second;
}
void phobos_autotune_cost(const PhTuneResult* r, int32_t i, double* makespan, double* compute, double* comm, uint64_t* peak,
                          uint64_t* fetch_bytes) {
  if (!r || i < 0 || i >= static_cast<int32_t>(r->ranked.size())) return;
  const RankedConfig& c = r->ranked[i];
  if (makespan) *makespan = c.makespan_sec;
  if (compute) *compute = c.compute_sec;
  if (comm) *comm = c.comm_sec;
  if (peak) *peak = c.peak_resident;
  if (fetch_bytes) *fetch_bytes = c.fetch_bytes;
}

}  // extern "C"
