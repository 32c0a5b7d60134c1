// Instruction executor: the pod's Engine (phobos-pod/src/engine.rs) for one
// device, without the network.  It owns a device arena (TileStore,
// phobos-pod/src/tile_store.rs), keeps the dependency table of issued
// instructions and runs ALLOC / LOAD / FETCH / COMPUTE / STORE / FREE with the
// reference's semantics:
//   - an instruction becomes ready when every dependency that is present in
//     the table has completed (engine.rs:282-323, 777-789)
//   - ALLOCs that do not fit are parked and retried after each FREE
//     (engine.rs:400-410, 736-742); if nothing else can make progress the
//     parked ALLOCs fail with "device arena exhausted" (engine.rs:752-775)
//   - COMPUTE resolves the kernel id to an entry name, builds row-major tensor
//     descriptors from the tile table (engine.rs:588-601) and enqueues the
//     native kernel on the compute stream (the reference rotates kernels and copies over four
//     streams; here copies rotate over three and leaves have one of their own), completion by
//     event (engine.rs:632-650, 655-687); Write / RMW tiles become resident then
//   - FETCH pulls a resident tile from a peer executor; on one box this is a
//     device-to-device copy over NVLink (cudaMemcpyPeerAsync) where the
//     reference stages through host memory and gRPC (engine.rs:511-540)
//   - FREE waits until the tile was served `expected_serves` times
//     (engine.rs:412-422)
// Tiles carry their element type, so f16 jobs work (the reference's store
// sizes every tile as 4-byte elements, tile_store.rs:110-113).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/phobos_leaf.h"
#include "host.h"

using namespace ph;

namespace {

struct Slab {
  uint64_t addr;
  uint64_t cls;
};

// One cudaMalloc slab, bump allocation, exact-fit size classes with free
// lists (tile_store.rs:13-83).
struct Arena {
  char* base = nullptr;
  uint64_t cap = 0, bump = 0, used = 0;
  std::map<uint64_t, std::vector<uint64_t>> free_lists;

  bool can_alloc(uint64_t bytes) const {
    const uint64_t cls = phobos_size_class(bytes);
    auto it = free_lists.find(cls);
    if (it != free_lists.end() && !it->second.empty()) return true;
    const uint64_t off = (bump + 255) & ~uint64_t(255);
    return off + cls <= cap;
  }
  bool alloc(uint64_t bytes, Slab* out) {
    const uint64_t cls = phobos_size_class(bytes);
    auto it = free_lists.find(cls);
    if (it != free_lists.end() && !it->second.empty()) {
      out->addr = it->second.back();
      out->cls = cls;
      it->second.pop_back();
      used += cls;
      return true;
    }
    const uint64_t off = (bump + 255) & ~uint64_t(255);
    if (off + cls > cap) return false;
    bump = off + cls;
    out->addr = reinterpret_cast<uint64_t>(base) + off;
    out->cls = cls;
    used += cls;
    return true;
  }
  void dealloc(const Slab& s) {
    free_lists[s.cls].push_back(s.addr);
    used -= s.cls;
  }
};

struct TileBuf {
  Slab slab;
  std::vector<uint64_t> shape;
  int dtype = PH_F32;
  uint64_t elems = 0;
  bool resident = false;
  uint32_t serves = 0, expected_serves = 0;
};

struct Node {
  PhInstr in;  // pointers inside are re-pointed at the owned copies below
  std::vector<uint64_t> deps;
  std::vector<PhTileArg> args;
  std::vector<PhScalar> scalars;
  int remaining = 0;
  std::vector<uint64_t> dependents;
};

struct Inflight {
  cudaEvent_t event;
  uint64_t iid;
  std::vector<uint64_t> wrote;  // tiles that become resident when the event completes
  void* host_stage;             // pinned staging buffer to release on completion (LOAD)
  PhExecutor* served_by;        // FETCH: the peer whose tile `wrote[0]` is being copied, to be credited with a serve
  uint64_t serve_bytes;
};

struct KernelEntry {
  std::string entry;
  int kind_hint;
};

struct TensorMetaOwned {
  std::string uri;
  int dtype;
  std::vector<uint64_t> shape;
  int mode;
  // device://<gpu>/0x<address>: the tensor lives row-major in that GPU's memory (HBM-resident storage); LOAD and
  // STORE are then 2-D device copies over NVLink instead of file reads through pinned staging
  bool on_device = false;
  int storage_device = -1;
  char* storage_base = nullptr;
};

// Parses device://<gpu>/0x<hex address>; false when the URI is of another scheme.
bool parse_device_uri(const std::string& uri, int* dev, char** base) {
  if (uri.compare(0, 9, "device://") != 0) return false;
  char* end = nullptr;
  const char* p = uri.c_str() + 9;
  const long d = strtol(p, &end, 10);
  if (end == p || *end != '/' || d < 0) return false;
  const char* q = end + 1;
  const unsigned long long a = strtoull(q, &end, 16);
  if (end == q || *end != 0 || a == 0) return false;
  *dev = static_cast<int>(d);
  *base = reinterpret_cast<char*>(static_cast<uintptr_t>(a));
  return true;
}

}  // namespace

struct PhExecutor {
  int device = 0;
  uint32_t node_id = 0;
  Arena arena;
  std::unordered_map<uint64_t, TileBuf> tiles;
  std::vector<TensorMetaOwned> tensors;
  std::unordered_map<uint32_t, KernelEntry> kernels;
  std::unordered_map<uint32_t, PhExecutor*> peers;
  std::unordered_map<uint64_t, Node> table;
  std::deque<uint64_t> ready;
  std::vector<Inflight> inflight;
  std::vector<uint64_t> deferred_allocs, deferred_frees, deferred_fetches;
  std::vector<PhCompletion> completions;
  cudaStream_t streams[4] = {nullptr, nullptr, nullptr, nullptr};
  int next_stream = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  uint64_t served_bytes = 0;
  cudaEvent_t run_start = nullptr;   // recorded on the device when phobos_executor_run starts
  float last_run_ms = -1.0f;         // device time from there to the last operation of the run
  int first_failure = 0;
  std::string first_failure_msg;
  // guards the tile table and counters against a peer's FETCH running on another host thread
  std::mutex mu;
};

namespace {

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

void complete(PhExecutor* ex, uint64_t iid) {
  auto it = ex->table.find(iid);
  if (it == ex->table.end()) return;
  std::vector<uint64_t> dependents = std::move(it->second.dependents);
  ex->table.erase(it);
  for (uint64_t d : dependents) {
    auto dn = ex->table.find(d);
    if (dn != ex->table.end() && --dn->second.remaining == 0) ex->ready.push_back(d);
  }
  ex->completions.push_back({iid, 0u, 0ull});
}

void fail_instr(PhExecutor* ex, uint64_t iid, int code, const std::string& msg) {
  // engine.rs:744-750: report the failure; the instruction never completes
  if (ex->first_failure == 0) {
    ex->first_failure = code;
    ex->first_failure_msg = "instr " + std::to_string(iid) + ": " + msg;
  }
  ex->completions.push_back({iid, static_cast<uint32_t>(-code), 0ull});
  ex->table.erase(iid);
}

bool try_alloc(PhExecutor* ex, uint64_t iid, const Node& n) {
  uint64_t elems = 1;
  for (int d = 0; d < n.in.shape_rank; d++) elems *= n.in.shape[d];
  const uint64_t bytes = elems * phobos_dtype_bytes(n.in.data_type);
  if (!ex->arena.can_alloc(bytes)) return false;
  TileBuf tb;
  ex->arena.alloc(bytes, &tb.slab);
  tb.shape.assign(n.in.shape, n.in.shape + n.in.shape_rank);
  tb.dtype = n.in.data_type;
  tb.elems = elems;
  ex->tiles[n.in.tile] = tb;
  complete(ex, iid);
  return true;
}

void retry_allocs(PhExecutor* ex) {
  std::vector<uint64_t> parked;
  parked.swap(ex->deferred_allocs);
  for (uint64_t iid : parked) {
    auto it = ex->table.find(iid);
    if (it == ex->table.end()) continue;
    if (!try_alloc(ex, iid, it->second)) ex->deferred_allocs.push_back(iid);
  }
}

bool try_free(PhExecutor* ex, uint64_t iid, uint64_t tile) {
  auto t = ex->tiles.find(tile);
  if (t == ex->tiles.end()) {
    fail_instr(ex, iid, PH_ERR_STATE, "free of unknown tile");
    return false;
  }
  if (t->second.serves < t->second.expected_serves) return false;
  ex->arena.dealloc(t->second.slab);
  ex->tiles.erase(t);
  complete(ex, iid);
  return true;
}

void retry_frees(PhExecutor* ex) {
  std::vector<uint64_t> parked;
  parked.swap(ex->deferred_frees);
  bool freed = false;
  for (uint64_t iid : parked) {
    auto it = ex->table.find(iid);
    if (it == ex->table.end()) continue;
    if (try_free(ex, iid, it->second.in.tile)) freed = true;
    else if (ex->table.count(iid)) ex->deferred_frees.push_back(iid);
  }
  if (freed) retry_allocs(ex);
}

// Copies (LOAD, FETCH, STORE) rotate over streams 1..3; stream 0 belongs to the leaves, so that a
// COMPUTE whose operands are resident never queues behind a transfer it does not depend on (seen in a
// host-side timeline of the 16384^3 plan on four GPUs: init leaves of 30 us completing 3 ms late behind
// 64 MB peer copies that shared their stream).
cudaStream_t pick_stream(PhExecutor* ex) {
  cudaStream_t s = ex->streams[1 + ex->next_stream];
  ex->next_stream = (ex->next_stream + 1) % 3;
  return s;
}

bool track(PhExecutor* ex, cudaStream_t s, uint64_t iid, std::vector<uint64_t> wrote, void* stage,
           PhExecutor* served_by = nullptr, uint64_t serve_bytes = 0) {
  cudaEvent_t ev;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(ev, s) != cudaSuccess) {
    fail_instr(ex, iid, PH_ERR_DEVICE, "event record failed");
    return false;
  }
  ex->inflight.push_back({ev, iid, std::move(wrote), stage, served_by, serve_bytes});
  return true;
}

// A region of a device-resident tensor as a 2-D copy: rows x row_bytes at `ptr`, rows `pitch` bytes apart.
// Returns false (with the error set) when the region does not lie inside the tensor.
bool device_region(const TensorMetaOwned& m, const PhRegion& rg, size_t es, char** ptr, size_t* pitch, size_t* row_bytes,
                   size_t* rows) {
  if (rg.rank == 1) {
    uint64_t total = 1;
    for (uint64_t d : m.shape) total *= d;
    if (rg.offset[0] > total || rg.shape[0] > total - rg.offset[0]) {
      fail(PH_ERR_INVALID, "region exceeds the tensor's %llu elements", (unsigned long long)total);
      return false;
    }
    *ptr = m.storage_base + rg.offset[0] * es;
    *pitch = *row_bytes = rg.shape[0] * es;
    *rows = 1;
    return true;
  }
  if (rg.rank != 2 || m.shape.size() != 2) {
    fail(PH_ERR_UNSUPPORTED, "device storage supports rank <= 2 regions of rank-2 tensors");
    return false;
  }
  for (int d = 0; d < 2; d++)
    if (rg.offset[d] > m.shape[d] || rg.shape[d] > m.shape[d] - rg.offset[d]) {
      fail(PH_ERR_INVALID, "region axis %d exceeds the tensor extent %llu", d, (unsigned long long)m.shape[d]);
      return false;
    }
  *pitch = m.shape[1] * es;
  *ptr = m.storage_base + rg.offset[0] * *pitch + rg.offset[1] * es;
  *row_bytes = rg.shape[1] * es;
  *rows = rg.shape[0];
  return true;
}

void do_load(PhExecutor* ex, uint64_t iid, const Node& n) {
  if (n.in.tensor >= ex->tensors.size()) return fail_instr(ex, iid, PH_ERR_STATE, "LOAD of unknown tensor");
  auto t = ex->tiles.find(n.in.tile);
  if (t == ex->tiles.end()) return fail_instr(ex, iid, PH_ERR_STATE, "LOAD into unknown tile");
  const TensorMetaOwned& m = ex->tensors[n.in.tensor];
  const size_t es = phobos_dtype_bytes(m.dtype);
  uint64_t total = 1;
  for (int d = 0; d < n.in.region.rank; d++) total *= n.in.region.shape[d];
  if (total != t->second.elems || m.dtype != t->second.dtype)
    return fail_instr(ex, iid, PH_ERR_STATE, "LOAD region does not match the tile");
  if (m.on_device) {
    // gather the region's rows into the contiguous tile, device to device (peer copy when the tensor lives on
    // another GPU); asynchronous, completion by event like every other operation
    char* src;
    size_t pitch, row_bytes, rows;
    if (!device_region(m, n.in.region, es, &src, &pitch, &row_bytes, &rows))
      return fail_instr(ex, iid, PH_ERR_INVALID, std::string("LOAD: ") + last_error());
    cudaStream_t s = pick_stream(ex);
    cudaError_t e = cudaMemcpy2DAsync(reinterpret_cast<void*>(t->second.slab.addr), row_bytes, src, pitch, row_bytes, rows,
                                      cudaMemcpyDefault, s);
    if (e != cudaSuccess) return fail_instr(ex, iid, PH_ERR_DEVICE, std::string("LOAD: ") + cudaGetErrorString(e));
    track(ex, s, iid, {n.in.tile}, nullptr);
    return;
  }
  void* stage = nullptr;
  if (cudaMallocHost(&stage, total * es) != cudaSuccess) return fail_instr(ex, iid, PH_ERR_DEVICE, "pinned staging alloc");
  int rc = phobos_storage_load(m.uri.c_str(), m.shape.data(), (int32_t)m.shape.size(), &n.in.region, es, stage);
  if (rc) {
    cudaFreeHost(stage);
    return fail_instr(ex, iid, rc, std::string("LOAD: ") + last_error());
  }
  cudaStream_t s = pick_stream(ex);
  if (cudaMemcpyAsync(reinterpret_cast<void*>(t->second.slab.addr), stage, total * es, cudaMemcpyHostToDevice, s) !=
      cudaSuccess) {
    cudaFreeHost(stage);
    return fail_instr(ex, iid, PH_ERR_DEVICE, "LOAD: host-to-device copy failed");
  }
  track(ex, s, iid, {n.in.tile}, stage);
}

void do_store(PhExecutor* ex, uint64_t iid, const Node& n) {
  if (n.in.tensor >= ex->tensors.size()) return fail_instr(ex, iid, PH_ERR_STATE, "STORE of unknown tensor");
  auto t = ex->tiles.find(n.in.tile);
  if (t == ex->tiles.end()) return fail_instr(ex, iid, PH_ERR_STATE, "STORE of unknown tile");
  const TensorMetaOwned& m = ex->tensors[n.in.tensor];
  const size_t es = phobos_dtype_bytes(t->second.dtype);
  // storage.rs store_f32: "store data/region length mismatch"
  uint64_t total = 1;
  for (int d = 0; d < n.in.region.rank; d++) total *= n.in.region.shape[d];
  if (total != t->second.elems || m.dtype != t->second.dtype)
    return fail_instr(ex, iid, PH_ERR_STATE, "STORE region does not match the tile");
  if (m.on_device) {
    // the producer of the tile has completed (STORE depends on it and completion is event-based), so the scatter
    // may run on any stream
    char* dst;
    size_t pitch, row_bytes, rows;
    if (!device_region(m, n.in.region, es, &dst, &pitch, &row_bytes, &rows))
      return fail_instr(ex, iid, PH_ERR_INVALID, std::string("STORE: ") + last_error());
    cudaStream_t s = pick_stream(ex);
    cudaError_t e = cudaMemcpy2DAsync(dst, pitch, reinterpret_cast<void*>(t->second.slab.addr), row_bytes, row_bytes, rows,
                                      cudaMemcpyDefault, s);
    if (e != cudaSuccess) return fail_instr(ex, iid, PH_ERR_DEVICE, std::string("STORE: ") + cudaGetErrorString(e));
    track(ex, s, iid, {}, nullptr);
    return;
  }
  std::vector<char> host(t->second.elems * es);
  // device-to-host on the executor thread (engine.rs:472-473); all streams are
  // drained first because the producer may have run on any of them
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpy(host.data(), reinterpret_cast<void*>(t->second.slab.addr), host.size(), cudaMemcpyDeviceToHost) !=
          cudaSuccess)
    return fail_instr(ex, iid, PH_ERR_DEVICE, "STORE: device-to-host copy failed");
  int rc = phobos_storage_store(m.uri.c_str(), m.shape.data(), (int32_t)m.shape.size(), &n.in.region, es, host.data());
  if (rc) return fail_instr(ex, iid, rc, std::string("STORE: ") + last_error());
  complete(ex, iid);
}

// Returns false when the source tile is not resident yet (retry later).
bool do_fetch(PhExecutor* ex, uint64_t iid, const Node& n) {
  auto pe = ex->peers.find(n.in.from_node);
  if (pe == ex->peers.end()) {
    fail_instr(ex, iid, PH_ERR_STATE, "no peer for FETCH");
    return true;
  }
  PhExecutor* peer = pe->second;
  // try_lock: two executors fetching from each other must not wait on each other's lock.
  // A fetch from this executor itself already runs under its own lock.
  std::unique_lock<std::mutex> peer_lock(peer->mu, std::defer_lock);
  if (peer != ex && !peer_lock.try_lock()) return false;
  auto src = peer->tiles.find(n.in.tile);
  // served once resident (engine.rs:698-705); a tile is marked resident only after the event of its
  // producer has completed, so its bytes are final and no synchronisation with the peer's streams is needed
  if (src == peer->tiles.end() || !src->second.resident) return false;
  auto dst = ex->tiles.find(n.in.tile);
  if (dst == ex->tiles.end()) {
    fail_instr(ex, iid, PH_ERR_STATE, "FETCH into unknown tile");
    return true;
  }
  const size_t bytes = src->second.elems * phobos_dtype_bytes(src->second.dtype);
  if (dst->second.elems != src->second.elems || dst->second.dtype != src->second.dtype) {
    fail_instr(ex, iid, PH_ERR_STATE, "FETCH: tile shapes differ between peers");
    return true;
  }
  cudaStream_t s = pick_stream(ex);
  cudaError_t e = cudaMemcpyPeerAsync(reinterpret_cast<void*>(dst->second.slab.addr), ex->device,
                                      reinterpret_cast<void*>(src->second.slab.addr), peer->device, bytes, s);
  if (e != cudaSuccess) {
    fail_instr(ex, iid, PH_ERR_DEVICE, std::string("FETCH: ") + cudaGetErrorString(e));
    return true;
  }
  // Event-tracked like COMPUTE.  The serve is credited when the copy has completed (the reference
  // serves a finished device-to-host copy), so the home cannot FREE the tile under the copy.
  track(ex, s, iid, {n.in.tile}, nullptr, peer, bytes);
  return true;
}

void do_compute(PhExecutor* ex, uint64_t iid, const Node& n) {
  auto k = ex->kernels.find(n.in.kernel);
  if (k == ex->kernels.end()) return fail_instr(ex, iid, PH_ERR_STATE, "COMPUTE of unknown kernel id");
  std::vector<PhTensor> tensors(n.args.size());
  std::vector<uint64_t> wrote;
  for (size_t i = 0; i < n.args.size(); i++) {
    auto t = ex->tiles.find(n.args[i].tile);
    if (t == ex->tiles.end()) return fail_instr(ex, iid, PH_ERR_STATE, "COMPUTE argument is an unknown tile");
    const TileBuf& tb = t->second;
    PhTensor& d = tensors[i];
    memset(&d, 0, sizeof(d));
    d.ptr = reinterpret_cast<void*>(tb.slab.addr);
    d.dtype = tb.dtype;
    d.rank = (int32_t)tb.shape.size();
    // row-major strides, innermost 1 (engine.rs:592-600)
    int64_t stride = 1;
    for (int r = d.rank - 1; r >= 0; r--) {
      d.sizes[r] = (int64_t)tb.shape[r];
      d.strides[r] = stride;
      stride *= (int64_t)tb.shape[r];
    }
    if (n.args[i].mode == PH_WRITE || n.args[i].mode == PH_RMW) wrote.push_back(n.args[i].tile);
  }
  // a kernel that comes with an `<name>_init` leaf is the accumulate step of a chain
  int32_t hint = k->second.kind_hint;
  {
    const std::string init_name = k->second.entry + "_init";
    for (const auto& kv : ex->kernels)
      if (kv.second.entry == init_name) {
        hint = (hint < 0 ? PH_KIND_AUTO : (hint & 0xFF)) | PH_LAUNCH_STEP_LEAF;
        break;
      }
  }
  const size_t need = phobos_launch_workspace_bytes(k->second.entry.c_str(), tensors.data(), (int32_t)tensors.size(),
                                                    hint);
  if (need > ex->workspace_bytes) {
    // grown on demand, outside any steady state; kernels using the old buffer are drained first
    cudaDeviceSynchronize();
    if (ex->workspace) cudaFree(ex->workspace);
    ex->workspace = nullptr;
    ex->workspace_bytes = 0;
    if (cudaMalloc(&ex->workspace, need) != cudaSuccess) return fail_instr(ex, iid, PH_ERR_DEVICE, "workspace allocation failed");
    ex->workspace_bytes = need;
  }
  // leaves run on stream 0 in issue order (those that use the shared workspace must not overlap anyway)
  cudaStream_t s = ex->streams[0];
  int rc = phobos_launch(k->second.entry.c_str(), tensors.data(), (int32_t)tensors.size(), n.scalars.data(),
                         (int32_t)n.scalars.size(), n.in.grid, n.in.cta, hint, ex->workspace,
                         ex->workspace_bytes, s);
  if (rc) return fail_instr(ex, iid, rc, std::string("COMPUTE: ") + last_error());
  track(ex, s, iid, std::move(wrote), nullptr);
}

void issue(PhExecutor* ex, uint64_t iid) {
  auto it = ex->table.find(iid);
  if (it == ex->table.end()) return;
  const Node& n = it->second;
  switch (n.in.op) {
    case PH_OP_ALLOC:
      if (!try_alloc(ex, iid, n)) ex->deferred_allocs.push_back(iid);
      break;
    case PH_OP_LOAD: do_load(ex, iid, n); break;
    case PH_OP_FETCH:
      if (!do_fetch(ex, iid, n)) ex->deferred_fetches.push_back(iid);
      break;
    case PH_OP_COMPUTE: do_compute(ex, iid, n); break;
    case PH_OP_STORE: do_store(ex, iid, n); break;
    case PH_OP_FREE: {
      auto t = ex->tiles.find(n.in.tile);
      if (t != ex->tiles.end()) t->second.expected_serves = n.in.expected_serves;
      if (try_free(ex, iid, n.in.tile)) retry_allocs(ex);
      else if (ex->table.count(iid)) ex->deferred_frees.push_back(iid);
      break;
    }
    default: fail_instr(ex, iid, PH_ERR_INVALID, "unknown opcode");
  }
}

bool poll_inflight(PhExecutor* ex) {
  bool progressed = false;
  for (size_t i = 0; i < ex->inflight.size();) {
    cudaError_t q = cudaEventQuery(ex->inflight[i].event);
    if (q == cudaErrorNotReady) {
      i++;
      continue;
    }
    if (q == cudaSuccess && ex->inflight[i].served_by != nullptr) {
      // a finished FETCH: credit the home with the serve (under its lock; try again next round if it is busy)
      PhExecutor* home = ex->inflight[i].served_by;
      std::unique_lock<std::mutex> home_lock(home->mu, std::defer_lock);
      if (home != ex && !home_lock.try_lock()) {
        i++;
        continue;
      }
      auto src = home->tiles.find(ex->inflight[i].wrote[0]);
      if (src != home->tiles.end()) src->second.serves++;
      home->served_bytes += ex->inflight[i].serve_bytes;
    }
    Inflight f = std::move(ex->inflight[i]);
    ex->inflight[i] = std::move(ex->inflight.back());
    ex->inflight.pop_back();
    cudaEventDestroy(f.event);
    if (f.host_stage) cudaFreeHost(f.host_stage);
    progressed = true;
    if (q != cudaSuccess) {
      fail_instr(ex, f.iid, PH_ERR_DEVICE, std::string("device error: ") + cudaGetErrorString(q));
      continue;
    }
    for (uint64_t w : f.wrote) {
      auto t = ex->tiles.find(w);
      if (t != ex->tiles.end()) t->second.resident = true;
    }
    complete(ex, f.iid);
  }
  return progressed;
}

}  // namespace

extern "C" {

PhExecutor* phobos_executor_create(int32_t device, uint32_t node_id, uint64_t arena_bytes) {
  clear_error();
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
    fail(PH_ERR_DEVICE, "executor: device %d not available", device);
    return nullptr;
  }
  DeviceGuard g(device);
  PhExecutor* ex = new PhExecutor();
  ex->device = device;
  ex->node_id = node_id;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, arena_bytes ? arena_bytes : 256);
  if (e != cudaSuccess) {
    fail(PH_ERR_DEVICE, "executor: arena of %llu bytes: %s", (unsigned long long)arena_bytes, cudaGetErrorString(e));
    delete ex;
    return nullptr;
  }
  ex->arena.base = static_cast<char*>(p);
  ex->arena.cap = arena_bytes;
  for (int i = 0; i < 4; i++) {
    if (cudaStreamCreateWithFlags(&ex->streams[i], cudaStreamNonBlocking) != cudaSuccess) {
      fail(PH_ERR_DEVICE, "executor: stream creation failed");
      phobos_executor_destroy(ex);
      return nullptr;
    }
  }
  return ex;
}

void phobos_executor_destroy(PhExecutor* ex) {
  if (!ex) return;
  DeviceGuard g(ex->device);
  cudaDeviceSynchronize();
  for (auto& f : ex->inflight) {
    cudaEventDestroy(f.event);
    if (f.host_stage) cudaFreeHost(f.host_stage);
  }
  for (int i = 0; i < 4; i++)
    if (ex->streams[i]) cudaStreamDestroy(ex->streams[i]);
  if (ex->workspace) cudaFree(ex->workspace);
  if (ex->arena.base) cudaFree(ex->arena.base);
  if (ex->run_start) cudaEventDestroy(ex->run_start);
  delete ex;
}

int phobos_executor_set_tensors(PhExecutor* ex, const PhTensorMeta* tensors, int32_t n) {
  clear_error();
  if (!ex || (n > 0 && !tensors)) return fail(PH_ERR_INVALID, "null argument");
  ex->tensors.clear();
  for (int32_t i = 0; i < n; i++) {
    if (tensors[i].rank < 1 || tensors[i].rank > 2) return fail(PH_ERR_UNSUPPORTED, "tensor %d: rank %d (1 or 2 supported)", i, tensors[i].rank);
    TensorMetaOwned m;
    m.uri = tensors[i].uri ? tensors[i].uri : "";
    m.dtype = tensors[i].dtype;
    m.shape.assign(tensors[i].shape, tensors[i].shape + tensors[i].rank);
    m.mode = tensors[i].mode;
    if (m.uri.compare(0, 9, "device://") == 0) {
      if (!parse_device_uri(m.uri, &m.storage_device, &m.storage_base))
        return fail(PH_ERR_INVALID, "tensor %d: malformed storage URI '%s' (device://<gpu>/0x<address>)", i, m.uri.c_str());
      int count = 0;
      if (cudaGetDeviceCount(&count) != cudaSuccess || m.storage_device >= count)
        return fail(PH_ERR_DEVICE, "tensor %d: no GPU %d", i, m.storage_device);
      if (m.storage_device != ex->device) {
        DeviceGuard g(ex->device);
        int can = 0;
        cudaDeviceCanAccessPeer(&can, ex->device, m.storage_device);
        if (!can) return fail(PH_ERR_DEVICE, "tensor %d: GPU %d cannot reach GPU %d", i, ex->device, m.storage_device);
        cudaError_t e = cudaDeviceEnablePeerAccess(m.storage_device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return fail(PH_ERR_DEVICE, "enable peer access %d -> %d: %s", ex->device, m.storage_device, cudaGetErrorString(e));
        cudaGetLastError();
      }
      m.on_device = true;
    }
    ex->tensors.push_back(m);
  }
  return PH_OK;
}

int phobos_executor_set_kernel(PhExecutor* ex, uint32_t kernel_id, const char* entry, int32_t kind_hint) {
  clear_error();
  if (!ex || !entry) return fail(PH_ERR_INVALID, "null argument");
  ex->kernels[kernel_id] = {entry, kind_hint};
  return PH_OK;
}

int phobos_executor_connect_peer(PhExecutor* ex, uint32_t node_id, PhExecutor* peer) {
  clear_error();
  if (!ex || !peer) return fail(PH_ERR_INVALID, "null argument");
  if (peer->device != ex->device) {
    DeviceGuard g(ex->device);
    int can = 0;
    cudaDeviceCanAccessPeer(&can, ex->device, peer->device);
    if (can) {
      cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
        return fail(PH_ERR_DEVICE, "enable peer access %d -> %d: %s", ex->device, peer->device, cudaGetErrorString(e));
      cudaGetLastError();
    }
  }
  ex->peers[node_id] = peer;
  return PH_OK;
}

int phobos_executor_issue(PhExecutor* ex, const PhInstr* instrs, int32_t n) {
  clear_error();
  if (!ex || (n > 0 && !instrs)) return fail(PH_ERR_INVALID, "null argument");
  // the whole segment is validated before any of it enters the table
  for (int32_t i = 0; i < n; i++) {
    const PhInstr& in = instrs[i];
    if (in.op == PH_OP_ALLOC && (in.shape_rank < 1 || in.shape_rank > 2))
      return fail(PH_ERR_UNSUPPORTED, "instr %llu: ALLOC rank %d (1 or 2 supported)", (unsigned long long)in.iid, in.shape_rank);
    if (in.op == PH_OP_ALLOC && phobos_dtype_bytes(in.data_type) == 0)
      return fail(PH_ERR_INVALID, "instr %llu: ALLOC of unknown element type %d", (unsigned long long)in.iid, in.data_type);
    if ((in.n_deps > 0 && !in.deps) || (in.n_args > 0 && !in.args) || (in.n_scalars > 0 && !in.scalars))
      return fail(PH_ERR_INVALID, "instr %llu: a list has a count but no pointer", (unsigned long long)in.iid);
  }
  // add nodes, then wire dependency counters (engine.rs:297-322)
  for (int32_t i = 0; i < n; i++) {
    const PhInstr& in = instrs[i];
    Node nd;
    nd.in = in;
    if (in.n_deps > 0 && in.deps) nd.deps.assign(in.deps, in.deps + in.n_deps);
    if (in.n_args > 0 && in.args) nd.args.assign(in.args, in.args + in.n_args);
    if (in.n_scalars > 0 && in.scalars) nd.scalars.assign(in.scalars, in.scalars + in.n_scalars);
    nd.in.deps = nullptr;
    nd.in.args = nullptr;
    nd.in.scalars = nullptr;
    ex->table[in.iid] = std::move(nd);
  }
  for (int32_t i = 0; i < n; i++) {
    Node& nd = ex->table[instrs[i].iid];
    int remaining = 0;
    for (uint64_t d : nd.deps) {
      auto dep = ex->table.find(d);
      if (dep != ex->table.end() && d != instrs[i].iid) {
        dep->second.dependents.push_back(instrs[i].iid);
        remaining++;
      }
    }
    nd.remaining = remaining;
    if (remaining == 0) ex->ready.push_back(instrs[i].iid);
  }
  return PH_OK;
}

int phobos_executor_run(PhExecutor* ex) {
  clear_error();
  if (!ex) return fail(PH_ERR_INVALID, "null executor");
  DeviceGuard g(ex->device);
  // device-side clock of this run: an event at its start; events after its last operation on every stream
  if (ex->run_start == nullptr) cudaEventCreate(&ex->run_start);
  for (int i = 0; i < 4; i++) cudaStreamSynchronize(ex->streams[i]);
  cudaEventRecord(ex->run_start, ex->streams[0]);
  ex->last_run_ms = -1.0f;
  int idle_rounds = 0;
  while (true) {
    std::unique_lock<std::mutex> self_lock(ex->mu);
    bool progressed = poll_inflight(ex);
    while (!ex->ready.empty()) {
      uint64_t iid = ex->ready.front();
      ex->ready.pop_front();
      issue(ex, iid);
      progressed = true;
    }
    if (!ex->deferred_fetches.empty()) {
      std::vector<uint64_t> parked;
      parked.swap(ex->deferred_fetches);
      for (uint64_t iid : parked) {
        auto it = ex->table.find(iid);
        if (it == ex->table.end()) continue;
        if (do_fetch(ex, iid, it->second)) progressed = true;
        else ex->deferred_fetches.push_back(iid);
      }
    }
    if (!ex->deferred_frees.empty()) retry_frees(ex);
    if (ex->first_failure) break;
    if (ex->table.empty() && ex->inflight.empty()) break;
    if (!progressed && ex->inflight.empty() && ex->ready.empty()) {
      // nothing runnable here: parked FETCHes / FREEs wait for a peer; parked
      // ALLOCs with nothing else pending can never fit (engine.rs:752-775)
      if (ex->deferred_fetches.empty() && ex->deferred_frees.empty()) {
        if (!ex->deferred_allocs.empty()) {
          std::vector<uint64_t> stuck;
          stuck.swap(ex->deferred_allocs);
          for (uint64_t iid : stuck)
            fail_instr(ex, iid, PH_ERR_STATE,
                       "device arena exhausted: the resident working set already fills the arena; raise the arena size");
        } else {
          ex->first_failure = PH_ERR_STATE;
          ex->first_failure_msg = "dependency cycle or dependency on an instruction that failed";
        }
        break;
      }
      // waiting on a peer that is driven by another thread: give up after a while
      if (++idle_rounds > 200000) {
        ex->first_failure = PH_ERR_STATE;
        ex->first_failure_msg = "stalled waiting for a peer (FETCH source never became resident, or FREE never served)";
        break;
      }
      self_lock.unlock();
      struct timespec ts = {0, 100000};  // 100 us, as the reference's idle sleep (engine.rs:225-230)
      nanosleep(&ts, nullptr);
    } else {
      idle_rounds = 0;
    }
  }
  if (ex->first_failure) {
    int code = ex->first_failure;
    fail(code, "%s", ex->first_failure_msg.c_str());
    ex->first_failure = 0;
    return code;
  }
  {
    float worst = 0.0f;
    cudaEvent_t end;
    if (cudaEventCreate(&end) == cudaSuccess) {
      for (int i = 0; i < 4; i++) {
        float ms = 0.0f;
        if (cudaEventRecord(end, ex->streams[i]) == cudaSuccess && cudaEventSynchronize(end) == cudaSuccess &&
            cudaEventElapsedTime(&ms, ex->run_start, end) == cudaSuccess && ms > worst)
          worst = ms;
      }
      cudaEventDestroy(end);
      ex->last_run_ms = worst;
    }
  }
  return PH_OK;
}

int32_t phobos_executor_drain_completions(PhExecutor* ex, PhCompletion* out, int32_t cap) {
  if (!ex || !out || cap <= 0) return 0;
  int32_t n = 0;
  while (n < cap && n < (int32_t)ex->completions.size()) {
    out[n] = ex->completions[n];
    n++;
  }
  ex->completions.erase(ex->completions.begin(), ex->completions.begin() + n);
  return n;
}

float phobos_executor_last_run_ms(const PhExecutor* ex) { return ex ? ex->last_run_ms : -1.0f; }
uint64_t phobos_executor_arena_used(const PhExecutor* ex) { return ex ? ex->arena.used : 0; }
uint64_t phobos_executor_served_bytes(const PhExecutor* ex) { return ex ? ex->served_bytes : 0; }

int phobos_executor_tile_addr(const PhExecutor* ex, uint64_t tile, void** addr_out, int32_t* resident_out) {
  clear_error();
  if (!ex) return fail(PH_ERR_INVALID, "null executor");
  auto t = ex->tiles.find(tile);
  if (t == ex->tiles.end()) return fail(PH_ERR_STATE, "unknown tile %#llx", (unsigned long long)tile);
  if (addr_out) *addr_out = reinterpret_cast<void*>(t->second.slab.addr);
  if (resident_out) *resident_out = t->second.resident ? 1 : 0;
  return PH_OK;
}

}  // extern "C"
