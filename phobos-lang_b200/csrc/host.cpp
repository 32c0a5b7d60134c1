// Host side of the leaf executor that needs no device code: tile ids, arena
// size classes, the seeded generator on the host, file:// storage and the
// job-file reader.  Contracts are in include/phobos_leaf.h.
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/phobos_leaf.h"
#include "host.h"

using namespace ph;

namespace {

std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) return "";
  size_t b = s.find_last_not_of(" \t\r\n");
  return s.substr(a, b - a + 1);
}

std::vector<std::string> split_ws(const std::string& s) {
  std::vector<std::string> out;
  std::istringstream is(s);
  std::string w;
  while (is >> w) out.push_back(w);
  return out;
}

bool parse_u64(const std::string& s, uint64_t* out) {
  const std::string t = trim(s);
  if (t.empty() || t[0] == '-' || t[0] == '+') return false;
  errno = 0;
  char* end = nullptr;
  unsigned long long v = strtoull(t.c_str(), &end, 10);
  if (errno || *end) return false;
  *out = v;
  return true;
}

bool parse_i64(const std::string& s, int64_t* out) {
  const std::string t = trim(s);
  if (t.empty()) return false;
  errno = 0;
  char* end = nullptr;
  long long v = strtoll(t.c_str(), &end, 10);
  if (errno || *end) return false;
  *out = v;
  return true;
}

// phobos-base/src/shape.rs:3-11: extents separated by 'x', blanks ignored.
bool parse_shape(const std::string& s, std::vector<uint64_t>* out, std::string* bad) {
  out->clear();
  size_t pos = 0;
  while (true) {
    size_t x = s.find('x', pos);
    std::string part = trim(s.substr(pos, x == std::string::npos ? std::string::npos : x - pos));
    uint64_t v;
    if (!parse_u64(part, &v)) {
      *bad = part;
      return false;
    }
    out->push_back(v);
    if (x == std::string::npos) break;
    pos = x + 1;
  }
  return true;
}

int dtype_from_name(const std::string& s) {  // phobos-sched/src/job.rs:111-121
  if (s == "f16") return PH_F16;
  if (s == "f32") return PH_F32;
  if (s == "f64") return PH_F64;
  if (s == "i8") return PH_I8;
  if (s == "i32") return PH_I32;
  if (s == "i64") return PH_I64;
  if (s == "bool") return PH_BOOL;
  return -1;
}

// The kernel's name: the identifier after the first `kernel` keyword that
// starts a declaration (grammar: SPEC.md:5-58).  Comments (`// ...`) are skipped.
std::string kernel_name_of(const std::string& src) {
  std::istringstream is(src);
  std::string line;
  while (std::getline(is, line)) {
    size_t c = line.find("//");
    if (c != std::string::npos) line = line.substr(0, c);
    size_t k = line.find("kernel");
    while (k != std::string::npos) {
      const bool left_ok = k == 0 || !(isalnum((unsigned char)line[k - 1]) || line[k - 1] == '_');
      const size_t after = k + 6;
      if (left_ok && after < line.size() && (line[after] == ' ' || line[after] == '\t')) {
        size_t b = line.find_first_not_of(" \t", after);
        size_t e = b;
        while (e < line.size() && (isalnum((unsigned char)line[e]) || line[e] == '_')) e++;
        if (b != std::string::npos && e > b) return line.substr(b, e - b);
      }
      k = line.find("kernel", k + 1);
    }
  }
  return "";
}

}  // namespace

struct PhJob {
  std::string kernel;
  std::string source;
  struct Dim { std::string name; int64_t value; };
  struct Tensor { std::string name; int dtype; int mode; std::vector<uint64_t> shape; std::string uri; };
  struct Scalar { std::string name; int dtype; uint64_t bits; };
  std::vector<Dim> dims;
  std::vector<Tensor> tensors;
  std::vector<Scalar> scalars;
};

namespace {

// phobos-sched/src/job.rs:90-100
bool parse_scalar(const std::string& type, const std::string& value, int* dtype, uint64_t* bits, std::string* msg) {
  auto bad = [&](const char* kind) {
    *msg = "scalar value '" + value + "' is not a valid " + kind;
    return false;
  };
  errno = 0;
  char* end = nullptr;
  if (type == "f32") {
    float f = strtof(value.c_str(), &end);
    if (*end || end == value.c_str()) return bad("f32");
    uint32_t b;
    memcpy(&b, &f, 4);
    *dtype = PH_F32;
    *bits = b;
  } else if (type == "f64") {
    double d = strtod(value.c_str(), &end);
    if (*end || end == value.c_str()) return bad("f64");
    memcpy(bits, &d, 8);
    *dtype = PH_F64;
  } else if (type == "i32") {
    int64_t v;
    if (!parse_i64(value, &v) || v < INT32_MIN || v > INT32_MAX) return bad("i32");
    *dtype = PH_I32;
    *bits = static_cast<uint32_t>(static_cast<int32_t>(v));
  } else if (type == "i64") {
    int64_t v;
    if (!parse_i64(value, &v)) return bad("i64");
    *dtype = PH_I64;
    *bits = static_cast<uint64_t>(v);
  } else if (type == "bool") {
    if (value != "true" && value != "false") return bad("bool");
    *dtype = PH_BOOL;
    *bits = value == "true";
  } else {
    *msg = "unknown scalar data type '" + type + "'";
    return false;
  }
  return true;
}

PhJob* parse_job_text(const std::string& text, const std::string& path, const char* source_override) {
  PhJob* job = new PhJob();
  bool have_source = false;
  std::istringstream is(text);
  std::string raw;
  int lineno = 0;
  auto err = [&](const std::string& msg) {
    fail(PH_ERR_PARSE, "%s:%d: %s", path.c_str(), lineno, msg.c_str());
    delete job;
    return static_cast<PhJob*>(nullptr);
  };
  while (std::getline(is, raw)) {
    lineno++;
    std::string line = trim(raw.substr(0, raw.find('#')));
    if (line.empty()) continue;
    if (line.compare(0, 6, "source") == 0) {
      std::string rest = trim(line.substr(6));
      if (rest.empty() || rest[0] != '=') return err("expected `source = <path>`");
      std::string p = trim(rest.substr(1));
      if (source_override) {
        job->source = source_override;
      } else {
        std::ifstream f(p);
        if (!f) return err("reading source file '" + p + "'");
        std::stringstream ss;
        ss << f.rdbuf();
        job->source = ss.str();
      }
      have_source = true;
    } else if (line.compare(0, 4, "dim ") == 0) {
      std::string rest = line.substr(4);
      size_t eq = rest.find('=');
      if (eq == std::string::npos) return err("expected `dim NAME = VALUE`");
      int64_t v;
      if (!parse_i64(rest.substr(eq + 1), &v)) return err("dim value must be an integer");
      job->dims.push_back({trim(rest.substr(0, eq)), v});
    } else if (line.compare(0, 7, "tensor ") == 0) {
      std::string rest = line.substr(7);
      size_t eq = rest.find('=');
      if (eq == std::string::npos) return err("expected `tensor NAME = MODE DATA_TYPE SHAPE URI`");
      std::vector<std::string> parts = split_ws(rest.substr(eq + 1));
      if (parts.size() < 1) return err("tensor missing mode");
      if (parts.size() < 2) return err("tensor missing data type");
      if (parts.size() < 3) return err("tensor missing shape");
      if (parts.size() < 4) return err("tensor missing uri");
      PhJob::Tensor t;
      t.name = trim(rest.substr(0, eq));
      t.dtype = dtype_from_name(parts[1]);
      if (t.dtype < 0) return err("unknown data type '" + parts[1] + "'");
      std::string bad;
      if (!parse_shape(parts[2], &t.shape, &bad)) return err("bad shape extent '" + bad + "'");
      if (parts[0] == "read") t.mode = PH_READ;
      else if (parts[0] == "write") t.mode = PH_WRITE;
      else if (parts[0] == "rmw") t.mode = PH_RMW;
      else return err("unknown tensor mode '" + parts[0] + "' (read|write|rmw)");
      t.uri = parts[3];
      job->tensors.push_back(t);
    } else if (line.compare(0, 7, "scalar ") == 0) {
      std::string rest = line.substr(7);
      size_t eq = rest.find('=');
      if (eq == std::string::npos) return err("expected `scalar NAME = DATA_TYPE VALUE`");
      std::vector<std::string> parts = split_ws(rest.substr(eq + 1));
      if (parts.size() < 1) return err("scalar missing data type");
      if (parts.size() < 2) return err("scalar missing value");
      PhJob::Scalar s;
      s.name = trim(rest.substr(0, eq));
      std::string msg;
      if (!parse_scalar(parts[0], parts[1], &s.dtype, &s.bits, &msg)) return err(msg);
      job->scalars.push_back(s);
    } else {
      return err("unknown directive '" + line + "'");
    }
  }
  if (!have_source) {
    fail(PH_ERR_PARSE, "%s: job-file has no `source =` line", path.c_str());
    delete job;
    return nullptr;
  }
  job->kernel = kernel_name_of(job->source);
  return job;
}

// Byte spans of a region inside a row-major tensor: phobos-cluster/src/storage.rs:22-46.
int byte_spans(const uint64_t* tensor_shape, int32_t tensor_rank, const PhRegion* region, size_t es,
               std::vector<std::pair<uint64_t, uint64_t>>* spans) {
  if (region->rank == 1) {
    uint64_t total = 1;
    for (int32_t d = 0; d < tensor_rank; d++) total *= tensor_shape[d];
    if (region->offset[0] > total || region->shape[0] > total - region->offset[0])
      return fail(PH_ERR_INVALID, "region [%llu, +%llu) exceeds the tensor's %llu elements",
                  (unsigned long long)region->offset[0], (unsigned long long)region->shape[0], (unsigned long long)total);
    spans->push_back({region->offset[0] * es, region->shape[0] * es});
    return PH_OK;
  }
  if (region->rank == 2) {
    if (tensor_rank != 2) return fail(PH_ERR_INVALID, "rank-2 region needs a rank-2 tensor");
    for (int d = 0; d < 2; d++)
      if (region->offset[d] > tensor_shape[d] || region->shape[d] > tensor_shape[d] - region->offset[d])
        return fail(PH_ERR_INVALID, "region axis %d: [%llu, +%llu) exceeds the tensor extent %llu", d,
                    (unsigned long long)region->offset[d], (unsigned long long)region->shape[d],
                    (unsigned long long)tensor_shape[d]);
    const uint64_t pitch = tensor_shape[1];
    for (uint64_t r = 0; r < region->shape[0]; r++)
      spans->push_back({((region->offset[0] + r) * pitch + region->offset[1]) * es, region->shape[1] * es});
    return PH_OK;
  }
  return fail(PH_ERR_UNSUPPORTED, "file:// storage supports rank <= 2, got rank %d", region->rank);
}

}  // namespace

extern "C" {

// ---- tile ids: phobos-cluster/src/tile.rs:12-30 ------------------------------------------
uint64_t phobos_tile_id(uint32_t tensor, uint32_t version, uint64_t coord) {
  return (static_cast<uint64_t>(tensor & 0xFFF) << 52) | (static_cast<uint64_t>(version & 0xFFFF) << 36) |
         (coord & ((1ull << 36) - 1));
}
uint32_t phobos_tile_tensor(uint64_t id) { return static_cast<uint32_t>(id >> 52); }
uint32_t phobos_tile_version(uint64_t id) { return static_cast<uint32_t>((id >> 36) & 0xFFFF); }
uint64_t phobos_tile_coord(uint64_t id) { return id & ((1ull << 36) - 1); }

// phobos-pod/src/tile_store.rs:22-27: round up to 256 bytes, at least 256.
uint64_t phobos_size_class(uint64_t bytes) {
  const uint64_t c = (bytes + 255) / 256 * 256;
  return c < 256 ? 256 : c;
}

// ---- generator on the host: phobos-base/src/rng.rs:9-25 ------------------------------------
int phobos_fill_random_host(float* out, uint64_t n, uint64_t seed, uint64_t first, float scale) {
  clear_error();
  if (!out && n) return fail(PH_ERR_INVALID, "null output");
  unsigned long long s = lcg_skip_host(seed, first);
  for (uint64_t i = 0; i < n; i++) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    out[i] = scale * (static_cast<float>(s >> 33) / 2147483648.0f - 1.0f);
  }
  return PH_OK;
}

// ---- storage: phobos-cluster/src/storage.rs ---------------------------------------------------
int phobos_storage_path(const char* uri, char* out, size_t out_len) {
  clear_error();
  if (!uri || !out) return fail(PH_ERR_INVALID, "null argument");
  if (strncmp(uri, "file://", 7) != 0) return fail(PH_ERR_IO, "unsupported storage URI '%s' (expected file://)", uri);
  const char* rest = uri + 7;
  // "/C:/..." -> "C:/..." (storage.rs:14-18)
  if (rest[0] == '/' && rest[1] != 0 && rest[2] == ':') rest++;
  if (strlen(rest) + 1 > out_len) return fail(PH_ERR_INVALID, "path buffer too small");
  strcpy(out, rest);
  return PH_OK;
}

int phobos_storage_load(const char* uri, const uint64_t* tensor_shape, int32_t tensor_rank, const PhRegion* region,
                        size_t elem_bytes, void* host_out) {
  clear_error();
  char path[4096];
  int rc = phobos_storage_path(uri, path, sizeof(path));
  if (rc) return rc;
  if (!region || !host_out || !tensor_shape) return fail(PH_ERR_INVALID, "null argument");
  std::vector<std::pair<uint64_t, uint64_t>> spans;
  if ((rc = byte_spans(tensor_shape, tensor_rank, region, elem_bytes, &spans))) return rc;
  FILE* f = fopen(path, "rb");
  if (!f) return fail(PH_ERR_IO, "open %s: %s", path, strerror(errno));
  char* dst = static_cast<char*>(host_out);
  for (auto& sp : spans) {
    if (fseeko(f, static_cast<off_t>(sp.first), SEEK_SET) != 0 || fread(dst, 1, sp.second, f) != sp.second) {
      fclose(f);
      return fail(PH_ERR_IO, "read %s at byte %llu: short read", path, (unsigned long long)sp.first);
    }
    dst += sp.second;
  }
  fclose(f);
  return PH_OK;
}

int phobos_storage_store(const char* uri, const uint64_t* tensor_shape, int32_t tensor_rank, const PhRegion* region,
                         size_t elem_bytes, const void* host_in) {
  clear_error();
  char path[4096];
  int rc = phobos_storage_path(uri, path, sizeof(path));
  if (rc) return rc;
  if (!region || !host_in || !tensor_shape) return fail(PH_ERR_INVALID, "null argument");
  std::vector<std::pair<uint64_t, uint64_t>> spans;
  if ((rc = byte_spans(tensor_shape, tensor_rank, region, elem_bytes, &spans))) return rc;
  // region writes keep the rest of the file (storage.rs:65-72): open without truncation, create if absent
  FILE* f = fopen(path, "r+b");
  if (!f) f = fopen(path, "w+b");
  if (!f) return fail(PH_ERR_IO, "open %s: %s", path, strerror(errno));
  const char* src = static_cast<const char*>(host_in);
  for (auto& sp : spans) {
    if (fseeko(f, static_cast<off_t>(sp.first), SEEK_SET) != 0 || fwrite(src, 1, sp.second, f) != sp.second) {
      fclose(f);
      return fail(PH_ERR_IO, "write %s at byte %llu failed", path, (unsigned long long)sp.first);
    }
    src += sp.second;
  }
  if (fclose(f) != 0) return fail(PH_ERR_IO, "close %s: %s", path, strerror(errno));
  return PH_OK;
}

// ---- job file: phobos-sched/src/job.rs:5-88 -----------------------------------------------------
PhJob* phobos_job_parse(const char* path) {
  clear_error();
  if (!path) {
    fail(PH_ERR_INVALID, "null path");
    return nullptr;
  }
  std::ifstream f(path);
  if (!f) {
    fail(PH_ERR_IO, "reading job-file %s", path);
    return nullptr;
  }
  std::stringstream ss;
  ss << f.rdbuf();
  return parse_job_text(ss.str(), path, nullptr);
}

PhJob* phobos_job_parse_text(const char* text, const char* origin, const char* source_text) {
  clear_error();
  if (!text) {
    fail(PH_ERR_INVALID, "null text");
    return nullptr;
  }
  return parse_job_text(text, origin ? origin : "<text>", source_text);
}

void phobos_job_free(PhJob* job) { delete job; }
const char* phobos_job_kernel_name(const PhJob* j) { return j ? j->kernel.c_str() : ""; }
const char* phobos_job_source(const PhJob* j) { return j ? j->source.c_str() : ""; }
int32_t phobos_job_n_dims(const PhJob* j) { return j ? (int32_t)j->dims.size() : 0; }
const char* phobos_job_dim_name(const PhJob* j, int32_t i) { return j->dims.at(i).name.c_str(); }
int64_t phobos_job_dim_value(const PhJob* j, int32_t i) { return j->dims.at(i).value; }
int32_t phobos_job_n_tensors(const PhJob* j) { return j ? (int32_t)j->tensors.size() : 0; }
const char* phobos_job_tensor_name(const PhJob* j, int32_t i) { return j->tensors.at(i).name.c_str(); }
int32_t phobos_job_tensor_dtype(const PhJob* j, int32_t i) { return j->tensors.at(i).dtype; }
int32_t phobos_job_tensor_mode(const PhJob* j, int32_t i) { return j->tensors.at(i).mode; }
int32_t phobos_job_tensor_rank(const PhJob* j, int32_t i) { return (int32_t)j->tensors.at(i).shape.size(); }
int64_t phobos_job_tensor_dim(const PhJob* j, int32_t i, int32_t d) { return (int64_t)j->tensors.at(i).shape.at(d); }
const char* phobos_job_tensor_uri(const PhJob* j, int32_t i) { return j->tensors.at(i).uri.c_str(); }
int32_t phobos_job_n_scalars(const PhJob* j) { return j ? (int32_t)j->scalars.size() : 0; }
const char* phobos_job_scalar_name(const PhJob* j, int32_t i) { return j->scalars.at(i).name.c_str(); }
int32_t phobos_job_scalar_dtype(const PhJob* j, int32_t i) { return j->scalars.at(i).dtype; }
uint64_t phobos_job_scalar_bits(const PhJob* j, int32_t i) { return j->scalars.at(i).bits; }

}  // extern "C"
