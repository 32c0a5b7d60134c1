// Protobuf wire format of instruction segments: `phobos.v1.Segment` and the messages under
// it (phobos-cluster/proto/v1/phobos_v1_isa.proto:5-113), read and written without a
// protobuf runtime.  Decoding turns a segment a phobos scheduler emitted into the
// executor's PhInstr records; encoding does the reverse for plans made here, so either
// side of the reference's scheduler / pod boundary can be replaced on its own.
//
// Field numbers (proto3; repeated scalars are packed, unpacked input is accepted too):
//   Segment{1 id, 2 instructions*}  Instruction{1 iid, 2 dependencies*, 3 operation}
//   Operation oneof{1 allocate, 2 load, 3 fetch, 4 compute, 5 store, 6 free}
//   Allocate{1 tile, 2 shape*, 3 data_type}  Load{1 tile, 2 source}  Fetch{1 tile, 2 from}
//   Compute{1 kernel, 2 arguments*, 3 grid, 4 cta, 5 scalars*}  Store{1 tile, 2 destination}
//   Free{1 tile, 2 expected_serves}  StorageReference{1 tensor, 2 region}  Region{1 offset*, 2 shape*}
//   Dim3{1 x, 2 y, 3 z}  ComputeArgument{1 tile, 2 mode}  ScalarArgument{1 position, 2 value}
//   ScalarValue oneof{1 f32 (fixed32), 2 f64 (fixed64), 3 i32, 4 i64, 5 boolean}
// The enums DataType and AccessMode are the C enums plus one (0 is UNSPECIFIED on the wire).
#include <cstdint>
#include <cstring>
#include <string>

#include "host.h"
#include "plan.h"

using namespace ph;
using ph::plan::OwnedInstr;

namespace {

// ---- reading -------------------------------------------------------------------------------------
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  bool done() const { return p >= end || !ok; }
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 70; shift += 7) {
      if (p >= end) {
        ok = false;
        return 0;
      }
      const uint8_t b = *p++;
      v |= static_cast<uint64_t>(b & 0x7F) << (shift < 64 ? shift : 63);
      if (!(b & 0x80)) return v;
    }
    ok = false;
    return 0;
  }
  uint32_t fixed32() {
    if (end - p < 4) {
      ok = false;
      return 0;
    }
    uint32_t v;
    memcpy(&v, p, 4);
    p += 4;
    return v;
  }
  uint64_t fixed64() {
    if (end - p < 8) {
      ok = false;
      return 0;
    }
    uint64_t v;
    memcpy(&v, p, 8);
    p += 8;
    return v;
  }
  Reader sub() {   // a length-delimited field
    const uint64_t n = varint();
    if (!ok || n > static_cast<uint64_t>(end - p)) {
      ok = false;
      return Reader{p, p, false};
    }
    Reader r{p, p + n};
    p += n;
    return r;
  }
  void skip(uint32_t wt) {
    switch (wt) {
      case 0: varint(); break;
      case 1: fixed64(); break;
      case 2: sub(); break;
      case 5: fixed32(); break;
      default: ok = false;
    }
  }
};

// a repeated uint64: packed (wire type 2) or one element (wire type 0)
void read_repeated_u64(Reader& r, uint32_t wt, std::vector<uint64_t>* out) {
  if (wt == 2) {
    Reader s = r.sub();
    while (!s.done()) out->push_back(s.varint());
    if (!s.ok) r.ok = false;
  } else if (wt == 0) {
    out->push_back(r.varint());
  } else {
    r.ok = false;
  }
}

bool read_region(Reader r, PhRegion* out) {
  std::vector<uint64_t> off, shp;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f == 1) read_repeated_u64(r, wt, &off);
    else if (f == 2) read_repeated_u64(r, wt, &shp);
    else r.skip(wt);
  }
  if (!r.ok || off.size() != shp.size() || shp.size() > 2) return false;
  out->rank = static_cast<int32_t>(shp.size());
  for (size_t i = 0; i < shp.size(); i++) {
    out->offset[i] = off[i];
    out->shape[i] = shp[i];
  }
  return true;
}

bool read_storage_ref(Reader r, uint32_t* tensor, PhRegion* region) {
  *tensor = 0;
  bool have_region = false;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f == 1 && wt == 0) *tensor = static_cast<uint32_t>(r.varint());
    else if (f == 2 && wt == 2) have_region = read_region(r.sub(), region);
    else r.skip(wt);
  }
  return r.ok && have_region;
}

void read_dim3(Reader r, uint32_t out[3], bool* ok) {
  out[0] = out[1] = out[2] = 0;   // proto3 omits zeros
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f >= 1 && f <= 3 && wt == 0) out[f - 1] = static_cast<uint32_t>(r.varint());
    else r.skip(wt);
  }
  if (!r.ok) *ok = false;
}

bool read_scalar_value(Reader r, PhScalar* s) {
  bool have = false;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f == 1 && wt == 5) {
      s->dtype = PH_F32;
      s->bits = r.fixed32();
      have = true;
    } else if (f == 2 && wt == 1) {
      s->dtype = PH_F64;
      s->bits = r.fixed64();
      have = true;
    } else if (f == 3 && wt == 0) {
      s->dtype = PH_I32;
      s->bits = static_cast<uint32_t>(r.varint());   // int32 travels sign-extended to 64 bits
      have = true;
    } else if (f == 4 && wt == 0) {
      s->dtype = PH_I64;
      s->bits = r.varint();
      have = true;
    } else if (f == 5 && wt == 0) {
      s->dtype = PH_BOOL;
      s->bits = r.varint() != 0;
      have = true;
    } else {
      r.skip(wt);
    }
  }
  return r.ok && have;
}

bool read_operation(Reader r, OwnedInstr* oi, std::string* err) {
  bool have = false;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f < 1 || f > 6 || wt != 2) {
      r.skip(wt);
      continue;
    }
    Reader m = r.sub();
    have = true;
    PhInstr& in = oi->in;
    in.op = static_cast<int32_t>(f - 1);   // the oneof's field numbers follow PhOpCode + 1
    std::vector<uint64_t> shape;
    bool sub_ok = true;
    while (!m.done()) {
      const uint64_t k2 = m.varint();
      const uint32_t g = static_cast<uint32_t>(k2 >> 3), w2 = k2 & 7;
      if (g == 1 && w2 == 0 && f != 4) {
        in.tile = m.varint();
      } else if (f == 1 && g == 2) {
        read_repeated_u64(m, w2, &shape);
      } else if (f == 1 && g == 3 && w2 == 0) {
        const uint64_t dt = m.varint();
        if (dt == 0 || dt > 7) {
          *err = "ALLOC with unspecified data type";
          return false;
        }
        in.data_type = static_cast<int32_t>(dt - 1);
      } else if ((f == 2 || f == 5) && g == 2 && w2 == 2) {
        sub_ok = read_storage_ref(m.sub(), &in.tensor, &in.region) && sub_ok;
      } else if (f == 3 && g == 2 && w2 == 0) {
        in.from_node = static_cast<uint32_t>(m.varint());
      } else if (f == 6 && g == 2 && w2 == 0) {
        in.expected_serves = static_cast<uint32_t>(m.varint());
      } else if (f == 4 && g == 1 && w2 == 0) {
        in.kernel = static_cast<uint32_t>(m.varint());
      } else if (f == 4 && g == 2 && w2 == 2) {
        Reader a = m.sub();
        PhTileArg arg{0, -1};
        while (!a.done()) {
          const uint64_t k3 = a.varint();
          const uint32_t h = static_cast<uint32_t>(k3 >> 3), w3 = k3 & 7;
          if (h == 1 && w3 == 0) arg.tile = a.varint();
          else if (h == 2 && w3 == 0) arg.mode = static_cast<int32_t>(a.varint()) - 1;
          else a.skip(w3);
        }
        if (!a.ok || arg.mode < 0 || arg.mode > 2) {
          *err = "COMPUTE argument without an access mode";
          return false;
        }
        oi->args.push_back(arg);
      } else if (f == 4 && (g == 3 || g == 4) && w2 == 2) {
        read_dim3(m.sub(), g == 3 ? in.grid : in.cta, &sub_ok);
      } else if (f == 4 && g == 5 && w2 == 2) {
        Reader a = m.sub();
        PhScalar s{};
        bool have_value = false;
        while (!a.done()) {
          const uint64_t k3 = a.varint();
          const uint32_t h = static_cast<uint32_t>(k3 >> 3), w3 = k3 & 7;
          if (h == 1 && w3 == 0) s.pos = static_cast<uint32_t>(a.varint());
          else if (h == 2 && w3 == 2) have_value = read_scalar_value(a.sub(), &s);
          else a.skip(w3);
        }
        if (!a.ok || !have_value) {
          *err = "scalar argument without a value";
          return false;
        }
        oi->scalars.push_back(s);
      } else {
        m.skip(w2);
      }
    }
    if (!m.ok || !sub_ok) {
      *err = "malformed operation";
      return false;
    }
    if (f == 1) {
      if (shape.size() > 2) {
        *err = "ALLOC of rank " + std::to_string(shape.size()) + " (rank <= 2 supported)";
        return false;
      }
      in.shape_rank = static_cast<int32_t>(shape.size());
      for (size_t i = 0; i < shape.size(); i++) in.shape[i] = shape[i];
    }
  }
  if (!r.ok || !have) {
    *err = "instruction without an operation";
    return false;
  }
  return true;
}

// ---- writing -------------------------------------------------------------------------------------
struct Writer {
  std::string s;
  void varint(uint64_t v) {
    while (v >= 0x80) {
      s.push_back(static_cast<char>((v & 0x7F) | 0x80));
      v >>= 7;
    }
    s.push_back(static_cast<char>(v));
  }
  void key(uint32_t field, uint32_t wt) { varint((static_cast<uint64_t>(field) << 3) | wt); }
  void u64(uint32_t field, uint64_t v) {   // proto3: zero is the default and is not written
    if (v == 0) return;
    key(field, 0);
    varint(v);
  }
  void bytes(uint32_t field, const std::string& b) {
    key(field, 2);
    varint(b.size());
    s += b;
  }
  void packed(uint32_t field, const uint64_t* v, int n) {
    if (n == 0) return;
    Writer w;
    for (int i = 0; i < n; i++) w.varint(v[i]);
    bytes(field, w.s);
  }
};

std::string enc_storage_ref(uint32_t tensor, const PhRegion& r) {
  Writer reg;
  reg.packed(1, r.offset, r.rank);
  reg.packed(2, r.shape, r.rank);
  Writer w;
  w.u64(1, tensor);
  w.bytes(2, reg.s);
  return w.s;
}
std::string enc_dim3(const uint32_t d[3]) {
  Writer w;
  for (int i = 0; i < 3; i++) w.u64(i + 1, d[i]);
  return w.s;
}

bool enc_instr(const PhInstr& in, Writer* out, std::string* err) {
  Writer op;
  switch (in.op) {
    case PH_OP_ALLOC:
      op.u64(1, in.tile);
      op.packed(2, in.shape, in.shape_rank);
      op.u64(3, static_cast<uint64_t>(in.data_type) + 1);
      break;
    case PH_OP_LOAD:
    case PH_OP_STORE:
      op.u64(1, in.tile);
      op.bytes(2, enc_storage_ref(in.tensor, in.region));
      break;
    case PH_OP_FETCH:
      op.u64(1, in.tile);
      op.u64(2, in.from_node);
      break;
    case PH_OP_FREE:
      op.u64(1, in.tile);
      op.u64(2, in.expected_serves);
      break;
    case PH_OP_COMPUTE: {
      op.u64(1, in.kernel);
      for (int i = 0; i < in.n_args; i++) {
        Writer a;
        a.u64(1, in.args[i].tile);
        a.u64(2, static_cast<uint64_t>(in.args[i].mode) + 1);
        op.bytes(2, a.s);
      }
      op.bytes(3, enc_dim3(in.grid));
      op.bytes(4, enc_dim3(in.cta));
      for (int i = 0; i < in.n_scalars; i++) {
        const PhScalar& sc = in.scalars[i];
        Writer v;
        switch (sc.dtype) {
          case PH_F32: {
            v.key(1, 5);
            const uint32_t b = static_cast<uint32_t>(sc.bits);
            v.s.append(reinterpret_cast<const char*>(&b), 4);
            break;
          }
          case PH_F64:
            v.key(2, 1);
            v.s.append(reinterpret_cast<const char*>(&sc.bits), 8);
            break;
          case PH_I32:   // oneof members are written even when zero
            v.key(3, 0);
            v.varint(static_cast<uint64_t>(static_cast<int64_t>(static_cast<int32_t>(sc.bits))));
            break;
          case PH_I64:
            v.key(4, 0);
            v.varint(sc.bits);
            break;
          case PH_BOOL:
            v.key(5, 0);
            v.varint(sc.bits != 0);
            break;
          default:
            *err = "scalar of a type the wire format cannot carry";
            return false;
        }
        Writer a;
        a.u64(1, sc.pos);
        a.bytes(2, v.s);
        op.bytes(5, a.s);
      }
      break;
    }
    default:
      *err = "unknown op code";
      return false;
  }
  Writer operation;
  operation.bytes(static_cast<uint32_t>(in.op) + 1, op.s);
  Writer ins;
  ins.u64(1, in.iid);
  ins.packed(2, in.deps, in.n_deps);
  ins.bytes(3, operation.s);
  out->bytes(2, ins.s);
  return true;
}

}  // namespace

struct PhSegmentMsg {
  ph::plan::Segment seg;
};

extern "C" {

PhSegmentMsg* phobos_segment_decode(const void* data, size_t n) {
  clear_error();
  if (!data && n) {
    fail(PH_ERR_INVALID, "null segment bytes");
    return nullptr;
  }
  PhSegmentMsg* msg = new PhSegmentMsg();
  Reader r{static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + n};
  std::string err;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t f = static_cast<uint32_t>(key >> 3), wt = key & 7;
    if (f == 1 && wt == 0) {
      msg->seg.id = r.varint();
    } else if (f == 2 && wt == 2) {
      Reader ir = r.sub();
      OwnedInstr oi;
      oi.in.grid[0] = oi.in.grid[1] = oi.in.grid[2] = 0;
      bool have_op = false;
      while (!ir.done()) {
        const uint64_t k2 = ir.varint();
        const uint32_t g = static_cast<uint32_t>(k2 >> 3), w2 = k2 & 7;
        if (g == 1 && w2 == 0) oi.in.iid = ir.varint();
        else if (g == 2) read_repeated_u64(ir, w2, &oi.deps);
        else if (g == 3 && w2 == 2) {
          if (!read_operation(ir.sub(), &oi, &err)) {
            fail(PH_ERR_PARSE, "segment: instruction %llu: %s", static_cast<unsigned long long>(oi.in.iid), err.c_str());
            delete msg;
            return nullptr;
          }
          have_op = true;
        } else {
          ir.skip(w2);
        }
      }
      if (!ir.ok || !have_op) {
        fail(PH_ERR_PARSE, "segment: malformed instruction %llu", static_cast<unsigned long long>(oi.in.iid));
        delete msg;
        return nullptr;
      }
      msg->seg.instrs.push_back(std::move(oi));
    } else {
      r.skip(wt);
    }
  }
  if (!r.ok) {
    fail(PH_ERR_PARSE, "segment: truncated or malformed message");
    delete msg;
    return nullptr;
  }
  for (OwnedInstr& oi : msg->seg.instrs) {
    oi.in.deps = oi.deps.data();
    oi.in.n_deps = static_cast<int32_t>(oi.deps.size());
    oi.in.args = oi.args.data();
    oi.in.n_args = static_cast<int32_t>(oi.args.size());
    oi.in.scalars = oi.scalars.data();
    oi.in.n_scalars = static_cast<int32_t>(oi.scalars.size());
    msg->seg.flat.push_back(oi.in);
  }
  return msg;
}

void phobos_segment_free(PhSegmentMsg* m) { delete m; }
uint64_t phobos_segment_id(const PhSegmentMsg* m) { return m ? m->seg.id : 0; }
int32_t phobos_segment_n_instrs(const PhSegmentMsg* m) { return m ? static_cast<int32_t>(m->seg.flat.size()) : 0; }
const PhInstr* phobos_segment_instrs(const PhSegmentMsg* m) { return (m && !m->seg.flat.empty()) ? m->seg.flat.data() : nullptr; }

/* Writes Segment{id, instructions} into out (when it fits) and returns the encoded size; SIZE_MAX on error. */
size_t phobos_segment_encode(uint64_t id, const PhInstr* instrs, int32_t n, void* out, size_t cap) {
  clear_error();
  if (n > 0 && !instrs) {
    fail(PH_ERR_INVALID, "null instruction list");
    return SIZE_MAX;
  }
  Writer w;
  w.u64(1, id);
  std::string err;
  for (int32_t i = 0; i < n; i++)
    if (!enc_instr(instrs[i], &w, &err)) {
      fail(PH_ERR_INVALID, "instruction %llu: %s", static_cast<unsigned long long>(instrs[i].iid), err.c_str());
      return SIZE_MAX;
    }
  if (out && cap >= w.s.size()) memcpy(out, w.s.data(), w.s.size());
  return w.s.size();
}

}  // extern "C"
