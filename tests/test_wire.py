"""Segments on the wire (phobos.v1.Segment): the hand-written reader / writer against the protobuf
runtime.  The message layout below restates phobos-cluster/proto/v1/phobos_v1_isa.proto:5-113 as a
descriptor built in code (no protoc here); the Python protobuf package then is the independent
implementation both directions are checked against."""
import struct

import pytest

pb = pytest.importorskip("google.protobuf")


def _messages():
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    F = descriptor_pb2.FieldDescriptorProto
    f = descriptor_pb2.FileDescriptorProto(name="isa_restated.proto", package="phobos.v1", syntax="proto3")

    def enum(name, values):
        e = f.enum_type.add(name=name)
        for i, v in enumerate(values):
            e.value.add(name=v, number=i)

    enum("DataType", ["DATA_TYPE_UNSPECIFIED", "DATA_TYPE_F16", "DATA_TYPE_F32", "DATA_TYPE_F64", "DATA_TYPE_I8",
                      "DATA_TYPE_I32", "DATA_TYPE_I64", "DATA_TYPE_BOOL"])
    enum("AccessMode", ["ACCESS_MODE_UNSPECIFIED", "ACCESS_MODE_READ", "ACCESS_MODE_WRITE", "ACCESS_MODE_RMW"])
    T = {"u64": F.TYPE_UINT64, "u32": F.TYPE_UINT32, "f32": F.TYPE_FLOAT, "f64": F.TYPE_DOUBLE, "i32": F.TYPE_INT32,
         "i64": F.TYPE_INT64, "bool": F.TYPE_BOOL}

    def msg(name, fields, oneof=None):
        m = f.message_type.add(name=name)
        if oneof:
            m.oneof_decl.add(name=oneof)
        for num, (fname, ftype, rep) in enumerate(fields, start=1):
            fd = m.field.add(name=fname, number=num, label=F.LABEL_REPEATED if rep else F.LABEL_OPTIONAL)
            if ftype in T:
                fd.type = T[ftype]
            elif ftype in ("DataType", "AccessMode"):
                fd.type, fd.type_name = F.TYPE_ENUM, ".phobos.v1." + ftype
            else:
                fd.type, fd.type_name = F.TYPE_MESSAGE, ".phobos.v1." + ftype
            if oneof:
                fd.oneof_index = 0

    msg("Region", [("offset", "u64", True), ("shape", "u64", True)])
    msg("StorageReference", [("tensor", "u32", False), ("region", "Region", False)])
    msg("Dim3", [("x", "u32", False), ("y", "u32", False), ("z", "u32", False)])
    msg("ComputeArgument", [("tile", "u64", False), ("mode", "AccessMode", False)])
    msg("ScalarValue", [("f32", "f32", False), ("f64", "f64", False), ("i32", "i32", False), ("i64", "i64", False),
                        ("boolean", "bool", False)], oneof="value")
    msg("ScalarArgument", [("position", "u32", False), ("value", "ScalarValue", False)])
    msg("Allocate", [("tile", "u64", False), ("shape", "u64", True), ("data_type", "DataType", False)])
    msg("Load", [("tile", "u64", False), ("source", "StorageReference", False)])
    msg("Fetch", [("tile", "u64", False), ("from", "u32", False)])
    msg("Compute", [("kernel", "u32", False), ("arguments", "ComputeArgument", True), ("grid", "Dim3", False),
                    ("cta", "Dim3", False), ("scalars", "ScalarArgument", True)])
    msg("Store", [("tile", "u64", False), ("destination", "StorageReference", False)])
    msg("Free", [("tile", "u64", False), ("expected_serves", "u32", False)])
    msg("Operation", [("allocate", "Allocate", False), ("load", "Load", False), ("fetch", "Fetch", False),
                      ("compute", "Compute", False), ("store", "Store", False), ("free", "Free", False)], oneof="kind")
    msg("Instruction", [("iid", "u64", False), ("dependencies", "u64", True), ("operation", "Operation", False)])
    msg("Segment", [("id", "u64", False), ("instructions", "Instruction", True)])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("phobos.v1." + n))
            for n in ("Segment", "Instruction")}


def _plan_instrs(ph):
    from test_planner import GEMM
    pl = ph.plan(ph.Program(GEMM), {"M": 1024, "N": 512, "K": 512}, nodes=2, policy=ph.HOME_LOAD_PEER_FETCH,
                 scalars={"alpha": ph.scalar_f32(0, 0.125), "beta": ph.scalar_f32(0, -1.5)})
    return pl.node_instrs(0) + pl.node_instrs(1)


def _key(i):
    return (i.iid, i.op, i.deps, i.tile, i.data_type if i.op == 0 else 0, i.shape, i.tensor if i.op in (1, 4) else 0,
            i.region_offset, i.region_shape, i.from_node, i.kernel, i.args,
            tuple((s.pos, s.dtype, s.bits) for s in i.scalars), i.grid if i.op == 3 else 0, i.cta if i.op == 3 else 0,
            i.expected_serves)


def test_encoded_plan_parses_with_the_protobuf_runtime(ph):
    M = _messages()
    instrs = _plan_instrs(ph)
    data = ph.encode_segment(7, instrs)
    seg = M["Segment"]()
    seg.ParseFromString(data)
    assert seg.id == 7 and len(seg.instructions) == len(instrs)
    kinds = ["allocate", "load", "fetch", "compute", "store", "free"]
    for want, got in zip(instrs, seg.instructions):
        assert got.iid == want.iid and tuple(got.dependencies) == want.deps
        assert got.operation.WhichOneof("kind") == kinds[want.op]
        if want.op == ph.OP_ALLOC:
            assert got.operation.allocate.tile == want.tile and tuple(got.operation.allocate.shape) == want.shape
            assert got.operation.allocate.data_type == want.data_type + 1
        if want.op == ph.OP_COMPUTE:
            c = got.operation.compute
            assert [(a.tile, a.mode - 1) for a in c.arguments] == list(want.args)
            assert (c.grid.x, c.grid.y, c.grid.z) == want.grid and (c.cta.x, c.cta.y, c.cta.z) == want.cta
            assert [(s.position, struct.pack("<f", s.value.f32)) for s in c.scalars] == \
                   [(s.pos, struct.pack("<I", s.bits)) for s in want.scalars]
        if want.op == ph.OP_STORE:
            d = got.operation.store.destination
            assert d.tensor == want.tensor and tuple(d.region.offset) == want.region_offset
        if want.op == ph.OP_FREE:
            assert got.operation.free.expected_serves == want.expected_serves
    # the same bytes as the runtime's own serialisation (field order and packing are canonical)
    assert seg.SerializeToString() == data


def test_runtime_encoded_segment_is_read(ph):
    M = _messages()
    seg = M["Segment"](id=3)
    a = seg.instructions.add(iid=11)
    a.operation.allocate.tile = ph.tile_id(1, 2, 5)
    a.operation.allocate.shape.extend([64, 128])
    a.operation.allocate.data_type = 1           # f16
    ld = seg.instructions.add(iid=12, dependencies=[11])
    ld.operation.load.tile = ph.tile_id(1, 2, 5)
    ld.operation.load.source.tensor = 1
    ld.operation.load.source.region.offset.extend([0, 256])     # a zero inside a packed list
    ld.operation.load.source.region.shape.extend([64, 128])
    ft = seg.instructions.add(iid=13)
    ft.operation.fetch.tile = 9
    setattr(ft.operation.fetch, "from", 2)
    c = seg.instructions.add(iid=14, dependencies=[12, 13])
    c.operation.compute.kernel = 0                # default values are absent on the wire
    c.operation.compute.arguments.add(tile=9, mode=1)
    c.operation.compute.arguments.add(tile=ph.tile_id(1, 2, 5), mode=3)
    c.operation.compute.grid.x, c.operation.compute.grid.y, c.operation.compute.grid.z = 4, 2, 1
    c.operation.compute.cta.x, c.operation.compute.cta.y, c.operation.compute.cta.z = 128, 1, 1
    for pos, field, val in ((3, "f32", 0.5), (4, "f64", -2.25), (5, "i32", -7), (6, "i64", -(1 << 40)), (7, "boolean", True),
                            (8, "i32", 0)):
        s = c.operation.compute.scalars.add(position=pos)
        setattr(s.value, field, val)
    fr = seg.instructions.add(iid=15, dependencies=[14])
    fr.operation.free.tile = 9
    fr.operation.free.expected_serves = 3
    sid, ins = ph.decode_segment(seg.SerializeToString())
    assert sid == 3 and [i.iid for i in ins] == [11, 12, 13, 14, 15]
    assert (ins[0].op, ins[0].shape, ins[0].data_type, ins[0].tile) == (ph.OP_ALLOC, (64, 128), ph.F16, ph.tile_id(1, 2, 5))
    assert (ins[1].op, ins[1].deps, ins[1].tensor, ins[1].region_offset, ins[1].region_shape) == \
           (ph.OP_LOAD, (11,), 1, (0, 256), (64, 128))
    assert (ins[2].op, ins[2].tile, ins[2].from_node) == (ph.OP_FETCH, 9, 2)
    cm = ins[3]
    assert cm.op == ph.OP_COMPUTE and cm.kernel == 0 and cm.args == ((9, ph.READ), (ph.tile_id(1, 2, 5), ph.RMW))
    assert cm.grid == (4, 2, 1) and cm.cta == (128, 1, 1)
    got = [(s.pos, s.dtype, s.bits) for s in cm.scalars]
    assert got == [(3, ph.F32, struct.unpack("<I", struct.pack("<f", 0.5))[0]),
                   (4, ph.F64, struct.unpack("<Q", struct.pack("<d", -2.25))[0]),
                   (5, ph.I32, (-7) & 0xFFFFFFFF), (6, ph.I64, (-(1 << 40)) & ((1 << 64) - 1)), (7, ph.BOOL, 1),
                   (8, ph.I32, 0)]
    assert (ins[4].op, ins[4].expected_serves) == (ph.OP_FREE, 3)
    # and back: the round trip through our writer gives the runtime's bytes again
    assert ph.encode_segment(3, ins) == seg.SerializeToString()


def test_round_trip_and_malformed_input(ph):
    instrs = _plan_instrs(ph)
    sid, back = ph.decode_segment(ph.encode_segment(41, instrs))
    assert sid == 41 and [_key(i) for i in back] == [_key(i) for i in instrs]
    assert ph.decode_segment(b"") == (0, [])
    data = ph.encode_segment(1, instrs[:4])
    for bad in (data[:-3], data[:10] + b"\xff" * 12, b"\x12\x7f"):
        with pytest.raises(ph.PhobosError):
            ph.decode_segment(bad)
