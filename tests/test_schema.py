"""Flatbuffer toolkit: writer/reader round trip, generated header freshness, verifier."""

import os
import struct

import pytest

from ttmlir_b200 import graphs
from ttmlir_b200.schema import gen_cpp
from ttmlir_b200.schema.fbs import Reader, Writer
from ttmlir_b200.schema.ttnn_schema import FILE_IDENTIFIER, OP_TYPE_MEMBERS, S, UNDECLARED_OPS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_container_layout():
    buf = graphs.build_binary(graphs.mlp_graph)
    size = struct.unpack_from("<I", buf, 0)[0]
    assert size + 4 == len(buf)          # size prefix counts the rest of the file
    assert buf[8:12] == FILE_IDENTIFIER  # identifier follows the root offset
    assert len(buf) % 4 == 0


def test_round_trip_through_reader():
    buf = graphs.build_binary(graphs.quant_chain_graph, rows=32, cols=32, keep_intermediates=True)
    root = Reader(S, buf).root("TTNNBinary")
    prog = root["programs"][0]
    kinds = [op["type"][0] for op in prog["operations"]]
    assert kinds[0] == "GetDeviceOp"
    assert kinds.count("EltwiseQuantizationOp") == 3
    q = next(op["type"][1] for op in prog["operations"] if op["type"][0] == "EltwiseQuantizationOp")
    assert q["type"] == "Quantize" and q["axis"] is None and q["output_dtype"] == "Int32"
    assert q["params"][0] == "QuantizeDequantizeOpParams"
    assert abs(q["params"][1]["scale"][1]["scale"] - 0.02) < 1e-9
    # shared TensorRef: the producer's out id is the consumer's in id
    rq = [op["type"][1] for op in prog["operations"] if op["type"][0] == "EltwiseQuantizationOp"][1]
    assert rq["in"]["global_id"] == q["out"]["global_id"]
    assert prog["mesh_shape"] == {"y": 1, "x": 1}
    assert [o["desc"]["layout"]["memory_desc"]["data_type"] for o in prog["outputs"]] == ["Float32", "Int32", "Int32"]


def test_optional_scalars_are_absent_unless_set():
    w = Writer(S)
    off = w.create_table("AllReduceOp", {"reduce_type": 0, "cluster_axis": 1})
    buf = w.finish(off, b"TEST")
    t = Reader(S, buf).root("AllReduceOp")
    assert t["num_links"] is None and t["topology"] is None and t["cluster_axis"] == 1
    w = Writer(S)
    off = w.create_table("AllReduceOp", {"reduce_type": 0, "cluster_axis": 0, "num_links": 0})
    t = Reader(S, w.finish(off, b"TEST")).root("AllReduceOp")
    assert t["num_links"] == 0  # explicitly written zero survives


def test_op_type_union_ids():
    u = S.unions["OpType"]
    assert len(OP_TYPE_MEMBERS) == 131
    assert u.type_id("AdamWOp") == 1 and u.type_id("CopyOp") == 131
    assert u.type_id("MatmulOp") == OP_TYPE_MEMBERS.index("MatmulOp") + 1
    assert "MoeComputeOp" in UNDECLARED_OPS and "MatmulOp" not in UNDECLARED_OPS


def test_union_field_takes_two_slots():
    t = S.tables["Operation"]
    assert [f.id for f in t.fields] == [0, 2, 3]
    m = S.tables["MatmulOp"]
    ids = {f.name: f.id for f in m.fields}
    assert ids["matmul_program_config"] == 5 and ids["activation"] == 7 and ids["compute_config"] == 8


def test_generated_header_is_current():
    path = os.path.join(ROOT, "tt-mlir_b200", "runtime", "generated", "ttnn_schema.h")
    assert open(path).read() == gen_cpp.gen(S), "run python tt-mlir_b200/build.py to regenerate"


def test_struct_layout():
    assert S.structs["Dim2d"].size == 8
    assert S.structs["Placement"].size == 8 and S.structs["Placement"].offsets == [0, 4]
    assert S.structs["Version"].size == 8


def test_executor_dispatches_every_declared_op():
    """The executor has a case for every op type whose table the schema declares, and the op types it refuses are
    exactly the ones the schema leaves undeclared (they are rejected at submit by name, never run approximately)."""
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = open(os.path.join(root, "tt-mlir_b200", "runtime", "executor.cpp")).read()
    dispatched = set(re.findall(r"case OpType::(\w+)", src))
    declared = set(OP_TYPE_MEMBERS) - set(UNDECLARED_OPS)
    assert declared <= dispatched, f"declared but not dispatched: {sorted(declared - dispatched)}"
    assert set(UNDECLARED_OPS) == {
        "GenericOp", "MoeGptOp", "PrepareMoEComputeW0W1WeightsOp", "PrepareMoEComputeW2WeightsOp", "MoeComputeOp",
        "SDPAForwardOp", "SDPABackwardOp", "SelectiveReduceCombineOp"}
    assert not (set(UNDECLARED_OPS) & dispatched)
    assert len(OP_TYPE_MEMBERS) == 131
