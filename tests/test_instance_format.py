"""The older Instance record format: parser twin, wire codec, and the three tools around it."""
import numpy as np
import pytest

from parameter_server_b200.data import instance as I
from parameter_server_b200.runtime import host


def _schema():
    """instance.proto's Instance / FeatureGroup as a dynamic protobuf schema (field numbers as in the reference)."""
    pb = pytest.importorskip("google.protobuf")
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

    fd = descriptor_pb2.FileDescriptorProto(name="ins_test.proto", package="PSX", syntax="proto2")
    g = fd.message_type.add(name="FeatureGroup")
    T = descriptor_pb2.FieldDescriptorProto
    g.field.add(name="grp_id", number=1, type=T.TYPE_INT32, label=T.LABEL_OPTIONAL)
    f = g.field.add(name="fea_id", number=2, type=T.TYPE_UINT64, label=T.LABEL_REPEATED)
    f.options.packed = True
    f = g.field.add(name="fea_val", number=3, type=T.TYPE_FLOAT, label=T.LABEL_REPEATED)
    f.options.packed = True
    m = fd.message_type.add(name="Instance")
    m.field.add(name="label", number=1, type=T.TYPE_FLOAT, label=T.LABEL_OPTIONAL)
    m.field.add(name="fea_grp", number=2, type=T.TYPE_MESSAGE, label=T.LABEL_REPEATED, type_name=".PSX.FeatureGroup")
    m.field.add(name="ins_id", number=3, type=T.TYPE_INT64, label=T.LABEL_OPTIONAL)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("PSX.Instance"))


def test_wire_format_is_protobuf_both_ways():
    Msg = _schema()
    ins = I.Instance(label=-1.0, ins_id=-7, fea_grp=[
        I.FeatureGroup(3, np.array([1, 300, (1 << 64) - 2], np.uint64), np.array([0.5, -2.0, 1e-3], np.float32)),
        I.FeatureGroup(9, np.array([42], np.uint64))])
    m = Msg()
    m.ParseFromString(ins.encode())
    assert m.label == -1.0 and m.ins_id == -7 and len(m.fea_grp) == 2
    assert list(m.fea_grp[0].fea_id) == [1, 300, (1 << 64) - 2] and m.fea_grp[0].grp_id == 3
    assert np.allclose(list(m.fea_grp[0].fea_val), [0.5, -2.0, 1e-3]) and list(m.fea_grp[1].fea_val) == []
    back = I.Instance.decode(m.SerializeToString())                     # bytes written by the protobuf library
    assert back.label == -1.0 and back.ins_id == -7
    assert back.fea_grp[0].fea_id.tolist() == [1, 300, (1 << 64) - 2] and back.fea_grp[1].fea_id.tolist() == [42]
    assert np.allclose(back.fea_grp[0].fea_val, [0.5, -2.0, 1e-3])


def test_truncated_record_is_rejected():
    body = I.Instance(label=1.0, fea_grp=[I.FeatureGroup(1, np.arange(5, dtype=np.uint64))]).encode()
    with pytest.raises(ValueError):
        I.Instance.decode(body[:-2])


def test_parser_counts_groups_and_label_kinds():
    p = I.TextParser("LIBSVM")
    a = p.to_instance("1 3:0.5 7:1.5 10:2")
    assert a.label == 1.0 and a.fea_grp[0].grp_id == 1 and a.fea_grp[0].fea_id.tolist() == [3, 7, 10]
    assert p.to_instance("no label here") is None
    assert p.to_instance("-1 1:1 7:0.25") is not None
    info = p.info()
    assert info.num_ins == 2 and info.nnz_ele == 5 and (info.fea_begin, info.fea_end) == (1, 11)
    assert info.label_type == I.BINARY and [g.grp_id for g in info.fea_grp] == [1, I.LABEL_GROUP]
    assert info.fea_grp[0].nnz_ins == 2 and info.fea_grp[1].nnz_ele == 2
    p.to_instance("3 1:1")
    assert p.info().label_type == I.MULTICLASS
    p.to_instance("0.5 1:1")
    assert p.info().label_type == I.CONTINUOUS


def test_parser_matches_the_example_parser_on_grouped_text(tmp_path):
    H = host()
    lines = ["1 100;7:2 9:2 11:3 5:3", "0 101;8:2 5:3", "1 102;7:2"]
    fmt = "ADFEA"
    slots, _, bad = H.parse_text("\n".join(lines) + "\n", getattr(H.TextFormat, fmt), False, False, False)
    if bad:
        pytest.skip("sample lines are not in this parser's ADFEA dialect")
    p = I.TextParser(fmt)
    ins = [p.to_instance(l) for l in lines]
    assert all(i is not None for i in ins)
    for gid in (k for k in slots if k != 0):
        want = np.asarray(slots[gid]["index"], np.uint64)
        got = np.concatenate([g.fea_id for i in ins for g in i.fea_grp if g.grp_id == gid])
        assert got.tolist() == want.tolist()
    assert p.info().fea_type == I.SPARSE_BINARY and p.info().nnz_ele == sum(len(slots[g]["index"]) for g in slots if g != 0)


def test_text2proto_showins_proto2bin(tmp_path, capsys):
    src = tmp_path / "d.libsvm"
    src.write_text("1 3:0.5 7:1.5 10:2\n-1 1:1 7:0.25\nbroken\n1 2:3\n")
    out = str(tmp_path / "part")
    r = I.text2proto("LIBSVM", str(src), out)
    assert r == {"instances": 3, "skipped": 1, "nnz": 6}
    assert "num_ins: 3" in open(out + ".info").read()
    assert I.showins(out + ".recordio", 2) == 2
    assert capsys.readouterr().out.splitlines()[0] == "1 [1] 3:0.5 7:1.5 10:2"
    b = I.proto2bin(out + ".recordio", str(tmp_path / "bin"))
    assert b == {"rows": 3, "cols": 11, "nnz": 6, "binary": False}
    m = H = host().read_bin_matrix(str(tmp_path / "bin"))
    assert m["offset"].tolist() == [0, 3, 5, 6] and m["index"].tolist() == [3, 7, 10, 1, 7, 2]
    assert np.allclose(m["value"], [0.5, 1.5, 2, 1, 0.25, 3])
    assert np.fromfile(str(tmp_path / "bin") + ".label", np.float32).tolist() == [1, -1, 1]


def test_codec_roundtrip_property():
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    u64 = st.integers(min_value=0, max_value=(1 << 64) - 1)
    f32 = st.floats(width=32, allow_nan=False, allow_infinity=True)
    group = st.tuples(st.integers(0, 4095), st.lists(u64, max_size=12), st.booleans()).flatmap(
        lambda t: st.tuples(st.just(t[0]), st.just(t[1]), st.lists(f32, min_size=len(t[1]), max_size=len(t[1])) if t[2] else st.just([])))

    @settings(max_examples=150, deadline=None)
    @given(st.one_of(st.none(), f32), st.lists(group, max_size=5), st.one_of(st.none(), st.integers(-(1 << 63), (1 << 63) - 1)))
    def check(label, groups, ins_id):
        ins = I.Instance(label=label, ins_id=ins_id, fea_grp=[
            I.FeatureGroup(g, np.asarray(ids, np.uint64), np.asarray(vals, np.float32)) for g, ids, vals in groups])
        back = I.Instance.decode(ins.encode())
        assert (back.label is None) == (label is None) and (label is None or np.float32(back.label) == np.float32(label))
        assert back.ins_id == ins_id and len(back.fea_grp) == len(groups)
        for b, (g, ids, vals) in zip(back.fea_grp, groups):
            assert b.grp_id == g and b.fea_id.tolist() == ids
            assert np.array_equal(b.fea_val, np.asarray(vals, np.float32))

    check()
