"""Data ingest: text parsers, slot reader cache, stream reader, file search, binary matrices."""
import gzip
import os

import numpy as np
import pytest

from parameter_server_b200.runtime import host

H = host()

LIBSVM = "1 3:0.5 7:1.5 100:2\n-1 1:1 3:0.25\n+1 7:3\nbad line here\n-1 9:1 8:1\n"
ADFEA = "1001 1 1 11:1 12:1 99:7\n1002 1 0 13:1 98:7 97:7\n"
TERAFEA = "1 77 | %d %d %d\n0 78 | %d\n" % ((3 << 54) | 5, (3 << 54) | 2, (9 << 54) | 1, (9 << 54) | 4)


def test_libsvm_parser():
    slots, info, bad = H.parse_text(LIBSVM, H.TextFormat.LIBSVM)
    assert bad == 2 and info["num_ex"] == 3          # unordered ids and garbage are rejected
    assert slots[0]["value"].tolist() == [1.0, -1.0, 1.0]
    s = slots[1]
    assert s["offset"].tolist() == [0, 3, 5, 6] and s["index"].tolist() == [3, 7, 100, 1, 3, 7]
    assert s["value"].tolist() == [0.5, 1.5, 2.0, 1.0, 0.25, 3.0]
    si = info["slot"][1]
    assert (si["min_key"], si["max_key"], si["nnz_ele"], si["nnz_ex"], si["format"]) == (1, 101, 6, 3, "SPARSE")


def test_adfea_parser_groups_and_ignore():
    slots, info, bad = H.parse_text(ADFEA, H.TextFormat.ADFEA)
    assert bad == 0 and slots[0]["value"].tolist() == [1.0, -1.0]
    assert slots[1]["offset"].tolist() == [0, 2, 3] and slots[1]["index"].tolist() == [11, 12, 13]
    assert slots[7]["offset"].tolist() == [0, 1, 3] and slots[7]["index"].tolist() == [99, 98, 97]
    assert len(slots[7]["value"]) == 0 and info["slot"][7]["format"] == "SPARSE_BINARY"
    merged, minfo, _ = H.parse_text(ADFEA, H.TextFormat.ADFEA, True)
    assert sorted(merged.keys()) == [0, 1] and merged[1]["offset"].tolist() == [0, 3, 6]


def test_terafea_parser_sorts_groups_and_shuffles():
    slots, info, bad = H.parse_text(TERAFEA, H.TextFormat.TERAFEA)
    assert bad == 0 and slots[0]["value"].tolist() == [1.0, -1.0]
    assert slots[3]["index"].tolist() == [(3 << 54) | 2, (3 << 54) | 5] and slots[3]["offset"].tolist() == [0, 2, 2]
    assert slots[9]["offset"].tolist() == [0, 1, 2]
    sh, _, _ = H.parse_text(TERAFEA, H.TextFormat.TERAFEA, False, True)
    assert sh[3]["index"].tolist() == [H.shuffle_feature_id((3 << 54) | 2), H.shuffle_feature_id((3 << 54) | 5)]
    beta, binfo, _ = H.parse_text(TERAFEA, H.TextFormat.TERAFEA, False, False, True)
    assert beta[1023]["index"].tolist() == [0, 0]


def _write_parts(tmp_path, n_files=3, rows=40):
    rng = np.random.RandomState(0)
    files, all_rows = [], []
    d = tmp_path / "train"
    d.mkdir()
    for f in range(n_files):
        lines = []
        for _ in range(rows):
            idx = np.sort(rng.choice(500, size=rng.randint(1, 8), replace=False))
            val = rng.rand(len(idx)).round(3)
            y = 1 if rng.rand() < 0.5 else -1
            lines.append(f"{y} " + " ".join(f"{i}:{v}" for i, v in zip(idx, val)))
            all_rows.append((y, idx, val))
        p = d / f"part-{f:03d}"
        if f == 1:
            with gzip.open(str(p) + ".gz", "wt") as g:     # gz files are read transparently
                g.write("\n".join(lines) + "\n")
            files.append(str(p) + ".gz")
        else:
            p.write_text("\n".join(lines) + "\n")
            files.append(str(p))
    return files, all_rows


def test_search_and_divide_files(tmp_path):
    files, _ = _write_parts(tmp_path)
    (tmp_path / "train" / "other.txt").write_text("x")
    found = H.search_files([str(tmp_path / "train" / "part-.*")])
    assert found == sorted(files)
    parts = H.divide_files(found, 2)
    assert parts[0] == [found[0], found[2]] and parts[1] == [found[1]]
    assert H.divide_files(found, 2, 1) == [[found[0]], [found[1]]]


def test_slot_reader_cache_and_stream_reader(tmp_path):
    files, rows = _write_parts(tmp_path)
    cache = str(tmp_path / "cache")
    r = H.SlotReader()
    r.init(files, H.TextFormat.LIBSVM, cache)
    info, hits = r.read(3)
    assert hits == 0 and info["num_ex"] == len(rows)
    off, idx, val, y = r.offset(1), r.index(1), r.value(1), r.value(0)
    assert y.tolist() == [float(t[0]) for t in rows]
    assert off[-1] == sum(len(t[1]) for t in rows) == len(idx) == len(val)
    assert idx.tolist() == [int(i) for t in rows for i in t[1]]
    np.testing.assert_allclose(val, [v for t in rows for v in t[2]], rtol=1e-6)
    assert info["slot"][1]["nnz_ele"] == len(idx) and os.path.exists(r.cache_name(files[0], 1) + ".colidx.partition")
    r2 = H.SlotReader()
    r2.init(files, H.TextFormat.LIBSVM, cache)
    info2, hits2 = r2.read(2)
    assert hits2 == len(files) and info2["num_ex"] == info["num_ex"]
    assert np.array_equal(r2.index(1), idx) and np.array_equal(r2.offset(1), off)
    s = H.StreamReader()
    s.init(files, H.TextFormat.LIBSVM)
    seen, batches = 0, 0
    while True:
        out = s.read(25)
        if out is None:
            break
        slots, binfo = out
        n = binfo["num_ex"]
        assert slots[0]["value"].tolist() == [float(t[0]) for t in rows[seen:seen + n]]
        assert slots[1]["offset"][-1] == sum(len(t[1]) for t in rows[seen:seen + n])
        seen += n
        batches += 1
    assert seen == len(rows) and batches == 5


def test_bin_matrix_roundtrip(tmp_path):
    off = np.array([0, 2, 2, 5], dtype=np.uint64)
    idx = np.array([1, 4, 0, 2, 3], dtype=np.uint64)
    val = np.array([.5, 1, 2, 3, 4], dtype=np.float32)
    name = str(tmp_path / "m")
    assert H.write_bin_matrix(name, True, 3, 5, off, idx, val, 4)
    m = H.read_bin_matrix(name)
    assert (m["rows"], m["cols"], m["nnz"], m["row_major"], m["binary"]) == (3, 5, 5, True, False)
    assert m["offset"].tolist() == off.tolist() and m["index"].tolist() == idx.tolist() and m["value"].tolist() == val.tolist()
    sub = H.read_bin_matrix(name, 1, 3)
    assert sub["rows"] == 2 and sub["offset"].tolist() == [0, 0, 3] and sub["index"].tolist() == [0, 2, 3]
    assert H.write_bin_matrix(name + "b", False, 3, 5, off, idx)
    assert H.read_bin_matrix(name + "b")["binary"] and H.read_bin_matrix(str(tmp_path / "nope")) is None
