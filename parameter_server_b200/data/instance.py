"""The older `Instance` record format: text lines -> per-example records with feature groups, and back.

The reference keeps a deprecated twin of its example parser that turns a text line into an ``Instance`` message
(label + feature groups of ids and optional values) and sums up an ``InstanceInfo`` (per group: non-zeros, non-empty
rows, id range; the label is reported as group 4096) — src/data/text_parser.{h,cc}, src/proto/instance.proto — and
three small programs around it: ``text2proto`` (text -> record file + ``.info``), ``showins`` (print the first
records) and ``proto2bin`` (record file -> binary matrix), src/data/{text2proto,showins,proto2bin}.cc.

Here a line is parsed by the native example parser (one line at a time) and re-shaped; the records are written in
the protobuf wire format of ``instance.proto`` by a small codec of our own (field numbers as in that schema), into
the framed record files of the host runtime (``record_write`` / ``record_read``), so files written here can be read
by any protobuf implementation that has the schema.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from ..runtime import host

LABEL_GROUP = 4096            # group id under which InstanceInfo reports the labels
_U64 = (1 << 64) - 1

# label / feature kinds of InstanceInfo
EMPTY, BINARY, MULTICLASS, CONTINUOUS = 1, 2, 3, 4
DENSE, SPARSE, SPARSE_BINARY = 1, 2, 3


# ---------------------------------------------------------------- protobuf wire format (the subset the schema needs)
def _varint(n: int) -> bytes:
    n &= _U64
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = val = 0
    while True:
        if pos >= len(buf) or shift > 63:
            raise ValueError("truncated or overlong varint")
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val & _U64, pos
        shift += 7


def _tag(fieldno: int, wire: int) -> bytes:
    return _varint(fieldno << 3 | wire)


def _fields(buf: bytes) -> Iterable[Tuple[int, int, object]]:
    """(field number, wire type, payload) of every field of one message."""
    pos = 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        fno, wire = key >> 3, key & 7
        if wire == 0:
            val, pos = _read_varint(buf, pos)
        elif wire == 1:
            val, pos = buf[pos:pos + 8], pos + 8
        elif wire == 2:
            n, pos = _read_varint(buf, pos)
            val, pos = buf[pos:pos + n], pos + n
            if len(val) != n:
                raise ValueError("truncated length-delimited field")
        elif wire == 5:
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield fno, wire, val


@dataclass
class FeatureGroup:
    grp_id: int = 0
    fea_id: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint64))
    fea_val: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))   # empty: binary features

    def encode(self) -> bytes:
        out = _tag(1, 0) + _varint(self.grp_id)
        if len(self.fea_id):
            ids = b"".join(_varint(int(k)) for k in self.fea_id)
            out += _tag(2, 2) + _varint(len(ids)) + ids
        if len(self.fea_val):
            vals = np.asarray(self.fea_val, "<f4").tobytes()
            out += _tag(3, 2) + _varint(len(vals)) + vals
        return out

    @staticmethod
    def decode(buf: bytes) -> "FeatureGroup":
        g, ids, vals = FeatureGroup(), [], []
        for fno, wire, val in _fields(buf):
            if fno == 1 and wire == 0:
                g.grp_id = int(val) if val < 1 << 31 else int(val) - (1 << 64)
            elif fno == 2 and wire == 2:                       # packed
                pos = 0
                while pos < len(val):
                    k, pos = _read_varint(val, pos)
                    ids.append(k)
            elif fno == 2 and wire == 0:                       # a writer that did not pack
                ids.append(val)
            elif fno == 3 and wire == 2:
                vals.extend(np.frombuffer(val, "<f4").tolist())
            elif fno == 3 and wire == 5:
                vals.append(struct.unpack("<f", val)[0])
        g.fea_id, g.fea_val = np.asarray(ids, np.uint64), np.asarray(vals, np.float32)
        return g


@dataclass
class Instance:
    label: Optional[float] = None
    fea_grp: List[FeatureGroup] = field(default_factory=list)
    ins_id: Optional[int] = None

    def encode(self) -> bytes:
        out = b""
        if self.label is not None:
            out += _tag(1, 5) + struct.pack("<f", self.label)
        for g in self.fea_grp:
            body = g.encode()
            out += _tag(2, 2) + _varint(len(body)) + body
        if self.ins_id is not None:
            out += _tag(3, 0) + _varint(self.ins_id)
        return out

    @staticmethod
    def decode(buf: bytes) -> "Instance":
        ins = Instance()
        for fno, wire, val in _fields(buf):
            if fno == 1 and wire == 5:
                ins.label = struct.unpack("<f", val)[0]
            elif fno == 2 and wire == 2:
                ins.fea_grp.append(FeatureGroup.decode(val))
            elif fno == 3 and wire == 0:
                ins.ins_id = int(val) if val < 1 << 63 else int(val) - (1 << 64)
        return ins

    def __str__(self) -> str:
        parts = ["" if self.label is None else f"{self.label:g}"]
        for g in self.fea_grp:
            feats = (f"{int(k)}:{float(v):g}" for k, v in zip(g.fea_id, g.fea_val)) if len(g.fea_val) else \
                (str(int(k)) for k in g.fea_id)
            parts.append(f"[{g.grp_id}] " + " ".join(feats))
        return " ".join(parts)


@dataclass
class GroupInfo:
    grp_id: int = 0
    nnz_ele: int = 0
    nnz_ins: int = 0
    fea_begin: int = _U64
    fea_end: int = 0


@dataclass
class InstanceInfo:
    label_type: int = BINARY
    fea_type: int = SPARSE
    fea_grp: List[GroupInfo] = field(default_factory=list)
    num_ins: int = 0
    nnz_ele: int = 0
    fea_begin: int = _U64
    fea_end: int = 0

    def to_text(self) -> str:
        """Protobuf text format, the form of the reference's ``.info`` files."""
        lt = {EMPTY: "EMPTY", BINARY: "BINARY", MULTICLASS: "MULTICLASS", CONTINUOUS: "CONTINUOUS"}[self.label_type]
        ft = {DENSE: "DENSE", SPARSE: "SPARSE", SPARSE_BINARY: "SPARSE_BINARY"}[self.fea_type]
        lines = [f"label_type: {lt}", f"fea_type: {ft}"]
        for g in self.fea_grp:
            lines += ["fea_grp {", f"  grp_id: {g.grp_id}", f"  fea_begin: {g.fea_begin}", f"  fea_end: {g.fea_end}",
                      f"  nnz_ele: {g.nnz_ele}", f"  nnz_ins: {g.nnz_ins}", "}"]
        lines += [f"num_ins: {self.num_ins}", f"nnz_ele: {self.nnz_ele}", f"fea_begin: {self.fea_begin}",
                  f"fea_end: {self.fea_end}"]
        return "\n".join(lines) + "\n"


class TextParser:
    """One text line -> one ``Instance``; ``info()`` sums up what went through (src/data/text_parser.cc:12-87)."""

    def __init__(self, fmt: str, ignore_fea_grp: bool = False):
        self._H = host()
        self._fmt = getattr(self._H.TextFormat, fmt.upper())
        self._ignore = ignore_fea_grp
        self._groups: Dict[int, GroupInfo] = {}
        self._labels = 0
        self._num = 0
        self._label_type = BINARY
        self._fea_type = SPARSE if fmt.upper() == "LIBSVM" else SPARSE_BINARY

    def to_instance(self, line: str) -> Optional[Instance]:
        line = line.strip()
        if not line:
            return None
        slots, _, bad = self._H.parse_text(line + "\n", self._fmt, self._ignore, False, False)
        if bad or 0 not in slots or len(slots[0]["value"]) != 1:
            return None
        ins = Instance(label=float(slots[0]["value"][0]))
        for gid in sorted(k for k in slots if k != 0):
            if gid >= LABEL_GROUP:
                return None
            s = slots[gid]
            ins.fea_grp.append(FeatureGroup(int(gid), np.asarray(s["index"], np.uint64), np.asarray(s["value"], np.float32)))
        # bookkeeping only once the whole line is known to be good
        if ins.label != int(ins.label):
            self._label_type = CONTINUOUS
        elif ins.label not in (1.0, -1.0) and self._label_type != CONTINUOUS:
            self._label_type = MULTICLASS
        for g in ins.fea_grp:
            gi = self._groups.setdefault(g.grp_id, GroupInfo(g.grp_id))
            if len(g.fea_id):
                gi.fea_begin = min(gi.fea_begin, int(g.fea_id.min()))
                gi.fea_end = max(gi.fea_end, int(g.fea_id.max()) + 1)
            gi.nnz_ins += 1
            gi.nnz_ele += len(g.fea_id)
        self._labels += 1
        self._num += 1
        return ins

    def info(self) -> InstanceInfo:
        out = InstanceInfo(label_type=self._label_type, fea_type=self._fea_type, num_ins=self._num)
        for gid in sorted(self._groups):
            g = self._groups[gid]
            if g.nnz_ele == 0:
                continue
            out.fea_grp.append(g)
            out.fea_begin, out.fea_end = min(out.fea_begin, g.fea_begin), max(out.fea_end, g.fea_end)
            out.nnz_ele += g.nnz_ele
        if self._labels:
            out.fea_grp.append(GroupInfo(LABEL_GROUP, self._labels, self._labels, 0, 1))
        return out


# ---------------------------------------------------------------- the three programs
def text2proto(fmt: str, text_path: str, out: str, ignore_fea_grp: bool = False) -> dict:
    """``out.recordio`` (one framed Instance per good line) and ``out.info`` (text-format InstanceInfo)."""
    p = TextParser(fmt, ignore_fea_grp)
    recs, skipped = [], 0
    with open(text_path, "rt") as f:
        for line in f:
            if not line.strip():
                continue
            ins = p.to_instance(line)
            if ins is None:
                skipped += 1
            else:
                recs.append(ins.encode())
    if not host().record_write(out + ".recordio", recs):
        raise OSError(f"cannot write {out}.recordio")
    info = p.info()
    with open(out + ".info", "w") as f:
        f.write(info.to_text())
    return {"instances": info.num_ins, "skipped": skipped, "nnz": info.nnz_ele}


def read_instances(path: str, limit: int = 0) -> List[Instance]:
    recs = host().record_read(path)
    return [Instance.decode(bytes(r)) for r in (recs[:limit] if limit > 0 else recs)]


def showins(path: str, n: int = 10) -> int:
    ins = read_instances(path, n)
    for i in ins:
        print(i)
    return len(ins)


def proto2bin(path: str, out: str) -> dict:
    """Record file -> binary matrix ``out.{info,offset,index,value}`` + ``out.label`` (all groups in one key space)."""
    ins = read_instances(path)
    offset, index, value, label = [0], [], [], []
    binary = all(len(g.fea_val) == 0 for i in ins for g in i.fea_grp)
    for i in ins:
        label.append(0.0 if i.label is None else i.label)
        for g in i.fea_grp:
            index.append(g.fea_id)
            if not binary:
                value.append(g.fea_val if len(g.fea_val) else np.ones(len(g.fea_id), np.float32))
        offset.append(offset[-1] + sum(len(g.fea_id) for g in i.fea_grp))
    idx = np.concatenate(index) if index else np.zeros(0, np.uint64)
    val = None if binary else (np.concatenate(value) if value else np.zeros(0, np.float32)).astype(np.float32)
    cols = int(idx.max()) + 1 if len(idx) else 0
    if not host().write_bin_matrix(out, True, len(ins), cols, np.asarray(offset, np.uint64), idx.astype(np.uint64), val, 8):
        raise OSError(f"cannot write {out}")
    np.asarray(label, np.float32).tofile(out + ".label")
    return {"rows": len(ins), "cols": cols, "nnz": int(len(idx)), "binary": binary}
