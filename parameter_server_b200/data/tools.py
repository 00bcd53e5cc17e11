"""Data tools: convert text data to the binary matrix format and inspect data sets.

Counterparts of the reference's ``text2proto`` / ``proto2bin`` / ``showins`` programs
(src/data/text2proto.cc, proto2bin.cc, showins.cc) and of its MATLAB converters
(src/data/matlab/*.m: bin↔mat, ``saveas_pserver``).  Binary matrices are
``name.info`` + ``.offset`` + ``.index`` + ``.value`` (+ ``name.label`` for the labels).

  python -m parameter_server_b200.data.tools text2bin LIBSVM 'data/train/part-.*' out/train
  python -m parameter_server_b200.data.tools show out/train
  python -m parameter_server_b200.data.tools info ADFEA 'data/ctr/part-.*'
  python -m parameter_server_b200.data.tools bin2text out/train out/train.libsvm
  python -m parameter_server_b200.data.tools split rcv1_train.binary rcv1 1000 13   # train/part-000.. + test/part-013..
  python -m parameter_server_b200.data.tools rcv1 rcv1                               # fetch + unpack + split (data/rcv1_binary.sh)
  python -m parameter_server_b200.data.tools text2proto LIBSVM data/part-000 out/part   # out/part.recordio + out/part.info
  python -m parameter_server_b200.data.tools showins out/part.recordio 10
  python -m parameter_server_b200.data.tools proto2bin out/part.recordio out/part_bin
"""
from __future__ import annotations

import sys

import numpy as np

from ..runtime import host


def text2bin(fmt: str, pattern: str, out: str, cache: str = "/tmp/psb200_cache/tools/") -> dict:
    H = host()
    files = H.search_files([pattern])
    if not files:
        raise FileNotFoundError(pattern)
    r = H.SlotReader()
    r.init(files, getattr(H.TextFormat, fmt), cache, True)
    info, _ = r.read(4)
    off, idx, val = r.offset(1), r.index(1), r.value(1)
    cols = int(idx.max()) + 1 if len(idx) else 0
    H.write_bin_matrix(out, True, info["num_ex"], cols, off, idx, val if len(val) else None, 8)
    r.value(0).astype(np.float32).tofile(out + ".label")
    return {"rows": info["num_ex"], "cols": cols, "nnz": int(len(idx)), "files": len(files)}


def show(name: str, rows: int = 5) -> dict:
    H = host()
    m = H.read_bin_matrix(name)
    if m is None:
        raise FileNotFoundError(name + ".info")
    out = {k: m[k] for k in ("rows", "cols", "nnz", "row_major", "binary", "sparse")}
    for r in range(min(rows, m["rows"])):
        a, b = int(m["offset"][r]), int(m["offset"][r + 1])
        feats = " ".join(f"{int(i)}" + ("" if m["binary"] else f":{float(v):g}") for i, v in
                         zip(m["index"][a:b], m["value"][a:b] if not m["binary"] else [0] * (b - a)))
        print(f"row {r}: {feats}")
    return out


def info(fmt: str, pattern: str) -> str:
    H = host()
    files = H.search_files([pattern])
    r = H.StreamReader()
    r.init(files, getattr(H.TextFormat, fmt))
    total = None
    while True:
        out = r.read(100000)
        if out is None:
            break
        _, i = out
        if total is None:
            total = {"num_ex": 0, "slots": {}}
        total["num_ex"] += i["num_ex"]
        for sid, s in i["slot"].items():
            t = total["slots"].setdefault(sid, {"nnz_ele": 0, "nnz_ex": 0, "min_key": 2**64 - 1, "max_key": 0})
            t["nnz_ele"] += s["nnz_ele"]
            t["nnz_ex"] += s["nnz_ex"]
            t["min_key"], t["max_key"] = min(t["min_key"], s["min_key"]), max(t["max_key"], s["max_key"])
    return str(total)


def bin2text(name: str, out_path: str) -> int:
    """Binary matrix (+ ``.label``) back to LIBSVM text (the MATLAB ``saveas_pserver`` direction)."""
    H = host()
    m = H.read_bin_matrix(name)
    y = np.fromfile(name + ".label", dtype=np.float32)
    with open(out_path, "w") as f:
        for r in range(m["rows"]):
            a, b = int(m["offset"][r]), int(m["offset"][r + 1])
            vals = np.ones(b - a) if m["binary"] else m["value"][a:b]
            f.write(f"{int(y[r]):+d} " + " ".join(f"{int(i)}:{float(v):g}" for i, v in zip(m["index"][a:b], vals)) + "\n")
    return m["rows"]


def split_parts(path: str, out_dir: str, lines_per_part: int = 1000, train_parts: int = 13) -> dict:
    """Cut a text data set (plain, gzip or bzip2) into ``part-NNN`` files of ``lines_per_part`` lines: the first
    ``train_parts`` go to ``<out_dir>/train``, the rest to ``<out_dir>/test`` — the layout the reference's dataset
    script produces for rcv1 (data/rcv1_binary.sh:11-36; its download step needs a network and is left to the user)."""
    import bz2
    import gzip
    import os

    opener = bz2.open if path.endswith(".bz2") else gzip.open if path.endswith(".gz") else open
    train, test = os.path.join(out_dir, "train"), os.path.join(out_dir, "test")
    for d in (train, test):
        os.makedirs(d, exist_ok=True)
        for old in os.listdir(d):
            if old.startswith("part-"):
                os.remove(os.path.join(d, old))
    counts = {"train": 0, "test": 0, "lines": 0}
    out, part = None, -1
    with opener(path, "rt") as f:
        for n, line in enumerate(f):
            if n % lines_per_part == 0:
                if out:
                    out.close()
                part += 1
                which = "train" if part < train_parts else "test"
                counts[which] += 1
                out = open(os.path.join(train if which == "train" else test, f"part-{part:03d}"), "w")
            out.write(line)
            counts["lines"] += 1
    if out:
        out.close()
    return counts


RCV1_URL = "http://www.csie.ntu.edu.tw/~cjlin/libsvmtools/datasets/binary/rcv1_train.binary.bz2"


def rcv1(out_dir: str = "rcv1", url: str = RCV1_URL, lines_per_part: int = 1000, train_parts: int = 13) -> dict:
    """The reference's data set script (data/rcv1_binary.sh): fetch ``rcv1_train.binary.bz2`` unless
    ``rcv1_train.binary`` is already in the current directory, unpack it, and cut it into ``<out_dir>/train/part-000..``
    (the first ``train_parts`` parts of ``lines_per_part`` lines) and ``<out_dir>/test/part-...`` (the rest).  Without a
    network the download fails with the URL in the message: put the file there by hand and run the command again."""
    import bz2
    import os
    import shutil
    import urllib.request

    plain = "rcv1_train.binary"
    if not os.path.exists(plain):
        packed = plain + ".bz2"
        if not os.path.exists(packed):
            try:
                with urllib.request.urlopen(url, timeout=60) as r, open(packed + ".tmp", "wb") as f:
                    shutil.copyfileobj(r, f)
            except OSError as e:
                if os.path.exists(packed + ".tmp"):
                    os.remove(packed + ".tmp")
                raise OSError(f"cannot fetch {url} ({e}); download it to ./{packed} by hand and run this again") from e
            os.replace(packed + ".tmp", packed)
        with bz2.open(packed, "rb") as src, open(plain + ".tmp", "wb") as dst:
            shutil.copyfileobj(src, dst)
        os.replace(plain + ".tmp", plain)
    return split_parts(plain, out_dir, lines_per_part, train_parts)


def main(argv=None) -> int:
    a = list(sys.argv[1:] if argv is None else argv)
    if not a:
        print(__doc__)
        return 2
    if a[0] == "text2bin":
        print(text2bin(a[1], a[2], a[3]))
    elif a[0] == "show":
        print(show(a[1]))
    elif a[0] == "info":
        print(info(a[1], a[2]))
    elif a[0] == "bin2text":
        print(bin2text(a[1], a[2]))
    elif a[0] == "text2proto":
        from .instance import text2proto
        print(text2proto(a[1], a[2], a[3]))
    elif a[0] == "showins":
        from .instance import showins
        showins(a[1], int(a[2]) if len(a) > 2 else 10)
    elif a[0] == "proto2bin":
        from .instance import proto2bin
        print(proto2bin(a[1], a[2]))
    elif a[0] == "rcv1":
        print(rcv1(a[1] if len(a) > 1 else "rcv1", a[2] if len(a) > 2 else RCV1_URL))
    elif a[0] == "split":
        print(split_parts(a[1], a[2], int(a[3]) if len(a) > 3 else 1000, int(a[4]) if len(a) > 4 else 13))
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
