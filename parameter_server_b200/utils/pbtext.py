"""Protocol-buffer *text format* reader/writer driven by a small declarative schema.

The job files of the reference are text-format ``PS.AppConfig`` messages
(src/system/postoffice.cc:72, schema in src/proto/*.proto).  There is no ``protoc`` in
this environment, so the schema is declared in Python (see ``parameter_server_b200.config``)
and this module implements the grammar: ``name: value``, ``name { ... }``, ``name: { ... }``,
``name < ... >``, ``#`` comments, quoted strings with escapes and adjacent-string
concatenation, enum names or numbers, ``[a, b]`` lists for repeated scalars, optional ``,``/``;``
separators.  Unknown fields and enum names are errors, as with protobuf.
"""
from __future__ import annotations

import re
from typing import Any, Dict, List, Optional, Tuple

SCALARS = {"string", "bytes", "bool", "int32", "int64", "uint32", "uint64", "float", "double"}


class Enum:
    def __init__(self, name: str, **values: int):
        self.name, self.values = name, dict(values)
        self.names = {v: k for k, v in values.items()}

    def parse(self, tok: str) -> str:
        if tok in self.values:
            return tok
        try:
            n = int(tok, 0)
        except ValueError:
            raise ValueError(f"unknown value {tok!r} for enum {self.name}") from None
        if n not in self.names:
            raise ValueError(f"unknown number {n} for enum {self.name}")
        return self.names[n]


class Field:
    def __init__(self, name: str, ftype, label: str = "optional", default: Any = None):
        self.name, self.type, self.label, self.default = name, ftype, label, default

    @property
    def repeated(self) -> bool:
        return self.label == "repeated"


class Schema:
    """A message type: ordered fields by name."""

    def __init__(self, name: str, *fields: Field):
        self.name = name
        self.fields: Dict[str, Field] = {f.name: f for f in fields}

    def add(self, *fields: Field) -> "Schema":
        for f in fields:
            self.fields[f.name] = f
        return self

    def __call__(self, **kw) -> "Message":
        m = Message(self)
        for k, v in kw.items():
            setattr(m, k, v)
        return m


class Message:
    """Instance of a :class:`Schema`.  Unset optional fields read as their default
    (sub-messages read as an empty message); ``has(name)`` tells whether a field was set."""

    def __init__(self, schema: Schema):
        object.__setattr__(self, "_schema", schema)
        object.__setattr__(self, "_values", {})

    def has(self, name: str) -> bool:
        v = self._values.get(name)
        return v is not None and (not isinstance(v, list) or len(v) > 0)

    def __getattr__(self, name: str):
        sch: Schema = object.__getattribute__(self, "_schema")
        vals = object.__getattribute__(self, "_values")
        if name not in sch.fields:
            raise AttributeError(f"{sch.name} has no field {name!r}")
        f = sch.fields[name]
        if name in vals:
            return vals[name]
        if f.repeated:
            vals[name] = []
            return vals[name]
        if isinstance(f.type, Schema):
            return Message(f.type)          # detached empty default
        if f.default is not None:
            return f.default
        if isinstance(f.type, Enum):
            return next(iter(f.type.values))
        return {"string": "", "bytes": b"", "bool": False, "float": 0.0, "double": 0.0}.get(f.type, 0)

    def __setattr__(self, name: str, value):
        if name not in self._schema.fields:
            raise AttributeError(f"{self._schema.name} has no field {name!r}")
        self._values[name] = value

    def get(self, name: str):
        """Field access by string, for names that are Python keywords (``lambda``, ``in``)."""
        return self.__getattr__(name)

    def set(self, name: str, value) -> None:
        self.__setattr__(name, value)

    def mutable(self, name: str) -> "Message":
        f = self._schema.fields[name]
        if name not in self._values:
            self._values[name] = Message(f.type)
        return self._values[name]

    def add(self, name: str, value=None):
        f = self._schema.fields[name]
        lst = self.__getattr__(name)
        if value is None and isinstance(f.type, Schema):
            value = Message(f.type)
        lst.append(value)
        return value

    def copy(self) -> "Message":
        return parse(dumps(self), self._schema)

    def __repr__(self) -> str:
        return f"<{self._schema.name} {dumps(self, oneline=True)}>"

    def __eq__(self, other) -> bool:
        return isinstance(other, Message) and dumps(self) == dumps(other)


# ------------------------------------------------------------------ tokenizer
_TOKEN = re.compile(r"""
    (?P<ws>\s+|\#[^\n]*)
  | (?P<str>"(?:\\.|[^"\\])*"|'(?:\\.|[^'\\])*')
  | (?P<sym>[{}<>\[\]:,;])
  | (?P<word>[^\s{}<>\[\]:,;"'#]+)
""", re.X)

_ESC = {"n": "\n", "t": "\t", "r": "\r", "\\": "\\", '"': '"', "'": "'", "0": "\0"}


def _unescape(s: str) -> str:
    out, i = [], 0
    while i < len(s):
        c = s[i]
        if c == "\\" and i + 1 < len(s):
            n = s[i + 1]
            if n in _ESC:
                out.append(_ESC[n]); i += 2; continue
            if n == "x":
                out.append(chr(int(s[i + 2:i + 4], 16))); i += 4; continue
            if n.isdigit():
                j = i + 1
                while j < len(s) and j < i + 4 and s[j].isdigit():
                    j += 1
                out.append(chr(int(s[i + 1:j], 8))); i = j; continue
        out.append(c); i += 1
    return "".join(out)


def _tokenize(text: str) -> List[Tuple[str, str]]:
    toks, pos = [], 0
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m:
            raise ValueError(f"cannot tokenize at offset {pos}: {text[pos:pos + 20]!r}")
        pos = m.end()
        if m.lastgroup == "ws":
            continue
        toks.append((m.lastgroup, m.group(m.lastgroup)))
    return toks


# ------------------------------------------------------------------ parser
class _Parser:
    def __init__(self, toks):
        self.toks, self.i = toks, 0

    def peek(self) -> Optional[Tuple[str, str]]:
        return self.toks[self.i] if self.i < len(self.toks) else None

    def next(self) -> Tuple[str, str]:
        t = self.peek()
        if t is None:
            raise ValueError("unexpected end of input")
        self.i += 1
        return t

    def accept(self, sym: str) -> bool:
        t = self.peek()
        if t and t[0] == "sym" and t[1] == sym:
            self.i += 1
            return True
        return False

    def message(self, schema: Schema, close: Optional[str]) -> Message:
        msg = Message(schema)
        while True:
            t = self.peek()
            if t is None:
                if close is None:
                    return msg
                raise ValueError(f"missing {close!r} in {schema.name}")
            if t[0] == "sym" and t[1] == close:
                self.i += 1
                return msg
            if t[0] == "sym" and t[1] in ",;":
                self.i += 1
                continue
            kind, name = self.next()
            if kind != "word":
                raise ValueError(f"expected a field name in {schema.name}, got {name!r}")
            if name not in schema.fields:
                raise ValueError(f"message {schema.name} has no field named {name!r}")
            f = schema.fields[name]
            if isinstance(f.type, Schema):
                self.accept(":")
                t = self.next()
                if t[0] != "sym" or t[1] not in "{<":
                    raise ValueError(f"expected '{{' after {schema.name}.{name}")
                sub = self.message(f.type, "}" if t[1] == "{" else ">")
                if f.repeated:
                    msg.__getattr__(name).append(sub)
                else:
                    msg._values[name] = sub
            else:
                if not self.accept(":"):
                    raise ValueError(f"expected ':' after {schema.name}.{name}")
                if self.accept("["):
                    if not f.repeated:
                        raise ValueError(f"list value for non-repeated field {schema.name}.{name}")
                    while not self.accept("]"):
                        msg.__getattr__(name).append(self.scalar(f, schema))
                        self.accept(",")
                else:
                    v = self.scalar(f, schema)
                    if f.repeated:
                        msg.__getattr__(name).append(v)
                    else:
                        msg._values[name] = v

    def scalar(self, f: Field, schema: Schema):
        kind, tok = self.next()
        if isinstance(f.type, Enum):
            if kind != "word":
                raise ValueError(f"expected an enum value for {schema.name}.{f.name}")
            return f.type.parse(tok)
        if f.type in ("string", "bytes"):
            if kind != "str":
                raise ValueError(f"expected a quoted string for {schema.name}.{f.name}, got {tok!r}")
            s = _unescape(tok[1:-1])
            while self.peek() and self.peek()[0] == "str":      # adjacent strings concatenate
                s += _unescape(self.next()[1][1:-1])
            return s
        if kind != "word":
            raise ValueError(f"expected a value for {schema.name}.{f.name}, got {tok!r}")
        if f.type == "bool":
            low = tok.lower()
            if low in ("true", "t", "1"):
                return True
            if low in ("false", "f", "0"):
                return False
            raise ValueError(f"bad bool {tok!r} for {schema.name}.{f.name}")
        if f.type in ("float", "double"):
            t = tok.rstrip("fF") if not tok.lower().startswith("0x") else tok
            low = t.lower()
            if low in ("inf", "infinity"):
                return float("inf")
            if low in ("-inf", "-infinity"):
                return float("-inf")
            return float(t)
        v = int(tok, 0)
        lo, hi = {"int32": (-2**31, 2**31 - 1), "int64": (-2**63, 2**63 - 1), "uint32": (0, 2**32 - 1),
                  "uint64": (0, 2**64 - 1)}[f.type]
        if not lo <= v <= hi:
            raise ValueError(f"{v} out of range for {f.type} field {schema.name}.{f.name}")
        return v


def parse(text: str, schema: Schema) -> Message:
    p = _Parser(_tokenize(text))
    msg = p.message(schema, None)
    check_required(msg)
    return msg


def parse_file(path: str, schema: Schema) -> Message:
    with open(path) as f:
        return parse(f.read(), schema)


def check_required(msg: Message) -> None:
    for f in msg._schema.fields.values():
        if f.label == "required" and f.name not in msg._values:
            raise ValueError(f"missing required field {msg._schema.name}.{f.name}")
        v = msg._values.get(f.name)
        if isinstance(f.type, Schema) and v is not None:
            for sub in (v if f.repeated else [v]):
                check_required(sub)


# ------------------------------------------------------------------ printer
def _fmt(f: Field, v) -> str:
    if isinstance(f.type, Enum):
        return str(v)
    if f.type in ("string", "bytes"):
        s = v.decode("latin1") if isinstance(v, bytes) else v
        return '"' + s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'
    if f.type == "bool":
        return "true" if v else "false"
    if f.type in ("float", "double"):
        return repr(float(v))
    return str(int(v))


def dumps(msg: Message, indent: int = 0, oneline: bool = False) -> str:
    out: List[str] = []
    pad = "" if oneline else "  " * indent
    for f in msg._schema.fields.values():
        if f.name not in msg._values:
            continue
        vals = msg._values[f.name] if f.repeated else [msg._values[f.name]]
        for v in vals:
            if isinstance(f.type, Schema):
                if oneline:
                    out.append(f"{f.name} {{ {dumps(v, 0, True)} }}")
                else:
                    out.append(f"{pad}{f.name} {{\n{dumps(v, indent + 1)}{pad}}}\n")
            else:
                out.append(f"{pad}{f.name}: {_fmt(f, v)}" + ("" if oneline else "\n"))
    return (" " if oneline else "").join(out)
