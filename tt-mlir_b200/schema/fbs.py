"""A small FlatBuffers toolkit: schema model, binary writer and binary reader.

There is no `flatc` and no flatbuffers runtime on the build machine, so the wire
format (https://flatbuffers.dev/internals) is implemented here directly:

* `Schema` holds enum / struct / table / union declarations.  Field ids are
  positional, exactly as flatc assigns them when no `id:` attribute is used; a
  union field occupies two consecutive ids (`<name>_type` then `<name>`).
* `Writer` serialises nested Python dicts into a buffer, children first and
  back to front, with vtable de-duplication.  A dict that is passed twice (same
  object identity) is emitted once and shared, which is how the tt-mlir
  serialiser shares one `TensorRef` table between an op's result and its uses
  (include/ttmlir/Target/Utils/FlatbufferObjectCache.h).
* `Reader` turns a buffer back into dicts (used by tests and the JSON dump).
"""

from __future__ import annotations

import struct as _struct
from dataclasses import dataclass, field as _field
from typing import Any, Dict, List, Optional, Tuple

SCALARS = {
    "bool": ("?", 1), "u8": ("B", 1), "i8": ("b", 1), "u16": ("H", 2), "i16": ("h", 2),
    "u32": ("I", 4), "i32": ("i", 4), "u64": ("Q", 8), "i64": ("q", 8),
    "f32": ("f", 4), "f64": ("d", 8),
}

CPP_SCALARS = {
    "bool": "bool", "u8": "uint8_t", "i8": "int8_t", "u16": "uint16_t", "i16": "int16_t",
    "u32": "uint32_t", "i32": "int32_t", "u64": "uint64_t", "i64": "int64_t",
    "f32": "float", "f64": "double",
}


class _Null:
    """Marker for `= null` optional scalars (absent unless explicitly set)."""

    def __repr__(self):
        return "OPT"


OPT = _Null()


@dataclass
class Enum:
    name: str
    base: str
    values: Dict[str, int]
    ns: str

    def value(self, v) -> int:
        if isinstance(v, str):
            return self.values[v]
        return int(v)

    def name_of(self, v: int) -> str:
        for k, x in self.values.items():
            if x == v:
                return k
        return str(v)


@dataclass
class Field:
    name: str
    type: str
    default: Any = None  # None -> 0 / absent; OPT -> optional scalar
    id: int = 0          # vtable slot (first of two for unions)


@dataclass
class Struct:
    name: str
    fields: List[Field]
    ns: str
    size: int = 0
    align: int = 1
    offsets: List[int] = _field(default_factory=list)


@dataclass
class Table:
    name: str
    fields: List[Field]
    ns: str
    nslots: int = 0


@dataclass
class Union:
    name: str
    members: List[Tuple[str, str]]  # (alias, table name); type id = index + 1
    ns: str

    def type_id(self, alias: str) -> int:
        for i, (a, t) in enumerate(self.members):
            if a == alias or t == alias:
                return i + 1
        raise KeyError(f"{alias} is not a member of union {self.name}")


class Schema:
    def __init__(self):
        self.enums: Dict[str, Enum] = {}
        self.structs: Dict[str, Struct] = {}
        self.tables: Dict[str, Table] = {}
        self.unions: Dict[str, Union] = {}
        self.order: List[Tuple[str, str]] = []  # declaration order (kind, name)
        self.ns = ""

    # ---- declaration helpers -------------------------------------------------
    def namespace(self, ns: str):
        self.ns = ns

    def enum(self, name, base, values):
        if isinstance(values, (list, tuple)):
            values = {v: i for i, v in enumerate(values)}
        self.enums[name] = Enum(name, base, dict(values), self.ns)
        self.order.append(("enum", name))

    def struct(self, name, fields):
        fs = [Field(*f) for f in fields]
        st = Struct(name, fs, self.ns)
        off = 0
        for f in fs:
            sz, al = self._inline_size_align(f.type)
            off = (off + al - 1) // al * al
            st.offsets.append(off)
            off += sz
            st.align = max(st.align, al)
        st.size = (off + st.align - 1) // st.align * st.align
        self.structs[name] = st
        self.order.append(("struct", name))

    def table(self, name, fields):
        fs = []
        slot = 0
        for f in fields:
            fld = Field(*f)
            fld.id = slot
            slot += 2 if self.is_union(fld.type) or fld.type == "opaque_union" else 1
            fs.append(fld)
        self.tables[name] = Table(name, fs, self.ns, slot)
        self.order.append(("table", name))

    def union(self, name, members):
        ms = [(m, m) if isinstance(m, str) else tuple(m) for m in members]
        self.unions[name] = Union(name, ms, self.ns)
        self.order.append(("union", name))

    # ---- type classification -------------------------------------------------
    def is_union(self, t):
        return t in self.unions

    def is_scalar(self, t):
        return t in SCALARS or t in self.enums

    def scalar_fmt(self, t):
        if t in self.enums:
            t = self.enums[t].base
        return SCALARS[t]

    def _inline_size_align(self, t):
        if self.is_scalar(t):
            sz = self.scalar_fmt(t)[1]
            return sz, sz
        if t in self.structs:
            return self.structs[t].size, self.structs[t].align
        raise TypeError(f"type {t} has no inline layout")


# ==============================================================================
# Writer
# ==============================================================================


class Writer:
    def __init__(self, schema: Schema, initial: int = 1 << 16):
        self.s = schema
        self.buf = bytearray(initial)
        self.head = initial
        self.minalign = 1
        self.vtables: Dict[bytes, int] = {}
        self.shared: Dict[int, int] = {}
        self._keepalive: List[Any] = []

    # ---- low level -----------------------------------------------------------
    def offset(self) -> int:
        return len(self.buf) - self.head

    def _grow(self, need: int):
        while self.head < need:
            old = len(self.buf)
            new = bytearray(old * 2)
            new[old:] = self.buf  # keep content at the end
            self.buf = new
            self.head += old

    def _pad(self, n):
        for _ in range(n):
            self.head -= 1
            self.buf[self.head] = 0

    def prep(self, size: int, additional: int):
        if size > self.minalign:
            self.minalign = size
        align = (-(self.offset() + additional)) & (size - 1)
        self._grow(align + size + additional)
        self._pad(align)

    def place(self, fmt: str, size: int, v):
        self.head -= size
        _struct.pack_into("<" + fmt, self.buf, self.head, v)

    def prepend(self, fmt, size, v):
        self.prep(size, 0)
        self.place(fmt, size, v)

    def prepend_uoffset(self, off: int):
        self.prep(4, 0)
        assert off <= self.offset()
        self.place("I", 4, self.offset() - off + 4)

    def create_string(self, s) -> int:
        b = s.encode("utf-8") if isinstance(s, str) else bytes(s)
        self.prep(4, len(b) + 1)
        self.place("B", 1, 0)
        self._grow(len(b))
        self.head -= len(b)
        self.buf[self.head:self.head + len(b)] = b
        self.place("I", 4, len(b))
        return self.offset()

    def create_bytes_vector(self, b: bytes, align: int = 1) -> int:
        self.prep(4, len(b))
        self.prep(align, len(b))
        self._grow(len(b))
        self.head -= len(b)
        self.buf[self.head:self.head + len(b)] = b
        self.place("I", 4, len(b))
        return self.offset()

    # ---- schema driven -------------------------------------------------------
    def _struct_bytes(self, st: Struct, v) -> bytes:
        out = bytearray(st.size)
        if isinstance(v, dict):
            vals = [v.get(f.name, 0) for f in st.fields]
        else:
            vals = list(v)
        for f, off, x in zip(st.fields, st.offsets, vals):
            if f.type in self.s.structs:
                sub = self._struct_bytes(self.s.structs[f.type], x)
                out[off:off + len(sub)] = sub
            else:
                fmt, _ = self.s.scalar_fmt(f.type)
                if f.type in self.s.enums:
                    x = self.s.enums[f.type].value(x)
                _struct.pack_into("<" + fmt, out, off, x)
        return bytes(out)

    def create_vector(self, elem: str, values) -> int:
        s = self.s
        if s.is_scalar(elem):
            fmt, sz = s.scalar_fmt(elem)
            if isinstance(values, (bytes, bytearray, memoryview)) and sz == 1:
                return self.create_bytes_vector(bytes(values))
            if elem in s.enums:
                values = [s.enums[elem].value(v) for v in values]
            data = _struct.pack("<%d%s" % (len(values), fmt), *values)
            self.prep(4, len(data))
            self.prep(sz, len(data))
            self._grow(len(data))
            self.head -= len(data)
            self.buf[self.head:self.head + len(data)] = data
            self.place("I", 4, len(values))
            return self.offset()
        if elem in s.structs:
            st = s.structs[elem]
            data = b"".join(self._struct_bytes(st, v) for v in values)
            self.prep(4, len(data))
            self.prep(st.align, len(data))
            self._grow(len(data))
            self.head -= len(data)
            self.buf[self.head:self.head + len(data)] = data
            self.place("I", 4, len(values))
            return self.offset()
        # offsets: strings or tables
        if elem == "string":
            offs = [self.create_string(v) for v in values]
        elif elem in s.tables:
            offs = [self.create_table(elem, v) for v in values]
        else:
            raise TypeError(f"unsupported vector element type {elem}")
        self.prep(4, 4 * len(offs))
        for o in reversed(offs):
            self.prepend_uoffset(o)
        self.place("I", 4, len(offs))
        return self.offset()

    def create_table(self, tname: str, v: Dict[str, Any]) -> int:
        s = self.s
        key = id(v)
        if key in self.shared:
            return self.shared[key]
        t = s.tables[tname]
        unknown = set(v.keys()) - {f.name for f in t.fields}
        if unknown:
            raise KeyError(f"table {tname} has no field(s) {sorted(unknown)}")
        # 1. children first
        pre: Dict[str, Any] = {}
        for f in t.fields:
            if f.name not in v or v[f.name] is None:
                continue
            x = v[f.name]
            ft = f.type
            if ft == "string":
                pre[f.name] = self.create_string(x)
            elif ft.startswith("["):
                pre[f.name] = self.create_vector(ft[1:-1], x)
            elif ft in s.tables:
                pre[f.name] = self.create_table(ft, x)
            elif ft in s.unions:
                alias, val = x
                u = s.unions[ft]
                tid = u.type_id(alias)
                pre[f.name] = (tid, self.create_table(u.members[tid - 1][1], val))
            elif ft in ("opaque", "opaque_union"):
                raise TypeError(f"{tname}.{f.name} is opaque and cannot be written")
        # 2. the table itself
        slots = [0] * t.nslots
        object_end = self.offset()
        # Larger scalars first keeps padding small, as flatc does; ids are what matter.
        for f in sorted(t.fields, key=lambda f: -self._field_size(f)):
            if f.name not in v or v[f.name] is None:
                continue
            x = v[f.name]
            ft = f.type
            if s.is_scalar(ft):
                fmt, sz = s.scalar_fmt(ft)
                if ft in s.enums:
                    x = s.enums[ft].value(x)
                    dflt = 0 if f.default in (None, OPT) else s.enums[ft].value(f.default)
                else:
                    dflt = 0 if f.default in (None, OPT) else f.default
                if f.default is not OPT and x == dflt:
                    continue
                self.prepend(fmt, sz, x)
                slots[f.id] = self.offset()
            elif ft in s.structs:
                st = s.structs[ft]
                data = self._struct_bytes(st, x)
                self.prep(st.align, len(data))
                self._grow(len(data))
                self.head -= len(data)
                self.buf[self.head:self.head + len(data)] = data
                slots[f.id] = self.offset()
            elif ft in s.unions:
                tid, off = pre[f.name]
                self.prepend_uoffset(off)
                slots[f.id + 1] = self.offset()
                self.prepend("B", 1, tid)
                slots[f.id] = self.offset()
            else:
                self.prepend_uoffset(pre[f.name])
                slots[f.id] = self.offset()
        off = self._end_table(slots, object_end)
        self.shared[key] = off
        self._keepalive.append(v)  # ids stay unique while the writer lives
        return off

    def _field_size(self, f: Field) -> int:
        if self.s.is_scalar(f.type):
            return self.s.scalar_fmt(f.type)[1]
        if f.type in self.s.structs:
            return self.s.structs[f.type].align
        return 4

    def _end_table(self, slots: List[int], object_end: int) -> int:
        self.prepend("i", 4, 0)
        object_offset = self.offset()
        n = len(slots)
        while n > 0 and slots[n - 1] == 0:
            n -= 1
        vt = [(n + 2) * 2, object_offset - object_end]
        vt += [(object_offset - slots[i]) if slots[i] else 0 for i in range(n)]
        vt_bytes = _struct.pack("<%dH" % len(vt), *vt)
        existing = self.vtables.get(vt_bytes)
        if existing is None:
            self.prep(2, len(vt_bytes))
            self._grow(len(vt_bytes))
            self.head -= len(vt_bytes)
            self.buf[self.head:self.head + len(vt_bytes)] = vt_bytes
            existing = self.offset()
            self.vtables[vt_bytes] = existing
        _struct.pack_into("<i", self.buf, len(self.buf) - object_offset, existing - object_offset)
        return object_offset

    def finish(self, root: int, identifier: bytes, size_prefixed: bool = True) -> bytes:
        assert len(identifier) == 4
        extra = 4 + 4 + (4 if size_prefixed else 0)
        self.prep(self.minalign, extra)
        for b in reversed(identifier):
            self.place("B", 1, b)
        self.prepend_uoffset(root)
        if size_prefixed:
            self.place("I", 4, self.offset())
        return bytes(self.buf[self.head:])


# ==============================================================================
# Reader (to dicts)
# ==============================================================================


class Reader:
    def __init__(self, schema: Schema, buf: bytes, size_prefixed: bool = True):
        self.s = schema
        self.buf = memoryview(buf)
        self.base = 4 if size_prefixed else 0

    def _u(self, fmt, pos):
        return _struct.unpack_from("<" + fmt, self.buf, pos)[0]

    def identifier(self) -> bytes:
        return bytes(self.buf[self.base + 4:self.base + 8])

    def root(self, tname: str, max_bytes_vector: Optional[int] = None):
        pos = self.base + self._u("I", self.base)
        self.max_bytes_vector = max_bytes_vector
        return self.table(tname, pos)

    def _slot(self, pos, fid):
        vt = pos - self._u("i", pos)
        vsize = self._u("H", vt)
        at = 4 + 2 * fid
        if at >= vsize:
            return 0
        return self._u("H", vt + at)

    def _struct(self, st: Struct, pos):
        out = {}
        for f, off in zip(st.fields, st.offsets):
            if f.type in self.s.structs:
                out[f.name] = self._struct(self.s.structs[f.type], pos + off)
            else:
                out[f.name] = self._scalar(f.type, pos + off)
        return out

    def _scalar(self, t, pos):
        fmt, _ = self.s.scalar_fmt(t)
        v = self._u(fmt, pos)
        if t in self.s.enums:
            return self.s.enums[t].name_of(v)
        return v

    def string(self, pos):
        n = self._u("I", pos)
        return bytes(self.buf[pos + 4:pos + 4 + n]).decode("utf-8", "replace")

    def vector(self, elem, pos):
        n = self._u("I", pos)
        p = pos + 4
        s = self.s
        if s.is_scalar(elem):
            fmt, sz = s.scalar_fmt(elem)
            if sz == 1 and elem not in s.enums:
                if self.max_bytes_vector is not None and n > self.max_bytes_vector:
                    return f"<{n} bytes>"
                return bytes(self.buf[p:p + n])
            vals = list(_struct.unpack_from("<%d%s" % (n, fmt), self.buf, p))
            if elem in s.enums:
                vals = [s.enums[elem].name_of(v) for v in vals]
            return vals
        if elem in s.structs:
            st = s.structs[elem]
            return [self._struct(st, p + i * st.size) for i in range(n)]
        out = []
        for i in range(n):
            q = p + 4 * i
            tgt = q + self._u("I", q)
            out.append(self.string(tgt) if elem == "string" else self.table(elem, tgt))
        return out

    def table(self, tname, pos):
        s = self.s
        t = s.tables[tname]
        out: Dict[str, Any] = {}
        for f in t.fields:
            ft = f.type
            if ft in ("opaque", "opaque_union"):
                continue
            off = self._slot(pos, f.id)
            if s.is_scalar(ft):
                if off:
                    out[f.name] = self._scalar(ft, pos + off)
                elif f.default is OPT:
                    out[f.name] = None
                else:
                    d = f.default if f.default is not None else (False if ft == "bool" else 0)
                    if ft in s.enums and not isinstance(d, str):
                        d = s.enums[ft].name_of(d)
                    out[f.name] = d
                continue
            if ft in s.unions:
                tid = self._u("B", pos + off) if off else 0
                voff = self._slot(pos, f.id + 1)
                if tid == 0 or not voff:
                    out[f.name] = None
                else:
                    alias, mt = s.unions[ft].members[tid - 1]
                    q = pos + voff
                    out[f.name] = (alias, self.table(mt, q + self._u("I", q)))
                continue
            if not off:
                out[f.name] = None
                continue
            if ft in s.structs:
                out[f.name] = self._struct(s.structs[ft], pos + off)
                continue
            q = pos + off
            tgt = q + self._u("I", q)
            if ft == "string":
                out[f.name] = self.string(tgt)
            elif ft.startswith("["):
                out[f.name] = self.vector(ft[1:-1], tgt)
            else:
                out[f.name] = self.table(ft, tgt)
        return out
