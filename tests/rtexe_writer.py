"""A minimal writer of the compiled-executable container (`.rtexe`) for tests: FlatBuffers binary encoding of the
tables of executor/include/mlir-executor/Runtime/API/Executable.fbs that carry data segments, laid out as the
64-bit builder lays them out (the 64-bit section -- segment names and data, reached through 64-bit offsets -- at the
back of the buffer; 32-bit offsets point forwards).  Written from the published FlatBuffers format; there is no
`flatc` on this machine."""
import struct


def _align(buf: bytearray, n: int) -> None:
    while len(buf) % n:
        buf.append(0)


def build_rtexe(name: str, segments, source: str = "-- lua") -> bytes:
    """segments: list of dicts {name, data (bytes), alignment, constant, address_space, uninitialized_size}."""
    # The buffer is assembled front to back here (offsets are patched once positions are known); FlatBuffers only
    # requires that unsigned offsets point forwards and that scalars are aligned to their size.
    buf = bytearray(b"\x00" * 4)     # root offset, patched last
    patches32, patches64 = [], []    # (position of the offset field, key of the target)
    where = {}

    def table(fields):
        """fields: list of (kind, value) per schema slot; kind in {None, 'u8','u32','u64','off32','off64'}.  Returns the
        table position.  Layout: vtable, then the table (soffset, then fields in slot order, each aligned)."""
        sizes = {"u8": 1, "u32": 4, "u64": 8, "off32": 4, "off64": 8, "i32": 4}
        # the table body: the vtable back-reference, then the fields largest first (keeps every field aligned)
        fields = [f if f else (None, None) for f in fields]
        order = sorted([i for i, (k, _) in enumerate(fields) if k], key=lambda i: -sizes[fields[i][0]])
        offs, cur = {}, 4
        for i in order:
            sz = sizes[fields[i][0]]
            cur = (cur + sz - 1) // sz * sz
            offs[i] = cur
            cur += sz
        tsize = (cur + 3) // 4 * 4
        vt_entries = len(fields)
        vt_bytes = 4 + 2 * vt_entries
        _align(buf, 2)
        # place the vtable so that the table that follows it starts on an 8-byte boundary
        while (len(buf) + vt_bytes) % 8:
            buf.append(0)
        vt_pos = len(buf)
        buf.extend(struct.pack("<HH", vt_bytes, tsize))
        for i in range(vt_entries):
            buf.extend(struct.pack("<H", offs.get(i, 0)))
        tpos = len(buf)
        body = bytearray(tsize)
        struct.pack_into("<i", body, 0, tpos - vt_pos)
        for i, off in offs.items():
            kind, val = fields[i]
            if kind == "u8":
                struct.pack_into("<B", body, off, val)
            elif kind in ("u32", "i32"):
                struct.pack_into("<I" if kind == "u32" else "<i", body, off, val)
            elif kind == "u64":
                struct.pack_into("<Q", body, off, val)
            elif kind == "off32":
                patches32.append((tpos + off, val))
            else:
                patches64.append((tpos + off, val))
        buf.extend(body)
        return tpos

    def string(key, text):
        raw = text.encode()
        _align(buf, 4)
        where[key] = len(buf)
        buf.extend(struct.pack("<I", len(raw)) + raw + b"\x00")

    # 32-bit section: root table, the vector of segment tables, the segment tables, 32-bit strings
    seg_fields = []
    for i, s in enumerate(segments):
        seg_fields.append([("off64", ("segname", i)), ("off64", ("segdata", i)), ("u32", s.get("alignment", 16)),
                           ("u8", 1 if s.get("constant", True) else 0), ("u64", s.get("uninitialized_size", 0)),
                           ("u8", s.get("address_space", 0))])
    where["root"] = table([("off32", "name"), ("off32", "source"), ("off32", "segvec"), None, None, ("i32", 1), ("u32", 0)])
    _align(buf, 4)
    where["segvec"] = len(buf)
    buf.extend(struct.pack("<I", len(segments)))
    vec_slots = []
    for i in range(len(segments)):
        vec_slots.append(len(buf))
        buf.extend(b"\x00" * 4)
    for i, f in enumerate(seg_fields):
        where[("seg", i)] = table(f)
        patches32.append((vec_slots[i], ("seg", i)))
    string("name", name)
    string("source", source)
    # 64-bit section at the back
    for i, s in enumerate(segments):
        string(("segname", i), s["name"])
    for i, s in enumerate(segments):
        _align(buf, 8)
        where[("segdata", i)] = len(buf)
        buf.extend(struct.pack("<Q", len(s["data"])) + bytes(s["data"]))
    for pos, key in patches32:
        struct.pack_into("<I", buf, pos, where[key] - pos)
    for pos, key in patches64:
        struct.pack_into("<Q", buf, pos, where[key] - pos)
    struct.pack_into("<I", buf, 0, where["root"])
    return bytes(buf)
