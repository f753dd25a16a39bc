"""strixw: the converted-weights file strixite's serving path loads (strixite formats/strixw.hpp, formats/strixw.cpp) -
reader, writer, and the loaders that turn its tensors into the device weights of the MoE layer.

Layout (all little-endian):
  header, 128 bytes   magic "STRIXWT\\0" | u32 version (1..4) | u32 header bytes (128) | u64 index offset (128) |
                      u64 index bytes | u64 data offset (4096-aligned) | u64 file bytes | u64 index hash | ... zeros ... |
                      u64 hash of header bytes 0..119 at offset 120
  index               u32 n_meta, n_meta x (str16 key, u32 length + value bytes);
                      u32 n_tensors, per tensor: str16 name, u8 encoding, u8 ndim, ndim x i64 shape, i64 group size,
                      i64 experts, u16 n_parts x (str16 source, i64 row offset, i64 rows),
                      u8 n_components x (u8 role, u64 offset, u64 bytes, u64 hash)
  data                tensors start on 4096-byte boundaries, their components on 256-byte boundaries
Quantized tensors are [N, K] with components q (the row-major code bytes of formats/q4.hpp ... q8.hpp), scale and min
([N, K / G] BF16 bits each); an expert stack is one such tensor with `experts` > 0 and N = experts x rows per expert.
Hashes are strix_hash64 (the C library's entry point of that name).
"""
import ctypes as C
import mmap
import os
import struct

import numpy as np

from ._lib import StrixError, lib

MAGIC = b"STRIXWT\x00"
VERSION, OLDEST_VERSION = 4, 1
HEADER_BYTES, TENSOR_ALIGN, COMPONENT_ALIGN = 128, 4096, 256

# StrixwEncoding / StrixwRole (formats/strixw.hpp:19-21)
Q4_ROW, Q4_CHUNK, BF16, F32, I64, Q8_ROW, Q8_CHUNK, Q6_ROW, Q5_ROW = 1, 2, 3, 4, 5, 6, 7, 8, 9
ENCODING_NAMES = {Q4_ROW: "q4", Q4_CHUNK: "q4-chunk-major", BF16: "bf16", F32: "f32", I64: "i64", Q8_ROW: "q8", Q8_CHUNK: "q8-chunk-major",
                  Q6_ROW: "q6", Q5_ROW: "q5"}
DATA, Q, SCALE, MIN = 0, 1, 2, 3
ROLE_NAMES = {DATA: "data", Q: "q", SCALE: "scale", MIN: "min"}
_ROW_MAJOR_BITS = {Q4_ROW: 4, Q5_ROW: 5, Q6_ROW: 6, Q8_ROW: 8}


def hash64(buf):
    """strix_hash64 of a bytes-like object / numpy array."""
    a = np.frombuffer(buf, dtype=np.uint8) if not isinstance(buf, np.ndarray) else np.ascontiguousarray(buf).view(np.uint8).reshape(-1)
    return int(lib.strix_hash64(a.ctypes.data_as(C.c_void_p) if a.size else None, a.size))


def _align(v, a):
    return (v + a - 1) // a * a


class Part:
    """A run of rows that came from one checkpoint tensor (formats/strixw.hpp:29-32)."""

    def __init__(self, source, row_offset, rows):
        self.source, self.row_offset, self.rows = source, int(row_offset), int(rows)


class Component:
    def __init__(self, role, offset=0, nbytes=0, hash_=0):
        self.role, self.offset, self.bytes, self.hash = int(role), int(offset), int(nbytes), int(hash_)


class Tensor:
    """One index record (formats/strixw.hpp:39-48)."""

    def __init__(self, name, encoding, shape, group_size=0, experts=0, parts=()):
        self.name, self.encoding, self.shape = name, int(encoding), [int(d) for d in shape]
        self.group_size, self.experts, self.parts, self.components = int(group_size), int(experts), list(parts), []

    def numel(self):
        n = 1
        for d in self.shape:
            n *= d
        return n

    def component(self, role):
        for c in self.components:
            if c.role == role:
                return c
        raise StrixError("strixw tensor '%s' (%s) has no %s component" % (self.name, ENCODING_NAMES.get(self.encoding, "?"), ROLE_NAMES.get(role, role)))


def components_of(t):
    """The components an encoding has with their exact byte sizes (strixw_components, formats/strixw.cpp:132-195)."""
    enc = t.encoding
    if enc in (Q4_ROW, Q4_CHUNK, Q8_ROW, Q8_CHUNK, Q6_ROW, Q5_ROW):
        if len(t.shape) != 2:
            raise StrixError("strixw tensor '%s': %s needs shape [N, K], got %s" % (t.name, ENCODING_NAMES[enc], t.shape))
        N, K, G = t.shape[0], t.shape[1], t.group_size
        need = {Q6_ROW: 64, Q5_ROW: 128}.get(enc, 1)
        if G not in (32, 64, 128) or K % G != 0 or K % need != 0:
            raise StrixError("strixw tensor '%s': %s with K = %d, group size %d (must be 32/64/128 and divide K%s)"
                             % (t.name, ENCODING_NAMES[enc], K, G, "; K a multiple of %d" % need if need > 1 else ""))
        row = {Q4_ROW: K // 2, Q4_CHUNK: K // 2, Q8_ROW: K, Q8_CHUNK: K, Q6_ROW: K // 2 + K // 4, Q5_ROW: K // 2 + K // 8}[enc]
        return [Component(Q, 0, N * row), Component(SCALE, 0, N * (K // G) * 2), Component(MIN, 0, N * (K // G) * 2)]
    if enc in (BF16, F32, I64):
        if t.group_size != 0:
            raise StrixError("strixw tensor '%s': %s has group size %d, expected 0" % (t.name, ENCODING_NAMES[enc], t.group_size))
        return [Component(DATA, 0, t.numel() * {BF16: 2, F32: 4, I64: 8}[enc])]
    raise StrixError("strixw tensor '%s': unknown encoding %d" % (t.name, enc))


def _validate_record(t, where):
    """What writer and reader both require of a record (validate_record, formats/strixw.cpp:75-95)."""
    if not t.name:
        raise StrixError("%s: tensor with an empty name" % where)
    if not 1 <= len(t.shape) <= 8:
        raise StrixError("%s: tensor '%s' has %d dims, expected 1..8" % (where, t.name, len(t.shape)))
    if any(d < 1 for d in t.shape):
        raise StrixError("%s: tensor '%s' has shape %s" % (where, t.name, t.shape))
    if t.experts < 0 or (t.experts and t.shape[0] % t.experts):
        raise StrixError("%s: tensor '%s': %d rows don't split into %d experts" % (where, t.name, t.shape[0], t.experts))
    nxt = 0
    for p in t.parts:
        if not p.source or p.rows < 1 or p.row_offset != nxt:
            raise StrixError("%s: tensor '%s' part '%s' at row %d (%d rows), expected to start at row %d" % (where, t.name, p.source, p.row_offset, p.rows, nxt))
        nxt += p.rows
    if t.parts and nxt != t.shape[0]:
        raise StrixError("%s: tensor '%s' parts cover %d rows of %d" % (where, t.name, nxt, t.shape[0]))


def _str16(s, what):
    b = s.encode("utf-8")
    if len(b) > 0xFFFF:
        raise StrixError("strixw: %s '%s...' is %d bytes, limit 65535" % (what, s[:64], len(b)))
    return struct.pack("<H", len(b)) + b


def _encode_index(meta, tensors):
    out = [struct.pack("<I", len(meta))]
    for k in sorted(meta):  # the reference iterates a std::map: keys in byte order
        v = meta[k].encode("utf-8") if isinstance(meta[k], str) else bytes(meta[k])
        out += [_str16(k, "metadata key"), struct.pack("<I", len(v)), v]
    out.append(struct.pack("<I", len(tensors)))
    for t in tensors:
        out += [_str16(t.name, "tensor name"), struct.pack("<BB", t.encoding, len(t.shape)), struct.pack("<%dq" % len(t.shape), *t.shape),
                struct.pack("<qqH", t.group_size, t.experts, len(t.parts))]
        for p in t.parts:
            out += [_str16(p.source, "part source name"), struct.pack("<qq", p.row_offset, p.rows)]
        out.append(struct.pack("<B", len(t.components)))
        for c in t.components:
            out.append(struct.pack("<BQQQ", c.role, c.offset, c.bytes, c.hash))
    return b"".join(out)


def write(path, meta, tensors, data):
    """Writes a strixw file (StrixwWriter, formats/strixw.cpp:225-372). tensors: Tensor records (name, encoding, shape,
    group size, experts, parts); data: {(tensor name, role): bytes-like of exactly the planned size}."""
    where = "strixw.write('%s')" % path
    if not tensors:
        raise StrixError("%s: no tensors" % where)
    seen = set()
    for t in tensors:
        _validate_record(t, where)
        if t.name in seen:
            raise StrixError("%s: tensor '%s' planned twice" % (where, t.name))
        seen.add(t.name)
        t.components = components_of(t)
    index_bytes = len(_encode_index(meta, tensors))  # hashes are fixed-width: the size is final
    data_offset = _align(HEADER_BYTES + index_bytes, TENSOR_ALIGN)
    cur = data_offset
    for t in tensors:
        cur = _align(cur, TENSOR_ALIGN)
        for c in t.components:
            cur = _align(cur, COMPONENT_ALIGN)
            c.offset = cur
            cur += c.bytes
    file_bytes = cur
    with open(path, "wb") as f:
        f.truncate(file_bytes)
        for t in tensors:
            for c in t.components:
                key = (t.name, c.role)
                if key not in data:
                    raise StrixError("%s: tensor '%s' %s was never written" % (where, t.name, ROLE_NAMES[c.role]))
                b = np.ascontiguousarray(data[key]).view(np.uint8).reshape(-1) if isinstance(data[key], np.ndarray) else np.frombuffer(data[key], dtype=np.uint8)
                if b.size != c.bytes:
                    raise StrixError("%s: '%s' %s is %d bytes, planned %d (%s %s)" % (where, t.name, ROLE_NAMES[c.role], b.size, c.bytes, ENCODING_NAMES[t.encoding], t.shape))
                f.seek(c.offset)
                f.write(b.tobytes())
                c.hash = hash64(b)
        index = _encode_index(meta, tensors)
        h = bytearray(HEADER_BYTES)
        h[0:8] = MAGIC
        struct.pack_into("<IIQQQQQ", h, 8, VERSION, HEADER_BYTES, HEADER_BYTES, len(index), data_offset, file_bytes, hash64(index))
        struct.pack_into("<Q", h, 120, hash64(bytes(h[:120])))
        f.seek(0)
        f.write(bytes(h))
        f.write(index)
    return file_bytes


class StrixwFile:
    """Maps and validates a strixw file: header, index, every record (StrixwFile, formats/strixw.cpp:376-489)."""

    def __init__(self, path):
        self.path = path
        where = "strixw '%s'" % path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise StrixError("%s: open failed: %s" % (where, e.strerror)) from None
        if size < HEADER_BYTES:
            self._f.close()
            raise StrixError("%s: %d bytes, smaller than the %d-byte header" % (where, size, HEADER_BYTES))
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._np = np.frombuffer(self._map, dtype=np.uint8)
        b = self._map
        try:
            if b[0:8] != MAGIC:
                raise StrixError("%s: not a strixw file (bad magic)" % where)
            version, hsize, index_off, index_bytes, self.data_offset, file_bytes, index_hash = struct.unpack_from("<IIQQQQQ", b, 8)
            if not OLDEST_VERSION <= version <= VERSION:
                raise StrixError("%s: format version %d, this build reads %d..%d (re-run the converter)" % (where, version, OLDEST_VERSION, VERSION))
            if hsize != HEADER_BYTES:
                raise StrixError("%s: header size %d, expected %d" % (where, hsize, HEADER_BYTES))
            if struct.unpack_from("<Q", b, 120)[0] != hash64(b[0:120]):
                raise StrixError("%s: header hash mismatch (corrupt header)" % where)
            if file_bytes != size:
                raise StrixError("%s: header says %d bytes, the file has %d (truncated or appended to)" % (where, file_bytes, size))
            if index_off != HEADER_BYTES or index_bytes > size - index_off:
                raise StrixError("%s: index at %d (%d bytes) doesn't fit the %d-byte file" % (where, index_off, index_bytes, size))
            if self.data_offset % TENSOR_ALIGN or self.data_offset < index_off + index_bytes or self.data_offset > size:
                raise StrixError("%s: data offset %d (index ends at %d, alignment %d)" % (where, self.data_offset, index_off + index_bytes, TENSOR_ALIGN))
            if index_hash != hash64(b[index_off:index_off + index_bytes]):
                raise StrixError("%s: index hash mismatch (corrupt index)" % where)
            self.version, self.file_bytes = version, size
            self.meta, self.tensors, self._by_name = {}, [], {}
            self._parse_index(b, index_off, index_bytes, where)
        except Exception:
            self.close()
            raise

    def _parse_index(self, b, off, n, where):
        end = off + n
        at = [off]

        def get(fmt, what):
            sz = struct.calcsize(fmt)
            if end - at[0] < sz:
                raise StrixError("%s: index ends inside %s (at index byte %d of %d)" % (where, what, at[0] - off, n))
            v = struct.unpack_from(fmt, b, at[0])
            at[0] += sz
            return v[0] if len(v) == 1 else v

        def text(length, what):
            if end - at[0] < length:
                raise StrixError("%s: index ends inside %s (%d bytes at index byte %d of %d)" % (where, what, length, at[0] - off, n))
            s = bytes(b[at[0]:at[0] + length])
            at[0] += length
            return s

        for _ in range(get("<I", "metadata count")):
            k = text(get("<H", "metadata key length"), "metadata key").decode("utf-8", "replace")
            v = text(get("<I", "metadata value length"), "metadata value").decode("utf-8", "replace")
            if k in self.meta:
                raise StrixError("%s: metadata key '%s' twice" % (where, k))
            self.meta[k] = v
        nt = get("<I", "tensor count")
        if nt < 1:
            raise StrixError("%s: no tensors" % where)
        spans = []
        for _ in range(nt):
            name = text(get("<H", "tensor name length"), "tensor name").decode("utf-8", "replace")
            enc, ndim = get("<B", "encoding"), get("<B", "ndim")
            shape = [get("<q", "shape") for _ in range(ndim)]
            t = Tensor(name, enc, shape, get("<q", "group size"), get("<q", "experts"))
            for _ in range(get("<H", "part count")):
                src = text(get("<H", "part name length"), "part name").decode("utf-8", "replace")
                t.parts.append(Part(src, get("<q", "part row offset"), get("<q", "part rows")))
            for _ in range(get("<B", "component count")):
                t.components.append(Component(get("<B", "component role"), get("<Q", "component offset"), get("<Q", "component bytes"), get("<Q", "component hash")))
            _validate_record(t, where)
            want = components_of(t)
            if len(want) != len(t.components):
                raise StrixError("%s: tensor '%s' (%s) has %d components, expected %d" % (where, t.name, ENCODING_NAMES.get(enc, "?"), len(t.components), len(want)))
            for k, (g, w) in enumerate(zip(t.components, want)):
                if g.role != w.role or g.bytes != w.bytes:
                    raise StrixError("%s: tensor '%s' component %d is %s of %d bytes, expected %s of %d for %s %s"
                                     % (where, t.name, k, ROLE_NAMES.get(g.role, g.role), g.bytes, ROLE_NAMES[w.role], w.bytes, ENCODING_NAMES[enc], t.shape))
                if g.offset < self.data_offset or g.offset % COMPONENT_ALIGN or g.bytes > self.file_bytes - g.offset:
                    raise StrixError("%s: tensor '%s' %s at %d (%d bytes) is outside the data region [%d, %d) or not %d-aligned"
                                     % (where, t.name, ROLE_NAMES[g.role], g.offset, g.bytes, self.data_offset, self.file_bytes, COMPONENT_ALIGN))
                spans.append((g.offset, g.offset + g.bytes))
            if t.name in self._by_name:
                raise StrixError("%s: tensor '%s' twice" % (where, t.name))
            self._by_name[t.name] = len(self.tensors)
            self.tensors.append(t)
        if at[0] != end:
            raise StrixError("%s: %d unread bytes after the last index record" % (where, end - at[0]))
        spans.sort()
        for (a0, a1), (b0, _) in zip(spans, spans[1:]):
            if b0 < a1:
                raise StrixError("%s: components overlap at byte %d" % (where, b0))

    def close(self):
        self._np = None
        try:
            if getattr(self, "_map", None) is not None:
                self._map.close()
        except BufferError:
            pass  # views handed out by data() are still alive; the map goes with them
        self._map = None
        if getattr(self, "_f", None) is not None:
            self._f.close()
            self._f = None

    def find(self, name):
        i = self._by_name.get(name)
        return None if i is None else self.tensors[i]

    def get(self, name):
        t = self.find(name)
        if t is None:
            raise StrixError("strixw '%s': no tensor '%s'" % (self.path, name))
        return t

    def data(self, t, role):
        """The component's bytes as a read-only uint8 view of the mapping."""
        c = t.component(role)
        return self._np[c.offset:c.offset + c.bytes]

    def verify_hashes(self):
        """Recomputes every component hash; raises naming the first mismatch."""
        for t in self.tensors:
            for c in t.components:
                if hash64(self._np[c.offset:c.offset + c.bytes]) != c.hash:
                    raise StrixError("strixw '%s': tensor '%s' %s hash mismatch (corrupt data)" % (self.path, t.name, ROLE_NAMES[c.role]))

    # ---- loaders: tensors of the file as the device weights the MoE layer takes --------------------------------------

    def qweight(self, name, device="cuda"):
        """A row-major quantized tensor (q4/q5/q6/q8) as kernels.QWeight on the device; an expert stack keeps its stacked
        [experts x rows, K] form, which is what the expert kernels take (runtime/strixw_loader.hpp:24-48)."""
        from . import kernels as K

        t = self.get(name)
        bits = _ROW_MAJOR_BITS.get(t.encoding)
        if bits is None:
            raise StrixError("strixw '%s': tensor '%s' is %s, not a row-major quantized tensor" % (self.path, name, ENCODING_NAMES.get(t.encoding, "?")))
        N, Kdim = t.shape
        return K.QWeight.upload(bits, N, Kdim, t.group_size, np.array(self.data(t, Q)), np.array(self.data(t, SCALE)).view(np.uint16),
                                np.array(self.data(t, MIN)).view(np.uint16), device)

    def dense(self, name, device="cuda"):
        """A BF16 / F32 / I64 tensor as a torch tensor of its shape on the device."""
        import torch

        t = self.get(name)
        raw = np.array(self.data(t, DATA))
        if t.encoding == BF16:
            return torch.from_numpy(raw.view(np.int16).reshape(t.shape)).to(device).view(torch.bfloat16)
        if t.encoding == F32:
            return torch.from_numpy(raw.view(np.float32).reshape(t.shape)).to(device)
        if t.encoding == I64:
            return torch.from_numpy(raw.view(np.int64).reshape(t.shape)).to(device)
        raise StrixError("strixw '%s': tensor '%s' is %s, not a dense tensor" % (self.path, name, ENCODING_NAMES.get(t.encoding, "?")))
