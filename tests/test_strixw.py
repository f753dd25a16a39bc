"""CPU: the strixw weights-file reader and writer (strixite_b200/strixw.py, strix_hash64 of the C library) against the
reference: a file written by the reference's own StrixwWriter (tests/golden/demo.strixw) must read back record by record,
the writer here must reproduce that file byte for byte, and - where the reference is compiled (oracle/_ref) - the
reference's reader must accept what the writer here produces."""
import ctypes as C
import json
import os
import shutil

import numpy as np
import pytest

from strixite_b200 import StrixError
from strixite_b200 import strixw as SW

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEMO = os.path.join(GOLDEN, "demo.strixw")
SEED = 7
REF_SO = os.path.join(os.path.dirname(GOLDEN), "..", "oracle", "_ref", "libstrix_formats_ref.so")


def fill(nbytes, seed, ti, role):
    """The filler of oracle/ref_strixw_shim.cpp: byte i of component (tensor ti, role) of the demonstration file."""
    m = (1 << 64) - 1
    s = (seed * 0x9E3779B97F4A7C15 + ti * 0x100000001B3 + role * 0xD6E8FEB86659FD93 + 1) & m
    out = bytearray(nbytes)
    for i in range(nbytes):
        s ^= (s << 13) & m
        s ^= s >> 7
        s ^= (s << 17) & m
        out[i] = (s >> 32) & 0xFF
    return bytes(out)


def demo_plan():
    ts = [SW.Tensor("layers.0.moe.router", SW.BF16, [5, 128]),
          SW.Tensor("layers.0.moe.experts.gate_up", SW.Q4_ROW, [3 * 64, 128], 32, 3,
                    [SW.Part("model.layers.0.mlp.experts.gate_up_proj", 0, 128), SW.Part("model.layers.0.mlp.shared_expert.gate_up", 128, 64)]),
          SW.Tensor("layers.0.moe.experts.down", SW.Q5_ROW, [3 * 128, 128], 128, 3),
          SW.Tensor("layers.0.moe.shared.down", SW.Q8_ROW, [128, 64], 64),
          SW.Tensor("layers.0.moe.shared.gate_up", SW.Q6_ROW, [64, 128], 64),
          SW.Tensor("norm.weight", SW.F32, [128]),
          SW.Tensor("positions", SW.I64, [2, 3])]
    meta = {"model": "demo", "converter": "reference StrixwWriter", "empty": ""}
    return meta, ts


def demo_data(ts):
    data = {}
    for ti, t in enumerate(ts):
        for c in SW.components_of(t):
            data[(t.name, c.role)] = fill(c.bytes, SEED, ti, c.role)
    return data


def test_hash_matches_the_reference_values():
    cases = json.load(open(os.path.join(GOLDEN, "strixw_hashes.json")))["cases"]
    rng = np.random.default_rng(2026)
    for n, rec in cases.items():
        b = rng.integers(0, 256, int(n), dtype=np.uint8)
        assert b[:4].tolist() == rec["first"]
        assert "%016x" % SW.hash64(b) == rec["hash"], "length %s" % n


def test_reads_the_file_the_reference_wrote():
    f = SW.StrixwFile(DEMO)
    meta, ts = demo_plan()
    assert f.meta == meta and f.version == 4 and f.file_bytes == os.path.getsize(DEMO)
    assert [t.name for t in f.tensors] == [t.name for t in ts]
    for ti, (got, want) in enumerate(zip(f.tensors, ts)):
        assert (got.encoding, got.shape, got.group_size, got.experts) == (want.encoding, want.shape, want.group_size, want.experts)
        assert [(p.source, p.row_offset, p.rows) for p in got.parts] == [(p.source, p.row_offset, p.rows) for p in want.parts]
        comps = SW.components_of(want)
        assert [(c.role, c.bytes) for c in got.components] == [(c.role, c.bytes) for c in comps]
        assert got.components[0].offset % SW.TENSOR_ALIGN == 0
        for c in got.components:
            assert c.offset % SW.COMPONENT_ALIGN == 0 and c.offset >= f.data_offset
            assert bytes(f.data(got, c.role)) == fill(c.bytes, SEED, ti, c.role)
    f.verify_hashes()
    assert f.find("nope") is None
    with pytest.raises(StrixError, match="no tensor 'nope'"):
        f.get("nope")
    with pytest.raises(StrixError, match="has no scale component"):
        f.data(f.get("norm.weight"), SW.SCALE)
    f.close()


def test_writer_reproduces_the_reference_file_byte_for_byte(tmp_path):
    meta, ts = demo_plan()
    out = str(tmp_path / "ours.strixw")
    n = SW.write(out, meta, ts, demo_data(ts))
    assert n == os.path.getsize(DEMO)
    assert open(out, "rb").read() == open(DEMO, "rb").read()


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="the reference is not compiled here (oracle/_ref)")
def test_reference_reader_accepts_our_file(tmp_path):
    ref = C.CDLL(REF_SO)
    ref.ref_strixw_last_error.restype = C.c_char_p
    rng = np.random.default_rng(5)
    ts = [SW.Tensor("a.q8", SW.Q8_ROW, [6, 256], 32, 2, [SW.Part("src.a", 0, 6)]), SW.Tensor("b.bf16", SW.BF16, [3, 5, 7]),
          SW.Tensor("c.q4", SW.Q4_ROW, [9, 128], 128)]
    data = {(t.name, c.role): rng.integers(0, 256, c.bytes, dtype=np.uint8) for t in ts for c in SW.components_of(t)}
    out = str(tmp_path / "ours.strixw")
    SW.write(out, {"k": "v", "a": "b"}, ts, data)
    nt, nb = C.c_int64(), C.c_uint64()
    assert ref.ref_strixw_check(out.encode(), C.byref(nt), C.byref(nb)) == 0, ref.ref_strixw_last_error().decode()
    assert nt.value == 3 and nb.value == os.path.getsize(out)
    # and a corrupted component is caught by the reference's hash pass as by ours
    raw = bytearray(open(out, "rb").read())
    raw[SW.StrixwFile(out).get("c.q4").component(SW.Q).offset + 3] ^= 0x10
    bad = str(tmp_path / "bad.strixw")
    open(bad, "wb").write(raw)
    assert ref.ref_strixw_check(bad.encode(), C.byref(nt), C.byref(nb)) != 0
    with pytest.raises(StrixError, match="hash mismatch"):
        SW.StrixwFile(bad).verify_hashes()


def _corrupt(tmp_path, name, edit):
    raw = bytearray(open(DEMO, "rb").read())
    raw = edit(raw) or raw
    p = str(tmp_path / name)
    open(p, "wb").write(raw)
    return p


def test_rejects_corrupt_files(tmp_path):
    def flip(at):
        def e(raw):
            raw[at] ^= 1
        return e

    with pytest.raises(StrixError, match="bad magic"):
        SW.StrixwFile(_corrupt(tmp_path, "magic", flip(0)))
    with pytest.raises(StrixError, match="header hash mismatch"):
        SW.StrixwFile(_corrupt(tmp_path, "header", flip(33)))
    with pytest.raises(StrixError, match="index hash mismatch"):
        SW.StrixwFile(_corrupt(tmp_path, "index", flip(SW.HEADER_BYTES + 10)))
    with pytest.raises(StrixError, match="smaller than the 128-byte header"):
        SW.StrixwFile(_corrupt(tmp_path, "tiny", lambda raw: raw[:100]))
    with pytest.raises(StrixError, match="truncated or appended"):
        SW.StrixwFile(_corrupt(tmp_path, "short", lambda raw: raw[:-256]))
    with pytest.raises(StrixError, match="open failed"):
        SW.StrixwFile(str(tmp_path / "absent.strixw"))
    f = SW.StrixwFile(_corrupt(tmp_path, "data", flip(SW.StrixwFile(DEMO).tensors[2].components[0].offset)))
    with pytest.raises(StrixError, match="layers.0.moe.experts.down' q hash mismatch"):
        f.verify_hashes()


def test_writer_checks_its_plan(tmp_path):
    out = str(tmp_path / "x.strixw")
    with pytest.raises(StrixError, match="no tensors"):
        SW.write(out, {}, [], {})
    with pytest.raises(StrixError, match="group size 48"):
        SW.write(out, {}, [SW.Tensor("t", SW.Q4_ROW, [4, 96], 48)], {})
    with pytest.raises(StrixError, match="K a multiple of 128"):
        SW.write(out, {}, [SW.Tensor("t", SW.Q5_ROW, [4, 64], 32)], {})
    with pytest.raises(StrixError, match="don't split into 3 experts"):
        SW.write(out, {}, [SW.Tensor("t", SW.Q4_ROW, [4, 128], 32, 3)], {})
    with pytest.raises(StrixError, match="parts cover 2 rows of 4"):
        SW.write(out, {}, [SW.Tensor("t", SW.F32, [4, 2], 0, 0, [SW.Part("s", 0, 2)])], {})
    with pytest.raises(StrixError, match="planned twice"):
        SW.write(out, {}, [SW.Tensor("t", SW.F32, [2]), SW.Tensor("t", SW.F32, [2])], {})
    with pytest.raises(StrixError, match="never written"):
        SW.write(out, {}, [SW.Tensor("t", SW.F32, [2])], {})
    with pytest.raises(StrixError, match="is 4 bytes, planned 8"):
        SW.write(out, {}, [SW.Tensor("t", SW.F32, [2])], {("t", SW.DATA): b"abcd"})
