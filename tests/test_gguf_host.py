"""CPU tests of the GGUF header parser (host logic of the loader; no device involved)."""
import ctypes as C

import numpy as np
import pytest

from gguf_util import write_gguf


def _open(lib, path):
    h = C.c_void_p()
    rc = lib.tlc_gguf_open(str(path).encode(), C.byref(h))
    return rc, h


def _tensors(lib, h):
    out = {}
    for i in range(lib.tlc_gguf_tensor_count(h)):
        name, t, r, c, off, nb = C.c_char_p(), C.c_int32(), C.c_int64(), C.c_int64(), C.c_uint64(), C.c_uint64()
        assert lib.tlc_gguf_tensor_info(h, i, C.byref(name), C.byref(t), C.byref(r), C.byref(c), C.byref(off),
                                        C.byref(nb)) == 0
        out[name.value.decode()] = (t.value, r.value, c.value, off.value, nb.value)
    return out


@pytest.mark.parametrize("alignment", [32, 128])
def test_parse_matches_gguf_package(lib, tmp_path, alignment):
    import gguf
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import LlamaArch, synthetic_host_weights
    arch = LlamaArch(n_layers=1, d_model=128, n_heads=2, n_kv_heads=1, head_dim=64, ffn_dim=256, vocab=96)
    weights = synthetic_host_weights(arch, seed=1)
    weights["blk.0.ffn_up.weight"] = (8, synth.blocks(8, 1, 5, 256, 128))
    weights["blk.0.ffn_norm.weight"] = (0, weights["blk.0.ffn_norm.weight"][1].astype(np.float32))
    path = tmp_path / "t.gguf"
    write_gguf(path, weights, arch, alignment=alignment)
    rc, h = _open(lib, path)
    assert rc == 0, lib.tlc_last_error()
    got = _tensors(lib, h)
    rd = gguf.GGUFReader(str(path))
    assert lib.tlc_gguf_data_start(h) == rd.data_offset and rd.data_offset % alignment == 0
    assert set(got) == {t.name for t in rd.tensors} == set(weights)
    raw = open(path, "rb").read()
    for t in rd.tensors:
        gtype, rows, cols, off, nb = got[t.name]
        assert gtype == int(t.tensor_type)
        assert off == t.data_offset and nb == t.n_bytes
        dims = [int(x) for x in t.shape]             # file order, fastest first
        assert cols == dims[0] and rows == int(np.prod(dims[1:])) if len(dims) > 1 else rows == 1
        src_type, arr = weights[t.name]
        assert raw[off:off + nb] == np.ascontiguousarray(arr).tobytes()   # the bytes we wrote, at that offset
    # metadata: 1- and 2-byte values and arrays must not derail the walk
    v = C.c_double()
    for key, want in [("test.u8", 7), ("test.flag", 1), ("test.u16", 513), ("test.i8", -3), ("test.u64", float(1 << 40)),
                      ("test.f64", 2.5), ("test.tokens.length", 3), ("llama.block_count", 1),
                      ("llama.attention.head_count_kv", 1)]:
        assert lib.tlc_gguf_meta_num(h, key.encode(), C.byref(v)) == 0, key
        assert v.value == want, key
    assert lib.tlc_gguf_meta_str(h, b"test.note") == b"synthetic"
    assert lib.tlc_gguf_meta_str(h, b"general.architecture") == b"llama"
    assert lib.tlc_gguf_meta_num(h, b"nope", C.byref(v)) != 0
    lib.tlc_gguf_close(h)


def test_parse_errors(lib, tmp_path):
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.model import LlamaArch, synthetic_host_weights
    arch = LlamaArch(n_layers=1, d_model=128, n_heads=2, n_kv_heads=1, head_dim=64, ffn_dim=256, vocab=96)
    good = tmp_path / "g.gguf"
    write_gguf(good, synthetic_host_weights(arch, 1), arch)
    raw = open(good, "rb").read()
    cases = {
        "magic": (b"GGUX" + raw[4:], b"Invalid GGUF magic"),
        "version": (raw[:4] + (1).to_bytes(4, "little") + raw[8:], b"Unsupported GGUF version"),
        "truncated_header": (raw[:30], b"truncated"),
        "truncated_kv": (raw[:200], b"truncated"),
        "truncated_data": (raw[:-64], b"runs past the end"),
    }
    for name, (data, msg) in cases.items():
        p = tmp_path / f"{name}.gguf"
        open(p, "wb").write(data)
        rc, h = _open(lib, p)
        assert rc == _lib.ERR_LOAD and not h.value, name
        assert msg in lib.tlc_last_error(), (name, lib.tlc_last_error())
    rc, _ = _open(lib, tmp_path / "missing.gguf")
    assert rc == _lib.ERR_LOAD and b"Failed to open" in lib.tlc_last_error()


def test_unsupported_type_is_listed_not_fatal_at_parse(lib, tmp_path):
    """A Q6_K tensor (type 14) parses; it is only rejected when uploaded."""
    import gguf
    p = tmp_path / "k.gguf"
    w = gguf.GGUFWriter(str(p), "llama")
    w.add_tensor("output.weight", np.zeros((4, 210), np.uint8), raw_dtype=gguf.GGMLQuantizationType.Q6_K)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    rc, h = _open(lib, p)
    assert rc == 0
    t = _tensors(lib, h)["output.weight"]
    assert t[0] == 14 and (t[1], t[2]) == (4, 256)
    lib.tlc_gguf_close(h)


def _handmade_gguf(dims, ggml_type, offset=0, kv=b"", n_kv=0, payload=b"\0" * 64):
    """A minimal GGUF v3 file with one tensor whose header fields are taken as given."""
    import struct
    name = b"t"
    head = struct.pack("<IIQQ", 0x46554747, 3, 1, n_kv) + kv
    head += struct.pack("<Q", len(name)) + name + struct.pack("<I", len(dims))
    head += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ggml_type, offset)
    pad = (-len(head)) % 32
    return head + b"\0" * pad + payload


def test_header_sizes_that_wrap_are_rejected(lib, tmp_path):
    """Shapes, offsets and lengths whose products or sums wrap around 2^64 must not pass the end-of-file test."""
    import struct
    from tensorlogic_b200 import _lib
    big = 1 << 62
    arr_kv = struct.pack("<Q", 1) + b"a" + struct.pack("<IIQ", 9, 10, (1 << 61) + 1)  # array of u64, n*8 wraps to 8
    str_kv = struct.pack("<Q", 1) + b"s" + struct.pack("<IQ", 8, 1 << 63)              # string longer than the file
    cases = {
        "rows_x_cols": _handmade_gguf([1 << 33, 1 << 33], 1),             # 2^66 elements
        "elems_x_4": _handmade_gguf([big, 1], 0),                         # 2^62 * 4 wraps to 0
        "three_dims": _handmade_gguf([32, 1 << 32, 1 << 32], 2),          # rows wrap to 0
        "zero_dim": _handmade_gguf([0, 4], 1),
        "offset_wraps": _handmade_gguf([32], 1, offset=(1 << 64) - 32),   # data_start + offset wraps
        "offset_past_end": _handmade_gguf([32], 1, offset=1 << 40),
        "array_len": _handmade_gguf([32], 1, kv=arr_kv, n_kv=1),
        "string_len": _handmade_gguf([32], 1, kv=str_kv, n_kv=1),
    }
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        open(p, "wb").write(data)
        rc, h = _open(lib, p)
        assert rc == _lib.ERR_LOAD and not h.value, (name, lib.tlc_last_error())
    # the same file with an honest shape parses
    p = tmp_path / "ok.gguf"
    open(p, "wb").write(_handmade_gguf([32], 1))
    rc, h = _open(lib, p)
    assert rc == 0, lib.tlc_last_error()
    lib.tlc_gguf_close(h)
