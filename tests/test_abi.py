"""CPU-side checks of the C-ABI boundary: the library loads, exports every
symbol include/tlcuda.h declares, refuses to run without a CUDA device, and its
host-side generator matches the numpy restatement."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tlcuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"TLC_API\s+[\w\s\*]+?\b(tlc_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from tensorlogic_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in tlcuda.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert set(_lib.PROTOTYPES) <= set(names), set(_lib.PROTOTYPES) - set(names)


def test_no_oracle_in_product():
    """The shipped package must not reach into oracle/ (it is test infrastructure)."""
    pkg = os.path.join(ROOT, "tensorlogic_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "tl_ref" not in src and "libtlref" not in src, f


def test_init_fails_loudly_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    h = C.c_void_p()
    rc = lib.tlc_init(0, C.byref(h))
    from tensorlogic_b200 import _lib
    assert rc == _lib.ERR_DEVICE and not h.value
    assert b"no CPU path" in lib.tlc_last_error()
    from tensorlogic_b200.api import Device, TensorError
    with pytest.raises(TensorError):
        Device(0)


def test_version_string(lib):
    assert b"sm_100a" in lib.tlc_version()


@pytest.mark.parametrize("qtype,bb", [(2, 18), (8, 34)])
def test_host_generator_matches_numpy(lib, qtype, bb):
    from tensorlogic_b200 import synth
    seed, tid = 7, synth.tensor_id("blk.3.ffn_gate.weight")
    n_rows, n_cols = 6, 256
    want = synth.blocks(qtype, seed, tid, n_rows, n_cols)
    got = np.empty((n_rows * (n_cols // 32), bb), np.uint8)
    assert lib.tlc_synth_blocks_host(qtype, seed, tid, 0, 0, got.shape[0], got.ctypes.data) == 0
    assert np.array_equal(got.reshape(want.shape), want)
    # a shard generated on its own equals the slice of the whole
    part = synth.blocks(qtype, seed, tid, n_rows, n_cols, row0=2, rows=3)
    assert np.array_equal(part, want[2:5])
    got2 = np.empty((3 * 8, bb), np.uint8)
    assert lib.tlc_synth_blocks_host(qtype, seed, tid, 0, 2 * 8, 24, got2.ctypes.data) == 0
    assert np.array_equal(got2.reshape(part.shape), part)
    # scaled variant: d * 2^-2, same quantized values
    sc = synth.blocks(qtype, seed, tid, n_rows, n_cols, scale_log2=-2)
    got3 = np.empty_like(got)
    assert lib.tlc_synth_blocks_host(qtype, seed, tid, -2, 0, got3.shape[0], got3.ctypes.data) == 0
    assert np.array_equal(got3.reshape(sc.shape), sc)
    assert np.array_equal(sc[..., 2:], want[..., 2:])
    d0 = want[..., :2].copy().view(np.float16).astype(np.float32)
    d2 = sc[..., :2].copy().view(np.float16).astype(np.float32)
    assert np.allclose(d2, d0 / 4, rtol=1e-3)


def test_synthetic_distributions():
    from tensorlogic_b200 import synth
    b = synth.q4_0_blocks(0, 1, 64, 2048)
    d = b[..., :2].copy().view(np.float16).astype(np.float32)
    assert 0.0019 < d.min() and d.max() < 0.0201 and abs(d.mean() - 0.011) < 3e-4
    nib = np.concatenate([(b[..., 2:] & 15).ravel(), (b[..., 2:] >> 4).ravel()])
    assert abs(nib.mean() - 7.5) < 0.02 and set(np.unique(nib)) == set(range(16))
    q = synth.q8_0_blocks(0, 2, 64, 2048)[..., 2:].view(np.int8)
    assert q.min() == -127 and q.max() == 127 and abs(q.astype(np.float64).mean()) < 0.6
    x = synth.activations(0, "x", (1, 65536)).astype(np.float64)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1.0) < 0.02
    ids = synth.token_ids(0, "ids", 4096, 32000)
    assert ids.min() >= 0 and ids.max() < 32000 and len(np.unique(ids)) > 3800


def _tile_numpy(qtype, n_rows, n_cols, raw):
    """The tiled weight layout restated with numpy index arithmetic (the header's description)."""
    bb, tb, tile = (18, 4, 1152) if qtype == 2 else (34, 2, 1088)
    bpr = n_cols // 32
    ktiles = -(-bpr // tb)
    slabs = -(-n_rows // 16)
    out = np.zeros(slabs * ktiles * tile, np.uint8)
    blocks = np.asarray(raw, np.uint8).reshape(n_rows, bpr, bb)
    for r in range(n_rows):
        for b in range(bpr):
            base = ((r // 16) * ktiles + b // tb) * tile
            rr, j = r % 16, b % tb
            group = base + (rr // 8) * 512 + (rr % 8) * 64
            qs = blocks[r, b, 2:]
            for w in range((bb - 2) // 4):
                if qtype == 2:
                    off = group + w * 16 + j * 4
                else:
                    off = group + (w // 2) * 16 + (j * 2 + (w & 1)) * 4
                out[off:off + 4] = qs[4 * w:4 * w + 4]
            so = base + 1024 + (rr * tb + j) * 2
            out[so:so + 2] = blocks[r, b, :2]
    return out


@pytest.mark.parametrize("qtype,bb", [(2, 18), (8, 34)])
@pytest.mark.parametrize("n_rows,n_cols", [(16, 128), (1, 32), (17, 96), (40, 416)])
def test_tiled_layout_host(lib, qtype, bb, n_rows, n_cols):
    """The host restatement of the device layout: sizes, positions of every byte, zero padding."""
    rng = np.random.default_rng(n_rows * 1000 + n_cols + qtype)
    raw = rng.integers(0, 256, n_rows * (n_cols // 32) * bb, dtype=np.uint8)
    want = _tile_numpy(qtype, n_rows, n_cols, raw)
    assert lib.tlc_tiled_bytes(qtype, n_rows, n_cols) == want.size
    got = np.full(want.size, 0xAA, np.uint8)
    assert lib.tlc_tile_blocks_host(qtype, n_rows, n_cols, raw.ctypes.data, got.ctypes.data) == 0
    assert np.array_equal(got, want)
    # every input byte appears exactly once: the regrouping is a permutation plus zero padding
    assert np.array_equal(np.sort(got[got != 0]), np.sort(raw[raw != 0]))
    assert lib.tlc_tiled_bytes(1, n_rows, n_cols) == 0            # f16 tensors are not tiled
    assert lib.tlc_tile_blocks_host(1, n_rows, n_cols, raw.ctypes.data, got.ctypes.data) != 0


def test_integration_doc_binds_every_symbol():
    """The Rust extern block a TensorLogic maintainer would add lists every entry point of the header."""
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    missing = [s for s in _declared_symbols() if f"fn {s}(" not in doc]
    assert not missing, missing


def test_rust_shim_matches_header():
    """rust/src/device/cuda_ffi.rs is generated from the header and must not be stale; the hand-
    written Rust files may only call entry points the header declares (they cannot be compiled
    here, so this is what keeps them honest)."""
    import re
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "rust", "gen_ffi.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    header = open(os.path.join(ROOT, "include", "tlcuda.h")).read()
    declared = set(re.findall(r"\b(tlc_\w+)\s*\(", header))
    ffi = open(os.path.join(ROOT, "rust", "src", "device", "cuda_ffi.rs")).read()
    assert set(re.findall(r"pub fn (tlc_\w+)\(", ffi)) == {n for n in declared if re.search(r"TLC_API[^;]*\b%s\s*\(" % n, header)}
    for dirpath, _, files in os.walk(os.path.join(ROOT, "rust", "src")):
        for f in files:
            if f.endswith(".rs") and f != "cuda_ffi.rs":
                text = open(os.path.join(dirpath, f)).read()
                for name in set(re.findall(r"ffi::(tlc_\w+)\s*\(", text)):
                    assert name in declared, (f, name)
                for const in set(re.findall(r"ffi::(TLC_\w+)", text)):
                    assert re.search(r"pub const %s:" % const, ffi), (f, const)


def test_every_option_is_documented_in_the_header():
    """tlc_set_option's names (the parser in tlc_context.cu) and the list in the header's comment
    are the same set."""
    import re
    src = open(os.path.join(ROOT, "tensorlogic_b200", "csrc", "tlc_context.cu")).read()
    body = src[src.index("tlc_set_option("):]
    body = body[:body.index("unknown option")]
    parsed = set(re.findall(r'n == "(\w+)"', body))
    header = open(os.path.join(ROOT, "include", "tlcuda.h")).read()
    comment = header[header.index("Runtime switches the reference reads"):header.index("tlc_set_option(")]
    documented = set(re.findall(r'^ \*   "(\w+)"', comment, flags=re.M))
    assert parsed and parsed == documented, (sorted(parsed - documented), sorted(documented - parsed))
