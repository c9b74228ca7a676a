"""GPU parity tests of the quantized linear path, through the C ABI.

Dequantization must be bit-exact with the oracle; linear outputs must be
within rel-L2 1e-2 of the oracle's dequant + f32-accumulate linear (the
tolerance stated for this path).  In practice they are ~1e-4.
"""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-2        # stated tolerance
TIGHT = 2e-3      # what the kernels are expected to reach; a regression alarm

Q4, Q8 = 2, 8


def _weights(qtype, n, k, seed=0, name="w"):
    from tensorlogic_b200 import synth
    return synth.blocks(qtype, seed, synth.tensor_id(name), n, k)


def _x(m, k, seed=0, name="x"):
    from tensorlogic_b200 import synth
    return synth.activations(seed, name, (m, k))


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_dequant_bit_exact_config0(dev, ref, qtype):
    """Config 0: W [5632, 2048]; all 11,534,336 values bit-exact."""
    from tensorlogic_b200.api import QTensor
    n, k = 5632, 2048
    raw = _weights(qtype, n, k)
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    got = w.dequantize().numpy()
    want = ref.dequant(qtype, raw, n * k).reshape(n, k)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # stored bytes are the GGUF bytes, verbatim (K multiple of 256 -> no row padding)
    assert np.array_equal(w.raw_bytes().reshape(-1), raw.reshape(-1))


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_dequant_edge_scales_and_golden(dev, ref, golden, qtype):
    from tensorlogic_b200.api import QTensor
    raw = golden["q4_0_bytes" if qtype == Q4 else "q8_0_bytes"]  # zero / negative / subnormal / large scales
    w = QTensor.from_blocks(dev, qtype, 3, 256, raw)
    got = w.dequantize().numpy().reshape(-1)
    want = ref.dequant(qtype, raw, 768)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    with np.errstate(over="ignore"):
        gold = golden["q4_0_gguf_f32" if qtype == Q4 else "q8_0_gguf_f32"].astype(np.float16)
    assert np.array_equal(got.view(np.uint16), gold.view(np.uint16))


def test_reference_kats_on_device(dev):
    """The Rust loader's known-answer tests (src/model/formats/gguf.rs:622-718), on the GPU."""
    from tensorlogic_b200.api import QTensor
    b = np.zeros((8, 18), np.uint8)
    b[:, 0:2] = np.array([0.5], np.float16).view(np.uint8)
    b[:, 2:] = 0xFF
    out = QTensor.from_blocks(dev, Q4, 1, 256, b).dequantize().numpy()
    assert np.all(out == np.float16(3.5))
    q = np.zeros((8, 34), np.uint8)
    q[:, 0:2] = np.array([2.0], np.float16).view(np.uint8)
    q[:, 2:] = np.arange(32, dtype=np.uint8)
    out = QTensor.from_blocks(dev, Q8, 1, 256, q).dequantize().numpy().reshape(8, 32)
    assert out[0, 10] == 20.0 and out[7, 31] == 62.0


def test_config0_linear(dev, ref):
    """Config 0: y = x . W^T, W [5632, 2048] Q4_0, x [1, 2048]."""
    from tensorlogic_b200.api import QTensor, linear
    n, k = 5632, 2048
    raw = _weights(Q4, n, k)
    x = _x(1, k)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, n, k, raw)).numpy()
    want = ref.linear_q(Q4, raw, n, k, x)
    err = rel_l2(y, want)
    assert err < TOL and err < TIGHT, err
    # distance to the reference's literal CPU path (f16 running sum) is recorded, and is
    # dominated by that path's own rounding noise
    lit = ref.linear_literal(x, ref.dequant(Q4, raw, n * k).reshape(n, k)[:256])
    assert rel_l2(y[:, :256], lit) < 5e-2


# Config 1 shapes (K -> N); lm_head is cut to 4000 rows here, the full 32000 runs once below.
SHAPES = [(2048, 2048), (2048, 256), (2048, 5632), (5632, 2048), (2048, 4000)]


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_config1_sweep(dev, ref, qtype, k, n, m):
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=1, name=f"w{k}x{n}")
    x = _x(m, k, seed=1, name=f"x{m}x{k}")
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, qtype, n, k, raw)).numpy()
    want = ref.linear_q(qtype, raw, n, k, x)
    err = rel_l2(y, want)
    assert err < TOL and err < TIGHT, err
    # element-wise: the oracle rounds each dequantized weight to f16 first (as the
    # reference's loader does) while the kernel multiplies d*(q-8) exactly, so single
    # outputs differ by a random-walk of 2^-11 relative errors: small against the
    # output's rms, whatever the element's own magnitude
    yf, wf = y.astype(np.float32), want.astype(np.float32)
    assert np.max(np.abs(yf - wf)) < 2e-3 * max(float(np.max(np.abs(wf))), 1.0)  # ~2 f16 steps of the largest output


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_lm_head_full(dev, ref, qtype):
    from tensorlogic_b200.api import QTensor, linear
    n, k = 32000, 2048
    raw = _weights(qtype, n, k, seed=2)
    x = _x(1, k, seed=2)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, qtype, n, k, raw)).numpy()
    want = ref.linear_q(qtype, raw, n, k, x)
    assert rel_l2(y, want) < TIGHT
    assert ref.argmax_last(y) == ref.argmax_last(want) or \
        abs(float(y[0, ref.argmax_last(y)]) - float(want[0, ref.argmax_last(want)])) < 2e-2


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k,m", [(16, 32, 1), (1, 32, 1), (17, 64, 3), (33, 96, 5), (50, 288, 7), (130, 1056, 9),
                                   (48, 2080, 16), (31, 4128, 2), (20, 6144, 13),
                                   (512, 64, 1), (512, 64, 5), (512, 128, 1), (2048, 64, 16)])
def test_ragged_shapes(dev, ref, qtype, n, k, m):
    """N not a multiple of the 16-row slab, K not a multiple of 256 (padded row pitch), odd block counts."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=3, name=f"r{n}x{k}")
    x = _x(m, k, seed=3, name=f"rx{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    got_w = w.dequantize().numpy()
    assert np.array_equal(got_w.view(np.uint16), ref.dequant(qtype, raw, n * k).reshape(n, k).view(np.uint16))
    y = linear(dev.tensor(x), w).numpy()
    want = ref.linear_q(qtype, raw, n, k, x)
    assert y.shape == (m, n)
    # a handful of outputs cannot average out the oracle's f16 rounding of each weight
    assert rel_l2(y, want) < (TIGHT if n * m >= 64 else TOL)


def test_more_than_16_rows_is_chunked(dev, ref):
    from tensorlogic_b200.api import QTensor, linear
    n, k, m = 96, 512, 37
    raw = _weights(Q4, n, k, seed=4)
    x = _x(m, k, seed=4)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, n, k, raw)).numpy()
    assert rel_l2(y, ref.linear_q(Q4, raw, n, k, x)) < TIGHT


def test_extreme_activations_and_scales(dev, ref, golden):
    """Large / tiny activations and the edge scales (0, negative, subnormal, 123.5)."""
    from tensorlogic_b200.api import QTensor, linear
    raw = golden["q4_0_bytes"]          # W [3, 256]
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((4, 256)) * np.array([[1e-3], [1.0], [3.0], [1e-5]])).astype(np.float16)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, 3, 256, raw)).numpy()
    want = ref.linear_q(Q4, raw, 3, 256, x)
    assert np.all(np.isfinite(y.astype(np.float32)) == np.isfinite(want.astype(np.float32)))
    fin = np.isfinite(want.astype(np.float32))
    for r in range(4):
        if fin[r].all():
            assert rel_l2(y[r], want[r]) < 5e-3, r


def test_f16_weight_and_bias(dev, ref):
    from tensorlogic_b200.api import QTensor, linear
    rng = np.random.default_rng(9)
    w = (0.05 * rng.standard_normal((40, 96))).astype(np.float16)
    x = rng.standard_normal((3, 96)).astype(np.float16)
    b = rng.standard_normal(40).astype(np.float16)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, 1, 40, 96, w), dev.tensor(b)).numpy()
    want = ref.add(ref.linear_f32acc(x, w), np.broadcast_to(b, (3, 40)).copy())
    assert rel_l2(y, want) < TIGHT
    # f32 source tensors are rounded to f16 on upload
    y32 = linear(dev.tensor(x), QTensor.from_blocks(dev, 0, 40, 96, w.astype(np.float32))).numpy()
    assert rel_l2(y32, ref.linear_f32acc(x, w)) < TIGHT
    # bias on the quantized path: separate f16 add after the f16 rounding of the product
    raw = _weights(Q8, 40, 96, seed=5)
    yq = linear(dev.tensor(x), QTensor.from_blocks(dev, Q8, 40, 96, raw), dev.tensor(b)).numpy()
    wantq = ref.add(ref.linear_q(Q8, raw, 40, 96, x), np.broadcast_to(b, (3, 40)).copy())
    assert rel_l2(yq, wantq) < TIGHT


def test_linear_host_entry(dev, ref, lib):
    """The host-buffer variant of the ABI (upload, run, download)."""
    from tensorlogic_b200.api import QTensor
    from tensorlogic_b200._lib import check
    n, k, m = 256, 2048, 2
    raw = _weights(Q4, n, k, seed=6)
    x = _x(m, k, seed=6)
    w = QTensor.from_blocks(dev, Q4, n, k, raw)
    y = np.empty((m, n), np.float16)
    check(lib.tlc_linear_host(dev.handle, w.handle, x.ctypes.data, m, k, y.ctypes.data, None))
    assert rel_l2(y, ref.linear_q(Q4, raw, n, k, x)) < TIGHT


def test_linearity_property_full_size(dev):
    """Size-independent check at lm_head size: W.(a+b) == W.a + W.b up to f16 rounding."""
    from tensorlogic_b200.api import QTensor, linear
    from tensorlogic_b200 import synth
    n, k = 32000, 2048
    w = QTensor.synthetic(dev, Q4, n, k, 11, synth.tensor_id("output.weight"))
    a = _x(1, k, seed=11, name="a").astype(np.float32) * 0.5
    b = _x(1, k, seed=11, name="b").astype(np.float32) * 0.5
    a, b = a.astype(np.float16), b.astype(np.float16)
    s = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    ya = linear(dev.tensor(a), w).numpy().astype(np.float32)
    yb = linear(dev.tensor(b), w).numpy().astype(np.float32)
    ys = linear(dev.tensor(s), w).numpy().astype(np.float32)
    assert rel_l2(ys, ya + yb) < 3e-3


def test_device_generator_matches_host(dev):
    from tensorlogic_b200.api import QTensor
    from tensorlogic_b200 import synth
    for qtype in (Q4, Q8):
        tid = synth.tensor_id("blk.0.attn_q.weight")
        w = QTensor.synthetic(dev, qtype, 64, 512, 5, tid)
        want = synth.blocks(qtype, 5, tid, 64, 512)
        assert np.array_equal(w.raw_bytes().reshape(-1), want.reshape(-1))
        # row- and column-sharded generation equals slices of the whole
        wr = QTensor.synthetic(dev, qtype, 64, 512, 5, tid, tp_rank=1, tp_size=4, split=1)
        assert wr.shape == (16, 512)
        assert np.array_equal(wr.raw_bytes().reshape(16, 16, -1), want[16:32])
        wc = QTensor.synthetic(dev, qtype, 64, 512, 5, tid, tp_rank=3, tp_size=4, split=2)
        assert wc.shape == (64, 128)
        bb = want.shape[-1]
        assert np.array_equal(wc.raw_bytes()[:, :4 * bb].reshape(64, 4, bb), want[:, 12:16])


def test_sharded_upload(dev, ref):
    """Row- and column-split uploads keep exactly the rank's slice; partial sums add up."""
    from tensorlogic_b200.api import QTensor, linear
    n, k, tp = 64, 1024, 4
    raw = _weights(Q4, n, k, seed=7)
    x = _x(2, k, seed=7)
    full = ref.linear_q(Q4, raw, n, k, x)
    xd = dev.tensor(x)
    rows = [linear(xd, QTensor.from_blocks(dev, Q4, n, k, raw, r, tp, 1)).numpy() for r in range(tp)]
    assert rel_l2(np.concatenate(rows, axis=1), full) < TIGHT
    part = np.zeros((2, n), np.float32)
    for r in range(tp):
        xs = dev.tensor(np.ascontiguousarray(x[:, r * k // tp:(r + 1) * k // tp]))
        part += linear(xs, QTensor.from_blocks(dev, Q4, n, k, raw, r, tp, 2)).numpy().astype(np.float32)
    assert rel_l2(part, full) < 3e-3


def test_error_behaviour(dev):
    from tensorlogic_b200.api import QTensor, TensorError, linear
    raw = _weights(Q4, 16, 64)
    w = QTensor.from_blocks(dev, Q4, 16, 64, raw)
    with pytest.raises(TensorError) as e:       # K mismatch (src/ops/matmul.rs:266-273)
        linear(dev.tensor(np.zeros((1, 32), np.float16)), w)
    assert e.value.kind == "InvalidOperation" and "shape mismatch" in str(e.value)
    with pytest.raises(TensorError) as e:       # rank != 2 (matmul.rs:249-253)
        linear(dev.tensor(np.zeros((64,), np.float16)), w)
    assert "2D" in str(e.value)
    with pytest.raises(TensorError) as e:       # quantized K must be a multiple of 32
        QTensor.from_blocks(dev, Q4, 4, 48, np.zeros(100, np.uint8))
    assert e.value.kind == "LoadError"
    with pytest.raises(TensorError) as e:       # truncated tensor data
        QTensor.from_blocks(dev, Q4, 16, 64, raw.reshape(-1)[:100])
    assert e.value.kind == "LoadError"
    with pytest.raises(TensorError):            # unsupported type id (Q4_K = 12)
        QTensor.from_blocks(dev, 12, 16, 256, np.zeros(16 * 144, np.uint8))
    with pytest.raises(TensorError) as e:       # rows do not divide over ranks
        QTensor.from_blocks(dev, Q4, 16, 64, raw, 0, 3, 1)
    assert e.value.kind == "ShapeMismatch"


def test_pool_reuse_and_stats(dev):
    s0 = dev.pool_stats()
    t = dev.empty((1000,))       # 2000 B -> 2 KiB class
    p = t.ptr
    del t
    t2 = dev.empty((900,))
    assert t2.ptr == p           # same size class is served from the pool
    s1 = dev.pool_stats()
    assert s1["reuse_count"] >= s0["reuse_count"] + 1
    big = dev.empty((9 * 1024 * 1024,))   # above the largest class: exact size
    assert dev.pool_stats()["live_bytes"] >= 18 * 1024 * 1024
    del big, t2
    dev.pool_trim(0)
    assert dev.pool_stats()["total_pooled"] == 0


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_bounded_wait_reports_timeout_and_context_survives(dev, ref, kind):
    """Failure detection without a fault: a device-side wait that nothing satisfies (an mbarrier of the
    GEMV pipeline; the peer flags of the all-reduce; the flagged words of its short-vector form) runs out, the kernel returns, synchronize reports it
    once, and the next launch on the same context works."""
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.api import QTensor, TensorError, check, linear
    dev.set_option("wait_limit_ms", 40)
    try:
        check(dev.lib.tlc_selftest_wait_timeout(dev.handle, kind))
        with pytest.raises(TensorError) as e:
            dev.synchronize()
        assert e.value.code == _lib.ERR_TIMEOUT
        dev.synchronize()                      # reported once, then clear
    finally:
        dev.set_option("wait_limit_ms", 2000)
    raw = _weights(Q4, 64, 256, seed=31)
    x = _x(2, 256, seed=31)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, 64, 256, raw)).numpy()
    assert rel_l2(y, ref.linear_q(Q4, raw, 64, 256, x)) < TIGHT


@pytest.mark.gpu
@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k", [(48, 256), (33, 96), (130, 1056)])
def test_device_storage_is_the_tiled_layout(dev, qtype, n, k):
    """HBM holds exactly the bytes of the host-side regrouping; tlc_qtensor_blocks undoes it bit for bit."""
    from tensorlogic_b200.api import QTensor, check
    raw = _weights(qtype, n, k, seed=11, name=f"t{n}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    size = dev.lib.tlc_tiled_bytes(qtype, n, k)
    want = np.empty(size, np.uint8)
    flat = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    check(dev.lib.tlc_tile_blocks_host(qtype, n, k, flat.ctypes.data, want.ctypes.data))
    got = np.empty(size, np.uint8)
    check(dev.lib.tlc_download(dev.handle, got.ctypes.data, w.ptr, size))
    assert np.array_equal(got, want)
    assert np.array_equal(w.raw_bytes().reshape(-1), flat)


@pytest.mark.parametrize("n,k", [(2048, 2048), (512, 5632), (130, 1056), (48, 8192)])
def test_fp8_limb_form_of_one_row(dev, ref, n, k):
    """With option gemv_f8 = 1 one activation row against a Q4_0 weight runs on the FP8 tensor-core
    form (nibbles as e4m3 values, the row as four e4m3 limbs under a power-of-two scale).  Same answers as the f16
    fragments (option gemv_f8 = 0) and as the oracle, also for a row with a huge outlier, a tiny
    row, a zero row, with a fused RMSNorm, and non-finite in, non-finite out."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, norm_linear_multi
    raw = synth.blocks(Q4, 21, synth.tensor_id(f"f8_{n}x{k}"), n, k)
    w = QTensor.from_blocks(dev, Q4, n, k, raw)
    base = synth.activations(21, f"f8x{k}", (1, k))
    outlier = base.copy()
    outlier[0, 3] = np.float16(900.0)
    outlier[0, 40:200] *= np.float16(1e-3)
    cases = {"normal": base, "outlier": outlier, "tiny": (base.astype(np.float32) * 3e-5).astype(np.float16),
             "zero": np.zeros_like(base)}

    def both(fn):
        out = {}
        for mode in (1, 0):
            dev.set_option("gemv_f8", mode)
            try:
                out[mode] = fn()
            finally:
                dev.set_option("gemv_f8", 0)
        return out[1], out[0]

    for name, x in cases.items():
        y8, y16 = both(lambda: linear(dev.tensor(x), w).numpy())
        want = ref.linear_q(Q4, raw, n, k, x)
        if name == "zero":
            assert not np.any(y8.astype(np.float32)) and not np.any(y16.astype(np.float32))
            continue
        assert rel_l2(y8, want) < TIGHT and rel_l2(y16, want) < TIGHT, name
        assert rel_l2(y8, y16) < 5e-4, name
    nw = synth.norm_weight(21, "f8norm", k)
    (y8,), (y16,) = both(lambda: [t.numpy() for t in norm_linear_multi(dev.tensor(outlier), [w], dev.tensor(nw), 1e-5)])
    want = ref.linear_q(Q4, raw, n, k, ref.rms_norm(outlier, nw, 1e-5))
    assert rel_l2(y8, want) < TIGHT and rel_l2(y8, y16) < 5e-4
    bad = base.copy()
    bad[0, 5] = np.float16(np.inf)
    y8, y16 = both(lambda: linear(dev.tensor(bad), w).numpy())
    assert not np.any(np.isfinite(y8.astype(np.float32))) and not np.any(np.isfinite(y16.astype(np.float32)))


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k", [(256, 8192), (100, 28672), (512, 14336)])
def test_split_k_for_many_rows_of_a_wide_input(dev, ref, qtype, n, k):
    """2 to 16 activation rows of a wide K do not fit the shared memory in fragment order: the K
    range is cut into windows (one pass over the weights, f32 partial sums, a finishing kernel with
    the epilogue) instead of several passes.  Same answers as the oracle and as the multi-pass form
    (option gemv_splitk = 0), for the plain, the residual, the SiLU.mul and the RoPE epilogues."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, linear_residual, norm_linear_multi, swiglu_gate_up
    raw = synth.blocks(qtype, 23, synth.tensor_id(f"sk{n}x{k}"), n, k, scale_log2=-3)
    raw2 = synth.blocks(qtype, 23, synth.tensor_id(f"sk2{n}x{k}"), n, k, scale_log2=-3)
    w, w2 = QTensor.from_blocks(dev, qtype, n, k, raw), QTensor.from_blocks(dev, qtype, n, k, raw2)
    nw = synth.norm_weight(23, "sknorm", k)
    for m in (2, 8, 13, 16):
        x = synth.activations(23, f"skx{m}", (m, k))
        want = ref.linear_q(qtype, raw, n, k, x)
        dev.set_option("gemv_splitk", 1)                      # windows sized for two CTAs per SM first
        try:
            l0 = dev.launch_count
            y = linear(dev.tensor(x), w).numpy()
            launches2 = dev.launch_count - l0
        finally:
            dev.set_option("gemv_splitk", 2)
        assert rel_l2(y, want) < TIGHT, m
        l0 = dev.launch_count
        y = linear(dev.tensor(x), w).numpy()
        launches = dev.launch_count - l0
        assert rel_l2(y, want) < TIGHT, m
        dev.set_option("gemv_splitk", 0)
        try:
            l0 = dev.launch_count
            y_passes = linear(dev.tensor(x), w).numpy()
            passes = dev.launch_count - l0
        finally:
            dev.set_option("gemv_splitk", 2)
        assert rel_l2(y, y_passes) < 5e-4
        if passes > 1:
            assert launches == 2 and launches2 == 2, (m, launches, launches2, passes)  # one pass + the finish
        res = synth.activations(23, f"skr{m}", (m, n))
        assert rel_l2(linear_residual(dev.tensor(x), w, dev.tensor(res)).numpy(), ref.add(res, want)) < TIGHT
        xn = ref.rms_norm(x, nw, 1e-5)
        act = swiglu_gate_up(dev.tensor(x), w, w2, dev.tensor(nw), 1e-5).numpy()
        want_act = ref.swiglu(ref.linear_q(qtype, raw, n, k, xn), ref.linear_q(qtype, raw2, n, k, xn))
        assert rel_l2(act, want_act) < 2 * TIGHT
        if n % 64 == 0:
            pos = (np.arange(m, dtype=np.int32) * 11) % 500
            q, v = norm_linear_multi(dev.tensor(x), [w, w2], dev.tensor(nw), 1e-5, rope_heads=[n // 64, 0], positions=pos)
            want_q = ref.rope(ref.linear_q(qtype, raw, n, k, xn).reshape(m, n // 64, 64), 0, 10000, positions=pos).reshape(m, n)
            assert rel_l2(q.numpy(), want_q) < 2 * TIGHT
            assert rel_l2(v.numpy(), ref.linear_q(qtype, raw2, n, k, xn)) < 2 * TIGHT
