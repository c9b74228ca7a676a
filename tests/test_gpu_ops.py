"""GPU parity tests of the per-token ops and of the fused entry points, through the C ABI."""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

Q4, Q8 = 2, 8
TIGHT = 2e-3


def _ulp_diff(a, b):
    """Largest distance in f16 representation steps (same-sign finite values)."""
    a = a.view(np.uint16).astype(np.int32)
    b = b.view(np.uint16).astype(np.int32)
    return int(np.max(np.abs(a - b)))


def test_rms_norm_kat_and_parity(dev, ref, golden):
    from tensorlogic_b200.api import rms_norm
    # src/ops/normalization.rs:736-790
    y = rms_norm(dev.tensor(np.array([[2, 4, 6, 8]], np.float16)), dev.tensor(np.ones(4, np.float16)), 1e-6).numpy()
    assert np.allclose(y.astype(np.float32).ravel(), [0.3652, 0.7305, 1.0957, 1.4609], atol=0.01)
    for rows, d, eps in [(3, 256, 1e-5), (1, 2048, 1e-5), (16, 2048, 1e-6), (2, 8192, 1e-5), (5, 100, 1e-6)]:
        rng = np.random.default_rng(d + rows)
        x = (rng.standard_normal((rows, d)) * 3).astype(np.float16)
        w = (1 + 0.02 * rng.standard_normal(d)).astype(np.float16)
        got = rms_norm(dev.tensor(x), dev.tensor(w), eps).numpy()
        want = ref.rms_norm(x, w, eps)
        # the reduction order differs from the oracle's sequential sum: at most one f16 step
        assert _ulp_diff(got, want) <= 1
        assert rel_l2(got, want) < 2e-4
    got = rms_norm(dev.tensor(golden["rms_x"]), dev.tensor(golden["rms_w"]), 1e-5).numpy()
    assert rel_l2(got, golden["rms_y_eps1e-5"]) < 5e-4


@pytest.mark.parametrize("pos", [0, 7, 513, 2047])
def test_rope_parity(dev, ref, golden, pos):
    from tensorlogic_b200.api import rope
    x = golden["rope_x"]
    got = rope(dev.tensor(x), pos).numpy()
    want = ref.rope(x, pos)
    # powf/cosf/sinf of libm vs CUDA differ in the last bits (more so after the range reduction of
    # large angles); the reference's own tests allow 1e-2 absolute here
    assert np.max(np.abs(got.astype(np.float32) - want.astype(np.float32))) < 5e-3 and rel_l2(got, want) < 5e-4
    if f"rope_y_pos{pos}" in golden:
        assert np.max(np.abs(got.astype(np.float64) - golden[f"rope_y_pos{pos}"])) < 1e-2
    rng = np.random.default_rng(pos)
    for shape in [(1, 32, 64), (3, 4, 64), (2, 8, 128)]:
        x = rng.standard_normal(shape).astype(np.float16)
        assert rel_l2(rope(dev.tensor(x), pos).numpy(), ref.rope(x, pos)) < 3e-4
    p = np.array([5, 0, pos], np.int32)
    x = rng.standard_normal((3, 4, 64)).astype(np.float16)
    assert rel_l2(rope(dev.tensor(x), positions=p).numpy(), ref.rope(x, positions=p)) < 3e-4


def test_rope_properties_and_errors(dev):
    from tensorlogic_b200.api import TensorError, rope
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 3, 8)).astype(np.float16)
    y0 = rope(dev.tensor(x), 0).numpy()
    assert np.array_equal(y0[0].view(np.uint16), x[0].view(np.uint16))   # position 0 is the identity
    y = rope(dev.tensor(x), 9).numpy().astype(np.float32).reshape(-1, 2)
    xm = x.astype(np.float32).reshape(-1, 2)
    assert np.allclose(np.hypot(y[:, 0], y[:, 1]), np.hypot(xm[:, 0], xm[:, 1]), atol=5e-3)
    with pytest.raises(TensorError):          # src/ops/rope.rs: rank < 3
        rope(dev.tensor(np.zeros((4, 8), np.float16)))
    with pytest.raises(TensorError):          # odd head_dim
        rope(dev.tensor(np.zeros((1, 2, 7), np.float16)))


def test_sigmoid_mul_add_swiglu(dev, ref):
    from tensorlogic_b200.api import add, mul, sigmoid, silu, swiglu
    rng = np.random.default_rng(2)
    a = (rng.standard_normal(10007) * 4).astype(np.float16)
    b = (rng.standard_normal(10007) * 4).astype(np.float16)
    ta, tb = dev.tensor(a), dev.tensor(b)
    assert np.array_equal(mul(ta, tb).numpy().view(np.uint16), ref.mul(a, b).view(np.uint16))
    assert np.array_equal(add(ta, tb).numpy().view(np.uint16), ref.add(a, b).view(np.uint16))
    assert _ulp_diff(sigmoid(ta).numpy(), ref.sigmoid(a)) <= 1
    # src/ops/activations.rs:778-840
    kat = silu(dev.tensor(np.array([-2, -1, 0, 1, 2], np.float16))).numpy().astype(np.float32)
    assert np.allclose(kat, [-0.2384, -0.2689, 0.0, 0.7311, 1.7616], atol=2e-3)
    got = swiglu(ta, tb).numpy()
    want = ref.swiglu(a, b)
    assert rel_l2(got, want) < 5e-4
    assert rel_l2(mul(silu(ta), tb).numpy(), want) < 5e-4


def test_softmax(dev, ref):
    from tensorlogic_b200.api import softmax
    rng = np.random.default_rng(3)
    for shape in [(4, 37), (32, 512), (3, 5, 129), (1, 1)]:
        x = (rng.standard_normal(shape) * 3).astype(np.float16)
        got = softmax(dev.tensor(x)).numpy()
        want = ref.softmax(x)
        assert np.max(np.abs(got.astype(np.float32) - want.astype(np.float32))) < 1e-3
        assert np.allclose(got.astype(np.float32).sum(-1), 1.0, atol=1e-2)
    z = np.array([[np.inf, 0.0, -np.inf, np.nan], [-np.inf] * 4, [-10000, 1, 2, -10000]], np.float16)
    got = softmax(dev.tensor(z)).numpy().astype(np.float32)
    assert np.array_equal(got[0], [0, 1, 0, 0]) and np.allclose(got[1], 0.25)
    assert np.allclose(got[2], ref.softmax(z).astype(np.float32)[2], atol=1e-3)


def test_embedding(dev, ref):
    from tensorlogic_b200.api import TensorError, embedding
    rng = np.random.default_rng(4)
    for vocab, d in [(1000, 2048), (50, 20)]:
        t = rng.standard_normal((vocab, d)).astype(np.float16)
        ids = rng.integers(0, vocab, 9)
        assert np.array_equal(embedding(dev.tensor(t), ids).numpy().view(np.uint16), t[ids].view(np.uint16))
        assert np.array_equal(embedding(dev.tensor(t), 3).numpy().view(np.uint16), t[3:4].view(np.uint16))
        with pytest.raises(TensorError) as e:
            embedding(dev.tensor(t), [vocab])
        assert e.value.kind == "IndexOutOfBounds"


# ---- fused entry points == composition of the unfused oracle ops ---------------------

def _blocks(qtype, n, k, name):
    from tensorlogic_b200 import synth
    return synth.blocks(qtype, 21, synth.tensor_id(name), n, k)


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("m,pos", [(1, 0), (1, 700), (5, 31), (16, 500)])
def test_fused_norm_qkv_rope(dev, ref, qtype, m, pos):
    """TinyLlama attention front end: rms_norm -> q/k/v linears -> rope(q), rope(k) in one launch."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, norm_linear_multi
    d, H, Hkv, hd = 2048, 32, 4, 64
    x = synth.activations(21, "h", (m, d))
    nw = synth.norm_weight(21, "attn_norm", d)
    rq, rk, rv = _blocks(qtype, H * hd, d, "q"), _blocks(qtype, Hkv * hd, d, "k"), _blocks(qtype, Hkv * hd, d, "v")
    ws = [QTensor.from_blocks(dev, qtype, r.shape[0], d, r) for r in (rq, rk, rv)]
    q, k, v = norm_linear_multi(dev.tensor(x), ws, dev.tensor(nw), 1e-5, rope_heads=[H, Hkv, 0], position_offset=pos)
    xn = ref.rms_norm(x, nw, 1e-5)
    wq = ref.rope(ref.linear_q(qtype, rq, H * hd, d, xn).reshape(m, H, hd), pos).reshape(m, -1)
    wk = ref.rope(ref.linear_q(qtype, rk, Hkv * hd, d, xn).reshape(m, Hkv, hd), pos).reshape(m, -1)
    wv = ref.linear_q(qtype, rv, Hkv * hd, d, xn)
    for got, want in ((q, wq), (k, wk), (v, wv)):
        assert rel_l2(got.numpy(), want) < TIGHT
    # batched-decode form: explicit per-row positions
    p = (np.arange(m, dtype=np.int32) * 37 + pos) % 2048
    q2, _, _ = norm_linear_multi(dev.tensor(x), ws, dev.tensor(nw), 1e-5, rope_heads=[H, Hkv, 0], positions=p)
    wq2 = ref.rope(ref.linear_q(qtype, rq, H * hd, d, xn).reshape(m, H, hd), positions=p).reshape(m, -1)
    assert rel_l2(q2.numpy(), wq2) < TIGHT


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("m", [1, 3, 16])
def test_fused_swiglu_and_residual(dev, ref, qtype, m):
    """TinyLlama FFN: rms_norm -> gate/up -> silu*mul in one launch, then down + residual in one."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear_residual, swiglu_gate_up
    d, f = 2048, 5632
    x = synth.activations(22, "h", (m, d))
    nw = synth.norm_weight(22, "ffn_norm", d)
    if qtype == Q8:
        # synthetic Q8_0 weights are ~50x larger than Q4_0 ones (|q| up to 127): keep the FFN inside f16 range
        nw = (nw.astype(np.float32) * 0.05).astype(np.float16)
    rg, ru, rd = _blocks(qtype, f, d, "gate"), _blocks(qtype, f, d, "up"), _blocks(qtype, d, f, "down")
    wg, wu, wd = (QTensor.from_blocks(dev, qtype, r.shape[0], r.shape[1] * 32, r) for r in (rg, ru, rd))
    act = swiglu_gate_up(dev.tensor(x), wg, wu, dev.tensor(nw), 1e-5)
    xn = ref.rms_norm(x, nw, 1e-5)
    want_act = ref.swiglu(ref.linear_q(qtype, rg, f, d, xn), ref.linear_q(qtype, ru, f, d, xn))
    assert rel_l2(act.numpy(), want_act) < TIGHT
    y = linear_residual(act, wd, dev.tensor(x)).numpy()
    want = ref.add(x, ref.linear_q(qtype, rd, d, f, want_act))
    assert rel_l2(y, want) < TIGHT
    # without the norm prologue
    act2 = swiglu_gate_up(dev.tensor(x), wg, wu).numpy()
    assert rel_l2(act2, ref.swiglu(ref.linear_q(qtype, rg, f, d, x), ref.linear_q(qtype, ru, f, d, x))) < TIGHT


def test_fused_small_and_ragged(dev, ref):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear_residual, norm_linear_multi, swiglu_gate_up
    d = 96
    x = synth.activations(23, "h", (3, d))
    nw = synth.norm_weight(23, "n", d)
    ra, rb = _blocks(Q4, 40, d, "a"), _blocks(Q4, 24, d, "b")
    wa, wb = QTensor.from_blocks(dev, Q4, 40, d, ra), QTensor.from_blocks(dev, Q4, 24, d, rb)
    ya, yb = norm_linear_multi(dev.tensor(x), [wa, wb], dev.tensor(nw), 1e-6, rope_heads=[5, 0], position_offset=3)
    xn = ref.rms_norm(x, nw, 1e-6)
    assert rel_l2(ya.numpy(), ref.rope(ref.linear_q(Q4, ra, 40, d, xn).reshape(3, 5, 8), 3).reshape(3, 40)) < TIGHT
    assert rel_l2(yb.numpy(), ref.linear_q(Q4, rb, 24, d, xn)) < TIGHT
    rg, ru = _blocks(Q4, 40, d, "g"), _blocks(Q4, 40, d, "u")
    act = swiglu_gate_up(dev.tensor(x), QTensor.from_blocks(dev, Q4, 40, d, rg), QTensor.from_blocks(dev, Q4, 40, d, ru))
    assert rel_l2(act.numpy(), ref.swiglu(ref.linear_q(Q4, rg, 40, d, x), ref.linear_q(Q4, ru, 40, d, x))) < TIGHT
    res = synth.activations(23, "res", (3, 40))
    y = linear_residual(dev.tensor(x), wa, dev.tensor(res)).numpy()
    assert rel_l2(y, ref.add(res, ref.linear_q(Q4, ra, 40, d, x))) < TIGHT


def test_rope_with_tables(dev, ref):
    """rope(x, cos, sin) on the device is bit for bit the oracle's restatement of rope_candle_f16,
    for the pair-indexed table and for the reference builtin's duplicated one; shape errors as upstream."""
    from tensorlogic_b200 import _lib
    from tensorlogic_b200._lib import TensorError
    from tensorlogic_b200.api import rope, rope_table
    rng = np.random.default_rng(41)
    for seq, heads, d in [(7, 4, 64), (33, 2, 128), (1, 32, 64)]:
        x = rng.standard_normal((seq, heads, d)).astype(np.float16)
        for paired in (True, False):
            cos, sin = ref.precompute_rope_tables(d, seq + 5, 10000.0, paired=paired)
            got = rope_table(dev.tensor(x), dev.tensor(cos), dev.tensor(sin)).numpy()
            assert np.array_equal(got.view(np.uint16), ref.rope_table(x, cos, sin).view(np.uint16))
        cos, sin = ref.precompute_rope_tables(d, seq, 10000.0, paired=True)
        close = rope_table(dev.tensor(x), dev.tensor(cos), dev.tensor(sin)).numpy().astype(np.float32)
        assert np.max(np.abs(close - rope(dev.tensor(x)).numpy().astype(np.float32))) < 2e-2
    x = dev.tensor(rng.standard_normal((4, 2, 64)).astype(np.float16))
    cos, sin = ref.precompute_rope_tables(64, 3, 10000.0)
    with pytest.raises(TensorError) as e:                     # fewer table rows than positions
        rope_table(x, dev.tensor(cos), dev.tensor(sin))
    assert e.value.code == _lib.ERR_INVALID_OPERATION and "first dim must be >= seq_len" in str(e.value)
    cos, sin = ref.precompute_rope_tables(32, 8, 10000.0)
    with pytest.raises(TensorError) as e:                     # tables made for another head_dim
        rope_table(x, dev.tensor(cos[:, :24]), dev.tensor(sin[:, :24]))
    assert "last dim must be head_dim" in str(e.value)
    with pytest.raises(TensorError):
        rope_table(dev.tensor(np.zeros((4, 64), np.float16)), dev.tensor(cos), dev.tensor(sin))


def test_matmul_builtin(dev, ref):
    """matmul(a, b): the reference's KAT ([[1,2,3],[4,5,6]] @ [[1,2],[3,4],[5,6]] = [[22,28],[49,64]],
    src/ops/matmul.rs:466-504), ragged shapes against the oracle's f32-accumulating product, the
    shape-mismatch message."""
    from tensorlogic_b200 import _lib
    from tensorlogic_b200._lib import TensorError
    from tensorlogic_b200.api import matmul
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float16)
    b = np.array([[1, 2], [3, 4], [5, 6]], np.float16)
    assert np.array_equal(matmul(dev.tensor(a), dev.tensor(b)).numpy(), np.array([[22, 28], [49, 64]], np.float16))
    rng = np.random.default_rng(42)
    for m, k, n in [(1, 2048, 2048), (10, 2048, 300), (65, 17, 129), (128, 100, 64), (3, 1, 5)]:
        a = rng.standard_normal((m, k)).astype(np.float16)
        b = (rng.standard_normal((k, n)) * 0.05).astype(np.float16)
        got = matmul(dev.tensor(a), dev.tensor(b)).numpy()
        want = ref.linear_f32acc(a, np.ascontiguousarray(b.T))          # a @ b, f32 sums in k order
        assert got.shape == (m, n) and rel_l2(got, want) < 1e-3
    with pytest.raises(TensorError) as e:
        matmul(dev.tensor(np.zeros((2, 3), np.float16)), dev.tensor(np.zeros((4, 2), np.float16)))
    assert e.value.code == _lib.ERR_INVALID_OPERATION and "matmul shape mismatch: [2, 3] @ [4, 2]" in str(e.value)


def test_perf_switch_times_every_op(dev, ref, capfd):
    """Option "perf" (the reference's TL_PERF): each op prints "[PERF] op(shape): x.xxxms" on stderr
    and tlc_perf_report returns per-op call counts and device milliseconds; off again, nothing is
    printed or counted, and results are unchanged."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, rms_norm
    n, k = 256, 512
    raw = synth.blocks(2, 5, synth.tensor_id("perf"), n, k)
    w = QTensor.from_blocks(dev, 2, n, k, raw)
    x = synth.activations(5, "perfx", (3, k))
    nw = synth.norm_weight(5, "perfn", k)
    want = ref.linear_q(2, raw, n, k, x)
    dev.perf_report(reset=True)
    dev.set_option("perf", 1)
    try:
        y = linear(dev.tensor(x), w).numpy()
        linear(dev.tensor(x), w)
        rms_norm(dev.tensor(x), dev.tensor(nw), 1e-5)
    finally:
        dev.set_option("perf", 0)
    err = capfd.readouterr().err
    assert err.count("[PERF] linear(q4_0, m=3, n=256, k=512): ") == 2 and "[PERF] rms_norm(rows=3, d=512): " in err
    rep = dev.perf_report(reset=True)
    assert rep["linear"][0] == 2 and rep["rms_norm"][0] == 1
    assert all(0.0 < ms < 1000.0 for _, ms in rep.values())
    assert np.max(np.abs(y.astype(np.float32) - want.astype(np.float32))) < 2e-3 * max(float(np.max(np.abs(want))), 1.0)
    linear(dev.tensor(x), w)
    dev.synchronize()
    assert "[PERF]" not in capfd.readouterr().err and dev.perf_report() == {}
