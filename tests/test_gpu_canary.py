"""Out-of-bounds stand-in for a memory checker: every output of the linear paths is written into
the middle of a larger buffer whose guard bands (one output row's worth before, a row plus 64
elements after) hold a bit pattern no kernel produces.  After the call the bands must be intact and
the interior must match the oracle -- for ragged N and M on the GEMV (one pass, split K), the tcgen05
GEMM (single CTA, split K, CTA pairs) and the fused epilogues."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

Q4, Q8 = 2, 8
CANARY = np.uint16(0x7E5A)  # a NaN payload no computation here produces


def _guarded(dev, rows, cols):
    """A device buffer of (1 + rows + 1) rows of `cols` f16 plus 64 elements, all canaries."""
    total = (rows + 2) * cols + 64
    host = np.full(total, CANARY, np.uint16).view(np.float16)
    return dev.tensor(host), cols * 2  # tensor, byte offset of the interior


def _check(buf, rows, cols, want, tol=2e-3):
    got = buf.numpy().view(np.uint16)
    assert np.all(got[:cols] == CANARY), "write before the output"
    assert np.all(got[(rows + 1) * cols:] == CANARY), "write past the output"
    inner = got[cols:(rows + 1) * cols].view(np.float16).reshape(rows, cols)
    assert not np.any(inner.view(np.uint16) == CANARY), "an output element was never written"
    assert rel_l2(inner, want) < tol


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k", [(77, 64), (130, 1056), (200, 4096), (1000, 2048)])
@pytest.mark.parametrize("m", [1, 3, 16, 17, 37, 130])
def test_linear_writes_only_its_output(dev, ref, qtype, n, k, m):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, check
    raw = synth.blocks(qtype, 41, synth.tensor_id(f"cw{n}x{k}"), n, k)
    x = synth.activations(41, f"cx{m}x{k}", (m, k))
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    want = ref.linear_q(qtype, raw, n, k, x)
    xd = dev.tensor(x)
    for pair in (0, 1):
        dev.set_option("gemm_pair", pair)
        try:
            buf, off = _guarded(dev, m, n)
            check(dev.lib.tlc_linear(dev.handle, w.handle, xd.ptr, m, k, C.c_void_p(buf.ptr + off), None))
            _check(buf, m, n, want)
        finally:
            dev.set_option("gemm_pair", 0)


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("m", [1, 8, 13, 45, 300])
def test_fused_epilogues_write_only_their_output(dev, ref, qtype, m):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, check
    n, k = 328, 2048                     # ragged N (not a multiple of 16), K wide enough for split K
    raw = synth.blocks(qtype, 42, synth.tensor_id("cg"), n, k, scale_log2=-3)
    raw2 = synth.blocks(qtype, 42, synth.tensor_id("cu"), n, k, scale_log2=-3)
    w, w2 = QTensor.from_blocks(dev, qtype, n, k, raw), QTensor.from_blocks(dev, qtype, n, k, raw2)
    x = synth.activations(42, f"cfx{m}", (m, k))
    res = synth.activations(42, f"cfr{m}", (m, n))
    nw = synth.norm_weight(42, "cfn", k)
    xd, rd, nd = dev.tensor(x), dev.tensor(res), dev.tensor(nw)
    lin = ref.linear_q(qtype, raw, n, k, x)
    buf, off = _guarded(dev, m, n)
    check(dev.lib.tlc_linear_residual(dev.handle, w.handle, xd.ptr, m, rd.ptr, C.c_void_p(buf.ptr + off)))
    _check(buf, m, n, ref.add(res, lin))
    xn = ref.rms_norm(x, nw, 1e-5)
    want_act = ref.swiglu(ref.linear_q(qtype, raw, n, k, xn), ref.linear_q(qtype, raw2, n, k, xn))
    buf, off = _guarded(dev, m, n)
    check(dev.lib.tlc_swiglu_gate_up(dev.handle, w.handle, w2.handle, xd.ptr, m, nd.ptr, C.c_float(1e-5),
                                     C.c_void_p(buf.ptr + off)))
    _check(buf, m, n, want_act, tol=4e-3)
    buf, off = _guarded(dev, m, k)
    check(dev.lib.tlc_rms_norm(dev.handle, xd.ptr, nd.ptr, C.c_void_p(buf.ptr + off), m, k, C.c_float(1e-5)))
    _check(buf, m, k, xn)
