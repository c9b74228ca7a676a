"""GPU parity tests of the tensor-core (tcgen05) path of the quantized linears.

The path takes over from the GEMV for many activation rows (prefill).  Its
weight tile must hold exactly the oracle's dequantized f16 values (checked
bit-exactly through one-hot activations); its outputs must be within rel-L2
1e-2 of the oracle's dequant + f32-accumulate linear (observed ~1e-4) and agree
with the GEMV path on the same inputs.
"""
import contextlib

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-2
TIGHT = 2e-3
Q4, Q8 = 2, 8
NEVER = 1 << 30


@contextlib.contextmanager
def gemm_from(dev, min_m):
    """Route linears with at least min_m rows to the GEMM (NEVER: keep the GEMV)."""
    dev.set_option("gemm_min_m", min_m)
    try:
        yield
    finally:
        dev.set_option("gemm_min_m", 0)


def _bits(a):
    """f16 bit patterns with -0 folded into +0: a weight of -0 (zero scale, negative
    quant) passes through the accumulator as 0 + (-0) = +0."""
    a = np.ascontiguousarray(a, dtype=np.float16)
    return (a + np.float16(0)).view(np.uint16)


def _weights(qtype, n, k, seed=0, name="w"):
    from tensorlogic_b200 import synth
    return synth.blocks(qtype, seed, synth.tensor_id(name), n, k)


def _x(m, k, seed=0, name="x"):
    from tensorlogic_b200 import synth
    return synth.activations(seed, name, (m, k))


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k", [(128, 128), (200, 192), (77, 64)])
def test_weight_tile_is_bit_exact(dev, ref, golden, qtype, n, k):
    """One-hot activations read the dequantized weight tile back through the MMA, exactly."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=11, name=f"tile{n}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    x = np.eye(k, dtype=np.float16)                      # row j picks column j of W
    with gemm_from(dev, 1):
        y = linear(dev.tensor(x), w).numpy()             # [k, n] = W^T
    want = ref.dequant(qtype, raw, n * k).reshape(n, k).T
    assert np.array_equal(_bits(y), _bits(want))


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_edge_scales_through_gemm(dev, ref, golden, qtype):
    """Zero, negative, subnormal and large block scales (the golden blocks) survive the tile dequantizer."""
    from tensorlogic_b200.api import QTensor, linear
    raw = golden["q4_0_bytes" if qtype == Q4 else "q8_0_bytes"]     # W [3, 256]
    w = QTensor.from_blocks(dev, qtype, 3, 256, raw)
    x = np.eye(256, dtype=np.float16)
    with gemm_from(dev, 1):
        y = linear(dev.tensor(x), w).numpy()
    want = np.ascontiguousarray(ref.dequant(qtype, raw, 768).reshape(3, 256).T)
    assert np.array_equal(_bits(y), _bits(want))


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k,m", [(128, 64, 128), (130, 128, 37), (2048, 2048, 128), (256, 5632, 100),
                                   (4000, 2048, 17), (5632, 2048, 700), (96, 4096, 513),
                                   (200, 96, 130), (64, 1376, 40), (512, 64, 21), (512, 128, 21)])
def test_gemm_matches_oracle(dev, ref, qtype, n, k, m):
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=12, name=f"g{n}x{k}")
    x = _x(m, k, seed=12, name=f"gx{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    with gemm_from(dev, 1):
        y = linear(dev.tensor(x), w).numpy()
    want = ref.linear_q(qtype, raw, n, k, x)
    assert y.shape == (m, n)
    err = rel_l2(y, want)
    assert err < TOL and err < TIGHT, err
    yf, wf = y.astype(np.float32), want.astype(np.float32)
    assert np.max(np.abs(yf - wf)) < 2e-3 * max(float(np.max(np.abs(wf))), 1.0)


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("tile", [11, 12, 22])
@pytest.mark.parametrize("n,k,m", [(300, 640, 300), (512, 1088, 130), (40, 4096, 257)])
def test_every_tile_shape(dev, ref, qtype, tile, n, k, m):
    """128x128, 128x256 and 256x256 tiles on ragged shapes (several CTAs per axis, partial tiles, ring wrap-around)."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=17, name=f"t{n}x{k}")
    x = _x(m, k, seed=17, name=f"tx{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    want = ref.linear_q(qtype, raw, n, k, x)
    want_t = ref.dequant(qtype, raw, n * k).reshape(n, k).T[:m]
    dev.set_option("gemm_tile", tile)
    try:
        # one producer group, and (tiles of one activation sub-tile) two groups taking alternate K steps
        for pg in (1, 2):
            dev.set_option("gemm_pg", pg)
            with gemm_from(dev, 1):
                y = linear(dev.tensor(x), w).numpy()
                yt = linear(dev.tensor(np.eye(k, dtype=np.float16)[:m]), w).numpy()
            assert rel_l2(y, want) < TIGHT, pg
            assert np.array_equal(_bits(yt), _bits(want_t)), pg
    finally:
        dev.set_option("gemm_tile", 0)
        dev.set_option("gemm_pg", 0)


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k,m", [(300, 640, 300), (512, 1088, 130), (40, 4096, 257), (1000, 64, 129),
                                   (2100, 96, 2500), (256, 8192, 256)])
def test_cta_pair_tiles(dev, ref, qtype, n, k, m):
    """The CTA-pair kernel (option gemm_pair: two SMs per 256 x 256 tile, persistent): ragged
    shapes, a walk of several tiles per cluster (2100 x 2500: 90 tiles), both accumulators, ring
    wrap-around; the same shapes on the default single-CTA kernel give the same result."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=19, name=f"p{n}x{k}")
    x = _x(m, k, seed=19, name=f"px{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    want = ref.linear_q(qtype, raw, n, k, x)
    eye = np.eye(k, dtype=np.float16)[:m] if m <= k else None
    with gemm_from(dev, 1):
        y1 = linear(dev.tensor(x), w).numpy()
        dev.set_option("gemm_pair", 1)
        try:
            l0 = dev.launch_count
            y = linear(dev.tensor(x), w).numpy()
            assert dev.launch_count - l0 == 1
            yt = linear(dev.tensor(eye), w).numpy() if eye is not None else None
        finally:
            dev.set_option("gemm_pair", 0)
    assert rel_l2(y, want) < TIGHT
    assert rel_l2(y1, want) < TIGHT
    assert rel_l2(y, y1) < 1e-4
    if yt is not None:
        assert np.array_equal(_bits(yt), _bits(ref.dequant(qtype, raw, n * k).reshape(n, k).T[:m]))


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k,m", [(512, 2048, 100), (200, 4096, 37), (2048, 8192, 128), (96, 1088, 64), (300, 1056, 17)])
def test_gemm_split_k(dev, ref, qtype, n, k, m):
    """Up to 128 rows against a weight of few tiles: the K steps are shared out over several CTAs
    per tile (f32 shares in scratch, one finishing kernel).  Same answer as the oracle and as the
    unsplit GEMM (option gemm_splitk = 0); ragged N, K with a last step of one block, uneven shares."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=21, name=f"s{n}x{k}")
    x = _x(m, k, seed=21, name=f"sx{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    want = ref.linear_q(qtype, raw, n, k, x)
    with gemm_from(dev, 1):
        try:
            dev.set_option("gemm_splitk", 2)  # share K wherever possible, also where the cost model would not
            l0 = dev.launch_count
            y = linear(dev.tensor(x), w).numpy()
            launches = dev.launch_count - l0
            yt = linear(dev.tensor(np.eye(k, dtype=np.float16)[:m]), w).numpy()
            dev.set_option("gemm_splitk", 1)  # the default: by cost
            y2 = linear(dev.tensor(x), w).numpy()
            dev.set_option("gemm_splitk", 0)
            l0 = dev.launch_count
            y1 = linear(dev.tensor(x), w).numpy()
            assert dev.launch_count - l0 == 1
        finally:
            dev.set_option("gemm_splitk", 1)
    assert launches == 2, launches            # the GEMM with K shared out + the finishing kernel
    assert rel_l2(y2, want) < TIGHT
    assert rel_l2(y, want) < TIGHT and rel_l2(y1, want) < TIGHT
    assert rel_l2(y, y1) < 1e-4
    assert np.array_equal(_bits(yt), _bits(ref.dequant(qtype, raw, n * k).reshape(n, k).T[:m]))


@pytest.mark.parametrize("qtype", [Q4, Q8])
@pytest.mark.parametrize("n,k,m", [(300, 640, 300), (512, 2048, 100), (2100, 96, 2500), (64, 1376, 40)])
def test_gemm_with_cp_async_activation_loaders(dev, ref, qtype, n, k, m):
    """Option gemm_tma = 0: four warps copy the activation tile with cp.async instead of the TMA
    boxes (the path taken when no tensor map can be made); one and two producer groups, split K."""
    from tensorlogic_b200.api import QTensor, linear
    raw = _weights(qtype, n, k, seed=22, name=f"c{n}x{k}")
    x = _x(m, k, seed=22, name=f"cx{m}x{k}")
    w = QTensor.from_blocks(dev, qtype, n, k, raw)
    dev.set_option("gemm_tma", 0)
    try:
        with gemm_from(dev, 1):
            y = linear(dev.tensor(x), w).numpy()
            yt = linear(dev.tensor(np.eye(k, dtype=np.float16)[:m]), w).numpy() if m <= k else None
    finally:
        dev.set_option("gemm_tma", 1)
    assert rel_l2(y, ref.linear_q(qtype, raw, n, k, x)) < TIGHT
    if yt is not None:
        assert np.array_equal(_bits(yt), _bits(ref.dequant(qtype, raw, n * k).reshape(n, k).T[:m]))


def test_automatic_tile_choice_large(dev, ref):
    """Shapes large enough that the launcher picks the wide tiles by itself."""
    from tensorlogic_b200.api import QTensor, linear
    for n, k, m in [(4100, 512, 2390), (4100, 256, 1190)]:
        raw = _weights(Q4, n, k, seed=18, name=f"a{n}x{k}")
        x = _x(m, k, seed=18, name=f"ax{m}x{k}")
        y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, n, k, raw)).numpy()
        assert rel_l2(y, ref.linear_q(Q4, raw, n, k, x)) < TIGHT, (n, k, m)


def test_gemm_agrees_with_gemv(dev):
    from tensorlogic_b200.api import QTensor, linear
    n, k, m = 1024, 2048, 48
    w = QTensor.from_blocks(dev, Q4, n, k, _weights(Q4, n, k, seed=13))
    x = dev.tensor(_x(m, k, seed=13))
    with gemm_from(dev, 1):
        a = linear(x, w).numpy()
    with gemm_from(dev, NEVER):
        b = linear(x, w).numpy()
    # the GEMM rounds each dequantized weight to f16 (as the reference's loader does), the
    # GEMV scales the block's integer dot product by d: a random walk of 2^-11 relative steps
    assert rel_l2(a, b) < 1e-3


def test_default_dispatch(dev, ref):
    """Without an override: 16 rows stay on the GEMV, wide weights switch from 17 rows on."""
    from tensorlogic_b200.api import QTensor, linear
    n, k = 128 * 80, 256
    raw = _weights(Q4, n, k, seed=14)
    w = QTensor.from_blocks(dev, Q4, n, k, raw)
    for m in (16, 17, 64):
        x = _x(m, k, seed=14, name=f"d{m}")
        y = linear(dev.tensor(x), w).numpy()
        assert rel_l2(y, ref.linear_q(Q4, raw, n, k, x)) < TIGHT, m
    # an odd number of blocks (K = 96): the last K step of the GEMM holds one block and zero padding
    n, k, m = 64, 96, 80
    raw = _weights(Q4, n, k, seed=15)
    x = _x(m, k, seed=15)
    with gemm_from(dev, 1):
        y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q4, n, k, raw)).numpy()
    assert rel_l2(y, ref.linear_q(Q4, raw, n, k, x)) < TIGHT


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_fused_contract_on_gemm(dev, ref, qtype):
    """RMSNorm prologue, RoPE / residual / bias / SiLU.mul epilogues give what the GEMV path gives."""
    _fused_contract(dev, qtype, 45)


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_fused_contract_on_cta_pairs(dev, ref, qtype):
    """The same contract on the CTA-pair kernel (option gemm_pair, from 129 rows on)."""
    dev.set_option("gemm_pair", 1)
    try:
        _fused_contract(dev, qtype, 300)
    finally:
        dev.set_option("gemm_pair", 0)


@pytest.mark.parametrize("qtype", [Q4, Q8])
def test_fused_contract_on_split_k_gemm(dev, ref, qtype):
    """The same contract with K = 2048 and 45 rows: every GEMM of it shares K over several CTAs."""
    _fused_contract(dev, qtype, 45, d=2048)


def _fused_contract(dev, qtype, m, d=256):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, linear_residual, norm_linear_multi, swiglu_gate_up
    heads, kvh, hd, ffn = 4, 2, 64, 384
    wq = QTensor.from_blocks(dev, qtype, heads * hd, d, _weights(qtype, heads * hd, d, 16, "q"))
    wk = QTensor.from_blocks(dev, qtype, kvh * hd, d, _weights(qtype, kvh * hd, d, 16, "k"))
    wv = QTensor.from_blocks(dev, qtype, kvh * hd, d, _weights(qtype, kvh * hd, d, 16, "v"))
    wg = QTensor.from_blocks(dev, qtype, ffn, d, _weights(qtype, ffn, d, 16, "g"))
    wu = QTensor.from_blocks(dev, qtype, ffn, d, _weights(qtype, ffn, d, 16, "u"))
    x = dev.tensor(_x(m, d, 16))
    res = dev.tensor(_x(m, heads * hd, 16, "res"))
    bias = dev.tensor(_x(1, heads * hd, 16, "bias").reshape(-1))
    nw = dev.tensor((synth.norm_weight(16, "nw", d).astype(np.float32) * 0.05).astype(np.float16))
    positions = np.arange(m, dtype=np.int32)[::-1].copy() * 3

    def run():
        qkv = norm_linear_multi(x, [wq, wk, wv], nw, 1e-5, [heads, kvh, 0], position_offset=7)
        qkv_p = norm_linear_multi(x, [wq, wk], None, 1e-5, [heads, kvh], positions=positions)
        act = swiglu_gate_up(x, wg, wu, nw, 1e-5)
        r = linear_residual(x, wq, res)
        b = linear(x, wq, bias)
        return [t.numpy() for t in qkv + qkv_p + [act, r, b]]

    with gemm_from(dev, 1):
        a = run()
    with gemm_from(dev, NEVER):
        b = run()
    for i, (u, v) in enumerate(zip(a, b)):
        assert u.shape == v.shape
        assert rel_l2(u, v) < 1e-3, i


def test_long_prefill_uses_gemm_and_matches_oracle(dev, ref, tmp_path):
    """A 100-token prompt through the runner: GEMM prefill == GEMV prefill == oracle forward."""
    from gguf_util import write_gguf
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, LlamaArch, load_model, synthetic_host_weights
    from test_gpu_model import _ref_model
    arch = LlamaArch(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=1000)
    weights = synthetic_host_weights(arch, seed=6)
    path = tmp_path / "small.gguf"
    write_gguf(path, weights, arch)
    model = load_model(dev, path)
    ids = synth.token_ids(6, "prompt", 100, arch.vocab)
    out = {}
    for label, min_m in (("gemm", 1), ("gemv", NEVER)):
        with gemm_from(dev, min_m):
            llm = Llama(dev, model, arch, max_seq=256, max_prefill=128, logits_all_rows=True)
            launches0 = dev.launch_count
            nxt, logits = llm.prefill(ids, all_rows=True)
            out[label] = (nxt, logits, dev.launch_count - launches0)
            # the decode step after the prompt reads the cache the prefill wrote
            out[label + "_step"] = llm.decode([int(ids[0])], return_logits=True)[1]
    want = _ref_model(ref, weights, arch).forward(ids)
    assert rel_l2(out["gemm"][1], want) < TOL
    assert rel_l2(out["gemm"][1], out["gemv"][1]) < 5e-3
    assert rel_l2(out["gemm_step"], out["gemv_step"]) < 5e-3
    assert out["gemm"][2] != out["gemv"][2]          # different kernels ran
