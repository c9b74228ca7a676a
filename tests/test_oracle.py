"""Pins the CPU oracle against the reference's own known-answer tests and
against outputs of the reference's Python implementation (tests/golden)."""
import numpy as np
import pytest

from conftest import rel_l2


# ---- f16 conversion ----------------------------------------------------------

def test_f16_to_f32_exhaustive(ref):
    bits = np.arange(65536, dtype=np.uint16)
    h = bits.view(np.float16)
    got = ref.f16_to_f32(h)
    want = h.astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.all(np.isnan(got[nan]))


def test_f32_to_f16_matches_ieee_rne(ref):
    rng = np.random.default_rng(1)
    # every f16 value, midpoints between neighbours, and random floats over the whole range
    h = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float32)
    mids = ((h[:-1].astype(np.float64) + h[1:].astype(np.float64)) / 2).astype(np.float32)
    rnd = rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32)
    tiny = (rng.random(20000).astype(np.float32) * np.float32(2.0 ** -13))
    big = np.array([65504.0, 65519.9, 65520.0, 65536.0, 1e9, np.inf, -np.inf, 2.0 ** -25, 2.0 ** -24,
                    1.5 * 2.0 ** -25, -0.0, 0.0], np.float32)
    x = np.concatenate([h, -h, mids, -mids, np.nextafter(mids, np.float32(np.inf)),
                        np.nextafter(mids, np.float32(-np.inf)), rnd, tiny, big])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    got = ref.f32_to_f16(x)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


# ---- dequantizers: the reference's Rust known-answer tests ----------------------

def _q8_block(scale, qs):
    b = np.zeros(34, np.uint8)
    b[0:2] = np.array([scale], np.float16).view(np.uint8)
    b[2:] = np.asarray(qs, dtype=np.uint8)
    return b


def test_q8_0_kat_scale_one(ref):
    # src/model/formats/gguf.rs:622-643
    out = ref.dequant(ref.GGML_Q8_0, _q8_block(1.0, np.arange(32)), 32)
    assert out.shape == (32,)
    assert out[0] == 0.0 and out[1] == 1.0 and out[2] == 2.0
    assert np.array_equal(out.astype(np.float32), np.arange(32, dtype=np.float32))


def test_q8_0_kat_two_blocks(ref):
    # src/model/formats/gguf.rs:666-695
    data = np.concatenate([_q8_block(1.0, np.arange(32)), _q8_block(2.0, np.arange(32))])
    out = ref.dequant(ref.GGML_Q8_0, data, 64)
    assert out[0] == 0.0 and out[10] == 10.0 and out[32] == 0.0 and out[42] == 20.0


def test_q4_0_kat_scale_effect(ref):
    # src/model/formats/gguf.rs:697-718: scale 0.5, all nibbles 0xF -> 3.5
    b = np.zeros(18, np.uint8)
    b[0:2] = np.array([0.5], np.float16).view(np.uint8)
    b[2:] = 0xFF
    out = ref.dequant(ref.GGML_Q4_0, b, 32)
    assert out.shape == (32,)
    assert np.all(np.abs(out.astype(np.float32) - 3.5) < 0.01)
    assert np.all(out == np.float16(3.5))


def test_q4_0_kat_layout(ref):
    # src/model/formats/gguf.rs:645-664: byte 0x01 -> element 0 is -7*d, element 16 is -8*d
    b = np.zeros(18, np.uint8)
    b[0:2] = np.array([1.0], np.float16).view(np.uint8)
    b[2] = 0x01
    out = ref.dequant(ref.GGML_Q4_0, b, 32).astype(np.float32)
    assert out.shape == (32,)
    assert out[0] == -7.0 and out[16] == -8.0 and np.all(out[1:16] == -8.0) and np.all(out[17:] == -8.0)


def test_q4_0_truncated_input_leaves_zeros(ref):
    # gguf.rs:79-81: stop at the first block that does not fit; the rest stays zero
    b = np.zeros(18 + 10, np.uint8)
    b[0:2] = np.array([1.0], np.float16).view(np.uint8)
    b[2:18] = 0x99
    out = ref.dequant(ref.GGML_Q4_0, b, 64).astype(np.float32)
    assert np.all(out[:32] == 1.0) and np.all(out[32:] == 0.0)


def test_dequant_vs_reference_python_and_gguf_package(ref, golden):
    q4 = golden["q4_0_bytes"]
    got = ref.dequant(ref.GGML_Q4_0, q4, q4.shape[0] * 32)
    # the reference script and the gguf package both produce f32 d*(q-8); rounding that
    # exact product to f16 is precisely the Rust loader's single rounding
    with np.errstate(over="ignore"):
        assert np.array_equal(got.view(np.uint16), golden["q4_0_script_f32"].astype(np.float16).view(np.uint16))
        assert np.array_equal(got.view(np.uint16), golden["q4_0_gguf_f32"].astype(np.float16).view(np.uint16))
    q8 = golden["q8_0_bytes"]
    got8 = ref.dequant(ref.GGML_Q8_0, q8, q8.shape[0] * 32)
    with np.errstate(over="ignore"):
        assert np.array_equal(got8.view(np.uint16), golden["q8_0_gguf_f32"].astype(np.float16).view(np.uint16))


# ---- matmul / linear ---------------------------------------------------------------

def test_matmul_kat(ref):
    # src/ops/matmul.rs:466-504: [[1,2,3],[4,5,6]] @ [[1,2],[3,4],[5,6]] = [22,28,49,64]
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float16)
    b = np.array([[1, 2], [3, 4], [5, 6]], np.float16)
    assert np.array_equal(ref.matmul_f16acc(a, b).astype(np.float32).ravel(), [22, 28, 49, 64])
    assert np.array_equal(ref.linear_literal(a, b.T.copy()).astype(np.float32).ravel(), [22, 28, 49, 64])
    assert np.array_equal(ref.linear_f32acc(a, b.T.copy()).astype(np.float32).ravel(), [22, 28, 49, 64])


def test_linear_variants_agree_within_tolerance(ref):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 512)).astype(np.float16)
    w = (rng.uniform(-0.16, 0.16, (96, 512))).astype(np.float16)
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    f32 = ref.linear_f32acc(x, w)
    lit = ref.linear_literal(x, w)
    assert rel_l2(f32, exact) < 1e-3
    # the f16 running sum of the literal CPU path is visibly noisier
    assert rel_l2(lit, exact) < 3e-2
    assert rel_l2(f32, exact) < rel_l2(lit, exact)


def test_linear_q_equals_dequant_then_linear(ref, golden):
    rng = np.random.default_rng(4)
    q4 = golden["q4_0_bytes"][6:].copy()  # 18 blocks with ordinary scales -> W [3, 192]
    x = rng.standard_normal((2, 192)).astype(np.float16)
    w = ref.dequant(ref.GGML_Q4_0, q4, 18 * 32).reshape(3, 192)
    assert np.array_equal(ref.linear_q(ref.GGML_Q4_0, q4, 3, 192, x).view(np.uint16),
                          ref.linear_f32acc(x, w).view(np.uint16))


# ---- rms_norm / rope / sigmoid / softmax / attention --------------------------------

def test_rms_norm_kat(ref):
    # src/ops/normalization.rs:736-790: [2,4,6,8], w=1, eps=1e-6
    y = ref.rms_norm(np.array([[2, 4, 6, 8]], np.float16), np.ones(4, np.float16), 1e-6).astype(np.float32)
    assert np.allclose(y.ravel(), [0.3652, 0.7305, 1.0957, 1.4609], atol=0.01)


def test_rms_norm_vs_reference_python(ref, golden):
    y = ref.rms_norm(golden["rms_x"], golden["rms_w"], 1e-5)
    want = golden["rms_y_eps1e-5"]
    assert np.max(np.abs(y.astype(np.float64) - want)) <= 2e-3 * np.max(np.abs(want))
    assert rel_l2(y, want) < 5e-4


@pytest.mark.parametrize("pos", [0, 7, 513])
def test_rope_vs_reference_python(ref, golden, pos):
    y = ref.rope(golden["rope_x"], pos_offset=pos)
    want = golden[f"rope_y_pos{pos}"]
    # reference tests allow 1e-2 (tests/test_shader_mathematical_correctness.rs:156-185)
    assert np.max(np.abs(y.astype(np.float64) - want)) < 1e-2
    assert rel_l2(y, want) < 1e-3


def test_rope_properties(ref):
    # src/ops/rope.rs:322-640: position 0 is the identity; pair magnitudes are preserved
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 2, 8)).astype(np.float16)
    assert np.array_equal(ref.rope(x, 0).view(np.uint16), x.view(np.uint16))
    y = ref.rope(x, 11).astype(np.float32).reshape(-1, 2)
    xm = x.astype(np.float32).reshape(-1, 2)
    assert np.allclose(np.hypot(y[:, 0], y[:, 1]), np.hypot(xm[:, 0], xm[:, 1]), atol=5e-3)
    pos = np.array([3], np.int32)
    assert np.array_equal(ref.rope(x, 0, positions=pos).view(np.uint16), ref.rope(x, 3).view(np.uint16))


def test_silu_kat(ref):
    # src/ops/activations.rs:778-840: silu at -2,-1,0,1,2
    x = np.array([-2, -1, 0, 1, 2], np.float16)
    got = ref.mul(x, ref.sigmoid(x)).astype(np.float32)
    want = np.array([-0.2384, -0.2689, 0.0, 0.7311, 1.7616], np.float32)
    assert np.allclose(got, want, atol=2e-3)
    assert np.array_equal(ref.swiglu(x, np.ones(5, np.float16)).view(np.uint16), ref.mul(x, ref.sigmoid(x)).view(np.uint16))


def test_softmax(ref):
    # tests/test_shader_mathematical_correctness.rs:103-133 (CPU reference in the test)
    rng = np.random.default_rng(6)
    x = rng.standard_normal((4, 37)).astype(np.float16)
    y = ref.softmax(x).astype(np.float64)
    e = np.exp(x.astype(np.float64) - x.astype(np.float64).max(-1, keepdims=True))
    assert np.allclose(y, e / e.sum(-1, keepdims=True), atol=1e-3)
    assert np.allclose(y.sum(-1), 1.0, atol=5e-3)
    # non-finite inputs contribute zero; an all-masked row becomes uniform
    z = np.array([[np.inf, 0.0, -np.inf, np.nan]], np.float16)
    assert np.array_equal(ref.softmax(z).astype(np.float32), [[0, 1, 0, 0]])
    assert np.allclose(ref.softmax(np.full((1, 4), -np.inf, np.float16)).astype(np.float32), 0.25)


def test_attention_vs_reference_python(ref, golden):
    q, k, v = golden["attn_q"], golden["attn_k"], golden["attn_v"]
    S = q.shape[0]
    # full visibility (q_pos0 large) = the reference script's unmasked attention
    out = ref.attention(q, k, v, 1.0 / np.sqrt(q.shape[-1]), q_pos0=S, round_exp=True, f16_pv=False)
    assert rel_l2(out, golden["attn_full_out"]) < 3e-3
    # the shader's f16 running sum for P.V stays within the reference's 1e-2 tolerance
    lit = ref.attention(q, k, v, 1.0 / np.sqrt(q.shape[-1]), q_pos0=S, round_exp=True, f16_pv=True)
    assert rel_l2(lit, golden["attn_full_out"]) < 1e-2


def test_attention_causal_mask(ref):
    rng = np.random.default_rng(7)
    q = rng.standard_normal((3, 4, 8)).astype(np.float16)
    k = rng.standard_normal((5, 2, 8)).astype(np.float16)
    v = rng.standard_normal((5, 2, 8)).astype(np.float16)
    # queries at positions 2,3,4 over 5 keys == each query alone over its visible prefix
    out = ref.attention(q, k, v, 0.35, q_pos0=2)
    for i in range(3):
        alone = ref.attention(q[i:i + 1], k[:3 + i], v[:3 + i], 0.35, q_pos0=2 + i)
        assert rel_l2(out[i], alone[0]) < 2e-3


def test_swiglu_ffn_vs_reference_python(ref, golden):
    x = golden["ffn_x"]
    g = ref.linear_f32acc(x, golden["ffn_wg"])
    u = ref.linear_f32acc(x, golden["ffn_wu"])
    y = ref.linear_f32acc(ref.swiglu(g, u), golden["ffn_wd"])
    assert rel_l2(y, golden["ffn_y"]) < 5e-3


def test_argmax_last_on_ties(ref):
    # src/interpreter/builtin_sampling.rs:176-181: max_by keeps the last maximum
    assert ref.argmax_last(np.array([1, 5, 3, 5, 2], np.float16)) == 3
    assert ref.argmax_last(np.array([7], np.float16)) == 0


def test_embedding_bounds(ref):
    t = np.arange(12, dtype=np.float16).reshape(4, 3)
    assert np.array_equal(ref.embedding(t, [2, 0]), t[[2, 0]])
    with pytest.raises(IndexError):
        ref.embedding(t, [4])


def test_literal_matmul_hardware_and_software_conversions_agree(ref):
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((2, 300)) * 3).astype(np.float16)
    w = rng.uniform(-0.3, 0.3, (17, 300)).astype(np.float16)
    ref.set_f16c(True)
    hw = ref.linear_literal(x, w)
    ref.set_f16c(False)
    sw = ref.linear_literal(x, w)
    ref.set_f16c(True)
    assert np.array_equal(hw.view(np.uint16), sw.view(np.uint16))


def test_q6_k_against_gguf_package(ref):
    """Q6_K super-blocks: bit-exact with the gguf package's dequantizer (llama.cpp element order,
    the order GGUFLoader::dequantize_q6_k follows), including zero / negative / subnormal
    super-block scales, extreme sub-block scales and all-min / all-max quants."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "q6_k.npz"))
    raw, want = g["q6_k_bytes"], g["q6_k_gguf_f32"]
    got = ref.dequant(14, raw, raw.shape[0] * 256)
    with np.errstate(over="ignore"):
        assert np.array_equal(got.view(np.uint16), want.astype(np.float16).view(np.uint16))
    # hand-made block: d = 0.5, every sub-block scale 2, ql = 0x21, qh = 0b11100100:
    #   q1 = 1 | 0<<4 = 1, q2 = 1 | 1<<4 = 17, q3 = 2 | 2<<4 = 34, q4 = 2 | 3<<4 = 50  (minus 32)
    b = np.zeros(210, np.uint8)
    b[:128] = 0x21
    b[128:192] = 0b11100100
    b[192:208] = 2
    b[208:210] = np.array([0.5], np.float16).view(np.uint8)
    out = ref.dequant(14, b, 256).astype(np.float32).reshape(2, 4, 32)
    for j, q in enumerate((1, 17, 34, 50)):
        assert np.all(out[:, j, :] == 0.5 * 2 * (q - 32))
    # truncated data leaves zeros, partial element counts stop early
    assert np.all(ref.dequant(14, b[:100], 256) == 0)
    assert ref.dequant(14, b, 40).shape == (40,)


def test_q6_k_linear_is_dequant_plus_f16_linear(ref):
    g = np.load(__import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "q6_k.npz"))
    raw = g["q6_k_bytes"][7:11]                      # 4 ordinary super-blocks -> W [2, 512]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 512)).astype(np.float16)
    w = ref.dequant(14, raw, 1024).reshape(2, 512)
    assert np.array_equal(ref.linear_q(14, raw, 2, 512, x).view(np.uint16), ref.linear_f32acc(x, w).view(np.uint16))


def test_temperature_sample_kats(ref):
    """The reference's sampling tests (src/interpreter/builtin_sampling.rs:555-790), through the oracle."""
    # test_temperature_sample_greedy / _zero_equivalence: T = 0 picks the maximum, whatever the draw
    lg = np.array([1.0, 2.0, 0.5, 3.0, 1.5, 10.0, 2.5, 0.1], np.float16)
    for u in (0.0, 0.3, 0.999):
        assert ref.temperature_sample(lg, 0.0, u) == 5
    # test_softmax_probabilities_sum_to_one / test_exp_numerical_stability: large logits stay finite
    big = np.array([1000.0, 1001.0, 1000.5], np.float16)
    idx, cdf = ref.temperature_sample(big, 1.0, 0.5, return_cdf=True)
    assert np.all(np.isfinite(cdf)) and abs(cdf[-1] - 1.0) < 1e-5 and idx == 1
    # test_temperature_scaling_effects: lower temperature -> more mass on the maximum
    lg4 = np.array([1.0, 2.0, 3.0, 0.5], np.float16)
    mass = []
    for t in (0.5, 1.0, 2.0):
        _, cdf = ref.temperature_sample(lg4, t, 0.0, return_cdf=True)
        p = np.diff(np.concatenate([[0.0], cdf]))
        assert int(np.argmax(p)) == 2
        mass.append(p[2])
    assert mass[0] > mass[1] > mass[2]
    # the draw walks the cumulative sums; u at or above the final sum falls back to the last index
    _, cdf = ref.temperature_sample(lg4, 1.0, 0.0, return_cdf=True)
    assert ref.temperature_sample(lg4, 1.0, 0.0) == 0
    assert ref.temperature_sample(lg4, 1.0, float(cdf[0]) + 1e-4) == 1
    assert ref.temperature_sample(lg4, 1.0, 0.99999994) == 3
    # distribution check against the exact softmax
    rng = np.random.default_rng(3)
    lg = (rng.standard_normal(50) * 2).astype(np.float16)
    cnt = np.bincount([ref.temperature_sample(lg, 0.7, float(u)) for u in rng.random(20000, np.float32)], minlength=50)
    p = np.exp(lg.astype(np.float64) / 0.7)
    p /= p.sum()
    assert np.abs(cnt / 20000 - p).max() < 0.015


def test_rope_table_layouts(ref):
    """rope(x, cos, sin): with one table column per rotary pair the table form equals the
    computed form up to the f16 rounding of the tables; with the reference builtin's own table
    (every frequency stored twice, rows of head_dim) the kernel's pair-indexed read gives pair p
    the frequency p // 2 -- restated as the reference computes it, not corrected."""
    rng = np.random.default_rng(40)
    seq, heads, d = 9, 3, 64
    x = rng.standard_normal((seq, heads, d)).astype(np.float16)
    cos_p, sin_p = ref.precompute_rope_tables(d, 16, 10000.0, paired=True)
    assert cos_p.shape == (16, d // 2)
    y_tab = ref.rope_table(x, cos_p, sin_p)
    y_cmp = ref.rope(x, 0, 10000)
    assert np.max(np.abs(y_tab.astype(np.float32) - y_cmp.astype(np.float32))) < 8e-3   # tables are f16
    cos_r, sin_r = ref.precompute_rope_tables(d, 16, 10000.0)
    assert cos_r.shape == (16, d) and np.array_equal(cos_r[:, 0::2], cos_r[:, 1::2])
    y_ref_layout = ref.rope_table(x, cos_r, sin_r)
    # pair p reads column p of c0 c0 c1 c1 ...: the frequency of pair p // 2
    want = ref.rope_table(x, np.ascontiguousarray(cos_p[:, np.arange(d // 2) // 2]), np.ascontiguousarray(sin_p[:, np.arange(d // 2) // 2]))
    assert np.array_equal(y_ref_layout.view(np.uint16), want.view(np.uint16))
    # position 0 rotates nothing in either layout
    assert np.array_equal(y_tab[0].view(np.uint16), x[0].view(np.uint16))
    assert np.array_equal(y_ref_layout[0].view(np.uint16), x[0].view(np.uint16))
