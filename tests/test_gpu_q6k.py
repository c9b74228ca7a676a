"""GPU tests of Q6_K tensors: kept quantized in HBM (210-byte super-blocks padded to 224), dequantized
bit-exactly on demand, used by linear() through a fused kernel and by the runner; column shards
and option q6k_resident = 0 take the f16 expansion the reference's loader keeps in memory."""
import os

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

Q4, Q6K = 2, 14
HERE = os.path.dirname(__file__)


def _q6k_blocks(rng, rows, cols, d_lo=2e-4, d_hi=2e-3):
    """Random Q6_K super-blocks [rows, cols/256, 210] with sane scales."""
    nsb = cols // 256
    b = rng.integers(0, 256, (rows, nsb, 210), dtype=np.uint8)
    b[:, :, 192:208] = rng.integers(-60, 61, (rows, nsb, 16), dtype=np.int8).view(np.uint8)
    d = rng.uniform(d_lo, d_hi, (rows, nsb)).astype(np.float16)
    b[:, :, 208:210] = d.view(np.uint8).reshape(rows, nsb, 2)
    return b


def test_q6_k_upload_is_bit_exact(dev, ref):
    from tensorlogic_b200.api import QTensor
    g = np.load(os.path.join(HERE, "golden", "q6_k.npz"))
    raw = g["q6_k_bytes"]                                      # 12 super-blocks -> W [3, 1024]
    w = QTensor.from_blocks(dev, Q6K, 3, 1024, raw)
    assert w.type == Q6K and w.shape == (3, 1024)              # stays quantized in HBM
    assert np.array_equal(w.raw_bytes().reshape(-1), np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    got = w.dequantize().numpy()
    want = ref.dequant(Q6K, raw, 3072).reshape(3, 1024)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    with np.errstate(over="ignore"):
        assert np.array_equal(got.view(np.uint16), g["q6_k_gguf_f32"].astype(np.float16).reshape(3, 1024).view(np.uint16))


def test_q6_k_linear_and_shards(dev, ref):
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.api import QTensor, linear
    rng = np.random.default_rng(3)
    n, k, m = 96, 768, 5
    raw = _q6k_blocks(rng, n, k)
    x = rng.standard_normal((m, k)).astype(np.float16)
    want = ref.linear_q(Q6K, raw, n, k, x)
    y = linear(dev.tensor(x), QTensor.from_blocks(dev, Q6K, n, k, raw)).numpy()
    assert rel_l2(y, want) < 2e-3
    dense = ref.dequant(Q6K, raw, n * k).reshape(n, k)
    for rank in range(2):                                      # row and column shards are slices of the dense tensor
        wr = QTensor.from_blocks(dev, Q6K, n, k, raw, rank, 2, _lib.SPLIT_ROWS).dequantize().numpy()
        assert np.array_equal(wr.view(np.uint16), dense[rank * 48:(rank + 1) * 48].view(np.uint16))
        wc = QTensor.from_blocks(dev, Q6K, n, k, raw, rank, 2, _lib.SPLIT_COLS).dequantize().numpy()
        assert np.array_equal(wc.view(np.uint16), np.ascontiguousarray(dense[:, rank * 384:(rank + 1) * 384]).view(np.uint16))


def test_q6_k_errors(dev):
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.api import QTensor, TensorError
    with pytest.raises(TensorError) as e:
        QTensor.from_blocks(dev, Q6K, 2, 128, np.zeros(210, np.uint8))      # not a multiple of 256
    assert e.value.code == _lib.ERR_LOAD
    with pytest.raises(TensorError) as e:
        QTensor.from_blocks(dev, Q6K, 2, 256, np.zeros(210, np.uint8))      # one super-block short
    assert e.value.code == _lib.ERR_LOAD


def test_real_file_layout_q6_k_head_and_q4_0_embeddings(dev, ref, tmp_path):
    """The tensor types of a stock Q4_0 GGUF: token_embd Q4_0, output.weight Q6_K, the rest Q4_0."""
    from gguf_util import write_gguf
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, LlamaArch, load_model, synthetic_host_weights
    from test_gpu_model import _ref_model
    arch = LlamaArch(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=1000)
    weights = synthetic_host_weights(arch, seed=9)
    rng = np.random.default_rng(9)
    weights["output.weight"] = (Q6K, _q6k_blocks(rng, arch.vocab, arch.d_model))
    weights["token_embd.weight"] = (Q4, synth.blocks(Q4, 9, synth.tensor_id("emb"), arch.vocab, arch.d_model))
    path = tmp_path / "stock.gguf"
    write_gguf(path, weights, arch)
    model = load_model(dev, path)
    llm = Llama(dev, model, arch, max_seq=64, max_prefill=32, logits_all_rows=True)
    ids = synth.token_ids(9, "prompt", 12, arch.vocab)
    _, logits = llm.prefill(ids, all_rows=True)
    # oracle: the same file contents, embeddings dequantized the way the reference's loader would
    ow = dict(weights)
    emb = ref.dequant(Q4, weights["token_embd.weight"][1], arch.vocab * arch.d_model).reshape(arch.vocab, arch.d_model)
    ow["token_embd.weight"] = (1, emb)
    want = _ref_model(ref, ow, arch).forward(ids)
    assert rel_l2(logits, want) < 1e-2


@pytest.mark.parametrize("n,k", [(96, 768), (1000, 2048), (33, 256), (257, 4096)])
def test_q6_k_fused_linear(dev, ref, n, k):
    """linear() on resident Q6_K against the oracle (dequantize as the loader does, f32 sums) for
    1 .. 19 activation rows, with bias, with the fused residual and RMSNorm entry points, and
    against the f16 expansion (option q6k_resident = 0)."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, linear_residual, norm_linear_multi
    rng = np.random.default_rng(n + k)
    raw = _q6k_blocks(rng, n, k)
    w = QTensor.from_blocks(dev, Q6K, n, k, raw)
    assert w.type == Q6K
    dev.set_option("q6k_resident", 0)
    try:
        w16 = QTensor.from_blocks(dev, Q6K, n, k, raw)
    finally:
        dev.set_option("q6k_resident", 1)
    assert w16.type == 1
    for m in (1, 2, 5, 8, 19):
        x = rng.standard_normal((m, k)).astype(np.float16)
        want = ref.linear_q(Q6K, raw, n, k, x)
        l0 = dev.launch_count
        y = linear(dev.tensor(x), w).numpy()
        assert dev.launch_count - l0 == (m + 7) // 8
        assert y.shape == (m, n) and rel_l2(y, want) < 2e-3, m
        assert rel_l2(y, linear(dev.tensor(x), w16).numpy()) < 1e-3
    x = rng.standard_normal((3, k)).astype(np.float16)
    bias = rng.standard_normal(n).astype(np.float16)
    want = ref.add(ref.linear_q(Q6K, raw, n, k, x), np.broadcast_to(bias, (3, n)))
    assert rel_l2(linear(dev.tensor(x), w, dev.tensor(bias)).numpy(), want) < 2e-3
    res = rng.standard_normal((3, n)).astype(np.float16)
    want = ref.add(res, ref.linear_q(Q6K, raw, n, k, x))
    assert rel_l2(linear_residual(dev.tensor(x), w, dev.tensor(res)).numpy(), want) < 2e-3
    nw = synth.norm_weight(3, "q6norm", k)
    (got,) = norm_linear_multi(dev.tensor(x), [w], dev.tensor(nw), 1e-5)
    assert rel_l2(got.numpy(), ref.linear_q(Q6K, raw, n, k, ref.rms_norm(x, nw, 1e-5))) < 2e-3
