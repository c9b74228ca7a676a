"""GPU tests of Q6_K tensors: accepted on upload, dequantized on the device into F16 tensors
(what the reference's loader keeps in memory), used by linear() and the runner."""
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
    assert w.type == 1 and w.shape == (3, 1024)                # an F16 tensor from here on
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
