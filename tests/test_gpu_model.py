"""GPU tests of the GGUF loader and of the LLaMA forward pass against the CPU oracle."""
import os

import numpy as np
import pytest

from conftest import rel_l2
from gguf_util import write_gguf

pytestmark = pytest.mark.gpu

TOL = 1e-2  # rel-L2 on logits, the tolerance stated for the full forward


def _small_arch():
    from tensorlogic_b200.model import LlamaArch
    return LlamaArch(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=1000)


def _ref_model(ref, weights, arch):
    w = {}
    for name, (gtype, arr) in weights.items():
        if gtype == 1:
            w[name] = arr.reshape(-1) if name.endswith("norm.weight") else arr
        else:
            w[name] = (gtype, arr, (arr.shape[0], arr.shape[1] * (256 if gtype == 14 else 32)))
    return ref.RefLlama(w, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.head_dim, arch.rms_eps, arch.rope_base)


@pytest.mark.parametrize("alignment", [32, 64])
def test_gguf_round_trip(dev, ref, tmp_path, alignment):
    from tensorlogic_b200.model import load_model, synthetic_host_weights
    arch = _small_arch()
    weights = synthetic_host_weights(arch, seed=3, qtype=2)
    # mix in a Q8_0 and an F32 tensor
    from tensorlogic_b200 import synth
    weights["blk.1.ffn_up.weight"] = (8, synth.blocks(8, 3, 99, arch.ffn_dim, arch.d_model))
    weights["blk.0.attn_norm.weight"] = (0, weights["blk.0.attn_norm.weight"][1].astype(np.float32))
    path = tmp_path / "m.gguf"
    write_gguf(path, weights, arch, alignment=alignment)
    m = load_model(dev, path)
    assert sorted(m.names()) == sorted(weights)
    assert m.meta("llama.block_count") == 2 and m.meta("test.u16") == 513 and m.meta("test.flag") == 1
    assert m.meta("test.note") == "synthetic" and m.meta("test.tokens.length") == 3
    assert m.meta("general.alignment") in (None, alignment) or alignment == 32
    for name, (gtype, arr) in weights.items():
        t = m.get_tensor(name)
        got = t.dequantize().numpy()
        if gtype in (2, 8):
            rows, cols = arr.shape[0], arr.shape[1] * 32
            assert t.shape == (rows, cols) and t.type == gtype
            want = ref.dequant(gtype, arr, rows * cols).reshape(rows, cols)
            assert np.array_equal(t.raw_bytes().reshape(-1), arr.reshape(-1))     # blocks kept verbatim
        else:
            want = arr.astype(np.float16).reshape(got.shape)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), name
    with pytest.raises(Exception) as e:
        m.get_tensor("no.such.tensor")
    assert "not found" in str(e.value)


def test_gguf_errors(dev, tmp_path):
    from tensorlogic_b200.api import TensorError
    from tensorlogic_b200.model import load_model, synthetic_host_weights
    arch = _small_arch()
    weights = {k: v for k, v in synthetic_host_weights(arch, 1).items() if k.startswith(("output", "token"))}
    good = tmp_path / "g.gguf"
    write_gguf(good, weights, arch)
    raw = open(good, "rb").read()
    cases = {"magic": b"GGUX" + raw[4:], "version": raw[:4] + (9).to_bytes(4, "little") + raw[8:],
             "truncated_data": raw[:len(raw) - 1000], "truncated_header": raw[:40]}
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        open(p, "wb").write(data)
        with pytest.raises(TensorError) as e:
            load_model(dev, p)
        assert e.value.kind == "LoadError", name
    with pytest.raises(TensorError) as e:
        load_model(dev, tmp_path / "missing.gguf")
    assert e.value.kind == "LoadError"


def test_small_llama_prefill_and_decode(dev, ref, tmp_path):
    """2-layer model from a GGUF file: all-row prefill logits, then teacher-forced decode steps."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, load_model, synthetic_host_weights
    arch = _small_arch()
    weights = synthetic_host_weights(arch, seed=5)
    path = tmp_path / "small.gguf"
    write_gguf(path, weights, arch)
    model = load_model(dev, path)
    llm = Llama(dev, model, arch, max_seq=128, max_prefill=64, logits_all_rows=True)
    oracle = _ref_model(ref, weights, arch)
    ids = synth.token_ids(5, "prompt", 37, arch.vocab)
    nxt, logits = llm.prefill(ids, all_rows=True)
    want = oracle.forward(ids)
    assert logits.shape == want.shape == (37, arch.vocab)
    assert rel_l2(logits, want) < TOL
    assert rel_l2(logits[-1], want[-1]) < TOL
    tok = ref.argmax_last(want[-1])
    assert nxt == ref.argmax_last(logits[-1])
    for step in range(6):
        got_next, lg = llm.decode([tok], return_logits=True)   # teacher-forced with the oracle's token
        w = oracle.forward([tok])
        assert rel_l2(lg, w) < TOL, step
        assert got_next[0] == ref.argmax_last(lg[0])
        tok = ref.argmax_last(w[0])
    # chunked prefill == one-shot prefill
    llm2 = Llama(dev, model, arch, max_seq=128, max_prefill=64, logits_all_rows=True)
    llm2.prefill(ids[:20], pos0=0)
    _, lg2 = llm2.prefill(ids[20:], pos0=20, all_rows=True)
    assert rel_l2(lg2, want[20:]) < TOL


def test_graph_replay_matches_eager_and_free_running_decode(dev):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, model_from_host, synthetic_host_weights
    arch = _small_arch()
    model = model_from_host(dev, synthetic_host_weights(arch, seed=6))
    ids = synth.token_ids(6, "prompt", 16, arch.vocab)
    outs = []
    for use_graph in (True, False):
        llm = Llama(dev, model, arch, max_seq=96, max_prefill=16, use_graph=use_graph)
        first, _ = llm.prefill(ids)
        toks = [first]
        for _ in range(5):
            nxt, lg = llm.decode(None, batch=1, return_logits=True)
            toks.append(int(nxt[0]))
        outs.append((toks, lg.copy()))
    assert outs[0][0] == outs[1][0]
    assert np.array_equal(outs[0][1].view(np.uint16), outs[1][1].view(np.uint16))
    # free-running device-side loop == stepping through the host
    llm = Llama(dev, model, arch, max_seq=96, max_prefill=16)
    llm.prefill(ids)
    llm.decode_enqueue(1, 5)
    nxt, pos = llm.read_state(1)
    assert int(nxt[0]) == outs[0][0][5] and int(pos[0]) == 16 + 5
    assert llm.launches_per_step == 5 * arch.n_layers + 3


def test_decode_is_the_same_for_every_dependent_launch_setting(dev):
    """When a kernel lets its successor be scheduled changes the timing only: tokens, logits and
    positions are bit-identical with dependent launch off and with each of its trigger points
    (the decode attention reads its position before or after its dependency wait accordingly)."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, model_from_host, synthetic_host_weights
    arch = _small_arch()
    model = model_from_host(dev, synthetic_host_weights(arch, seed=9))
    ids = synth.token_ids(9, "prompt", 70, arch.vocab)  # more than one key tile: the early K/V fetch runs
    outs = []
    try:
        for pdl, mode in ((1, 4), (0, 4), (1, 0), (1, 1), (1, 2), (1, 3)):
            dev.set_option("pdl", pdl)
            dev.set_option("pdl_mode", mode)
            llm = Llama(dev, model, arch, max_seq=160, max_prefill=70)
            first, _ = llm.prefill(ids)
            toks = [first]
            for _ in range(6):
                nxt, lg = llm.decode(None, batch=1, return_logits=True)
                toks.append(int(nxt[0]))
            llm.decode_enqueue(1, 4)
            nxt, pos = llm.read_state(1)
            outs.append((toks, lg.copy(), int(nxt[0]), int(pos[0])))
    finally:
        dev.set_option("pdl", 1)
        dev.set_option("pdl_mode", 4)
    for o in outs[1:]:
        assert o[0] == outs[0][0] and o[2:] == outs[0][2:]
        assert np.array_equal(o[1].view(np.uint16), outs[0][1].view(np.uint16))
    assert outs[0][3] == 70 + 6 + 4
    with pytest.raises(Exception):
        dev.set_option("pdl_mode", 5)


def test_step_kernel_against_the_kernel_by_kernel_path(dev, ref):
    """Option step_kernel=1 runs single-sequence greedy decode as one persistent kernel per step;
    the default is the five-launches-per-layer path.  Same tokens, logits within the forward tolerance of
    each other and of the oracle (the attention's key splits differ, so not bit for bit), for
    Q4_0 and Q8_0, head_dim 64 and 128, in-kernel multi-step runs included."""
    from tensorlogic_b200 import _lib, synth
    from tensorlogic_b200.model import Llama, LlamaArch, model_from_host, synthetic_host_weights
    cases = [(_small_arch(), _lib.TYPE_Q4_0), (_small_arch(), _lib.TYPE_Q8_0),
             (LlamaArch(n_layers=3, d_model=512, n_heads=4, n_kv_heads=1, head_dim=128, ffn_dim=1376, vocab=515), _lib.TYPE_Q4_0)]
    dev.set_option("wait_limit_ms", 300)       # a lost barrier arrival shows up as TIMEOUT at once
    for arch, qtype in cases:
        weights = synthetic_host_weights(arch, seed=31, qtype=qtype)
        model = model_from_host(dev, weights)
        ids = synth.token_ids(31, "prompt", 70, arch.vocab)     # more than one 64-key tile
        runs = {}
        for mode in (1, 0):
            dev.set_option("step_kernel", mode)
            try:
                llm = Llama(dev, model, arch, max_seq=128, max_prefill=80)
                first, _ = llm.prefill(ids)
                toks, rows = [int(first)], []
                for _ in range(6):
                    nxt, lg = llm.decode([toks[-1]], return_logits=True)
                    toks.append(int(nxt[0]))
                    rows.append(lg[0].copy())
                nxt, _ = llm.decode(None, batch=1)              # continue with the device's own token
                toks.append(int(nxt[0]))
                llm.decode_enqueue(1, 9)                        # nine steps inside one launch
                last, pos = llm.read_state(1)
                runs[mode] = (toks, np.stack(rows), int(last[0]), int(pos[0]), llm.launches_per_step)
            finally:
                dev.set_option("step_kernel", 0)
        (t1, r1, last1, pos1, n1), (t0, r0, last0, pos0, n0) = runs[1], runs[0]
        assert n1 == 1 and n0 == 5 * arch.n_layers + 3
        assert t1 == t0 and last1 == last0 and pos1 == pos0 == 70 + 7 + 9
        assert rel_l2(r1, r0) < 2e-3
        oracle = _ref_model(ref, weights, arch)
        oracle.forward(ids)
        want = oracle.forward(np.array(t1[:6], np.int32))
        assert rel_l2(r1, want) < TOL
    # per-phase device timing of the persistent step: stamps grow along the step and across steps
    dev.set_option("step_kernel", 1)
    try:
        llm = Llama(dev, model, arch, max_seq=128, max_prefill=80)
        llm.prefill(ids)
        tr = llm.step_trace(2).astype(np.int64)
        assert tr.shape == (2, arch.n_layers * 5 + 2, 3)
        ends = tr[:, :, 2].reshape(-1)
        assert np.all(ends > 0) and np.all(np.diff(ends) >= 0)
        assert int(llm.read_state(1)[1][0]) == 70 + 2
    finally:
        dev.set_option("step_kernel", 0)
    with pytest.raises(Exception):
        llm.step_trace(1)                                   # not on the persistent kernel: refused
    dev.set_option("wait_limit_ms", 2000)


def test_batched_decode_matches_single(dev):
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, model_from_host, synthetic_host_weights
    arch = _small_arch()
    model = model_from_host(dev, synthetic_host_weights(arch, seed=7))
    B = 3
    prompts = [synth.token_ids(7, f"p{b}", 5 + 4 * b, arch.vocab) for b in range(B)]
    singles = []
    for b in range(B):
        llm = Llama(dev, model, arch, max_seq=64, max_prefill=32)
        first, _ = llm.prefill(prompts[b])
        _, lg = llm.decode([first], return_logits=True)
        singles.append((first, lg[0].copy()))
    # the batched runner: fill each sequence's cache slot by decoding its prompt token by token
    llm = Llama(dev, model, arch, max_seq=64, max_batch=B, max_prefill=32)
    maxlen = max(len(p) for p in prompts)
    for t in range(maxlen):
        # sequences whose prompt is exhausted re-feed their last token at the same position (idempotent)
        ids = [int(p[min(t, len(p) - 1)]) for p in prompts]
        pos = [min(t, len(p) - 1) for p in prompts]
        llm.set_state(ids, pos)
        llm.decode(None, batch=B)
    llm.set_state([s[0] for s in singles], [len(p) for p in prompts])
    _, lg = llm.decode(None, batch=B, return_logits=True)
    for b in range(B):
        assert rel_l2(lg[b], singles[b][1]) < 2e-3, b


def test_tinyllama_shape_step(dev, ref):
    """Full TinyLlama-1.1B architecture (22 layers, Q4_0): short prompt + one decode step vs the oracle."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import TINYLLAMA, Llama, synthetic_host_weights, synthetic_model
    arch = TINYLLAMA
    model = synthetic_model(dev, arch, seed=2)          # quantized weights generated on the device
    weights = synthetic_host_weights(arch, seed=2)      # the same bytes on the host for the oracle
    llm = Llama(dev, model, arch, max_seq=64, max_prefill=16)
    oracle = _ref_model(ref, weights, arch)
    ids = synth.token_ids(2, "prompt", 6, arch.vocab)
    nxt, logits = llm.prefill(ids)
    want = oracle.forward(ids)
    assert rel_l2(logits[0], want[-1]) < TOL
    tok = ref.argmax_last(want[-1])
    _, lg = llm.decode([tok], return_logits=True)
    assert rel_l2(lg, oracle.forward([tok])) < TOL


def test_temperature_sample_builtin(dev, ref):
    """temperature_sample on the device == the oracle's restatement, draw by draw."""
    from tensorlogic_b200.api import temperature_sample
    rng = np.random.default_rng(21)
    for vocab, rows in ((8, 3), (1000, 4), (32000, 2), (4099, 5)):
        lg = (rng.standard_normal((rows, vocab)) * 3).astype(np.float16)
        t = dev.tensor(lg)
        assert list(temperature_sample(t, 0.0)) == [ref.argmax_last(lg[r]) for r in range(rows)]
        for temp in (0.5, 1.0, 1.7):
            us = rng.random(rows, np.float32)
            got = temperature_sample(t, temp, us)
            for r in range(rows):
                want, cdf = ref.temperature_sample(lg[r], temp, float(us[r]), return_cdf=True)
                if int(got[r]) != want:
                    # only a draw that sits on a boundary of the cumulative sums may resolve differently
                    # (the device forms the sums in parallel)
                    lo, hi = sorted((int(got[r]), want))
                    assert hi - lo == 1 and abs(float(cdf[lo]) - float(us[r])) < 2e-6, (vocab, temp, r)
    # the last index when the draw is not below any running sum
    lg = np.array([[0.0, 0.0, 0.0, 0.0]], np.float16)
    assert temperature_sample(dev.tensor(lg), 1.0, [0.99999994])[0] == 3
    assert temperature_sample(dev.tensor(lg), 1.0, [0.0])[0] == 0


def test_runner_temperature_sampling_is_reproducible(dev, ref):
    """Decode with temperature: tokens follow the oracle given the same uniform draws; same seed, same text."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, model_from_host, synthetic_host_weights
    arch = _small_arch()
    weights = synthetic_host_weights(arch, seed=12)
    model = model_from_host(dev, weights)
    ids = synth.token_ids(12, "prompt", 9, arch.vocab)
    runs = []
    for seed in (5, 5, 6):
        llm = Llama(dev, model, arch, max_seq=64, max_prefill=16)
        llm.set_sampling(0.9, seed)
        tok, logits = llm.prefill(ids)
        # prefill samples from the last prompt row with the draw of position len(ids) - 1 ... the runner
        # keys draws by the position of the token fed to the step; prefill feeds position len(ids) - 1 last
        toks = [tok]
        pos = len(ids)
        for _ in range(6):
            nxt, lg = llm.decode(None, return_logits=True)
            u = llm.sample_uniform(seed, pos)
            want, cdf = ref.temperature_sample(lg[0], 0.9, u, return_cdf=True)
            if int(nxt[0]) != want:
                lo, hi = sorted((int(nxt[0]), want))
                assert hi - lo == 1 and abs(float(cdf[lo]) - u) < 2e-6
            toks.append(int(nxt[0]))
            pos += 1
        runs.append(toks)
    assert runs[0] == runs[1]
    assert runs[0] != runs[2]
    # greedy again after switching back
    llm.set_sampling(0.0)


def test_weight_cache_lru(dev, ref, tmp_path):
    """GGUFWeightCache: lazy upload, LRU eviction by tensor count, hit / miss accounting, errors."""
    from tensorlogic_b200 import _lib
    from tensorlogic_b200.api import TensorError, linear
    from tensorlogic_b200.model import WeightCache, synthetic_host_weights
    arch = _small_arch()
    weights = synthetic_host_weights(arch, seed=15)
    path = tmp_path / "cache.gguf"
    write_gguf(path, weights, arch)
    cache = WeightCache(dev, path, 2)
    assert cache.contains("blk.0.attn_q.weight") and not cache.contains("nope.weight")
    names = ["blk.0.attn_q.weight", "blk.0.ffn_down.weight", "blk.1.attn_k.weight"]
    x = None
    for name in names[:2]:
        w = cache.get_weight(name)
        gtype, raw = weights[name]
        n, k = raw.shape[0], raw.shape[1] * 32
        assert w.type == gtype and w.shape == (n, k)
        assert np.array_equal(w.dequantize().numpy().view(np.uint16), ref.dequant(gtype, raw, n * k).reshape(n, k).view(np.uint16))
        x = synth_x = np.random.default_rng(1).standard_normal((2, k)).astype(np.float16)
        assert rel_l2(linear(dev.tensor(synth_x), w).numpy(), ref.linear_q(gtype, raw, n, k, synth_x)) < 2e-3
    assert cache.stats() == {"len": 2, "capacity": 2, "hits": 0, "misses": 2, "evictions": 0}
    cache.get_weight(names[0])                                   # hit: q becomes the most recent
    cache.get_weight(names[2])                                   # miss: evicts ffn_down, the least recent
    st = cache.stats()
    assert (st["len"], st["hits"], st["misses"], st["evictions"]) == (2, 1, 3, 1)
    cache.get_weight(names[0])                                   # still resident
    assert cache.stats()["hits"] == 2
    cache.get_weight(names[1])                                   # reloaded
    assert cache.stats()["misses"] == 4
    with pytest.raises(TensorError) as e:
        cache.get_weight("blk.9.attn_q.weight")
    assert e.value.code == _lib.ERR_LOAD and "Weight not found" in str(e.value)
    cache.clear()
    assert cache.stats()["len"] == 0
    with pytest.raises(TensorError):
        WeightCache(dev, path, 0)
    with pytest.raises(TensorError):
        WeightCache(dev, tmp_path / "missing.gguf", 2)
    cache.close()
