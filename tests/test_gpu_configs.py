"""GPU parity at the sizes the benchmark runs, each against the CPU oracle.

The other GPU test files cover the kernels on small and ragged shapes; this one runs the
measured configurations themselves:

  * the TinyLlama-1.1B shape with a 512-token prompt and 128 greedy decode steps (every one of
    the 129 logit rows is compared);
  * the Llama-2-7B-shape prefill GEMMs at 2048 activation rows, whole and as 8-way
    tensor-parallel shards, on sub-sampled outputs;
  * one Llama-2-70B-shape layer plus an lm_head shard, unsharded through the runner (prefill,
    then decode at batch 1, 8 and 32) and as 8-way shard shapes through the fused linears.

The oracle's 512-token forward costs about a teraflop on the host; its logits are kept in a
git-ignored cache file keyed by the inputs, so only the first run pays for it.
"""
import hashlib
import os

import numpy as np
import pytest

from conftest import ROOT, rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-2      # rel-L2 stated for linears and full-forward logits
TIGHT = 2e-3    # regression alarm for a single linear (observed ~1e-4)
Q4 = 2
CACHE_DIR = os.path.join(ROOT, "baseline", "_ref", "oracle_cache")


def _ref_model(ref, weights, arch):
    w = {}
    for name, (gtype, arr) in weights.items():
        if gtype == 1:
            w[name] = arr.reshape(-1) if name.endswith("norm.weight") else arr
        else:
            w[name] = (gtype, arr, (arr.shape[0], arr.shape[1] * 32))
    return ref.RefLlama(w, arch.n_layers, arch.n_heads, arch.n_kv_heads, arch.head_dim, arch.rms_eps, arch.rope_base)


def _cached(key: str, compute):
    """compute() -> dict of arrays, stored under baseline/_ref/oracle_cache/<key>.npz."""
    path = os.path.join(CACHE_DIR, key + ".npz")
    if os.path.exists(path):
        try:
            with np.load(path) as z:
                return {k: z[k] for k in z.files}
        except Exception:
            pass
    out = compute()
    try:
        os.makedirs(CACHE_DIR, exist_ok=True)
        np.savez(path, **out)
    except OSError:
        pass  # a read-only tree only loses the cache
    return out


def test_tinyllama_512_token_prompt_and_128_greedy_steps(dev, ref):
    """22 layers, d 2048, 32/4 heads, FFN 5632, vocab 32000, Q4_0: a 512-token prompt through the
    tcgen05 GEMM path, then 128 greedy steps through the decode step the benchmark times.  The
    oracle is teacher-forced with the tokens the device produced, so every step's logits are
    compared on identical inputs and one argmax flip cannot cascade."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import TINYLLAMA, Llama, synthetic_host_weights, synthetic_model
    arch, seed, n_prompt, n_steps = TINYLLAMA, 2, 512, 128
    model = synthetic_model(dev, arch, seed=seed)
    llm = Llama(dev, model, arch, max_seq=1024, max_prefill=n_prompt)
    ids = synth.token_ids(seed, "prompt512", n_prompt, arch.vocab)
    first, lg0 = llm.prefill(ids)
    toks, rows = [int(first)], [lg0[0].copy()]
    for _ in range(n_steps):
        nxt, lg = llm.decode([toks[-1]], return_logits=True)
        toks.append(int(nxt[0]))
        rows.append(lg[0].copy())
    got = np.stack(rows)                                   # [129, vocab]: prompt's last row, then each step
    _, pos = llm.read_state(1)
    assert int(pos[0]) == n_prompt + n_steps
    for r in range(len(rows)):                             # greedy: the token fed on is the row's last maximum
        assert toks[r] == ref.argmax_last(got[r]), r

    fed = np.array(toks[:n_steps], np.int32)               # tokens the decode steps consumed
    key = "tinyllama_q4_seed%d_%s" % (seed, hashlib.sha1(ids.tobytes() + fed.tobytes()).hexdigest()[:16])

    def oracle_logits():
        weights = synthetic_host_weights(arch, seed=seed)
        oracle = _ref_model(ref, weights, arch)
        last = oracle.forward(ids)[-1:]
        return {"logits": np.concatenate([last, oracle.forward(fed)])}

    want = _cached(key, oracle_logits)["logits"]
    assert want.shape == got.shape
    errs = [rel_l2(got[r], want[r]) for r in range(got.shape[0])]
    assert max(errs) < TOL, (int(np.argmax(errs)), max(errs))
    # wherever the oracle's top-2 margin exceeds twice the largest deviation, its token is the device's
    for r in range(got.shape[0]):
        w = want[r].astype(np.float32)
        top2 = np.partition(w, -2)[-2:]
        if top2[1] - top2[0] > 2 * float(np.abs(got[r].astype(np.float32) - w).max()):
            assert ref.argmax_last(want[r]) == toks[r], r


def _sample(n, count, rng):
    """Sorted sample of indices that always includes both ends and a tile boundary."""
    fixed = {0, n - 1, min(n - 1, 127), min(n - 1, 128)}
    pick = set(int(i) for i in rng.choice(n, size=min(count, n), replace=False))
    return np.array(sorted(fixed | pick))


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008), (1376, 4096), (4096, 1376)])
def test_llama7b_prefill_gemm_shapes(dev, ref, n, k):
    """Per-layer GEMMs of the Llama-2-7B shape at 2048 activation rows: q/k/v/o 4096x4096, gate/up
    11008x4096, down 4096x11008, and the 8-way shards 1376x4096 (rows) and 4096x1376 (43 blocks of
    every row: the last k-tile holds one zero block).  Outputs are compared with the oracle on a
    sample of weight rows x activation rows."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear
    m = 2048
    raw = synth.blocks(Q4, 3, synth.tensor_id(f"c3_{n}x{k}"), n, k)
    x = synth.activations(3, f"c3x_{k}", (m, k))
    w = QTensor.from_blocks(dev, Q4, n, k, raw)
    l0 = dev.launch_count
    y = linear(dev.tensor(x), w).numpy()
    assert dev.launch_count - l0 == 1 and y.shape == (m, n)
    rng = np.random.default_rng(n * 7 + k)
    ns, ms = _sample(n, 96, rng), _sample(m, 96, rng)
    want = ref.linear_q(Q4, np.ascontiguousarray(raw[ns]), ns.size, k, np.ascontiguousarray(x[ms]))
    got = y[np.ix_(ms, ns)]
    err = rel_l2(got, want)
    assert err < TOL and err < TIGHT, err
    assert np.all(np.isfinite(y.astype(np.float32)))


def _shard_case(dev, ref, m, rng_seed):
    """The seven linears of one Llama-2-70B-shape layer as ONE rank of eight holds them, plus its
    lm_head shard, through the fused entry points the decode step uses."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.api import QTensor, linear, linear_residual, norm_linear_multi, swiglu_gate_up
    d, qd, kvd, ffn, vocab = 8192, 1024, 128, 3584, 4000
    eps = 1e-5
    mk = lambda name, n, k: synth.blocks(Q4, 4, synth.tensor_id(name), n, k, scale_log2=-3)
    raws = {"q": mk("q", qd, d), "k": mk("k", kvd, d), "v": mk("v", kvd, d), "o": mk("o", d, qd),
            "gate": mk("gate", ffn, d), "up": mk("up", ffn, d), "down": mk("down", d, ffn), "lm": mk("lm", vocab, d)}
    W = {k_: QTensor.from_blocks(dev, Q4, r.shape[0], r.shape[1] * 32, r) for k_, r in raws.items()}
    x = synth.activations(rng_seed, f"sx{m}", (m, d))
    nw = synth.norm_weight(rng_seed, "snorm", d)
    xt, nwt = dev.tensor(x), dev.tensor(nw)
    xn = ref.rms_norm(x, nw, eps)
    pos = np.arange(m, dtype=np.int32) * 37 % 2048
    errs = {}
    # norm + q/k/v (+ rope on q and k at per-row positions)
    q, kk, v = norm_linear_multi(xt, [W["q"], W["k"], W["v"]], nwt, eps, rope_heads=[8, 1, 0], positions=pos)
    wq = ref.rope(ref.linear_q(Q4, raws["q"], qd, d, xn).reshape(m, 8, 128), 0, 10000, positions=pos).reshape(m, qd)
    wk = ref.rope(ref.linear_q(Q4, raws["k"], kvd, d, xn).reshape(m, 1, 128), 0, 10000, positions=pos).reshape(m, kvd)
    errs["q"], errs["k"] = rel_l2(q.numpy(), wq), rel_l2(kk.numpy(), wk)
    errs["v"] = rel_l2(v.numpy(), ref.linear_q(Q4, raws["v"], kvd, d, xn))
    # o (K = 1024) and down (K = 3584) with the residual
    a = synth.activations(rng_seed, f"sa{m}", (m, qd))
    errs["o"] = rel_l2(linear_residual(dev.tensor(a), W["o"], xt).numpy(), ref.add(x, ref.linear_q(Q4, raws["o"], d, qd, a)))
    act = ref.swiglu(ref.linear_q(Q4, raws["gate"], ffn, d, xn), ref.linear_q(Q4, raws["up"], ffn, d, xn))
    errs["act"] = rel_l2(swiglu_gate_up(xt, W["gate"], W["up"], nwt, eps).numpy(), act)
    errs["down"] = rel_l2(linear_residual(dev.tensor(act), W["down"], xt).numpy(),
                          ref.add(x, ref.linear_q(Q4, raws["down"], d, ffn, act)))
    lm, = norm_linear_multi(xt, [W["lm"]], nwt, eps)
    errs["lm"] = rel_l2(lm.numpy(), ref.linear_q(Q4, raws["lm"], vocab, d, xn))
    return errs


@pytest.mark.parametrize("m", [1, 8, 32])
def test_llama70b_tp8_shard_linears(dev, ref, m):
    """q 1024x8192, k/v 128x8192, o 8192x1024, gate/up 3584x8192, down 8192x3584, lm_head 4000x8192
    at decode batch 1, 8 and 32."""
    errs = _shard_case(dev, ref, m, 40 + m)
    assert max(errs.values()) < TOL, errs
    assert max(errs.values()) < 3 * TIGHT, errs


def test_llama70b_one_layer_unsharded(dev, ref):
    """One layer of the Llama-2-70B shape (d 8192, 64/8 heads of 128, FFN 28672) and a 4000-row
    lm_head through the runner: a 40-token prompt, then decode at batch 1, 8 and 32 -- K = 8192 and
    28672 in the GEMV, head_dim 128 in the attention."""
    from tensorlogic_b200 import synth
    from tensorlogic_b200.model import Llama, LlamaArch, model_from_host, synthetic_host_weights
    arch = LlamaArch(n_layers=1, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn_dim=28672, vocab=4000)
    weights = synthetic_host_weights(arch, seed=4)
    model = model_from_host(dev, weights)
    oracle = _ref_model(ref, weights, arch)
    llm = Llama(dev, model, arch, max_seq=64, max_batch=32, max_prefill=48)
    ids = synth.token_ids(4, "p70", 40, arch.vocab)
    _, lg = llm.prefill(ids)
    want = oracle.forward(ids)
    assert rel_l2(lg[0], want[-1]) < TOL
    tok = ref.argmax_last(want[-1])
    for _ in range(2):                                     # batch 1, continuing sequence 0
        _, lg = llm.decode([tok], return_logits=True)
        w = oracle.forward([tok])
        assert rel_l2(lg, w) < TOL
        tok = ref.argmax_last(w[0])
    for B in (8, 32):                                      # B fresh sequences, two steps each
        caches = oracle.empty_caches(B)
        step_ids = synth.token_ids(4, f"b{B}", B, arch.vocab)
        llm.set_state(step_ids, [0] * B)
        for step in range(2):
            nxt, lg = llm.decode(step_ids, return_logits=True)
            w = oracle.forward_batch(step_ids, caches)
            errs = [rel_l2(lg[b], w[b]) for b in range(B)]
            assert max(errs) < TOL, (B, step, max(errs))
            step_ids = np.array([ref.argmax_last(w[b]) for b in range(B)], np.int32)


def test_decode_refuses_to_run_past_the_cache(dev):
    """A pre-allocated cache cannot grow like the reference's concatenating one: the step that
    would write row max_seq is refused on the host, before anything is launched."""
    from tensorlogic_b200 import _lib
    from tensorlogic_b200._lib import TensorError
    from tensorlogic_b200.model import Llama, LlamaArch, model_from_host, synthetic_host_weights
    arch = LlamaArch(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=1000)
    model = model_from_host(dev, synthetic_host_weights(arch, seed=8))
    for use_graph in (True, False):
        llm = Llama(dev, model, arch, max_seq=16, max_batch=2, max_prefill=16, use_graph=use_graph)
        llm.set_state([3, 4], [14, 15])                    # sequence 1 sits on the last row
        l0 = dev.launch_count
        llm.decode([3, 4])                                 # writes rows 14 and 15: fine
        assert dev.launch_count > l0
        l1 = dev.launch_count
        with pytest.raises(TensorError) as e:
            llm.decode([5, 6])                             # would write row 16 of sequence 1
        assert e.value.code == _lib.ERR_INDEX and dev.launch_count == l1
        with pytest.raises(TensorError) as e:
            llm.decode_enqueue(2, 1)
        assert e.value.code == _lib.ERR_INDEX and dev.launch_count == l1
        llm.set_state([3], [10])                           # sequence 0 alone has room for 6 more
        llm.decode_enqueue(1, 6)
        with pytest.raises(TensorError):
            llm.decode_enqueue(1, 1)
        dev.synchronize()
    # a prompt that fills the cache exactly leaves no room for a step either
    llm = Llama(dev, model, arch, max_seq=16, max_prefill=16)
    llm.prefill(np.arange(16) % arch.vocab)
    with pytest.raises(TensorError) as e:
        llm.decode(None, batch=1)
    assert e.value.code == _lib.ERR_INDEX
    dev.synchronize()
