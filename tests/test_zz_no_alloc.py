"""The allocation-free decode attention entry point, checked against the regular one.

Some users of this library decode from a place where they must not ask the driver
for device memory: while a CUDA graph is being captured, inside a serving loop that
cannot afford cudaMalloc's device-wide synchronisation, or in a process whose own
allocator has claimed all of HBM.  ``tlc_attention_decode_static`` serves them: same
kernel, but the split-key partials and ticket counters sit in a fixed array inside
the library instead of a cudaMalloc'ed scratch block, and the caller owns q / K / V /
out.  This file is collected last on purpose, so a failure here cannot hide the
results of the other tests in a stop-at-first-failure run.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

TIGHT = 4e-3  # the tolerance the attention tests use against the oracle


def _upload(dev, arr):
    from tensorlogic_b200._lib import check
    t = dev.empty((arr.size * arr.itemsize // 2,))
    check(dev.lib.tlc_upload(dev.handle, t.ptr, arr.ctypes.data, arr.nbytes))
    dev.synchronize()
    return t


def _run_both(dev, B, H, Hkv, D, lens, max_seq, seed):
    """Returns (regular, static) outputs [B, H, D] for one decode query per sequence."""
    from tensorlogic_b200._lib import check
    from tensorlogic_b200.api import KVCache
    rng = np.random.default_rng(seed)
    cache = KVCache(dev, 1, Hkv, D, max_seq=max_seq, max_batch=B)
    kp, vp = C.c_void_p(), C.c_void_p()
    check(dev.lib.tlc_kvcache_layer_ptrs(cache.handle, 0, C.byref(kp), C.byref(vp)))
    row = Hkv * D
    ks, vs = [], []
    for b, n in enumerate(lens):
        k = rng.standard_normal((n, Hkv, D)).astype(np.float16)
        v = rng.standard_normal((n, Hkv, D)).astype(np.float16)
        ks.append(k)
        vs.append(v)
        check(dev.lib.tlc_upload(dev.handle, kp.value + b * max_seq * row * 2, k.ctypes.data, k.nbytes))
        check(dev.lib.tlc_upload(dev.handle, vp.value + b * max_seq * row * 2, v.ctypes.data, v.nbytes))
        dev.synchronize()
    q = rng.standard_normal((B, H, D)).astype(np.float16)
    pos = np.array([n - 1 for n in lens], np.int32)
    qd = dev.tensor(q)
    regular = cache.attention(0, qd, H, batch=B, positions=pos).numpy()
    # the allocation-free entry point: caller-owned buffers, raw pointers, the library's stream
    out = dev.empty((B, H, D))
    pos_d = _upload(dev, pos)
    scale = float(1.0 / np.sqrt(D))
    check(dev.lib.tlc_attention_decode_static(dev.stream, qd.ptr, kp.value, vp.value, out.ptr, B, H, Hkv, D, max_seq,
                                              pos_d.ptr, int(pos.max()) + 1, scale))
    return regular, out.numpy(), cache, (q, ks, vs)


def _oracle(ref, q, ks, vs, D):
    """The CPU oracle's attention, sequence by sequence: q [B, H, D], ks/vs lists of [n, Hkv, D]."""
    scale = float(1.0 / np.sqrt(D))
    return np.stack([ref.attention(q[b:b + 1], ks[b], vs[b], scale, ks[b].shape[0] - 1)[0] for b in range(len(ks))])


def test_static_scratch_attention_matches_regular_twice(dev, ref):
    # first call: TinyLlama-like heads, several key splits
    reg1, st1, _c1, (q1, k1, v1) = _run_both(dev, B=1, H=32, Hkv=4, D=64, lens=[700], max_seq=1024, seed=1)
    assert rel_l2(st1, reg1) < TIGHT
    assert rel_l2(st1, _oracle(ref, q1, k1, v1, 64)) < TIGHT
    # second call straight after, different shape: the array still holds the first call's partials
    reg2, st2, _c2, (q2, k2, v2) = _run_both(dev, B=3, H=8, Hkv=1, D=128, lens=[5, 333, 64], max_seq=512, seed=2)
    assert rel_l2(st2, reg2) < TIGHT
    assert rel_l2(st2, _oracle(ref, q2, k2, v2, 128)) < TIGHT
    # and the first shape again gives the first answer again
    reg3, st3, _c3, _ = _run_both(dev, B=1, H=32, Hkv=4, D=64, lens=[700], max_seq=1024, seed=1)
    assert np.array_equal(st3.view(np.uint16), st1.view(np.uint16))
    assert rel_l2(st3, reg3) < TIGHT


def test_static_scratch_rejects_oversize_and_bad_arguments(dev):
    from tensorlogic_b200 import _lib
    lib = dev.lib
    buf = dev.empty((64,))
    # Rejections must not depend on how many key splits this GPU's SM count leads to: a request
    # that passed the size checks would launch a kernel on these 128-byte dummies.
    # 129 sequences x 8 KV heads = 1032 (sequence, KV head) pairs: over the 1024 built-in tickets
    # on any GPU (that many pairs get one key split each, so the partials check is passed first).
    rc = lib.tlc_attention_decode_static(dev.stream, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 129, 64, 8, 128, 2048,
                                         buf.ptr, 2048, 0.1)
    assert rc == _lib.ERR_BUFFER_EXHAUSTED and b"built-in tickets" in lib.tlc_last_error()
    if dev.sm_count >= 128:
        # 2 sequences x 128 heads x >= 16 key splits x 130 floats > 2 MiB of partials
        # (splits = ceil(2 * SMs / 16) here, so only asserted where that is at least 16)
        rc = lib.tlc_attention_decode_static(dev.stream, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 2, 128, 8, 128, 2048,
                                             buf.ptr, 2048, 0.1)
        assert rc == _lib.ERR_BUFFER_EXHAUSTED and b"built-in scratch" in lib.tlc_last_error()
    rc = lib.tlc_attention_decode_static(dev.stream, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 6, 2, 64, 64, buf.ptr, 8, 0.1)
    assert rc == _lib.ERR_INVALID_OPERATION          # group of 3 query heads per KV head
    rc = lib.tlc_attention_decode_static(dev.stream, buf.ptr, None, buf.ptr, buf.ptr, 1, 4, 2, 64, 64, buf.ptr, 8, 0.1)
    assert rc == _lib.ERR_INVALID_OPERATION          # null pointer
    rc = lib.tlc_attention_decode_static(dev.stream, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 4, 2, 64, 64, buf.ptr, 65, 0.1)
    assert rc == _lib.ERR_INDEX                      # more keys than the cache rows
    dev.synchronize()


def test_static_scratch_cuts_positions_at_max_keys(dev, ref):
    """A position at or beyond max_keys reads no row past max_keys: the keys are cut there and
    the status query says so once.  All buffers are real and large enough for the true position."""
    from tensorlogic_b200._lib import check
    B, H, Hkv, D, max_seq, n = 1, 8, 2, 64, 256, 100
    rng = np.random.default_rng(5)
    k = rng.standard_normal((n, Hkv, D)).astype(np.float16)
    v = rng.standard_normal((n, Hkv, D)).astype(np.float16)
    kc = np.zeros((max_seq, Hkv, D), np.float16)
    vc = np.zeros((max_seq, Hkv, D), np.float16)
    kc[:n], vc[:n] = k, v
    q = rng.standard_normal((B, H, D)).astype(np.float16)
    kd, vd, qd = _upload(dev, kc), _upload(dev, vc), dev.tensor(q)
    pos_d = _upload(dev, np.array([n - 1], np.int32))
    out = dev.empty((B, H, D))
    clamped = C.c_int32(-1)
    check(dev.lib.tlc_attention_decode_static_status(dev.stream, C.byref(clamped)))
    assert clamped.value == 0
    check(dev.lib.tlc_attention_decode_static(dev.stream, qd.ptr, kd.ptr, vd.ptr, out.ptr, B, H, Hkv, D, max_seq,
                                              pos_d.ptr, 64, 0.125))
    check(dev.lib.tlc_attention_decode_static_status(dev.stream, C.byref(clamped)))
    assert clamped.value == 1
    want = ref.attention(q, k[:64], v[:64], 0.125, 63)          # the first 64 keys only
    assert rel_l2(out.numpy(), want) < TIGHT
    check(dev.lib.tlc_attention_decode_static_status(dev.stream, C.byref(clamped)))
    assert clamped.value == 0                                    # the note is read once
