"""ctypes binding of the CPU oracle (``libtlref.so`` built from ``tl_ref.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg.  The product package never imports it.

All f16 tensors are numpy ``float16`` arrays (C-contiguous); quantized weights
are ``uint8`` arrays holding GGUF blocks verbatim.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtlref.so")

GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q6_K = 1, 2, 8, 14


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to it (gcc only)."""
    src = os.path.join(_HERE, "tl_ref.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtlref.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load() -> C.CDLL:
    build()
    lib = C.CDLL(_LIB_PATH)
    u16p, u8p, f32p, i32p = (C.POINTER(C.c_uint16), C.POINTER(C.c_uint8), C.POINTER(C.c_float),
                             C.POINTER(C.c_int32))
    sz = C.c_size_t
    sig = {
        "tlref_f16_to_f32_n": (None, [u16p, f32p, sz]),
        "tlref_f32_to_f16_n": (None, [f32p, u16p, sz]),
        "tlref_dequant_q4_0": (None, [u8p, sz, sz, u16p]),
        "tlref_dequant_q8_0": (sz, [u8p, sz, sz, u16p]),
        "tlref_dequant_q6_k": (sz, [u8p, sz, sz, u16p]),
        "tlref_matmul_f16acc": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int]),
        "tlref_linear_literal": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, u16p]),
        "tlref_linear_f32acc": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "tlref_linear_q_f32acc": (C.c_int, [C.c_int, u8p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "tlref_rms_norm": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_float]),
        "tlref_rope": (None, [u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint, i32p]),
        "tlref_rope_table": (None, [u16p, u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "tlref_sigmoid": (None, [u16p, u16p, sz]),
        "tlref_mul": (None, [u16p, u16p, u16p, sz]),
        "tlref_add": (None, [u16p, u16p, u16p, sz]),
        "tlref_swiglu": (None, [u16p, u16p, u16p, sz]),
        "tlref_softmax": (None, [u16p, u16p, C.c_int, C.c_int, C.c_int]),
        "tlref_embedding": (C.c_int, [u16p, C.c_int, C.c_int, i32p, C.c_int, u16p]),
        "tlref_attention": (None, [u16p, u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_float, C.c_int, C.c_int]),
        "tlref_argmax_last": (C.c_int, [u16p, C.c_int]),
        "tlref_temperature_sample": (C.c_int, [u16p, C.c_int, C.c_float, C.c_float, C.POINTER(C.c_float)]),
        "tlref_num_threads": (C.c_int, []),
        "tlref_set_f16c": (None, [C.c_int]),
        "tlref_uses_f16c": (C.c_int, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _h(a: np.ndarray):
    assert a.dtype == np.float16 and a.flags.c_contiguous, (a.dtype, a.flags.c_contiguous)
    return a.ctypes.data_as(C.POINTER(C.c_uint16))


def _b(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_uint8))


def _f16(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float16)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.float16)
    lib().tlref_f32_to_f16_n(x.ctypes.data_as(C.POINTER(C.c_float)), _h(out), x.size)
    return out


def f16_to_f32(x: np.ndarray) -> np.ndarray:
    x = _f16(x)
    out = np.empty(x.shape, np.float32)
    lib().tlref_f16_to_f32_n(_h(x), out.ctypes.data_as(C.POINTER(C.c_float)), x.size)
    return out


def dequant(qtype: int, data: np.ndarray, n_elem: int) -> np.ndarray:
    """Bit-exact GGUF dequantization to f16 (flat array of n_elem)."""
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    out = np.empty(n_elem, np.float16)
    if qtype == GGML_Q4_0:
        lib().tlref_dequant_q4_0(_b(data), data.size, n_elem, _h(out))
    elif qtype == GGML_Q8_0:
        lib().tlref_dequant_q8_0(_b(data), data.size, n_elem, _h(out))
    elif qtype == GGML_Q6_K:
        lib().tlref_dequant_q6_k(_b(data), data.size, n_elem, _h(out))
    elif qtype == GGML_F16:
        out[:] = data.view(np.float16)[:n_elem]
    else:
        raise ValueError(f"unsupported ggml type {qtype}")
    return out


def matmul_f16acc(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _f16(a), _f16(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float16)
    lib().tlref_matmul_f16acc(_h(a), _h(b), _h(c), m, k, n)
    return c


def linear_literal(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """transpose + f16-accumulating matmul: the reference's CPU linear."""
    x, w = _f16(x), _f16(w)
    m, k = x.shape
    n, k2 = w.shape
    assert k == k2
    y = np.empty((m, n), np.float16)
    scratch = np.empty((k, n), np.float16)
    lib().tlref_linear_literal(_h(x), _h(w), _h(y), m, k, n, _h(scratch))
    return y


def linear_f32acc(x: np.ndarray, w: np.ndarray, threads: int = 0) -> np.ndarray:
    x, w = _f16(x), _f16(w)
    m, k = x.shape
    n, k2 = w.shape
    assert k == k2
    y = np.empty((m, n), np.float16)
    lib().tlref_linear_f32acc(_h(x), _h(w), _h(y), m, k, n, threads)
    return y


def linear_q(qtype: int, wq: np.ndarray, n: int, k: int, x: np.ndarray, threads: int = 0) -> np.ndarray:
    """Parity target for a quantized linear: dequant (bit-exact) + f32-accumulate."""
    x = _f16(x)
    m, k2 = x.shape
    assert k == k2
    wq = np.ascontiguousarray(wq).view(np.uint8).reshape(-1)
    y = np.empty((m, n), np.float16)
    rc = lib().tlref_linear_q_f32acc(qtype, _b(wq), _h(x), _h(y), m, k, n, threads)
    if rc != 0:
        raise ValueError(f"tlref_linear_q_f32acc failed: {rc}")
    return y


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x, w = _f16(x), _f16(w)
    d = x.shape[-1]
    assert w.shape == (d,)
    y = np.empty_like(x)
    lib().tlref_rms_norm(_h(x), _h(w), _h(y), x.size // d, d, eps)
    return y


def rope(x: np.ndarray, pos_offset: int = 0, base: int = 10000, positions=None) -> np.ndarray:
    x = _f16(x)
    assert x.ndim >= 3 and x.shape[-1] % 2 == 0
    heads, d = x.shape[-2], x.shape[-1]
    seq = x.size // (heads * d)
    y = np.empty_like(x)
    pp = None
    if positions is not None:
        positions = np.ascontiguousarray(positions, dtype=np.int32)
        assert positions.size == seq
        pp = positions.ctypes.data_as(C.POINTER(C.c_int32))
    lib().tlref_rope(_h(x), _h(y), seq, heads, d, pos_offset, base, pp)
    return y


def rope_table(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x [seq, heads, d]; cos/sin f16 tables [rows >= seq, cols]: pair p of position s reads
    table[s, p] (cols = d reproduces the reference's call, cols = d/2 is one column per pair)."""
    x, cos, sin = _f16(x), _f16(cos), _f16(sin)
    seq, heads, d = x.shape
    assert cos.shape == sin.shape and cos.shape[0] >= seq and cos.shape[1] >= d // 2
    y = np.empty_like(x)
    lib().tlref_rope_table(_h(x), _h(cos), _h(sin), _h(y), seq, heads, d, cos.shape[1])
    return y


def precompute_rope_tables(head_dim: int, max_seq: int, base: float = 10000.0, paired: bool = False):
    """(cos, sin) f16 tables as the reference's builtin makes them
    (eval_precompute_rope_impl, src/interpreter/builtin_tensor.rs:640-722): f32 frequencies
    1 / base^(i / head_dim) for even i, f32 angle = pos * freq, f32 cos / sin, each value stored
    TWICE in rows of head_dim, then rounded to f16.  paired=True stores each value once
    ([max_seq, head_dim / 2]), the layout the kernel's index arithmetic expects."""
    i = np.arange(0, head_dim, 2, dtype=np.float32)
    theta = (np.float32(1.0) / np.power(np.float32(base), i / np.float32(head_dim))).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * theta[None, :]).astype(np.float32)
    c, s_ = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    if not paired:
        c, s_ = np.repeat(c, 2, axis=1), np.repeat(s_, 2, axis=1)
    return c.astype(np.float16), s_.astype(np.float16)


def sigmoid(x: np.ndarray) -> np.ndarray:
    x = _f16(x)
    y = np.empty_like(x)
    lib().tlref_sigmoid(_h(x), _h(y), x.size)
    return y


def mul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _f16(a), _f16(b)
    assert a.shape == b.shape
    y = np.empty_like(a)
    lib().tlref_mul(_h(a), _h(b), _h(y), a.size)
    return y


def add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _f16(a), _f16(b)
    assert a.shape == b.shape
    y = np.empty_like(a)
    lib().tlref_add(_h(a), _h(b), _h(y), a.size)
    return y


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate, up = _f16(gate), _f16(up)
    assert gate.shape == up.shape
    y = np.empty_like(gate)
    lib().tlref_swiglu(_h(gate), _h(up), _h(y), gate.size)
    return y


def softmax(x: np.ndarray, round_exp: bool = True) -> np.ndarray:
    x = _f16(x)
    last = x.shape[-1]
    y = np.empty_like(x)
    lib().tlref_softmax(_h(x), _h(y), x.size // last, last, int(round_exp))
    return y


def embedding(table: np.ndarray, ids) -> np.ndarray:
    table = _f16(table)
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    vocab, d = table.shape
    y = np.empty((ids.size, d), np.float16)
    rc = lib().tlref_embedding(_h(table), vocab, d, ids.ctypes.data_as(C.POINTER(C.c_int32)), ids.size, _h(y))
    if rc != 0:
        raise IndexError("token id out of range")
    return y


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, q_pos0: int,
              round_exp: bool = True, f16_pv: bool = False) -> np.ndarray:
    """q [I,H,D], k/v [J,Hkv,D] -> [I,H,D]; key j visible to query i iff j <= q_pos0+i."""
    q, k, v = _f16(q), _f16(k), _f16(v)
    I, H, D = q.shape
    J, Hkv, D2 = k.shape
    assert D == D2 and v.shape == k.shape and H % Hkv == 0
    out = np.empty_like(q)
    flags = (1 if round_exp else 0) | (2 if f16_pv else 0)
    lib().tlref_attention(_h(q), _h(k), _h(v), _h(out), I, J, H, Hkv, D, scale, q_pos0, flags)
    return out


def argmax_last(logits: np.ndarray) -> int:
    logits = _f16(logits).reshape(-1)
    return int(lib().tlref_argmax_last(_h(logits), logits.size))


def temperature_sample(logits: np.ndarray, temperature: float, u: float, return_cdf: bool = False):
    """temperature_sample(logits, T) with the uniform draw u passed in; optionally also the running sums."""
    logits = _f16(logits).reshape(-1)
    cdf = np.empty(logits.size, np.float32) if return_cdf else None
    idx = int(lib().tlref_temperature_sample(_h(logits), logits.size, temperature, u,
                                             cdf.ctypes.data_as(C.POINTER(C.c_float)) if return_cdf else None))
    return (idx, cdf) if return_cdf else idx


def num_threads() -> int:
    return int(lib().tlref_num_threads())


def set_f16c(enable: bool) -> None:
    """Allow / forbid the hardware f16 conversions in the literal matmul (bit-identical either way)."""
    lib().tlref_set_f16c(int(enable))


def uses_f16c() -> bool:
    return bool(lib().tlref_uses_f16c())


# --------------------------------------------------------------------------
# LLaMA forward assembled from the primitives above, op for op as the TL
# script debug/chat_demo_with_kvcache.tl does it (prefill :44-88 and the layer
# loop; decode :213-296), with one deliberate difference:
# RoPE takes the true position of each token (the script's decode branch calls
# rope() with its default offset 0).
# --------------------------------------------------------------------------

class RefLlama:
    """weights: dict name -> (ggml_type, raw uint8 bytes, (rows, cols)) for 2-D
    tensors or name -> float16 array for 1-D / f16 tensors, GGUF naming
    (token_embd.weight, blk.N.attn_q.weight, ..., output.weight)."""

    def __init__(self, weights: dict, n_layers: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 eps: float = 1e-5, rope_base: int = 10000, round_exp: bool = True, f16_pv: bool = False):
        self.w = weights
        self.n_layers, self.H, self.Hkv, self.D = n_layers, n_heads, n_kv_heads, head_dim
        self.eps, self.rope_base = eps, rope_base
        self.round_exp, self.f16_pv = round_exp, f16_pv
        self.k_cache = [np.zeros((0, n_kv_heads, head_dim), np.float16) for _ in range(n_layers)]
        self.v_cache = [np.zeros((0, n_kv_heads, head_dim), np.float16) for _ in range(n_layers)]

    def _lin(self, x, name):
        t = self.w[name]
        if isinstance(t, np.ndarray):
            return linear_f32acc(x, t)
        qtype, raw, (n, k) = t
        return linear_q(qtype, raw, n, k, x)

    def _f16w(self, name):
        t = self.w[name]
        if isinstance(t, np.ndarray):
            return t
        qtype, raw, (n, k) = t
        return dequant(qtype, raw, n * k).reshape(n, k)

    def forward(self, ids) -> np.ndarray:
        """Append len(ids) tokens to the cache; return logits [len(ids), vocab]."""
        ids = np.asarray(ids, dtype=np.int32).reshape(-1)
        m = ids.size
        pos0 = self.k_cache[0].shape[0]
        x = embedding(self._f16w("token_embd.weight"), ids)
        scale = 1.0 / float(np.sqrt(self.D))
        for l in range(self.n_layers):
            p = f"blk.{l}."
            xn = rms_norm(x, self.w[p + "attn_norm.weight"], self.eps)
            q = self._lin(xn, p + "attn_q.weight").reshape(m, self.H, self.D)
            k = self._lin(xn, p + "attn_k.weight").reshape(m, self.Hkv, self.D)
            v = self._lin(xn, p + "attn_v.weight").reshape(m, self.Hkv, self.D)
            q = rope(q, pos0, self.rope_base)
            k = rope(k, pos0, self.rope_base)
            self.k_cache[l] = np.concatenate([self.k_cache[l], k], axis=0)
            self.v_cache[l] = np.concatenate([self.v_cache[l], v], axis=0)
            a = attention(q, self.k_cache[l], self.v_cache[l], scale, pos0, self.round_exp, self.f16_pv)
            o = self._lin(a.reshape(m, self.H * self.D), p + "attn_output.weight")
            x1 = add(x, o)
            xn2 = rms_norm(x1, self.w[p + "ffn_norm.weight"], self.eps)
            g = self._lin(xn2, p + "ffn_gate.weight")
            u = self._lin(xn2, p + "ffn_up.weight")
            act = swiglu(g, u)
            dn = self._lin(act, p + "ffn_down.weight")
            x = add(x1, dn)
        xf = rms_norm(x, self.w["output_norm.weight"], self.eps)
        return self._lin(xf, "output.weight")

    def forward_batch(self, ids, caches) -> np.ndarray:
        """One decode step for len(ids) independent sequences: row b is the next token of
        sequence b, whose keys and values live in caches[b] = (k_list, v_list) (one array per
        layer, as k_cache / v_cache above; updated in place).  The row-wise operations run
        on all rows at once, attention runs sequence by sequence -- the same arithmetic as
        len(ids) separate forward() calls.  Returns logits [len(ids), vocab]."""
        ids = np.asarray(ids, dtype=np.int32).reshape(-1)
        B = ids.size
        assert len(caches) == B
        pos = np.array([caches[b][0][0].shape[0] for b in range(B)], np.int32)
        x = embedding(self._f16w("token_embd.weight"), ids)
        scale = 1.0 / float(np.sqrt(self.D))
        for l in range(self.n_layers):
            p = f"blk.{l}."
            xn = rms_norm(x, self.w[p + "attn_norm.weight"], self.eps)
            q = self._lin(xn, p + "attn_q.weight").reshape(B, self.H, self.D)
            k = self._lin(xn, p + "attn_k.weight").reshape(B, self.Hkv, self.D)
            v = self._lin(xn, p + "attn_v.weight").reshape(B, self.Hkv, self.D)
            q = rope(q, 0, self.rope_base, positions=pos)
            k = rope(k, 0, self.rope_base, positions=pos)
            a = np.empty_like(q)
            for b in range(B):
                kl, vl = caches[b]
                kl[l] = np.concatenate([kl[l], k[b:b + 1]], axis=0)
                vl[l] = np.concatenate([vl[l], v[b:b + 1]], axis=0)
                a[b] = attention(q[b:b + 1], kl[l], vl[l], scale, int(pos[b]), self.round_exp, self.f16_pv)[0]
            o = self._lin(a.reshape(B, self.H * self.D), p + "attn_output.weight")
            x1 = add(x, o)
            xn2 = rms_norm(x1, self.w[p + "ffn_norm.weight"], self.eps)
            act = swiglu(self._lin(xn2, p + "ffn_gate.weight"), self._lin(xn2, p + "ffn_up.weight"))
            x = add(x1, self._lin(act, p + "ffn_down.weight"))
        xf = rms_norm(x, self.w["output_norm.weight"], self.eps)
        return self._lin(xf, "output.weight")

    def empty_caches(self, batch: int):
        """Caches for forward_batch: `batch` sequences with no tokens yet."""
        return [([np.zeros((0, self.Hkv, self.D), np.float16) for _ in range(self.n_layers)],
                 [np.zeros((0, self.Hkv, self.D), np.float16) for _ in range(self.n_layers)]) for _ in range(batch)]
