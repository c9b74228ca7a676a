"""Host-side mirror of TensorLogic's builtin operator surface over libtlcuda.

Same names, argument meaning, defaults and error behaviour as the interpreter
builtins of the TensorLogic project:

    linear(x, W[, bias])      src/interpreter/builtin_math.rs:76-199
    rms_norm(x, w[, eps])     src/interpreter/builtin_nn.rs:44-151   (default eps 1e-6)
    rope(x[, position_offset]) src/interpreter/builtin_tensor.rs:514-567
    sigmoid(x)                src/interpreter/builtin_math.rs:203-230
    softmax(x[, dim])         src/interpreter/builtin_sampling.rs:25-58 (dim is ignored upstream too)
    embedding(table, ids)     src/interpreter/builtin_nn.rs:627-909
    mul / add                 src/ops/elementwise.rs:232-330, :48-140

Tensors are f16 device buffers handed out by the context's size-class pool;
weights are ``QTensor`` objects that keep their GGUF blocks in HBM.  Everything
runs through the C ABI of include/tlcuda.h; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import TensorError, check

__all__ = ["Device", "Tensor", "QTensor", "TensorError", "linear", "rms_norm", "rope", "sigmoid", "mul", "add",
           "silu", "swiglu", "softmax", "embedding", "norm_linear_multi", "swiglu_gate_up", "linear_residual"]


class Device:
    """One CUDA context + stream + buffer pool (MetalDevice, src/device/metal_device.rs)."""

    def __init__(self, ordinal: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        check(self.lib.tlc_init(ordinal, C.byref(h)))
        self.handle = h
        self.ordinal = ordinal

    def set_option(self, name: str, value: int) -> None:
        """Runtime switch by name (tlc_set_option): "gemm_min_m", "pdl", "pdl_mode"."""
        check(self.lib.tlc_set_option(self.handle, name.encode(), int(value)))

    def close(self) -> None:
        if self.handle:
            self.lib.tlc_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def name(self) -> str:
        buf = C.create_string_buffer(256)
        check(self.lib.tlc_device_name(self.handle, buf, 256))
        return buf.value.decode()

    @property
    def sm_count(self) -> int:
        n = C.c_int32()
        check(self.lib.tlc_sm_count(self.handle, C.byref(n)))
        return n.value

    @property
    def stream(self) -> int:
        return self.lib.tlc_stream(self.handle) or 0

    @property
    def launch_count(self) -> int:
        return int(self.lib.tlc_launch_count(self.handle))

    def perf_report(self, reset: bool = False) -> dict[str, tuple[int, float]]:
        """Per-op totals of the "perf" option (the reference's TL_PERF): {op: (calls, total ms)}."""
        need = C.c_size_t()
        check(self.lib.tlc_perf_report(self.handle, None, 0, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value + 1)
        check(self.lib.tlc_perf_report(self.handle, buf, len(buf), 1 if reset else 0, None))
        out = {}
        for line in buf.value.decode().splitlines():
            name, calls, ms = line.rsplit(" ", 2)
            out[name] = (int(calls), float(ms))
        return out

    def mem_info(self) -> tuple[int, int]:
        f, t = C.c_size_t(), C.c_size_t()
        check(self.lib.tlc_mem_info(self.handle, C.byref(f), C.byref(t)))
        return f.value, t.value

    def synchronize(self) -> None:
        check(self.lib.tlc_synchronize(self.handle))

    def pool_stats(self) -> dict:
        s = _lib.PoolStats()
        check(self.lib.tlc_pool_stats_get(self.handle, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in s._fields_}

    def pool_trim(self, max_idle_bytes: int = 0) -> None:
        check(self.lib.tlc_pool_trim(self.handle, max_idle_bytes))

    # -- tensors ---------------------------------------------------------
    def empty(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self, tuple(int(s) for s in shape))

    def tensor(self, array) -> "Tensor":
        """Upload a host array as an f16 tensor (Tensor::from_vec_gpu)."""
        a = np.ascontiguousarray(array, dtype=np.float16)
        t = Tensor(self, a.shape)
        if a.size:
            check(self.lib.tlc_upload(self.handle, t.ptr, a.ctypes.data, a.nbytes))
            self.synchronize()  # `a` may be a temporary
        return t


class Tensor:
    """f16 tensor on the device (Tensor<f16> with a pooled MetalBuffer upstream)."""

    def __init__(self, dev: Device, shape: tuple):
        self.dev = dev
        self.shape = tuple(shape)
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1
        h = C.c_void_p()
        check(dev.lib.tlc_alloc(dev.handle, max(self.size, 1) * 2, C.byref(h)))
        self._buf = h
        self.ptr = dev.lib.tlc_buf_ptr(h)

    def __del__(self):
        try:
            if self._buf and self.dev.handle:
                self.dev.lib.tlc_free(self._buf)
            self._buf = None
        except Exception:
            pass

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def numpy(self) -> np.ndarray:
        """sync_and_read (src/tensor/tensor_io.rs:103-135)."""
        out = np.empty(self.shape, np.float16)
        if self.size:
            check(self.dev.lib.tlc_download(self.dev.handle, out.ctypes.data, self.ptr, out.nbytes))
        return out

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        if int(np.prod(shape)) != self.size:
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"expected {self.size} elements, got shape {shape}")
        v = Tensor.__new__(Tensor)
        v.dev, v.shape, v.size, v.ptr = self.dev, shape, self.size, self.ptr
        v._buf = None
        v._base = self  # keeps the storage alive
        return v


class QTensor:
    """A weight [n_rows, n_cols] resident in HBM as GGUF blocks (or f16)."""

    def __init__(self, dev: Device, handle: C.c_void_p):
        self.dev = dev
        self.handle = handle
        t, r, c, pitch, p = C.c_int32(), C.c_int64(), C.c_int64(), C.c_size_t(), C.c_void_p()
        check(dev.lib.tlc_qtensor_info(handle, C.byref(t), C.byref(r), C.byref(c), C.byref(pitch), C.byref(p)))
        self.type, self.shape, self.row_pitch, self.ptr = t.value, (r.value, c.value), pitch.value, p.value

    @classmethod
    def from_blocks(cls, dev: Device, qtype: int, n_rows: int, n_cols: int, data, tp_rank: int = 0,
                    tp_size: int = 1, split: int = _lib.SPLIT_NONE) -> "QTensor":
        raw = np.ascontiguousarray(data)
        raw = raw.view(np.uint8).reshape(-1)
        h = C.c_void_p()
        check(dev.lib.tlc_qtensor_create(dev.handle, qtype, n_rows, n_cols, raw.ctypes.data, raw.nbytes, tp_rank,
                                         tp_size, split, C.byref(h)))
        return cls(dev, h)

    @classmethod
    def synthetic(cls, dev: Device, qtype: int, n_rows: int, n_cols: int, seed: int, tensor_id: int,
                  tp_rank: int = 0, tp_size: int = 1, split: int = _lib.SPLIT_NONE, scale_log2: int = 0) -> "QTensor":
        h = C.c_void_p()
        check(dev.lib.tlc_qtensor_create_synthetic(dev.handle, qtype, n_rows, n_cols, seed, tensor_id, scale_log2,
                                                   tp_rank, tp_size, split, C.byref(h)))
        return cls(dev, h)

    @classmethod
    def normal_f16(cls, dev: Device, n_rows: int, n_cols: int, seed: int, tensor_id: int, mean: float = 0.0,
                   std: float = 1.0) -> "QTensor":
        """f16 tensor filled on the device with N(mean, std) (large benchmark tensors only)."""
        h = C.c_void_p()
        check(dev.lib.tlc_qtensor_create_normal_f16(dev.handle, n_rows, n_cols, seed, tensor_id, mean, std, C.byref(h)))
        return cls(dev, h)

    def __del__(self):
        try:
            if self.handle and self.dev.handle:
                self.dev.lib.tlc_qtensor_destroy(self.handle)
            self.handle = None
        except Exception:
            pass

    def dequantize(self) -> Tensor:
        out = self.dev.empty(self.shape)
        check(self.dev.lib.tlc_dequant(self.dev.handle, self.handle, out.ptr))
        return out

    def raw_bytes(self) -> np.ndarray:
        """The shard's GGUF blocks (or f16 rows) in the file's order: uint8 [n_rows, bytes per row]."""
        per_row = {_lib.TYPE_Q4_0: 18, _lib.TYPE_Q8_0: 34}.get(self.type)
        row_bytes = self.shape[1] // 32 * per_row if per_row else self.shape[1] * 2
        if self.type == 14:                                   # Q6_K: 210-byte super-blocks of 256 values
            row_bytes = self.shape[1] // 256 * 210
        stage = self.dev.empty((self.shape[0] * row_bytes // 2,))
        check(self.dev.lib.tlc_qtensor_blocks(self.dev.handle, self.handle, stage.ptr))
        out = np.empty((self.shape[0], row_bytes), np.uint8)
        check(self.dev.lib.tlc_download(self.dev.handle, out.ctypes.data, stage.ptr, out.nbytes))
        return out


# ---------------------------------------------------------------------------
# builtins
# ---------------------------------------------------------------------------

def _rows_cols(x: Tensor) -> tuple[int, int]:
    if x.ndim != 2:
        raise TensorError(_lib.ERR_INVALID_OPERATION, "matmul_transposed_b requires 2D tensors")
    return x.shape


def linear(x: Tensor, weight: QTensor, bias: Optional[Tensor] = None) -> Tensor:
    """linear(x, weight[, bias]) = x @ weight.T (+ bias)."""
    if not isinstance(x, Tensor) or not isinstance(weight, QTensor):
        raise TypeError("linear() requires a tensor and a weight")
    if bias is not None and not isinstance(bias, Tensor):
        raise TypeError("linear() bias must be f16 tensor")
    m, k = _rows_cols(x)
    y = x.dev.empty((m, weight.shape[0]))
    check(x.dev.lib.tlc_linear(x.dev.handle, weight.handle, x.ptr, m, k, y.ptr, bias.ptr if bias is not None else None))
    return y


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    d = weight.size
    if x.shape[-1] != d:
        raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"rms_norm: last dim {x.shape[-1]} != weight {d}")
    y = x.dev.empty(x.shape)
    check(x.dev.lib.tlc_rms_norm(x.dev.handle, x.ptr, weight.ptr, y.ptr, x.size // d, d, eps))
    return y


def rope(x: Tensor, position_offset: int = 0, positions: Optional[np.ndarray] = None, base: int = 10000) -> Tensor:
    """rope(x[, position_offset]); x is [..., seq, heads, head_dim]."""
    if x.ndim < 3:
        raise TensorError(_lib.ERR_INVALID_OPERATION, "RoPE requires at least 3D tensor [seq, heads, head_dim]")
    heads, d = x.shape[-2], x.shape[-1]
    seq = x.size // (heads * d)
    y = x.dev.empty(x.shape)
    pos_t = None
    pos_ptr = None
    if positions is not None:
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        if pos.size != seq:
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"rope: {pos.size} positions for {seq} rows")
        pos_t = _upload_i32(x.dev, pos)
        pos_ptr = pos_t.ptr
    check(x.dev.lib.tlc_rope(x.dev.handle, x.ptr, y.ptr, seq, heads, d, position_offset, base, pos_ptr))
    return y


def rope_table(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """rope(x, cos, sin): the rope builtin's arm with precomputed f16 tables
    (src/interpreter/builtin_tensor.rs:634-722 -> Tensor::rope_candle, src/ops/rope.rs:18-65).

    x is [seq, heads, head_dim]; cos / sin are [rows >= seq, cols].  cols = head_dim / 2 is one
    column per rotary pair (the layout the kernel indexes) and equals rope(x); cols = head_dim
    is the reference builtin's table (every frequency stored twice), whose result -- pair p gets
    frequency p // 2 -- is reproduced as the reference computes it.  (Upstream, rope() with three
    arguments never reaches this op: eval_rope_candle_style returns a sine table instead.)"""
    if x.ndim != 3:
        raise TensorError(_lib.ERR_INVALID_OPERATION,
                          f"rope_candle requires 3D tensor [seq_len, n_heads, head_dim], got {x.ndim}D")
    if cos.ndim != 2 or sin.ndim != 2:
        raise TensorError(_lib.ERR_INVALID_OPERATION,
                          f"cos/sin must be 2D [max_seq_len, head_dim], got cos: {cos.ndim}D, sin: {sin.ndim}D")
    seq, heads, d = x.shape
    if cos.shape != sin.shape or cos.shape[1] not in (d, d // 2):
        raise TensorError(_lib.ERR_INVALID_OPERATION,
                          f"cos/sin last dim must be head_dim = {d}, got cos: {cos.shape[1]}, sin: {sin.shape[1]}")
    y = x.dev.empty(x.shape)
    check(x.dev.lib.tlc_rope_table(x.dev.handle, x.ptr, cos.ptr, sin.ptr, y.ptr, seq, heads, d, cos.shape[0],
                                   cos.shape[1]))
    return y


def matmul(a: Tensor, b: Tensor) -> Tensor:
    """matmul(a, b) -> a @ b for 2-D f16 tensors (src/interpreter/builtin_math.rs:39-66,
    Tensor::matmul src/ops/matmul.rs:13-75): f32 accumulation, one rounding to f16."""
    if a.ndim != 2 or b.ndim != 2:
        raise TensorError(_lib.ERR_INVALID_OPERATION, "matmul requires 2D tensors")
    y = a.dev.empty((a.shape[0], b.shape[1]))
    check(a.dev.lib.tlc_matmul(a.dev.handle, a.ptr, b.ptr, y.ptr, a.shape[0], a.shape[1], b.shape[0], b.shape[1]))
    return y


def sigmoid(x: Tensor) -> Tensor:
    y = x.dev.empty(x.shape)
    check(x.dev.lib.tlc_sigmoid(x.dev.handle, x.ptr, y.ptr, x.size))
    return y


def _binary(fn_name: str, a: Tensor, b: Tensor) -> Tensor:
    if a.shape != b.shape:
        raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"expected {list(a.shape)}, got {list(b.shape)}")
    y = a.dev.empty(a.shape)
    check(getattr(a.dev.lib, fn_name)(a.dev.handle, a.ptr, b.ptr, y.ptr, a.size))
    return y


def mul(a: Tensor, b: Tensor) -> Tensor:
    return _binary("tlc_mul", a, b)


def add(a: Tensor, b: Tensor) -> Tensor:
    return _binary("tlc_add", a, b)


def silu(x: Tensor) -> Tensor:
    """x * sigmoid(x), as the TL scripts define it (debug/chat_demo_with_kvcache.tl:26-28)."""
    return mul(x, sigmoid(x))


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """silu(gate) * up in one kernel (same roundings as the three-op composition)."""
    return _binary("tlc_swiglu", gate, up)


def softmax(x: Tensor, dim: int = -1) -> Tensor:
    del dim  # the reference builtin always normalises the last axis
    last = x.shape[-1]
    y = x.dev.empty(x.shape)
    check(x.dev.lib.tlc_softmax(x.dev.handle, x.ptr, y.ptr, x.size // last, last))
    return y


def temperature_sample(logits: Tensor, temperature: float = 1.0, uniforms=None) -> np.ndarray:
    """temperature_sample(logits, T) for every row of ``logits`` [rows, vocab]: sampled token ids.

    ``uniforms``: one draw in [0, 1) per row (the reference draws ``rand::thread_rng().gen::<f32>()``
    itself; here the caller owns the randomness).  temperature <= 1e-4 is greedy and needs none."""
    vocab = logits.shape[-1]
    rows = logits.size // vocab
    ids = np.empty(rows, np.int32)
    u = None
    if temperature > 1e-4:
        if uniforms is None:
            raise TensorError(_lib.ERR_INVALID_OPERATION, "temperature_sample() needs one uniform draw per row")
        u = np.ascontiguousarray(np.atleast_1d(uniforms), dtype=np.float32)
        if u.size != rows:
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"temperature_sample: {u.size} draws for {rows} rows")
    check(logits.dev.lib.tlc_temperature_sample(logits.dev.handle, logits.ptr, rows, vocab, float(temperature),
                                                u.ctypes.data_as(C.POINTER(C.c_float)) if u is not None else None,
                                                ids.ctypes.data_as(C.POINTER(C.c_int32))))
    return ids


def embedding(table: Tensor, ids) -> Tensor:
    if table.ndim != 2:
        raise TensorError(_lib.ERR_INVALID_OPERATION, "embedding table must be 2D [vocab, d]")
    ids = np.ascontiguousarray(np.atleast_1d(ids), dtype=np.int32)
    vocab, d = table.shape
    y = table.dev.empty((ids.size, d))
    check(table.dev.lib.tlc_embedding(table.dev.handle, table.ptr, vocab, d, ids.ctypes.data_as(C.POINTER(C.c_int32)),
                                      ids.size, y.ptr))
    return y


def _upload_i32(dev: Device, a: np.ndarray) -> Tensor:
    t = Tensor(dev, ((a.size * 4 + 1) // 2,))
    check(dev.lib.tlc_upload(dev.handle, t.ptr, a.ctypes.data, a.nbytes))
    dev.synchronize()
    return t


# -- fused entry points --------------------------------------------------------

def norm_linear_multi(x: Tensor, weights: Sequence[QTensor], norm_weight: Optional[Tensor] = None,
                      eps: float = 1e-6, rope_heads: Optional[Sequence[int]] = None, position_offset: int = 0,
                      positions: Optional[np.ndarray] = None, base: int = 10000) -> list[Tensor]:
    """[linear(rms_norm(x), W_i) (+ rope)] for up to three weights in one launch."""
    m, _ = _rows_cols(x)
    n = len(weights)
    outs = [x.dev.empty((m, w.shape[0])) for w in weights]
    wh = (C.c_void_p * n)(*[w.handle for w in weights])
    yh = (C.c_void_p * n)(*[o.ptr for o in outs])
    rh = (C.c_int32 * n)(*(rope_heads if rope_heads is not None else [0] * n))
    pos_t = _upload_i32(x.dev, np.ascontiguousarray(positions, dtype=np.int32)) if positions is not None else None
    check(x.dev.lib.tlc_norm_linear_multi(x.dev.handle, n, wh, yh, rh, x.ptr, m,
                                          norm_weight.ptr if norm_weight is not None else None, eps,
                                          position_offset, base, pos_t.ptr if pos_t is not None else None))
    return outs


def swiglu_gate_up(x: Tensor, w_gate: QTensor, w_up: QTensor, norm_weight: Optional[Tensor] = None,
                   eps: float = 1e-6) -> Tensor:
    m, _ = _rows_cols(x)
    act = x.dev.empty((m, w_gate.shape[0]))
    check(x.dev.lib.tlc_swiglu_gate_up(x.dev.handle, w_gate.handle, w_up.handle, x.ptr, m,
                                       norm_weight.ptr if norm_weight is not None else None, eps, act.ptr))
    return act


class KVCache:
    """KVCache::new_f16 (src/model/llama.rs:51-116) over pre-allocated device storage.

    ``append`` writes rows in place instead of concatenating the whole cache;
    ``attention`` is the fused replacement of the script-level GQA chain.
    """

    def __init__(self, dev: Device, n_layers: int, n_kv_heads: int, head_dim: int, max_seq: int = 2048,
                 max_batch: int = 1):
        self.dev = dev
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        self.max_seq, self.max_batch = max_seq, max_batch
        h = C.c_void_p()
        check(dev.lib.tlc_kvcache_create(dev.handle, n_layers, max_batch, max_seq, n_kv_heads, head_dim, C.byref(h)))
        self.handle = h
        self.lengths = [0] * n_layers  # sequence-0 token counts, like KVCache::seq_len upstream

    def __del__(self):
        try:
            if self.handle and self.dev.handle:
                self.dev.lib.tlc_kvcache_destroy(self.handle)
            self.handle = None
        except Exception:
            pass

    def append(self, layer: int, k: Tensor, v: Tensor, positions: Optional[np.ndarray] = None) -> None:
        """cache.append(layer, K, V): K/V are [m, n_kv_heads, head_dim] (or [m, n_kv_heads*head_dim])."""
        row = self.n_kv_heads * self.head_dim
        if k.size % row or k.size != v.size:
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"KV rows must have {row} elements")
        m = k.size // row
        pos_t = _upload_i32(self.dev, np.ascontiguousarray(positions, dtype=np.int32)) if positions is not None else None
        check(self.dev.lib.tlc_kvcache_append(self.dev.handle, self.handle, layer, k.ptr, v.ptr, m,
                                              self.lengths[layer] if positions is None else 0,
                                              pos_t.ptr if pos_t is not None else None))
        if positions is None:
            self.lengths[layer] += m

    def layer_arrays(self, layer: int, batch_index: int = 0, length: Optional[int] = None):
        """get_k / get_v (src/model/llama.rs:101-116): host copies [len, n_kv_heads, head_dim]."""
        kp, vp_ = C.c_void_p(), C.c_void_p()
        check(self.dev.lib.tlc_kvcache_layer_ptrs(self.handle, layer, C.byref(kp), C.byref(vp_)))
        n = self.lengths[layer] if length is None else length
        row = self.n_kv_heads * self.head_dim
        out = []
        for p in (kp.value, vp_.value):
            a = np.empty((n, self.n_kv_heads, self.head_dim), np.float16)
            if n:
                check(self.dev.lib.tlc_download(self.dev.handle, a.ctypes.data,
                                                p + batch_index * self.max_seq * row * 2, a.nbytes))
            out.append(a)
        return out

    def attention(self, layer: int, q: Tensor, n_heads: int, q_pos0: int = 0, batch: int = 1,
                  positions: Optional[np.ndarray] = None, scale: Optional[float] = None) -> Tensor:
        """softmax(q.K^T * scale + causal mask).V for q [batch*n_queries, n_heads, head_dim]."""
        D = self.head_dim
        if q.size % (n_heads * D * batch):
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, f"attention: q has {q.size} elements")
        nq = q.size // (n_heads * D * batch)
        out = self.dev.empty(q.shape)
        scale = float(1.0 / np.sqrt(D)) if scale is None else scale
        pos_t, max_keys = None, q_pos0 + nq
        if positions is not None:
            pos = np.ascontiguousarray(positions, dtype=np.int32)
            pos_t = _upload_i32(self.dev, pos)
            max_keys = int(pos.max()) + 1
        check(self.dev.lib.tlc_attention(self.dev.handle, self.handle, layer, q.ptr, out.ptr, batch, nq, n_heads,
                                         q_pos0, pos_t.ptr if pos_t is not None else None, max_keys, scale))
        return out


def linear_residual(x: Tensor, weight: QTensor, residual: Tensor) -> Tensor:
    m, _ = _rows_cols(x)
    y = x.dev.empty((m, weight.shape[0]))
    check(x.dev.lib.tlc_linear_residual(x.dev.handle, weight.handle, x.ptr, m, residual.ptr, y.ptr))
    return y
