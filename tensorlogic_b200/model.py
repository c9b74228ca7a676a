"""GGUF models and the LLaMA forward pass (host-side mirror).

    load_model(path)          src/interpreter/builtin_model.rs:106-131
    get_tensor(model, name)   src/interpreter/builtin_model.rs:203-246
    Llama.prefill / decode    the TL script debug/chat_demo_with_kvcache.tl:136-296
                              (LlamaModel::forward itself is a stub upstream,
                              src/model/llama.rs:257-266)

Weights stay in HBM as GGUF blocks; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib, synth
from ._lib import LlamaConfig, TensorError, check
from .api import Device, QTensor


@dataclass
class LlamaArch:
    """LlamaConfig (src/model/llama.rs:14-42); the defaults are TinyLlama-1.1B's."""
    n_layers: int = 22
    d_model: int = 2048
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 64
    ffn_dim: int = 5632
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope_base: int = 10000

    def tensor_shapes(self) -> dict:
        """GGUF tensor names -> (rows, cols) in the loader's [out, in] order."""
        d, qd, kvd = self.d_model, self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        shapes = {"token_embd.weight": (self.vocab, d), "output_norm.weight": (1, d), "output.weight": (self.vocab, d)}
        for l in range(self.n_layers):
            p = f"blk.{l}."
            shapes.update({p + "attn_norm.weight": (1, d), p + "attn_q.weight": (qd, d), p + "attn_k.weight": (kvd, d),
                           p + "attn_v.weight": (kvd, d), p + "attn_output.weight": (d, qd),
                           p + "ffn_norm.weight": (1, d), p + "ffn_gate.weight": (self.ffn_dim, d),
                           p + "ffn_up.weight": (self.ffn_dim, d), p + "ffn_down.weight": (d, self.ffn_dim)})
        return shapes


TINYLLAMA = LlamaArch()
LLAMA2_7B = LlamaArch(32, 4096, 32, 32, 128, 11008, 32000)
LLAMA2_70B = LlamaArch(80, 8192, 64, 8, 128, 28672, 32000)

_ROW_SPLIT = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "ffn_gate.weight", "ffn_up.weight")
_COL_SPLIT = ("attn_output.weight", "ffn_down.weight")


def split_for(name: str) -> int:
    if name.endswith(_ROW_SPLIT) or name == "output.weight":
        return _lib.SPLIT_ROWS
    if name.endswith(_COL_SPLIT):
        return _lib.SPLIT_COLS
    return _lib.SPLIT_NONE


class WeightCache:
    """GGUFWeightCache (src/model/gguf_weight_cache.rs): tensors of a GGUF file uploaded on first use,
    at most ``capacity`` of them resident (LRU).  ``load_weight_cache_gguf_f16(path, capacity)`` /
    ``get_weight(cache, name)`` of the builtin surface; the cached tensors stay quantized."""

    def __init__(self, dev: Device, path, capacity: int):
        self.dev = dev
        h = C.c_void_p()
        check(dev.lib.tlc_weight_cache_open(dev.handle, str(path).encode(), int(capacity), C.byref(h)))
        self.handle = h

    def close(self) -> None:
        if self.handle and self.dev.handle:
            self.dev.lib.tlc_weight_cache_close(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def get_weight(self, name: str) -> QTensor:
        """The tensor stays owned by the cache: valid until evicted, cleared or closed."""
        h = C.c_void_p()
        check(self.dev.lib.tlc_weight_cache_get(self.handle, name.encode(), C.byref(h)))
        t = QTensor(self.dev, h)
        t._owner = self
        t.__class__ = _BorrowedQTensor
        return t

    def contains(self, name: str) -> bool:
        return bool(self.dev.lib.tlc_weight_cache_contains(self.handle, name.encode()))

    def clear(self) -> None:
        check(self.dev.lib.tlc_weight_cache_clear(self.handle))

    def stats(self) -> dict:
        n, cap = C.c_int64(), C.c_int64()
        hits, misses, ev = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(self.dev.lib.tlc_weight_cache_stats(self.handle, C.byref(n), C.byref(cap), C.byref(hits), C.byref(misses),
                                                  C.byref(ev)))
        return {"len": n.value, "capacity": cap.value, "hits": hits.value, "misses": misses.value,
                "evictions": ev.value}


class Model:
    """Model<T> = name -> tensor map (src/model/mod.rs:39-45), tensors resident on the device."""

    def __init__(self, dev: Device, handle: Optional[C.c_void_p] = None):
        self.dev = dev
        if handle is None:
            handle = C.c_void_p()
            check(dev.lib.tlc_model_create(dev.handle, C.byref(handle)))
        self.handle = handle

    def __del__(self):
        try:
            if self.handle and self.dev.handle:
                self.dev.lib.tlc_model_destroy(self.handle)
            self.handle = None
        except Exception:
            pass

    def add(self, name: str, t: QTensor) -> None:
        check(self.dev.lib.tlc_model_add(self.handle, name.encode(), t.handle))
        t.handle = None  # ownership moved to the model

    def get_tensor(self, name: str) -> QTensor:
        h = C.c_void_p()
        check(self.dev.lib.tlc_model_get(self.handle, name.encode(), C.byref(h)))
        t = QTensor(self.dev, h)
        t._owner = self
        t.__class__ = _BorrowedQTensor
        return t

    def names(self) -> list[str]:
        n = self.dev.lib.tlc_model_tensor_count(self.handle)
        return [self.dev.lib.tlc_model_tensor_name(self.handle, i).decode() for i in range(n)]

    def meta(self, key: str):
        v = C.c_double()
        rc = self.dev.lib.tlc_model_meta_num(self.handle, key.encode(), C.byref(v))
        if rc == _lib.OK:
            return v.value
        s = self.dev.lib.tlc_model_meta_str(self.handle, key.encode())
        return s.decode() if s is not None else None


class _BorrowedQTensor(QTensor):
    """A QTensor whose storage belongs to a Model."""

    def __del__(self):
        self.handle = None


def load_model(dev: Device, path: str, tp_rank: int = 0, tp_size: int = 1) -> Model:
    h = C.c_void_p()
    check(dev.lib.tlc_model_load_gguf(dev.handle, str(path).encode(), tp_rank, tp_size, C.byref(h)))
    return Model(dev, h)


def get_tensor(model: Model, name: str) -> QTensor:
    return model.get_tensor(name)


def weight_scale_log2(qtype: int, cols: int, residual_writer: bool = False) -> int:
    """Power-of-two factor applied to the block scales of a model's linear weights.

    Blocks with d ~ U[0.002, 0.02] have rms 0.0565 (Q4_0) / 0.89 (Q8_0), so a linear over K inputs
    amplifies by rms*sqrt(K) (2.6x at K=2048 for Q4_0); stacked 22 or 80 times with residuals the f16
    activations overflow (the CPU oracle shows inf at layer 15 of the TinyLlama shape).  Full-model
    configurations therefore scale d by the power of two that brings that gain closest to 1; the
    single-linear configurations keep the unscaled range.  The projections that write into the
    residual stream (attn_output, ffn_down) get a further 2^-2: uniform nibbles have mean 7.5 - 8,
    so every weight row carries a small negative mean that accumulates layer after layer.
    """
    rms = 0.0565 if qtype == _lib.TYPE_Q4_0 else 0.892
    return -int(round(float(np.log2(rms * np.sqrt(cols))))) - (2 if residual_writer else 0)


def synthetic_host_weights(arch: LlamaArch, seed: int, qtype: int = _lib.TYPE_Q4_0) -> dict:
    """Seeded synthetic weights as host arrays: name -> (ggml_type, array).

    Linear weights are Q4_0/Q8_0 blocks from the counter-based generator (block scales
    U[0.002, 0.02] * 2^weight_scale_log2); embeddings f16 N(0,1)*0.02 and norm weights
    f16 1 + N(0, 0.02).
    """
    out = {}
    for name, (rows, cols) in arch.tensor_shapes().items():
        if name.endswith("norm.weight"):
            out[name] = (_lib.TYPE_F16, synth.norm_weight(seed, name, cols).reshape(1, cols))
        elif name == "token_embd.weight":
            out[name] = (_lib.TYPE_F16, synth.embedding_table(seed, name, rows, cols))
        else:
            out[name] = (qtype, synth.blocks(qtype, seed, synth.tensor_id(name), rows, cols,
                                             scale_log2=weight_scale_log2(qtype, cols, name.endswith(_COL_SPLIT))))
    return out


def synthetic_model(dev: Device, arch: LlamaArch, seed: int, qtype: int = _lib.TYPE_Q4_0, tp_rank: int = 0,
                    tp_size: int = 1, device_embeddings: bool = False) -> Model:
    """The same weights as ``synthetic_host_weights``; the quantized ones are generated on the device.

    device_embeddings: fill the f16 embedding table on the device too (same distribution, different
    samples than the host generator) -- for the large shapes whose 0.5 GB table is slow to make in numpy.
    """
    m = Model(dev)
    for name, (rows, cols) in arch.tensor_shapes().items():
        if name.endswith("norm.weight"):
            t = QTensor.from_blocks(dev, _lib.TYPE_F16, 1, cols, synth.norm_weight(seed, name, cols))
        elif name == "token_embd.weight" and device_embeddings:
            t = QTensor.normal_f16(dev, rows, cols, seed, synth.tensor_id(name), 0.0, 0.02)
        elif name == "token_embd.weight":
            t = QTensor.from_blocks(dev, _lib.TYPE_F16, rows, cols, synth.embedding_table(seed, name, rows, cols))
        else:
            t = QTensor.synthetic(dev, qtype, rows, cols, seed, synth.tensor_id(name), tp_rank, tp_size,
                                  split_for(name) if tp_size > 1 else _lib.SPLIT_NONE,
                                  scale_log2=weight_scale_log2(qtype, cols, name.endswith(_COL_SPLIT)))
        m.add(name, t)
    return m


def model_from_host(dev: Device, weights: dict, tp_rank: int = 0, tp_size: int = 1) -> Model:
    m = Model(dev)
    for name, (gtype, arr) in weights.items():
        arr = np.ascontiguousarray(arr)
        if gtype in (_lib.TYPE_F16, _lib.TYPE_F32):
            rows, cols = (1, arr.size) if arr.ndim == 1 else arr.shape
        else:
            rows, cols = arr.shape[0], arr.shape[1] * 32
        split = split_for(name) if tp_size > 1 and rows > 1 else _lib.SPLIT_NONE
        m.add(name, QTensor.from_blocks(dev, gtype, rows, cols, arr, tp_rank, tp_size, split))
    return m


class Llama:
    """Prefill + greedy decode over a Model with LLaMA tensor names."""

    def __init__(self, dev: Device, model: Model, arch: LlamaArch, max_seq: int = 2048, max_batch: int = 1,
                 max_prefill: int = 512, logits_all_rows: bool = False, use_graph: bool = True, tp_rank: int = 0,
                 tp_size: int = 1):
        self.dev, self.model, self.arch = dev, model, arch
        self.max_batch = max_batch
        self._max_seq, self._tp_size = max_seq, tp_size
        cfg = LlamaConfig(arch.n_layers, arch.d_model, arch.n_heads, arch.n_kv_heads, arch.head_dim, arch.ffn_dim,
                          arch.vocab, arch.rms_eps, arch.rope_base, max_seq, max_batch, max_prefill, tp_rank, tp_size,
                          int(logits_all_rows), int(not use_graph))
        h = C.c_void_p()
        check(dev.lib.tlc_llama_create(dev.handle, model.handle, C.byref(cfg), C.byref(h)))
        self.handle = h
        self.vocab_local = arch.vocab // max(tp_size, 1)

    def __del__(self):
        try:
            if self.handle and self.dev.handle:
                self.dev.lib.tlc_llama_destroy(self.handle)
            self.handle = None
        except Exception:
            pass

    def set_comm(self, comm) -> None:
        """Tensor parallelism: join this rank's runner to its communicator (tensorlogic_b200.comm.Comm)."""
        check(self.dev.lib.tlc_llama_set_comm(self.handle, comm.handle))
        self._comm = comm  # keep it alive
        self.vocab_local = self.arch.vocab  # logits handed back to the host are full rows

    def set_sampling(self, temperature: float = 0.0, seed: int = 0) -> None:
        """temperature <= 1e-4: greedy (default).  Otherwise temperature_sample on the device, with
        uniform draws that depend only on (seed, position, sequence): see ``sample_uniform``."""
        check(self.dev.lib.tlc_llama_set_sampling(self.handle, float(temperature), int(seed)))

    def sample_uniform(self, seed: int, position: int, sequence: int = 0) -> float:
        """The draw the device uses for the token fed at ``position`` of ``sequence``."""
        return float(self.dev.lib.tlc_sample_uniform_host(int(seed), int(position), int(sequence)))

    def prefill(self, ids, pos0: int = 0, return_logits: bool = True, all_rows: bool = False):
        """Returns (next_token, logits or None); logits are [1 or n, vocab] f16."""
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        rows = ids.size if all_rows else 1
        logits = np.empty((rows, self.vocab_local), np.float16) if return_logits else None
        nxt = C.c_int32()
        check(self.dev.lib.tlc_llama_prefill(self.handle, ids.ctypes.data_as(C.POINTER(C.c_int32)), ids.size, pos0,
                                             logits.ctypes.data if logits is not None else None, int(all_rows),
                                             C.byref(nxt)))
        return nxt.value, logits

    def set_state(self, ids, positions) -> None:
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        pos = np.ascontiguousarray(positions, dtype=np.int32).reshape(-1)
        if ids.size != pos.size:
            raise TensorError(_lib.ERR_SHAPE_MISMATCH, "ids and positions differ in length")
        check(self.dev.lib.tlc_llama_set_state(self.handle, ids.size, ids.ctypes.data_as(C.POINTER(C.c_int32)),
                                               pos.ctypes.data_as(C.POINTER(C.c_int32))))

    def decode(self, ids=None, batch: int = 1, return_logits: bool = False):
        """One greedy step through host buffers.  Returns (next_tokens[batch], logits or None)."""
        ids_p = None
        if ids is not None:
            ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
            batch = ids.size
            ids_p = ids.ctypes.data_as(C.POINTER(C.c_int32))
        nxt = np.empty(batch, np.int32)
        logits = np.empty((batch, self.vocab_local), np.float16) if return_logits else None
        check(self.dev.lib.tlc_llama_decode_host(self.handle, batch, ids_p, nxt.ctypes.data_as(C.POINTER(C.c_int32)),
                                                 logits.ctypes.data if logits is not None else None))
        return nxt, logits

    def fill_cache_random(self, seed: int, std: float = 1.0) -> None:
        """Fill the whole KV cache with f16 N(0, std) on the device: stands in for a context that is
        'already in the cache' (the 70B-shape decode workload) without running a 2048-token prefill."""
        cache = self.dev.lib.tlc_llama_cache(self.handle)
        kv_local = self.arch.n_kv_heads // max(self._tp_size, 1)
        n = self.max_batch * self._max_seq * kv_local * self.arch.head_dim
        for l in range(self.arch.n_layers):
            kp, vp_ = C.c_void_p(), C.c_void_p()
            check(self.dev.lib.tlc_kvcache_layer_ptrs(cache, l, C.byref(kp), C.byref(vp_)))
            check(self.dev.lib.tlc_fill_normal_f16(self.dev.handle, kp, n, seed, 2 * l, 0.0, std))
            check(self.dev.lib.tlc_fill_normal_f16(self.dev.handle, vp_, n, seed, 2 * l + 1, 0.0, std))

    def decode_enqueue(self, batch: int, steps: int, parts: int = 7) -> None:
        """Enqueue greedy steps on the device; parts (1 linears | 2 attention | 4 gather+sample) != 7
        replays only those launches, for per-kernel timing."""
        if parts == 7:
            check(self.dev.lib.tlc_llama_decode_enqueue(self.handle, batch, steps))
        else:
            check(self.dev.lib.tlc_llama_decode_enqueue_parts(self.handle, batch, steps, parts))

    def read_state(self, batch: int = 1):
        nxt, pos = np.empty(batch, np.int32), np.empty(batch, np.int32)
        check(self.dev.lib.tlc_llama_read_state(self.handle, batch, nxt.ctypes.data_as(C.POINTER(C.c_int32)),
                                                pos.ctypes.data_as(C.POINTER(C.c_int32))))
        return nxt, pos

    def step_trace(self, steps: int = 1) -> np.ndarray:
        """Device times (ns) of `steps` decode steps of sequence 0 as [steps, n_layers * 5 + 2, 3]:
        for every phase (input ready, dot products done, outputs stored); phases per layer A (norm + q/k/v + rope), B (attention), C (o +
        residual), D (norm + gate/up + SiLU.mul), E (down + residual), then F (norm + lm_head)
        and G (sample).  Only for models that run on the persistent step kernel."""
        per = self.arch.n_layers * 5 + 2
        out = np.zeros(steps * per * 3, np.uint64)
        check(self.dev.lib.tlc_llama_step_trace(self.handle, steps, out.ctypes.data_as(C.POINTER(C.c_uint64)), out.size))
        return out.reshape(steps, per, 3)

    def launches(self, parts: int = 7) -> int:
        return int(self.dev.lib.tlc_llama_launches_per_step(self.handle, parts))

    @property
    def launches_per_step(self) -> int:
        return self.launches(7)
