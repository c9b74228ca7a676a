"""Writes synthetic weights as a real GGUF v3 file with the `gguf` Python package."""
import numpy as np


def write_gguf(path, weights: dict, arch=None, alignment: int = 32, extra_kv: bool = True):
    """weights: name -> (ggml_type, array); quantized arrays are uint8 [rows, blocks, block_bytes]."""
    import gguf
    w = gguf.GGUFWriter(str(path), "llama")
    if alignment != 32:
        w.add_custom_alignment(alignment)
    if arch is not None:
        w.add_block_count(arch.n_layers)
        w.add_embedding_length(arch.d_model)
        w.add_head_count(arch.n_heads)
        w.add_head_count_kv(arch.n_kv_heads)
        w.add_feed_forward_length(arch.ffn_dim)
        w.add_layer_norm_rms_eps(arch.rms_eps)
        w.add_rope_freq_base(float(arch.rope_base))
    if extra_kv:
        # 1-, 2-byte and array values: a reader that skips them by the wrong size loses its place
        w.add_uint8("test.u8", 7)
        w.add_bool("test.flag", True)
        w.add_uint16("test.u16", 513)
        w.add_int8("test.i8", -3)
        w.add_array("test.tokens", ["<s>", "</s>", "hello"])
        w.add_array("test.scores", [0.5, -1.25, 3.0])
        w.add_string("test.note", "synthetic")
        w.add_uint64("test.u64", 1 << 40)
        w.add_float64("test.f64", 2.5)
    for name, (gtype, arr) in weights.items():
        arr = np.ascontiguousarray(arr)
        if gtype == 1:
            a = arr.astype(np.float16)
            w.add_tensor(name, a.reshape(-1) if a.shape[0] == 1 and name.endswith("norm.weight") else a)
        elif gtype == 0:
            a = arr.astype(np.float32)
            w.add_tensor(name, a.reshape(-1) if a.shape[0] == 1 and name.endswith("norm.weight") else a)
        else:
            rows = arr.shape[0]
            raw = arr.reshape(rows, -1).view(np.uint8)
            w.add_tensor(name, raw, raw_dtype=gguf.GGMLQuantizationType(gtype))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
