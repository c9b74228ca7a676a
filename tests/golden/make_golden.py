"""Generates tests/golden/reference_py.npz and q6_k.npz from the reference's own Python code.

Run where the TensorLogic checkout is available, with its path in TL_REFERENCE:

    TL_REFERENCE=<path to the tensorlogic checkout> python tests/golden/make_golden.py

It imports the reference's numpy implementation of the TinyLlama layer
(scripts/reference_impl.py, scripts/reference_with_gguf.py) and the `gguf`
Python package, feeds them seeded inputs, and stores inputs and outputs.  The
fixture travels with the repository; the reference checkout does not.
Outputs of the reference scripts are f32/f64 numpy results (the scripts print
while they run; that output is silenced here).
"""
from __future__ import annotations

import contextlib
import io
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TL_REFERENCE")


def main() -> None:
    if not REF or not os.path.isdir(os.path.join(REF, "scripts")):
        raise SystemExit("set TL_REFERENCE to the path of the tensorlogic checkout")
    sys.path.insert(0, os.path.join(REF, "scripts"))
    import reference_impl as ri  # noqa: E402
    import reference_with_gguf as rg  # noqa: E402
    import gguf  # noqa: E402
    from gguf import quants  # noqa: E402

    rng = np.random.default_rng(20251125)
    out: dict[str, np.ndarray] = {}

    # --- Q4_0 / Q8_0 blocks: reference script dequantizer + gguf package ---
    nblk = 24
    q4 = np.zeros((nblk, 18), np.uint8)
    scales = rng.uniform(0.002, 0.02, nblk).astype(np.float16)
    # a few edge scales: zero, negative, subnormal, large
    scales[:4] = np.array([0.0, -0.0125, 6.1e-5, 123.5], np.float16)
    q4[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    q4[:, 2:] = rng.integers(0, 256, (nblk, 16), dtype=np.uint8)
    q4[4, 2:] = 0x00
    q4[5, 2:] = 0xFF
    out["q4_0_bytes"] = q4
    with contextlib.redirect_stdout(io.StringIO()):
        out["q4_0_script_f32"] = rg.dequantize_q4_0(q4.reshape(-1), (nblk * 32,)).astype(np.float32)
    out["q4_0_gguf_f32"] = quants.dequantize(q4.reshape(-1), gguf.GGMLQuantizationType.Q4_0).astype(np.float32)

    q8 = np.zeros((nblk, 34), np.uint8)
    q8[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    q8[:, 2:] = rng.integers(-127, 128, (nblk, 32), dtype=np.int8).view(np.uint8)
    q8[4, 2:] = np.int8(-128).view(np.uint8)
    out["q8_0_bytes"] = q8
    out["q8_0_gguf_f32"] = quants.dequantize(q8.reshape(-1), gguf.GGMLQuantizationType.Q8_0).astype(np.float32)

    # --- per-token ops of the TinyLlama layer (f16-representable inputs) ---
    x = rng.standard_normal((5, 4, 64)).astype(np.float16)
    out["rope_x"] = x
    for pos in (0, 7, 513):
        out[f"rope_y_pos{pos}"] = ri.apply_rope(x.astype(np.float64), position=pos).astype(np.float64)

    xn = rng.standard_normal((3, 256)).astype(np.float16)
    wn = (1.0 + 0.02 * rng.standard_normal(256)).astype(np.float16)
    out["rms_x"], out["rms_w"] = xn, wn
    out["rms_y_eps1e-5"] = ri.rms_norm(xn.astype(np.float64), wn.astype(np.float64), eps=1e-5)

    S, H, HKV, D = 6, 8, 2, 16
    q = rng.standard_normal((S, H, D)).astype(np.float16)
    k = rng.standard_normal((S, HKV, D)).astype(np.float16)
    v = rng.standard_normal((S, HKV, D)).astype(np.float16)
    out["attn_q"], out["attn_k"], out["attn_v"] = q, k, v
    with contextlib.redirect_stdout(io.StringIO()):
        ke = ri.expand_kv_heads(k.astype(np.float64), n_q_heads=H)
        ve = ri.expand_kv_heads(v.astype(np.float64), n_q_heads=H)
        # The script's attention() has no causal mask; it is the single-query /
        # full-visibility case, which is what a decode step computes.
        out["attn_full_out"] = ri.attention(q.astype(np.float64), ke, ve)
    out["expand_kv_k"] = ke

    xs = rng.standard_normal((2, 64)).astype(np.float16)
    wg = (0.1 * rng.standard_normal((96, 64))).astype(np.float16)
    wu = (0.1 * rng.standard_normal((96, 64))).astype(np.float16)
    wd = (0.1 * rng.standard_normal((64, 96))).astype(np.float16)
    out["ffn_x"], out["ffn_wg"], out["ffn_wu"], out["ffn_wd"] = xs, wg, wu, wd
    out["ffn_y"] = ri.swiglu(xs.astype(np.float64), wg.astype(np.float64), wu.astype(np.float64),
                             wd.astype(np.float64))

    path = os.path.join(HERE, "reference_py.npz")
    np.savez_compressed(path, **out)
    print(path, {k_: v_.shape for k_, v_ in out.items()})

    # --- Q6_K super-blocks (own file and generator, so the vectors above keep their bytes):
    # the gguf package's dequantizer = the llama.cpp element order the Rust loader follows ---
    rng6 = np.random.default_rng(20250614)
    nsb = 12
    q6 = rng6.integers(0, 256, (nsb, 210), dtype=np.uint8)
    d6 = rng6.uniform(1e-4, 2e-3, nsb).astype(np.float16)
    d6[:3] = np.array([0.0, -7.5e-4, 6.1e-5], np.float16)  # zero, negative, subnormal super-block scales
    q6[:, 208:210] = d6.view(np.uint8).reshape(-1, 2)
    q6[3, 192:208] = np.int8(-128).view(np.uint8)          # extreme sub-block scales
    q6[4, 192:208] = 127
    q6[5, :192] = 0x00                                     # all quants -32
    q6[6, :192] = 0xFF                                     # all quants +31
    out6 = {"q6_k_bytes": q6}
    out6["q6_k_gguf_f32"] = quants.dequantize(q6.reshape(-1), gguf.GGMLQuantizationType.Q6_K).astype(np.float32)
    # (scripts/reference_with_gguf.py also has a dequantize_q6_k, with another element order; the
    # script itself leaves it unused and the Rust loader follows llama.cpp, as the gguf package does.)
    path6 = os.path.join(HERE, "q6_k.npz")
    np.savez_compressed(path6, **out6)
    print(path6, {k_: v_.shape for k_, v_ in out6.items()})


if __name__ == "__main__":
    main()
