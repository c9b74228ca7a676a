"""tensorlogic_b200: the CUDA (sm_100a) device layer for TensorLogic's quantized-LLM path.

``tensorlogic_b200.api`` mirrors the interpreter's builtin operator surface
(linear, rms_norm, rope, sigmoid, softmax, embedding, ...) over the C ABI of
``include/tlcuda.h``; ``tensorlogic_b200.build`` compiles the library in-tree.
"""
from ._lib import LIB_PATH, TensorError  # noqa: F401

__version__ = "0.1.0"
