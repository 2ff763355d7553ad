"""leafcutterllm_b200: the LeafcutterLLM token-generation path on B200 (sm_100a).

The product is libleafcutter_b200.so (CUDA kernels + a C ABI, include/leafcutter_b200.h);
this package is the ctypes binding and the host-side mirror of the reference's interfaces.
Importing it needs the built library -- there is no fallback path.
"""
from ._capi import (LeafcutterError, ModelConfig, QUANT_GEOMETRY, TYPE_F16, TYPE_F32, TYPE_IQ4_NL, TYPE_Q4_0, TYPE_Q4_K,
                    TYPE_Q5_K, TYPE_Q6_K, TYPE_Q8_0, load)
from .backend import (B200Backend, Q4Matrix, Q8Matrix, apply_rotary_emb, dequantize, q4_0_matmul, q8_0_matmul, qmatmul,
                      sample_top_p, scan_blocks, seeded_uniform, tensor_bytes)
from .engine import Engine, ShardEngine, inspect_gguf

__all__ = ["B200Backend", "Engine", "ShardEngine", "LeafcutterError", "ModelConfig", "Q4Matrix", "Q8Matrix", "QUANT_GEOMETRY",
           "apply_rotary_emb", "dequantize", "q4_0_matmul", "q8_0_matmul", "qmatmul", "sample_top_p", "seeded_uniform", "scan_blocks", "inspect_gguf", "tensor_bytes", "load",
           "TYPE_F32", "TYPE_F16", "TYPE_Q4_0", "TYPE_Q8_0", "TYPE_Q4_K", "TYPE_Q5_K", "TYPE_Q6_K", "TYPE_IQ4_NL"]
