"""Synthetic models of the benchmark shapes: which tensors exist, their ggml types and GGUF dims.

Weights are N(0, 0.02) from the library's counter-based generator keyed by (seed, tensor name,
element index) and quantised in GGUF block order; norm gains are 1.0.  The same description
feeds the CUDA engine (tensors synthesised on the device or uploaded from the host generator)
and any checker that wants the identical bytes.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Iterator, Tuple

import numpy as np

from ._capi import TYPE_F32, TYPE_Q4_0, TYPE_Q4_K, TYPE_Q6_K, TYPE_Q8_0, check, load

SIGMA = 0.02
WEIGHT_SEED = 1234
PROMPT_SEED = 4321


@dataclass
class ModelSpec:
    name: str
    num_layers: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float = 10000.0
    layer_type: int = TYPE_Q4_K
    embed_type: int = TYPE_Q4_K
    head_type: int = TYPE_Q4_K
    tied_head: bool = False
    mix: str = ""        # "q4_k_m": the type mix of such a file (see mixed_type) instead of layer_type / head_type throughout
    n_experts: int = 0   # > 0: a mixture-of-experts FFN in every layer (f32 router + n_experts SwiGLU experts, top_k of them per token)
    top_k: int = 0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    def mixed_type(self, layer: int, which: str) -> int:
        """The type of attn_v / ffn_down of a layer (which = "v" | "down") and of the head (layer = -1).  With mix = "q4_k_m":
        Q6_K for the head and, for attn_v and ffn_down, in the first and last eighth of the layers and every third layer
        between; Q4_K elsewhere -- the placement the usual quantisation tool gives its "Q4_K_M" files."""
        if self.mix != "q4_k_m":
            return self.head_type if layer < 0 else self.layer_type
        if layer < 0:
            return TYPE_Q6_K
        n = self.num_layers
        more = layer < n // 8 or layer >= 7 * n // 8 or (layer - n // 8) % 3 == 2
        return TYPE_Q6_K if more else TYPE_Q4_K

    def tensors(self) -> Iterator[Tuple[str, int, Tuple[int, ...], str]]:
        """(gguf name, ggml type, dims fastest-first, 'normal' | 'ones')"""
        H, F, V = self.hidden_size, self.intermediate_size, self.vocab_size
        nq, nkv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        yield "token_embd.weight", self.embed_type, (H, V), "normal"
        yield "output_norm.weight", TYPE_F32, (H,), "ones"
        if not self.tied_head:
            yield "output.weight", self.mixed_type(-1, "head"), (H, V), "normal"
        for l in range(self.num_layers):
            p = f"blk.{l}."
            yield p + "attn_norm.weight", TYPE_F32, (H,), "ones"
            yield p + "attn_q.weight", self.layer_type, (H, nq), "normal"
            yield p + "attn_k.weight", self.layer_type, (H, nkv), "normal"
            yield p + "attn_v.weight", self.mixed_type(l, "v"), (H, nkv), "normal"
            yield p + "attn_output.weight", self.layer_type, (nq, H), "normal"
            yield p + "ffn_norm.weight", TYPE_F32, (H,), "ones"
            if self.n_experts > 0:
                yield p + "ffn_gate_inp.weight", TYPE_F32, (H, self.n_experts), "normal"
                for e in range(self.n_experts):
                    q = f"{p}expert.{e}."
                    yield q + "ffn_gate.weight", self.layer_type, (H, F), "normal"
                    yield q + "ffn_up.weight", self.layer_type, (H, F), "normal"
                    yield q + "ffn_down.weight", self.layer_type, (F, H), "normal"
                continue
            yield p + "ffn_gate.weight", self.layer_type, (H, F), "normal"
            yield p + "ffn_up.weight", self.layer_type, (H, F), "normal"
            yield p + "ffn_down.weight", self.mixed_type(l, "down"), (F, H), "normal"

    def with_layers(self, n: int) -> "ModelSpec":
        import dataclasses
        return dataclasses.replace(self, num_layers=n, name=f"{self.name}-L{n}")


# TinyLlama-1.1B shape: Q4_0 layers, Q8_0 embedding and head.
TINY = ModelSpec("tinyllama-1.1b-shape-q4_0", 22, 2048, 32, 4, 5632, 32000, 10000.0, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q8_0)
# Llama-2-7B shape, Q4_K throughout.
LLAMA7B = ModelSpec("llama2-7b-shape-q4_k", 32, 4096, 32, 32, 11008, 32000, 10000.0, TYPE_Q4_K, TYPE_Q4_K, TYPE_Q4_K)
# Llama-2-7B shape with the type mix of a "Q4_K_M" file: Q6_K head, Q6_K attn_v and ffn_down in about half of the layers.
LLAMA7B_Q4KM = ModelSpec("llama2-7b-shape-q4_k_m", 32, 4096, 32, 32, 11008, 32000, 10000.0, TYPE_Q4_K, TYPE_Q4_K, TYPE_Q4_K, mix="q4_k_m")
# Mixtral-8x7B shape: 8 experts of FFN 14336, two per token, 32 q / 8 kv heads, Q4_K (router f32).
MIXTRAL = ModelSpec("mixtral-8x7b-shape-q4_k", 32, 4096, 32, 8, 14336, 32000, 10000.0, TYPE_Q4_K, TYPE_Q4_K, TYPE_Q4_K, n_experts=8, top_k=2)
# Llama-3-70B shape, Q4_K.
LLAMA70B = ModelSpec("llama3-70b-shape-q4_k", 80, 8192, 64, 8, 28672, 128256, 500000.0, TYPE_Q4_K, TYPE_Q4_K, TYPE_Q4_K)


def host_tensor(typ: int, seed: int, name: str, n_elems: int, sigma: float = SIGMA) -> np.ndarray:
    """Raw block bytes of a synthetic tensor from the host generator (same bytes as the device one)."""
    lib = load()
    out = np.empty(lib.lc_tensor_bytes(typ, n_elems), np.uint8)
    check(lib.lc_synth_tensor_host(typ, seed, name.encode(), sigma, n_elems, out.ctypes.data_as(C.c_void_p)))
    return out


def tensor_bytes(spec: ModelSpec, name: str, typ: int, dims, kind: str, seed: int = WEIGHT_SEED) -> np.ndarray:
    n = int(np.prod(dims))
    if kind == "ones":
        return np.ones(n, np.float32).view(np.uint8)
    return host_tensor(typ, seed, name, n)


def prompt_tokens(n: int, vocab: int, seq_index: int = 0, seed: int = PROMPT_SEED) -> np.ndarray:
    out = np.empty(n, np.int64)
    check(load().lc_synth_tokens(seed + seq_index, n, vocab, out.ctypes.data_as(C.c_void_p)))
    return out


def build_engine(spec: ModelSpec, max_seq_len: int, seed: int = WEIGHT_SEED, on_device: bool = True, **engine_kwargs):
    """An `Engine` holding the synthetic model.  on_device=True synthesises every tensor with a CUDA
    kernel (no host copy); False runs the host generator and uploads."""
    from .engine import Engine
    eng = Engine(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size,
                 spec.vocab_size, max_seq_len=max_seq_len, rope_theta=spec.rope_theta, n_experts=spec.n_experts, top_k=spec.top_k,
                 **engine_kwargs)
    for name, typ, dims, kind in spec.tensors():
        if kind == "ones" or not on_device:
            eng.set_tensor(name, typ, dims, tensor_bytes(spec, name, typ, dims, kind, seed))
        else:
            eng.synth_tensor(name, typ, dims, seed, SIGMA)
    eng.finalize()
    return eng
