"""Host-side mirror of the reference's operator interface, bound to the C ABI.

`B200Backend` has the nine methods of `trait Backend` (rust/src/backend/mod.rs:18-46) with the
same argument meaning: flat f32 host slices in, a new f32 array out.  Shape errors raise
(the reference asserts, rust/src/model/tensor.rs:108-113).  The free functions mirror
kernels::dequantize_* (rust/src/kernels/mod.rs), Tensor::matmul on a quantised weight
(rust/src/model/tensor.rs:107-135) and the shard-order q8_0_matmul / q4_0_matmul
(rust/src/kernels/int8_gemm.rs:172-194, 336-358).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _capi
from ._capi import check, load


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class B200Backend:
    """`impl Backend for B200Backend` as a Python object; every call runs CUDA kernels."""

    def matmul(self, a, b, m: int, k: int, n: int) -> np.ndarray:
        a, b = _f32(a).ravel(), _f32(b).ravel()
        if a.size != m * k or b.size != k * n:
            raise ValueError("matmul: slice sizes do not match m, k, n")
        out = np.empty(m * n, np.float32)
        check(load().lc_matmul_f32(_p(a), _p(b), m, k, n, _p(out)))
        return out

    def _binary(self, fn, a, b):
        a, b = _f32(a).ravel(), _f32(b).ravel()
        if a.size != b.size:
            raise ValueError("vector lengths differ")
        out = np.empty(a.size, np.float32)
        check(fn(_p(a), _p(b), a.size, _p(out)))
        return out

    def vec_add(self, a, b):
        return self._binary(load().lc_vec_add, a, b)

    def vec_mul(self, a, b):
        return self._binary(load().lc_vec_mul, a, b)

    def vec_scale(self, a, scale: float):
        a = _f32(a).ravel()
        out = np.empty(a.size, np.float32)
        check(load().lc_vec_scale(_p(a), float(scale), a.size, _p(out)))
        return out

    def vec_scale_mul(self, a, scale: float, b):
        a, b = _f32(a).ravel(), _f32(b).ravel()
        if a.size != b.size:
            raise ValueError("vector lengths differ")
        out = np.empty(a.size, np.float32)
        check(load().lc_vec_scale_mul(_p(a), float(scale), _p(b), a.size, _p(out)))
        return out

    def rms_norm(self, x, weight, eps: float, hidden_size: int):
        x, weight = _f32(x).ravel(), _f32(weight).ravel()
        if hidden_size <= 0 or x.size % hidden_size or weight.size < hidden_size:
            raise ValueError("rms_norm: sizes do not match hidden_size")
        out = np.empty(x.size, np.float32)
        check(load().lc_rms_norm(_p(x), _p(weight), float(eps), hidden_size, x.size // hidden_size, _p(out)))
        return out

    def silu(self, x):
        x = _f32(x).ravel()
        out = np.empty(x.size, np.float32)
        check(load().lc_silu(_p(x), x.size, _p(out)))
        return out

    def softmax(self, x, hidden_size: int):
        x = _f32(x).ravel()
        if hidden_size <= 0 or x.size % hidden_size:
            raise ValueError("softmax: size is not a multiple of hidden_size")
        out = np.empty(x.size, np.float32)
        check(load().lc_softmax(_p(x), hidden_size, x.size // hidden_size, _p(out)))
        return out

    def sum_sq(self, x) -> float:
        x = _f32(x).ravel()
        out = np.empty(1, np.float32)
        check(load().lc_sum_sq(_p(x), x.size, _p(out)))
        return float(out[0])


def tensor_bytes(typ: int, count: int) -> int:
    return int(load().lc_tensor_bytes(typ, count))


def dequantize(typ: int, data, n_elems: int) -> np.ndarray:
    """kernels::dequantize_{q4_0,q8_0,q4_k,q5_k,q6_k,iq4_nl} / F32 / F16 -> f32, bit-exact with the reference."""
    data = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8))
    if data.size != tensor_bytes(typ, n_elems):
        raise ValueError(f"dequantize: {data.size} bytes given, {tensor_bytes(typ, n_elems)} expected")
    out = np.empty(n_elems, np.float32)
    check(load().lc_dequantize(typ, _p(data), n_elems, _p(out)))
    return out


def scan_blocks(typ: int, data, n_elems: int):
    """The per-tensor body of `scan_for_corruption` (rust/src/model/loader.rs:318-402) on the GPU: returns
    (blocks_total, blocks_bad).  Accepts every type code of the reference's type table; types without blocks give (0, 0)."""
    data = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8))
    total, bad = C.c_uint64(), C.c_uint64()
    check(load().lc_scan_blocks(typ, _p(data), n_elems, C.byref(total), C.byref(bad)))
    return int(total.value), int(bad.value)


def qmatmul(typ: int, a, w_blocks, m: int, k: int, n: int) -> np.ndarray:
    """a[m,k] . dequant(W)^T with W = raw GGUF blocks of an [n, k] weight (blocks along k)."""
    a = _f32(a).ravel()
    w = np.ascontiguousarray(w_blocks).view(np.uint8).ravel()
    if a.size != m * k or w.size != tensor_bytes(typ, n * k):
        raise ValueError("qmatmul: sizes do not match m, k, n")
    out = np.empty((m, n), np.float32)
    check(load().lc_qmatmul(typ, _p(a), _p(w), m, k, n, _p(out)))
    return out


@dataclass
class Q8Matrix:
    """kernels::q8_0::Matrix (rust/src/kernels/q8_0.rs:56-86): blocks [rows][cols/32]."""
    rows: int
    cols: int
    scales: np.ndarray  # f32 [rows, cols/32]
    qs: np.ndarray      # int8 [rows, cols]


@dataclass
class Q4Matrix:
    """kernels::q4_0::Matrix (rust/src/kernels/q4_0.rs:66-94): byte i of a block = elements 2i, 2i+1."""
    rows: int
    cols: int
    scales: np.ndarray  # f32 [rows, cols/32]
    qs: np.ndarray      # uint8 [rows, cols/2]


def q8_0_matmul(a, b: Q8Matrix, m: int, k: int, n: int) -> np.ndarray:
    a = _f32(a).ravel()
    if b.rows != k or b.cols != n or a.size != m * k:
        raise ValueError("q8_0_matmul: shapes do not match")
    sc = np.ascontiguousarray(b.scales, np.float32)
    qs = np.ascontiguousarray(b.qs, np.int8)
    out = np.empty((m, n), np.float32)
    check(load().lc_q8_0_matmul_shard(_p(a), _p(sc), _p(qs), m, k, n, _p(out)))
    return out


def q4_0_matmul(a, b: Q4Matrix, m: int, k: int, n: int) -> np.ndarray:
    a = _f32(a).ravel()
    if b.rows != k or b.cols != n or a.size != m * k:
        raise ValueError("q4_0_matmul: shapes do not match")
    sc = np.ascontiguousarray(b.scales, np.float32)
    qs = np.ascontiguousarray(b.qs, np.uint8)
    out = np.empty((m, n), np.float32)
    check(load().lc_q4_0_matmul_shard(_p(a), _p(sc), _p(qs), m, k, n, _p(out)))
    return out


def apply_rotary_emb(x, seq_len: int, num_heads: int, head_dim: int, theta: float, pos0: int = 0) -> np.ndarray:
    """attention::apply_rotary_emb (rust/src/inference/attention.rs:13-34); returns the rotated copy."""
    x = _f32(x).copy().ravel()
    if x.size != seq_len * num_heads * head_dim:
        raise ValueError("apply_rotary_emb: size mismatch")
    check(load().lc_rope(_p(x), seq_len, num_heads, head_dim, float(theta), pos0))
    return x


def sample_top_p(logits, temperature: float, top_p: float, u: float = None) -> int:
    """sampler::sample_top_p (rust/src/inference/sampler.rs:6-50).  Greedy for temperature <= 0; the stochastic branch
    needs the uniform draw `u` in [0, 1) that the reference takes from its unseeded generator (:38-39)."""
    v = _f32(logits).ravel()
    if temperature > 0.0 and u is None:
        raise ValueError("sample_top_p: the stochastic branch needs the uniform draw u (the reference's rng.gen::<f32>())")
    out = C.c_int64()
    check(load().lc_sample_top_p(_p(v), v.size, float(temperature), float(top_p), float(u or 0.0), C.byref(out)))
    return int(out.value)


def seeded_uniform(seed: int, index: int) -> float:
    """Draw `index` of a seeded generation (see Engine.generate(seed=...))."""
    return float(load().lc_seeded_uniform(seed, index))
