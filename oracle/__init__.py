"""ctypes wrapper of the CPU oracle (oracle.cpp).  TEST INFRASTRUCTURE: only tests/, the smoke
check and the CPU-baseline leg of bench.py may import this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB_PATH


class OrcConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_int32), ("num_layers", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
                ("intermediate_size", C.c_int32), ("max_seq_len", C.c_int32), ("vocab_size", C.c_int32),
                ("rope_theta", C.c_float), ("rms_eps", C.c_float), ("kv_f32", C.c_int32), ("rope_absolute", C.c_int32),
                ("n_experts", C.c_int32), ("top_k", C.c_int32)]


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        vp, sz, f, i32, u32 = C.c_void_p, C.c_size_t, C.c_float, C.c_int32, C.c_uint32
        sig = {
            "orc_num_threads": (C.c_int, []), "orc_set_num_threads": (None, [C.c_int]),
            "orc_f16_to_f32": (f, [C.c_uint16]), "orc_f32_to_f16": (C.c_uint16, [f]),
            "orc_f16_roundtrip": (None, [vp, vp, sz]),
            "orc_dequantize": (C.c_int, [u32, vp, sz, vp]), "orc_sanitize": (sz, [vp, sz]),
            "orc_tensor_bytes": (sz, [u32, sz]),
            "orc_matmul": (None, [vp, vp, sz, sz, sz, vp]), "orc_matmul_nk": (None, [vp, vp, sz, sz, sz, vp]),
            "orc_vec_add": (None, [vp, vp, sz, vp]), "orc_vec_mul": (None, [vp, vp, sz, vp]),
            "orc_vec_scale": (None, [vp, f, sz, vp]), "orc_vec_scale_mul": (None, [vp, f, vp, sz, vp]),
            "orc_rms_norm": (None, [vp, vp, f, sz, sz, vp]), "orc_silu": (None, [vp, sz, vp]),
            "orc_softmax": (None, [vp, sz, sz, vp]), "orc_sum_sq": (f, [vp, sz]),
            "orc_rope": (None, [vp, sz, sz, sz, f, sz]), "orc_argmax": (sz, [vp, sz]),
            "orc_qmatmul": (C.c_int, [u32, vp, vp, sz, sz, sz, vp]),
            "orc_q8_0_matmul_shard": (C.c_int, [vp, vp, vp, sz, sz, sz, vp]),
            "orc_q4_0_matmul_shard": (C.c_int, [vp, vp, vp, sz, sz, sz, vp]),
            "orc_quantize_q8_0_ref": (None, [vp, sz, vp]), "orc_quantize_q4_0_ref": (None, [vp, sz, vp]),
            "orc_model_create": (vp, [C.POINTER(OrcConfig)]), "orc_model_destroy": (None, [vp]),
            "orc_model_set_mode": (None, [vp, C.c_int, C.c_int]),
            "orc_model_set_tensor": (C.c_int, [vp, C.c_char_p, u32, C.POINTER(C.c_uint64), C.c_int, vp, sz]),
            "orc_kv_clear": (None, [vp]), "orc_kv_memory_bytes": (sz, [vp]),
            "orc_forward": (C.c_int, [vp, vp, sz, vp]), "orc_forward_hidden": (C.c_int, [vp, vp, sz, vp, vp]),
            "orc_generate": (C.c_int, [vp, vp, sz, sz, C.c_int, vp, C.POINTER(sz), vp]),
            "orc_sample_top_p": (sz, [vp, sz, C.c_float, C.c_float, C.c_float]),
            "orc_scan_blocks": (C.c_int, [C.c_uint32, vp, sz, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
            "orc_last_error": (C.c_char_p, [vp]), "orc_sanitized_count": (sz, [vp]),
            "orc_timers": (None, [vp, vp, C.c_int]),
            "orc_attention": (C.c_int, [vp, C.c_int, vp, sz, vp]), "orc_ffn": (C.c_int, [vp, C.c_int, vp, sz, vp]),
            "orc_synth_tensor": (C.c_int, [u32, C.c_uint64, C.c_char_p, f, sz, vp]),
            "orc_synth_tokens": (None, [C.c_uint64, sz, C.c_int64, vp]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def synth_tensor(typ: int, seed: int, name: str, sigma: float, n_elems: int) -> np.ndarray:
    """Raw block bytes of the benchmark's synthetic tensor (seed, name): the same bytes the CUDA library's generator makes."""
    out = np.empty(lib().orc_tensor_bytes(typ, n_elems), np.uint8)
    if lib().orc_synth_tensor(typ, seed, name.encode(), sigma, n_elems, _p(out)) != 0:
        raise ValueError(f"no synthetic generator for ggml type {typ}")
    return out


def synth_tokens(seed: int, n: int, vocab: int) -> np.ndarray:
    out = np.empty(n, np.int64)
    lib().orc_synth_tokens(seed, n, vocab, _p(out))
    return out


def dequantize(typ: int, data, n: int) -> np.ndarray:
    d = np.ascontiguousarray(data).view(np.uint8).ravel()
    out = np.empty(n, np.float32)
    if lib().orc_dequantize(typ, _p(d), n, _p(out)) != 0:
        raise ValueError(f"unsupported type {typ}")
    return out


def sample_top_p(logits, temperature: float, top_p: float, u: float = 0.0) -> int:
    """sampler::sample_top_p (rust/src/inference/sampler.rs:6-50) with the uniform draw `u` passed in."""
    v = _f32(logits).ravel()
    return int(lib().orc_sample_top_p(_p(v), v.size, temperature, top_p, u))


def scan_blocks(typ: int, data, n: int):
    """(blocks_total, blocks_bad) of one tensor as scan_for_corruption counts them (rust/src/model/loader.rs:318-402)."""
    d = np.ascontiguousarray(data).view(np.uint8).ravel()
    total, bad = C.c_uint64(), C.c_uint64()
    lib().orc_scan_blocks(typ, _p(d), n, C.byref(total), C.byref(bad))
    return int(total.value), int(bad.value)


def matmul(a, b, m, k, n):
    a, b = _f32(a).ravel(), _f32(b).ravel()
    out = np.empty(m * n, np.float32)
    lib().orc_matmul(_p(a), _p(b), m, k, n, _p(out))
    return out


def qmatmul(typ, a, w, m, k, n):
    a = _f32(a).ravel()
    w = np.ascontiguousarray(w).view(np.uint8).ravel()
    out = np.empty((m, n), np.float32)
    if lib().orc_qmatmul(typ, _p(a), _p(w), m, k, n, _p(out)) != 0:
        raise ValueError(f"unsupported type {typ}")
    return out


def vec_add(a, b):
    a, b = _f32(a).ravel(), _f32(b).ravel(); out = np.empty_like(a); lib().orc_vec_add(_p(a), _p(b), a.size, _p(out)); return out


def vec_mul(a, b):
    a, b = _f32(a).ravel(), _f32(b).ravel(); out = np.empty_like(a); lib().orc_vec_mul(_p(a), _p(b), a.size, _p(out)); return out


def vec_scale(a, s):
    a = _f32(a).ravel(); out = np.empty_like(a); lib().orc_vec_scale(_p(a), s, a.size, _p(out)); return out


def vec_scale_mul(a, s, b):
    a, b = _f32(a).ravel(), _f32(b).ravel(); out = np.empty_like(a); lib().orc_vec_scale_mul(_p(a), s, _p(b), a.size, _p(out)); return out


def rms_norm(x, w, eps, hidden):
    x, w = _f32(x).ravel(), _f32(w).ravel(); out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(w), eps, hidden, x.size // hidden, _p(out)); return out


def silu(x):
    x = _f32(x).ravel(); out = np.empty_like(x); lib().orc_silu(_p(x), x.size, _p(out)); return out


def softmax(x, hidden):
    x = _f32(x).ravel(); out = np.empty_like(x); lib().orc_softmax(_p(x), hidden, x.size // hidden, _p(out)); return out


def sum_sq(x):
    x = _f32(x).ravel(); return float(lib().orc_sum_sq(_p(x), x.size))


def rope(x, seq, heads, hd, theta, pos0=0):
    x = _f32(x).copy().ravel(); lib().orc_rope(_p(x), seq, heads, hd, theta, pos0); return x


def argmax(v):
    v = _f32(v).ravel(); return int(lib().orc_argmax(_p(v), v.size))


def f16_roundtrip(x):
    x = _f32(x).ravel(); out = np.empty_like(x); lib().orc_f16_roundtrip(_p(x), _p(out), x.size); return out


def q8_0_matmul_shard(a, scales, qs, m, k, n):
    a, scales, qs = _f32(a).ravel(), _f32(scales).ravel(), np.ascontiguousarray(qs, np.int8).ravel()
    out = np.empty((m, n), np.float32)
    assert lib().orc_q8_0_matmul_shard(_p(a), _p(scales), _p(qs), m, k, n, _p(out)) == 0
    return out


def q4_0_matmul_shard(a, scales, qs, m, k, n):
    a, scales, qs = _f32(a).ravel(), _f32(scales).ravel(), np.ascontiguousarray(qs, np.uint8).ravel()
    out = np.empty((m, n), np.float32)
    assert lib().orc_q4_0_matmul_shard(_p(a), _p(scales), _p(qs), m, k, n, _p(out)) == 0
    return out


def quantize_q8_0_ref(x):
    x = _f32(x).ravel(); out = np.empty(x.size // 32 * 34, np.uint8); lib().orc_quantize_q8_0_ref(_p(x), x.size, _p(out)); return out


def quantize_q4_0_ref(x):
    x = _f32(x).ravel(); out = np.empty(x.size // 32 * 18, np.uint8); lib().orc_quantize_q4_0_ref(_p(x), x.size, _p(out)); return out


class OracleModel:
    """Engine of the reference (rust/src/inference/engine.rs) restated on the CPU."""

    def __init__(self, hidden_size, num_layers, num_heads, num_kv_heads, intermediate_size, vocab_size, max_seq_len=4096,
                 rope_theta=10000.0, rms_eps=1e-5, kv_f32=False, rope_absolute=False, n_experts=0, top_k=0):
        c = OrcConfig(hidden_size, num_layers, num_heads, num_kv_heads, intermediate_size, max_seq_len, vocab_size,
                      rope_theta, rms_eps, int(kv_f32), int(rope_absolute), n_experts, top_k)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self._h = lib().orc_model_create(C.byref(c))

    def set_mode(self, reference_faithful: bool, cache_weights: bool = True):
        lib().orc_model_set_mode(self._h, int(reference_faithful), int(cache_weights))

    def set_tensor(self, name, typ, dims, data):
        d = np.ascontiguousarray(data).view(np.uint8).ravel()
        dd = (C.c_uint64 * len(dims))(*dims)
        rc = lib().orc_model_set_tensor(self._h, name.encode(), typ, dd, len(dims), _p(d), d.size)
        if rc != 0:
            raise ValueError(lib().orc_last_error(self._h).decode())

    def kv_clear(self):
        lib().orc_kv_clear(self._h)

    def kv_memory_bytes(self):
        return int(lib().orc_kv_memory_bytes(self._h))

    def forward(self, tokens, want_hidden=False):
        t = np.ascontiguousarray(list(tokens), np.int64)
        out = np.empty(self.vocab_size, np.float32)
        hid = np.empty(self.hidden_size, np.float32)
        rc = lib().orc_forward_hidden(self._h, _p(t), t.size, _p(out), _p(hid))
        if rc != 0:
            raise RuntimeError(lib().orc_last_error(self._h).decode())
        return (out, hid) if want_hidden else out

    def generate(self, tokens, max_tokens, stop_on_eos=True, want_margins=False):
        t = np.ascontiguousarray(list(tokens), np.int64)
        out = np.empty(max_tokens, np.int64)
        margins = np.empty(max_tokens, np.float32)
        n = C.c_size_t()
        rc = lib().orc_generate(self._h, _p(t), t.size, max_tokens, int(stop_on_eos), _p(out), C.byref(n), _p(margins))
        if rc != 0:
            raise RuntimeError(lib().orc_last_error(self._h).decode())
        toks = out[: n.value].tolist()
        return (toks, margins[: n.value]) if want_margins else toks

    def attention(self, layer, normed):
        x = _f32(normed); out = np.empty_like(x)
        lib().orc_attention(self._h, layer, _p(x), x.shape[0], _p(out)); return out

    def ffn(self, layer, x):
        x = _f32(x); out = np.empty_like(x)
        lib().orc_ffn(self._h, layer, _p(x), x.shape[0], _p(out)); return out

    def timers(self, reset=True):
        t = np.zeros(3, np.float64); lib().orc_timers(self._h, _p(t), int(reset))
        return {"dequant_s": t[0], "matmul_s": t[1], "attention_s": t[2]}

    def sanitized_count(self):
        return int(lib().orc_sanitized_count(self._h))

    def close(self):
        if self._h:
            lib().orc_model_destroy(self._h); self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
