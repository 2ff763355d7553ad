"""Host-side mirror of the reference's `Engine` (rust/src/inference/engine.rs) over the C ABI.

Same surface as the Rust type: `forward(tokens) -> logits of the last position`,
`generate(tokens, max_tokens, temperature, top_p) -> tokens`, a KV cache that can be cleared
and sized (rust/src/cache/mod.rs).  Weights arrive as raw GGUF blocks and stay on the device.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Iterable, Optional, Sequence

import numpy as np

from . import _capi
from ._capi import Counters, ModelConfig, check, load


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Engine:
    def __init__(self, hidden_size: int, num_layers: int, num_heads: int, num_kv_heads: int, intermediate_size: int,
                 vocab_size: int, max_seq_len: int = 4096, rope_theta: float = 10000.0, rms_eps: float = 1e-5,
                 kv_dtype: str = "f16", rope_mode: str = "call_relative", max_seqs: int = 1, kv_page_tokens: int = 16,
                 kv_pool_tokens: int = 0, device: int = 0, n_experts: int = 0, top_k: int = 0, tp_size: int = 0, tp_rank: int = 0):
        cfg = ModelConfig()
        cfg.n_experts, cfg.top_k = n_experts, top_k
        cfg.tp_size, cfg.tp_rank = tp_size, tp_rank
        cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads = hidden_size, num_layers, num_heads, num_kv_heads
        cfg.intermediate_size, cfg.max_seq_len, cfg.vocab_size = intermediate_size, max_seq_len, vocab_size
        cfg.rope_theta, cfg.rms_eps = rope_theta, rms_eps
        cfg.kv_dtype = {"f16": 0, "f32": 1}[kv_dtype]
        cfg.rope_mode = {"call_relative": 0, "absolute": 1}[rope_mode]
        cfg.max_seqs, cfg.kv_page_tokens, cfg.kv_pool_tokens, cfg.device = max_seqs, kv_page_tokens, kv_pool_tokens, device
        self.cfg = cfg
        self._h = C.c_void_p()
        check(load().lc_model_create(C.byref(cfg), C.byref(self._h)))
        self.vocab_size = vocab_size
        self.max_seqs = max_seqs

    @classmethod
    def load(cls, path: str, max_seq_len: int = 0, kv_dtype: str = "f16", rope_mode: str = "call_relative", max_seqs: int = 1,
             kv_page_tokens: int = 16, kv_pool_tokens: int = 0, device: int = 0) -> "Engine":
        """`Engine::load(path)` (rust/src/inference/engine.rs:18-49): a GGUF v3 file, parsed and uploaded by the library.
        max_seq_len > 0 caps the KV capacity (the file's context length can be far more than a test wants to allocate)."""
        over = ModelConfig()
        over.max_seq_len = max_seq_len
        over.kv_dtype = {"f16": 0, "f32": 1}[kv_dtype]
        over.rope_mode = {"call_relative": 0, "absolute": 1}[rope_mode]
        over.max_seqs, over.kv_page_tokens, over.kv_pool_tokens, over.device = max_seqs, kv_page_tokens, kv_pool_tokens, device
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        check(load().lc_model_load_gguf(str(path).encode(), C.byref(over), C.byref(self._h)))
        cfg = ModelConfig()
        check(load().lc_model_get_config(self._h, C.byref(cfg)))
        self.cfg = cfg
        self.vocab_size = cfg.vocab_size
        self.max_seqs = max(1, cfg.max_seqs)
        return self

    @staticmethod
    def group(engines: Sequence["Engine"]) -> "Engine":
        """Ranks 0 .. n-1 of one cut model, all in this process on one device: calls on the first engine then drive every
        rank in lock step (`lc_model_group`).  Returns that first engine."""
        arr = (C.c_void_p * len(engines))(*[e._h for e in engines])
        check(load().lc_model_group(arr, len(engines)))
        engines[0]._group = list(engines)
        return engines[0]

    # ---- weights -------------------------------------------------------
    def set_tensor(self, name: str, typ: int, dims: Sequence[int], data) -> None:
        """`dims` in GGUF order (fastest first); `data` = raw block bytes."""
        buf = np.ascontiguousarray(data).view(np.uint8).ravel()
        d = (C.c_uint64 * len(dims))(*dims)
        check(load().lc_model_set_tensor(self._h, name.encode(), typ, d, len(dims), _p(buf), buf.size))

    def synth_tensor(self, name: str, typ: int, dims: Sequence[int], seed: int, sigma: float) -> None:
        d = (C.c_uint64 * len(dims))(*dims)
        check(load().lc_model_synth_tensor(self._h, name.encode(), typ, d, len(dims), seed, sigma))

    def get_tensor(self, name: str, typ: int, dims: Sequence[int]) -> np.ndarray:
        count = int(np.prod(dims))
        out = np.empty(load().lc_tensor_bytes(typ, count), np.uint8)
        check(load().lc_model_get_tensor(self._h, name.encode(), _p(out), out.size))
        return out

    def finalize(self) -> None:
        check(load().lc_model_finalize(self._h))

    # ---- KV cache (rust/src/cache/mod.rs) --------------------------------
    def kv_clear(self, seq_id: int = -1) -> None:
        check(load().lc_kv_clear(self._h, seq_id))

    def kv_memory_bytes(self) -> int:
        out = C.c_uint64()
        check(load().lc_kv_memory_bytes(self._h, C.byref(out)))
        return out.value

    def kv_length(self, seq_id: int = 0) -> int:
        out = C.c_int32()
        check(load().lc_kv_length(self._h, seq_id, C.byref(out)))
        return out.value

    # ---- Engine::forward / generate ---------------------------------------
    def forward(self, tokens: Iterable[int]) -> np.ndarray:
        t = np.ascontiguousarray(list(tokens), dtype=np.int64)
        out = np.empty(self.vocab_size, np.float32)
        check(load().lc_forward(self._h, _p(t), t.size, _p(out)))
        return out

    def forward_batch(self, seq_ids: Sequence[int], token_lists: Sequence[Sequence[int]], want_logits: bool = True):
        n = len(seq_ids)
        ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        counts = np.ascontiguousarray([len(t) for t in token_lists], dtype=np.int32)
        flat = np.ascontiguousarray([x for t in token_lists for x in t], dtype=np.int64)
        logits = np.empty((n, self.vocab_size), np.float32) if want_logits else None
        nxt = np.empty(n, np.int64)
        check(load().lc_forward_batch(self._h, n, _p(ids), _p(flat), _p(counts), _p(logits) if want_logits else None, _p(nxt)))
        return logits, nxt

    def generate(self, tokens: Iterable[int], max_tokens: int, temperature: float = 0.0, top_p: float = 1.0,
                 stop_on_eos: bool = True, on_token: Optional[Callable[[int], None]] = None, seed: Optional[int] = None) -> list:
        """`Engine::generate` (rust/src/inference/engine.rs:51-76).  temperature > 0 needs `seed`: the reference draws from an
        unseeded generator, here token i uses `seeded_uniform(seed, i)` in `sample_top_p`'s arithmetic."""
        if seed is not None:
            check(load().lc_model_set_seed(self._h, int(seed)))
        t = np.ascontiguousarray(list(tokens), dtype=np.int64)
        out = np.empty(max_tokens, np.int64)
        n_out = C.c_int32()
        cb = _capi.TOKEN_CB((lambda tok, _u: on_token(int(tok))) if on_token else 0)
        check(load().lc_generate(self._h, _p(t), t.size, max_tokens, temperature, top_p, int(stop_on_eos), _p(out),
                                 C.byref(n_out), cb, None))
        return out[: n_out.value].tolist()

    def decode_loop(self, seq_ids: Sequence[int], first_tokens: Sequence[int], steps: int):
        """`steps` greedy steps per sequence without leaving the device; returns (tokens[steps, n], milliseconds)."""
        n = len(seq_ids)
        ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        first = np.ascontiguousarray(first_tokens, dtype=np.int64)
        out = np.empty((steps, n), np.int64)
        ms = C.c_float()
        check(load().lc_decode_loop(self._h, n, _p(ids), _p(first), steps, _p(out), C.byref(ms)))
        return out, ms.value

    # ---- probes / counters -------------------------------------------------
    def probe_attention(self, layer: int, normed: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(normed, np.float32)
        out = np.empty_like(x)
        check(load().lc_probe_attention(self._h, layer, _p(x), x.shape[0], _p(out)))
        return out

    def probe_ffn(self, layer: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        check(load().lc_probe_ffn(self._h, layer, _p(x), x.shape[0], _p(out)))
        return out

    def counters(self) -> dict:
        c = Counters()
        check(load().lc_get_counters(self._h, C.byref(c)))
        return {f: getattr(c, f) for f, _ in Counters._fields_ if f != "reserved"}

    def reset_counters(self) -> None:
        check(load().lc_reset_counters(self._h))

    def close(self) -> None:
        if self._h:
            load().lc_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def inspect_gguf(path: str, scan: bool = True, max_corrupt: int = 256) -> dict:
    """`GGUFModel::capability_report` (rust/src/model/loader.rs:54-104) and, with `scan`, `scan_for_corruption`
    (loader.rs:301-422, the block scales checked on the GPU) of one GGUF file, as a dict with the reference's field names."""
    rep = _capi.GgufReport()
    rows = (_capi.CorruptTensor * max(1, max_corrupt))()
    names = C.create_string_buffer(1 << 16)
    check(load().lc_gguf_inspect(str(path).encode(), 1 if scan else 0, C.byref(rep), rows, max_corrupt, names, len(names)))
    lines = names.value.decode().splitlines()
    by_type = {code: int(n) for code, n in enumerate(rep.tensors_by_type) if n}
    cfg = rep.config
    out = {
        "architecture": rep.architecture.decode(),
        "arch_supported": bool(rep.arch_supported),
        "quant_summary": {"total_tensors": int(rep.total_tensors), "types": by_type,
                          "unsupported": [c for c in range(32) if rep.unsupported_types >> c & 1]},
        "missing_tensors": [ln[len("missing "):] for ln in lines if ln.startswith("missing ")],
        "extra_tensors": [ln[len("extra "):] for ln in lines if ln.startswith("extra ")],
        "n_missing": int(rep.n_missing), "n_extra": int(rep.n_extra),
        "can_run": bool(rep.can_run),
        "config": {"hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
                   "num_key_value_heads": cfg.num_kv_heads, "intermediate_size": cfg.intermediate_size,
                   "max_position_embeddings": cfg.max_seq_len, "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_theta},
    }
    if scan:
        n = min(int(rep.n_corrupt_tensors), max_corrupt)
        out["corruption"] = {
            "corrupted_tensors": [{"name": rows[i].name.decode(), "quant_type": int(rows[i].ggml_type),
                                   "blocks_total": int(rows[i].blocks_total), "blocks_bad": int(rows[i].blocks_bad),
                                   "bad_percentage": 100.0 * rows[i].blocks_bad / max(1, rows[i].blocks_total)} for i in range(n)],
            "n_corrupt_tensors": int(rep.n_corrupt_tensors),
            "total_blocks_checked": int(rep.total_blocks_checked), "total_bad_blocks": int(rep.total_bad_blocks)}
    return out


class ShardEngine:
    """Host-side mirror of the reference's `ShardEngine` (rust/src/inference/shard_engine.rs:18-97): a model split into a
    manifest.json and per-layer LEAFSHDR shard files.  The reference maps one layer at a time from disk; here every shard
    is read once and kept in device memory, which is what `load_with_cache(path, num_layers)` asks for there."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def load(cls, manifest_path: str, max_seq_len: int = 0, device: int = 0) -> "ShardEngine":
        h = C.c_void_p()
        check(load().lc_shard_engine_load(str(manifest_path).encode(), max_seq_len, device, C.byref(h)))
        return cls(h)

    @classmethod
    def load_with_cache(cls, manifest_path: str, cache_slots: int, max_seq_len: int = 0, device: int = 0) -> "ShardEngine":
        del cache_slots  # every layer is resident
        return cls.load(manifest_path, max_seq_len, device)

    def forward(self, tokens: Iterable[int], vocab_size: int) -> np.ndarray:
        t = np.ascontiguousarray(list(tokens), dtype=np.int64)
        out = np.empty(vocab_size, np.float32)
        check(load().lc_shard_engine_forward(self._h, _p(t), t.size, _p(out), None))
        return out

    def generate(self, tokens: Iterable[int], max_tokens: int, temperature: float = 0.0, top_p: float = 1.0,
                 seed: Optional[int] = None) -> list:
        """`ShardEngine::generate` (rust/src/inference/shard_engine.rs:74-97); temperature > 0 needs `seed` (see Engine.generate)."""
        if seed is not None:
            check(load().lc_shard_engine_set_seed(self._h, int(seed)))
        t = np.ascontiguousarray(list(tokens), dtype=np.int64)
        out = np.empty(max_tokens, np.int64)
        n_out = C.c_int32()
        check(load().lc_shard_engine_generate(self._h, _p(t), t.size, max_tokens, temperature, top_p, _p(out), C.byref(n_out)))
        return out[: n_out.value].tolist()

    def reset_kv_cache(self) -> None:
        check(load().lc_shard_engine_reset_kv_cache(self._h))

    def kv_cache_memory_mb(self) -> float:
        out = C.c_uint64()
        check(load().lc_shard_engine_kv_cache_memory_bytes(self._h, C.byref(out)))
        return out.value / (1024.0 * 1024.0)

    def close(self) -> None:
        if self._h:
            load().lc_shard_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
