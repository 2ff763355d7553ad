"""A minimal writer of the reference's shard format for the loader tests: LEAFSHDR files (rust/src/shard/format.rs:1-23:
32-byte header, tensor table, data section aligned to 4096) and the manifest.json of rust/src/shard/loader.rs:13-43."""
import json
import os
import struct

import numpy as np

F32, Q8_0, Q4_0 = 0, 1, 2


def quantize_rows(x: np.ndarray, fmt: int):
    """Blocks of 32 along the flattened tensor.  Returns (raw block bytes, the f32 values those bytes stand for when the
    tensor is kept as a quantised matrix: q * scale, Q4_0 with element 2i in the low nibble of byte i, q4_0.rs:36-46)."""
    flat = np.ascontiguousarray(x, np.float32).ravel()
    if fmt == F32:
        return flat.tobytes(), flat.copy()
    blocks = flat.reshape(-1, 32)
    amax = np.abs(blocks).max(axis=1)
    if fmt == Q8_0:
        scale = (amax / 127.0).astype(np.float16)
        s32 = scale.astype(np.float32)
        q = np.where(s32[:, None] > 0, np.rint(blocks / np.where(s32 > 0, s32, 1)[:, None]), 0).clip(-127, 127).astype(np.int8)
        raw = np.zeros((blocks.shape[0], 34), np.uint8)
        raw[:, :2] = scale.view(np.uint8).reshape(-1, 2)
        raw[:, 2:] = q.view(np.uint8)
        return raw.tobytes(), (q.astype(np.float32) * s32[:, None]).ravel()
    scale = (amax / 7.0).astype(np.float16)
    s32 = scale.astype(np.float32)
    q = (np.where(s32[:, None] > 0, np.rint(blocks / np.where(s32 > 0, s32, 1)[:, None]), 0) + 8).clip(0, 15).astype(np.uint8)
    raw = np.zeros((blocks.shape[0], 18), np.uint8)
    raw[:, :2] = scale.view(np.uint8).reshape(-1, 2)
    raw[:, 2:] = q[:, 0::2] | (q[:, 1::2] << 4)
    return raw.tobytes(), ((q.astype(np.float32) - 8.0) * s32[:, None]).ravel()


def decode_flat_gguf_order(raw: bytes, fmt: int) -> np.ndarray:
    """What the reference makes of a tensor it does NOT keep quantised (1-D): the GGUF-order block decoders of
    rust/src/kernels/mod.rs:16-51 -- for Q4_0 element j in the low nibble of byte j, element j + 16 in the high one."""
    if fmt == F32:
        return np.frombuffer(raw, np.float32).copy()
    per = 34 if fmt == Q8_0 else 18
    b = np.frombuffer(raw, np.uint8).reshape(-1, per)
    s = b[:, :2].copy().view(np.float16).astype(np.float32)
    if fmt == Q8_0:
        return (b[:, 2:].copy().view(np.int8).astype(np.float32) * s).ravel()
    lo = (b[:, 2:] & 0x0F).astype(np.float32) - 8.0
    hi = (b[:, 2:] >> 4).astype(np.float32) - 8.0
    return (np.concatenate([lo, hi], axis=1) * s).ravel()


def write_shard(path: str, tensors, fmt: int, magic=b"LEAFSHDR", version=1):
    """tensors: list of (name, shape, raw bytes)."""
    table = 32
    for name, shape, raw in tensors:
        table += 4 + len(name.encode()) + 4 + 8 * len(shape) + 16
    data_start = (table + 4095) // 4096 * 4096
    head = magic + struct.pack("<IIQ", version, len(tensors), data_start) + bytes([fmt]) + b"\0" * 7
    off = data_start
    meta = b""
    for name, shape, raw in tensors:
        nb = name.encode()
        meta += struct.pack("<I", len(nb)) + nb + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        meta += struct.pack("<QQ", off, len(raw))
        off += len(raw)
    with open(path, "wb") as f:
        f.write(head + meta)
        f.write(b"\0" * (data_start - len(head) - len(meta)))
        for _n, _s, raw in tensors:
            f.write(raw)
    return os.path.getsize(path)


def write_model(directory: str, weights: dict, cfg: dict, fmt: int):
    """weights: engine-ready f32 arrays -- per layer l the nine names of shard_engine.rs under key (l, name), plus
    'model.embed_tokens.weight' [vocab, hidden], 'model.norm.weight', 'lm_head.weight' [hidden, vocab].
    Returns (manifest path, {key: f32 values the reference computes with})."""
    os.makedirs(directory, exist_ok=True)
    seen = {}

    def pack(key, arr):
        raw, kept = quantize_rows(arr, fmt)
        quantised_matrix = fmt != F32 and arr.ndim == 2 and arr.shape[1] % 32 == 0
        seen[key] = (kept if quantised_matrix else decode_flat_gguf_order(raw, fmt)).reshape(arr.shape)
        return raw

    layers = []
    for l in range(cfg["num_layers"]):
        names = [k[1] for k in weights if isinstance(k, tuple) and k[0] == l]
        tens = [(n, list(weights[(l, n)].shape), pack((l, n), weights[(l, n)])) for n in names]
        fn = f"layer_{l:03d}.shard"
        layers.append({"idx": l, "file": fn, "size": write_shard(os.path.join(directory, fn), tens, fmt)})
    special = {}
    for key, fn, field in [("model.embed_tokens.weight", "embed.shard", "embed"), ("model.norm.weight", "norm.shard", "norm"),
                           ("lm_head.weight", "lm_head.shard", "lm_head")]:
        size = write_shard(os.path.join(directory, fn), [(key, list(weights[key].shape), pack(key, weights[key]))], fmt)
        special[field] = fn
        special[field + "_size"] = size
    manifest = {"model": "test", "num_layers": cfg["num_layers"], "hidden_size": cfg["hidden_size"], "vocab_size": cfg["vocab_size"],
                "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
                "intermediate_size": cfg["intermediate_size"], "max_seq_len": cfg["max_seq_len"], "rope_theta": cfg["rope_theta"],
                "shard_dir": directory, "layers": layers, "special": special}
    path = os.path.join(directory, "manifest.json")
    with open(path, "w") as f:
        json.dump(manifest, f, indent=2)
    return path, seen
