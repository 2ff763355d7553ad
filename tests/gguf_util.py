"""A minimal GGUF v3 writer for the loader tests: header, metadata key/values, tensor infos, aligned data
(the layout rust/src/model/gguf.rs:76-119 parses)."""
import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _value(typ, v) -> bytes:
    fmt = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}
    if typ in fmt:
        return struct.pack(fmt[typ], v)
    if typ == T_BOOL:
        return struct.pack("<B", 1 if v else 0)
    if typ == T_STR:
        return _s(v)
    if typ == T_ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    raise ValueError(typ)


def write_gguf(path, metadata, tensors, alignment=32, version=3, magic=0x46554747, truncate_to=None):
    """metadata: list of (key, type, value); tensors: list of (name, ggml type, dims fastest-first, raw bytes)."""
    md = list(metadata)
    if alignment != 32:
        md.append(("general.alignment", T_U32, alignment))
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(md))
    for key, typ, v in md:
        head += _s(key) + struct.pack("<I", typ) + _value(typ, v)
    blobs, offset, infos = [], 0, b""
    for name, typ, dims, raw in tensors:
        raw = np.ascontiguousarray(raw).view(np.uint8).tobytes()
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, offset)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        offset += len(raw) + pad
    head += infos
    head += b"\0" * ((-len(head)) % alignment)
    data = head + b"".join(blobs)
    if truncate_to is not None:
        data = data[:truncate_to]
    with open(path, "wb") as f:
        f.write(data)
    return len(head)


def spec_metadata(spec, arch="llama", vocab_from_tokens=False, context=4096):
    md = [("general.architecture", T_STR, arch),
          (f"{'llama' if arch in ('llama', 'mistral') else arch}.embedding_length", T_U32, spec.hidden_size),
          (f"{'llama' if arch in ('llama', 'mistral') else arch}.block_count", T_U32, spec.num_layers),
          ("llama.attention.head_count", T_U32, spec.num_heads),
          ("llama.attention.head_count_kv", T_U64, spec.num_kv_heads),
          ("llama.feed_forward_length", T_ARR, (T_U32, [spec.intermediate_size])),  # one-element array form (gguf.rs:145-153)
          ("llama.context_length", T_U32, context),
          ("llama.rope.freq_base", T_F32, float(spec.rope_theta))]
    if vocab_from_tokens:
        md.append(("tokenizer.ggml.tokens", T_ARR, (T_STR, [f"t{i}" for i in range(spec.vocab_size)])))
    else:
        md.append(("llama.vocab_size", T_U32, spec.vocab_size))
    return md
