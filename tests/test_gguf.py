"""GGUF v3 loading (lc_model_load_gguf ≙ Engine::load, rust/src/inference/engine.rs:18-49)."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close, make_pair
from gguf_util import T_STR, T_U32, spec_metadata, write_gguf


def _tensors(spec, seed=1234, extra=()):
    from leafcutterllm_b200 import synth
    out = [(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind, seed)) for name, typ, dims, kind in spec.tensors()]
    return out + list(extra)


def _load_status(path):
    from leafcutterllm_b200 import _capi
    lib = _capi.load()
    h = C.c_void_p()
    st = lib.lc_model_load_gguf(str(path).encode(), None, C.byref(h))
    return st, lib.lc_last_error().decode()


def test_rejects_what_the_reference_rejects(tmp_path):
    """Bad magic, another version, a truncated header (gguf.rs:84-89 and GGUError::TruncatedData) -- no GPU involved:
    the file is parsed before a device is touched."""
    from leafcutterllm_b200 import synth, _capi
    spec = synth.TINY.with_layers(1)
    md = spec_metadata(spec)
    tiny = [("output_norm.weight", 0, (spec.hidden_size,), np.ones(spec.hidden_size, np.float32))]
    p = tmp_path / "m.gguf"
    write_gguf(p, md, tiny, magic=0x46554746)
    st, msg = _load_status(p)
    assert st == _capi.LC_ERR_INVALID and "magic" in msg
    write_gguf(p, md, tiny, version=2)
    st, msg = _load_status(p)
    assert st == _capi.LC_ERR_UNSUPPORTED and "version 2" in msg
    write_gguf(p, md, tiny, truncate_to=60)
    st, msg = _load_status(p)
    assert st == _capi.LC_ERR_INVALID and "truncated" in msg
    st, msg = _load_status(tmp_path / "missing.gguf")
    assert st == _capi.LC_ERR_INVALID and "cannot open" in msg


@pytest.mark.gpu
@pytest.mark.parametrize("alignment,vocab_from_tokens,arch", [(32, False, "llama"), (64, True, "mistral")])
def test_loaded_model_equals_the_tensor_by_tensor_model(gpu, oracle, tmp_path, alignment, vocab_from_tokens, arch):
    from leafcutterllm_b200 import synth
    from leafcutterllm_b200.engine import Engine
    spec = synth.TINY.with_layers(2)
    path = tmp_path / "tiny.gguf"
    extra = [("blk.0.attn_rot_embd", 0, (4,), np.zeros(4, np.float32)), ("rope_freqs.weight", 0, (8,), np.ones(8, np.float32))]
    write_gguf(path, spec_metadata(spec, arch=arch, vocab_from_tokens=vocab_from_tokens), _tensors(spec, extra=extra), alignment=alignment)
    eng = Engine.load(path, max_seq_len=96)
    assert (eng.cfg.hidden_size, eng.cfg.num_layers, eng.cfg.num_heads, eng.cfg.num_kv_heads) == (
        spec.hidden_size, 2, spec.num_heads, spec.num_kv_heads)
    assert eng.cfg.intermediate_size == spec.intermediate_size and eng.cfg.vocab_size == spec.vocab_size
    assert eng.cfg.max_seq_len == 96 and eng.cfg.rope_theta == spec.rope_theta
    ref, om = make_pair(gpu, oracle, spec, max_seq_len=96)
    prompt = synth.prompt_tokens(24, spec.vocab_size, 3)
    a, b = eng.forward(prompt), ref.forward(prompt)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # same bytes, same kernels
    assert_close(a, om.forward(prompt), 1e-2, 1e-3, "loaded model vs oracle")
    assert eng.generate(prompt, 12, stop_on_eos=False) == ref.generate(prompt, 12, stop_on_eos=False)
    eng.close()
    ref.close()


@pytest.mark.gpu
def test_load_reports_missing_and_unsupported_tensors(gpu, tmp_path):
    from leafcutterllm_b200 import synth, _capi
    from leafcutterllm_b200.engine import Engine
    spec = synth.TINY.with_layers(1)
    path = tmp_path / "bad.gguf"
    tensors = [t for t in _tensors(spec) if t[0] != "blk.0.ffn_down.weight"]
    write_gguf(path, spec_metadata(spec), tensors)
    with pytest.raises(_capi.LeafcutterError) as e:
        Engine.load(path, max_seq_len=64)
    assert "ffn_down" in str(e.value)
    tensors = _tensors(spec) + [("blk.0.odd.weight", 31, (32,), np.zeros(32, np.uint8))]
    write_gguf(path, spec_metadata(spec), tensors)
    with pytest.raises(_capi.LeafcutterError) as e:
        Engine.load(path, max_seq_len=64)
    assert "type 31" in str(e.value)


@pytest.mark.gpu
def test_mixture_of_experts_file(gpu, oracle, tmp_path):
    """A GGUF file of a mixture model: llama.expert_count / llama.expert_used_count in the metadata, the router as
    blk.N.ffn_gate_inp.weight and the experts as the stacked three-dimensional tensors blk.N.ffn_{gate,up,down}_exps.weight.
    The loaded model must give the logits of the tensor-by-tensor model (one tensor per expert) and of the oracle."""
    from leafcutterllm_b200 import synth
    from leafcutterllm_b200.engine import Engine
    from leafcutterllm_b200.synth import ModelSpec
    from gguf_util import T_U32
    spec = ModelSpec("moe-file", 2, 256, 2, 2, 512, 640, 10000.0, 12, 12, 12, n_experts=4, top_k=2)
    tensors, stacks = [], {}
    for name, typ, dims, kind in spec.tensors():
        data = synth.tensor_bytes(spec, name, typ, dims, kind)
        if ".expert." in name:
            layer, which = name.split(".")[1], name.split(".")[-2]
            stacks.setdefault((layer, which), []).append((typ, dims, data))
        else:
            tensors.append((name, typ, tuple(dims), data))
    for (layer, which), parts in stacks.items():
        typ, dims = parts[0][0], parts[0][1]
        tensors.append((f"blk.{layer}.{which}_exps.weight", typ, (dims[0], dims[1], spec.n_experts), np.concatenate([p[2] for p in parts])))
    path = tmp_path / "moe.gguf"
    md = spec_metadata(spec) + [("llama.expert_count", T_U32, spec.n_experts), ("llama.expert_used_count", T_U32, spec.top_k)]
    write_gguf(path, md, tensors)
    eng = Engine.load(path, max_seq_len=64)
    assert (eng.cfg.n_experts, eng.cfg.top_k) == (4, 2)
    ref, om = make_pair(gpu, oracle, spec, max_seq_len=64)
    prompt = synth.prompt_tokens(13, spec.vocab_size, 5)
    a, b = eng.forward(prompt), ref.forward(prompt)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert_close(a, om.forward(prompt), 1e-2, 1e-3, "mixture model from a file vs oracle")
    eng.close()
    ref.close()
