"""ShardEngine (rust/src/inference/shard_engine.rs) on the device: manifest + LEAFSHDR shards in the three formats of
rust/src/shard/format.rs, against the CPU oracle fed with the f32 values the reference computes with."""
import numpy as np
import pytest

import shard_util
from conftest import assert_close

pytestmark = pytest.mark.gpu
GGUF = {"self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
        "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
        "mlp.down_proj.weight": "ffn_down.weight", "input_layernorm.weight": "attn_norm.weight",
        "post_attention_layernorm.weight": "ffn_norm.weight"}
CFG = dict(num_layers=2, hidden_size=128, vocab_size=320, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
           max_seq_len=96, rope_theta=10000.0)


def random_weights(seed):
    r = np.random.default_rng(seed)
    H, F, V, nh, nkv = CFG["hidden_size"], CFG["intermediate_size"], CFG["vocab_size"], CFG["num_attention_heads"], CFG["num_key_value_heads"]
    hd = H // nh
    n = lambda *s: (r.standard_normal(s) * 0.06).astype(np.float32)
    w = {"model.embed_tokens.weight": n(V, H), "model.norm.weight": (1 + 0.1 * r.standard_normal(H)).astype(np.float32), "lm_head.weight": n(H, V)}
    for l in range(CFG["num_layers"]):
        w[(l, "self_attn.q_proj.weight")] = n(H, nh * hd)
        w[(l, "self_attn.k_proj.weight")] = n(H, nkv * hd)
        w[(l, "self_attn.v_proj.weight")] = n(H, nkv * hd)
        w[(l, "self_attn.o_proj.weight")] = n(nh * hd, H)
        w[(l, "mlp.gate_proj.weight")] = n(H, F)
        w[(l, "mlp.up_proj.weight")] = n(H, F)
        w[(l, "mlp.down_proj.weight")] = n(F, H)
        w[(l, "input_layernorm.weight")] = (1 + 0.1 * r.standard_normal(H)).astype(np.float32)
        w[(l, "post_attention_layernorm.weight")] = (1 + 0.1 * r.standard_normal(H)).astype(np.float32)
    return w


def oracle_model(oracle, seen):
    om = oracle.OracleModel(CFG["hidden_size"], CFG["num_layers"], CFG["num_attention_heads"], CFG["num_key_value_heads"],
                            CFG["intermediate_size"], CFG["vocab_size"], max_seq_len=CFG["max_seq_len"], rope_theta=CFG["rope_theta"])
    def put(name, arr):  # GGUF keeps [outputs][inputs]: the transpose of the engine-ready [k][n]; dims fastest first
        a = np.ascontiguousarray(arr.T if arr.ndim == 2 and name != "token_embd.weight" else arr, np.float32)
        om.set_tensor(name, 0, list(reversed(a.shape)), a.view(np.uint8).ravel())
    put("token_embd.weight", seen["model.embed_tokens.weight"])
    put("output_norm.weight", seen["model.norm.weight"])
    put("output.weight", seen["lm_head.weight"])
    for (key, arr) in seen.items():
        if isinstance(key, tuple):
            put(f"blk.{key[0]}.{GGUF[key[1]]}", arr)
    return om


@pytest.mark.parametrize("fmt", [shard_util.F32, shard_util.Q8_0, shard_util.Q4_0])
def test_shard_engine_matches_the_oracle(gpu, oracle, tmp_path, fmt):
    from leafcutterllm_b200 import ShardEngine
    path, seen = shard_util.write_model(str(tmp_path / "shards"), random_weights(11 + fmt), CFG, fmt)
    eng = ShardEngine.load_with_cache(path, CFG["num_layers"])
    om = oracle_model(oracle, seen)
    prompt = np.random.default_rng(5).integers(3, CFG["vocab_size"], 19).tolist()
    got = eng.forward(prompt, CFG["vocab_size"])
    want = om.forward(prompt)
    assert_close(got, want, 1e-2, 1e-3, f"prefill logits, shard format {fmt}")
    assert abs(eng.kv_cache_memory_mb() * 1024 * 1024 - 19 * CFG["num_layers"] * 2 * 2 * 32 * 2) < 1
    step = eng.forward([7], CFG["vocab_size"])   # one decode step over the cache
    assert_close(step, om.forward([7]), 1e-2, 1e-3, "decode logits")
    ref, margins = om.generate(prompt, 8, stop_on_eos=True, want_margins=True)
    assert eng.generate(prompt, 8) == ref, margins   # generate clears the cache first (shard_engine.rs:75)
    eng.reset_kv_cache()
    assert eng.kv_cache_memory_mb() == 0
    eng.close()


def test_shard_engine_seeded_sampling(gpu, oracle, tmp_path):
    """temperature > 0 after a seed: forward, sample_top_p (rust/src/inference/sampler.rs:12-50) with the documented draws."""
    from leafcutterllm_b200 import LeafcutterError, ShardEngine, seeded_uniform
    path, _ = shard_util.write_model(str(tmp_path / "shards"), random_weights(3), CFG, shard_util.Q8_0)
    eng = ShardEngine.load_with_cache(path, CFG["num_layers"])
    prompt = np.random.default_rng(8).integers(3, CFG["vocab_size"], 11).tolist()
    with pytest.raises(LeafcutterError, match="LC_ERR_UNSUPPORTED"):
        eng.generate(prompt, 4, temperature=0.7, top_p=0.9)
    got = eng.generate(prompt, 9, temperature=1.3, top_p=0.9, seed=5)
    assert got == eng.generate(prompt, 9, temperature=1.3, top_p=0.9, seed=5)
    eng.reset_kv_cache()
    want, feed = [], list(prompt)
    for i in range(9):
        tok = oracle.sample_top_p(eng.forward(feed, CFG["vocab_size"]), 1.3, 0.9, seeded_uniform(5, i))
        want.append(tok)
        feed = [tok]
        if tok == 2:   # ShardEngine::generate stops after token 2 (shard_engine.rs:84-86, 92-94)
            break
    assert got == want and got != eng.generate(prompt, 9)
    eng.close()


def test_shard_loader_rejects_broken_files(gpu, tmp_path):
    from leafcutterllm_b200 import LeafcutterError, ShardEngine
    w = random_weights(3)
    path, _ = shard_util.write_model(str(tmp_path / "ok"), w, CFG, shard_util.F32)
    d = str(tmp_path / "ok")
    # bad magic (loader.rs:305-307)
    shard_util.write_shard(f"{d}/layer_001.shard", [("x", [1], b"\0\0\0\0")], 0, magic=b"NOTSHARD")
    with pytest.raises(LeafcutterError, match="bad magic"):
        ShardEngine.load(path)
    # a tensor that reaches past the end of the file (loader.rs:315-317)
    shard_util.write_shard(f"{d}/layer_001.shard", [("self_attn.q_proj.weight", [128, 128], b"\0" * 16)], 0)
    with pytest.raises(LeafcutterError, match="size mismatch|out of bounds"):
        ShardEngine.load(path)
    # a layer without one of its nine tensors (shard_engine.rs: expect("Missing ..."))
    shard_util.write_shard(f"{d}/layer_001.shard", [("input_layernorm.weight", [128], np.ones(128, np.float32).tobytes())], 0)
    with pytest.raises(LeafcutterError, match="missing"):
        ShardEngine.load(path)
    with pytest.raises(LeafcutterError):
        ShardEngine.load(str(tmp_path / "nowhere.json"))
