"""The synthetic-weight generator and quantisers: deterministic, well distributed, and identical on host and device."""
import numpy as np
import pytest


def test_host_generator_is_deterministic_and_keyed(lc):
    from leafcutterllm_b200 import synth
    a = synth.host_tensor(0, 1234, "blk.0.attn_q.weight", 4096)
    b = synth.host_tensor(0, 1234, "blk.0.attn_q.weight", 4096)
    c = synth.host_tensor(0, 1234, "blk.1.attn_q.weight", 4096)
    d = synth.host_tensor(0, 1235, "blk.0.attn_q.weight", 4096)
    assert np.array_equal(a, b) and not np.array_equal(a, c) and not np.array_equal(a, d)
    # any slice can be generated on its own: element i does not depend on the tensor length
    assert np.array_equal(synth.host_tensor(0, 1234, "blk.0.attn_q.weight", 1024), a[:4096])


def test_host_generator_is_normal_0_02(lc):
    from leafcutterllm_b200 import synth
    x = synth.host_tensor(0, 7, "stats", 1 << 20).view(np.float32)
    assert abs(x.mean()) < 1e-4 and abs(x.std() - 0.02) < 1e-4
    z = x / 0.02
    assert abs((z ** 3).mean()) < 0.02 and abs((z ** 4).mean() - 3.0) < 0.05  # skewness, kurtosis
    assert np.abs(z).max() < 6.5


@pytest.mark.parametrize("typ,tol", [(8, 0.02 * 4.5 / 127 * 0.51), (2, 0.02 * 4.5 / 8 * 1.01), (12, 0.02 * 9 / 15 * 0.6),
                                     (13, 0.02 * 9 / 31 * 0.6), (14, 0.02 * 4.5 / 31 * 0.6)])
def test_quantisers_round_trip_through_the_reference_dequantisers(lc, oracle, typ, tol):
    from leafcutterllm_b200 import synth
    n = 256 * 64
    x = synth.host_tensor(0, 99, "rt", n).view(np.float32)
    q = synth.host_tensor(typ, 99, "rt", n)  # same seed and name: quantised form of exactly x
    back = oracle.dequantize(typ, q, n)
    assert np.abs(back - x).max() < tol
    assert oracle.lib().orc_sanitize(back.ctypes.data, n) == 0  # nothing for the reference's weight sanity pass to zero


def test_q8_0_and_q4_0_follow_the_reference_absmax_rule(lc, oracle):
    """Same scale rule as rust/src/kernels/q8_0.rs:99-118 and q4_0.rs:107-133 (max|x|/127, max|x|/8), GGUF element order."""
    from leafcutterllm_b200 import synth
    x = synth.host_tensor(0, 5, "rule", 32 * 40).view(np.float32)
    assert np.array_equal(synth.host_tensor(8, 5, "rule", x.size), oracle.quantize_q8_0_ref(x))
    ours = synth.host_tensor(2, 5, "rule", x.size).reshape(-1, 18)
    ref = oracle.quantize_q4_0_ref(x).reshape(-1, 18)  # shard order: byte i = elements 2i, 2i+1
    assert np.array_equal(ours[:, :2], ref[:, :2])
    nib = np.stack([ref[:, 2:] & 0x0F, ref[:, 2:] >> 4], axis=-1).reshape(-1, 32)  # element order
    regrouped = (nib[:, :16] | (nib[:, 16:] << 4)).astype(np.uint8)            # GGUF: byte j = elements j, j+16
    assert np.array_equal(ours[:, 2:], regrouped)


def test_prompt_tokens_are_uniform_and_seeded(lc):
    from leafcutterllm_b200 import synth
    a = synth.prompt_tokens(4096, 32000, 0)
    assert np.array_equal(a, synth.prompt_tokens(4096, 32000, 0)) and not np.array_equal(a, synth.prompt_tokens(4096, 32000, 1))
    assert a.min() >= 0 and a.max() < 32000 and abs(a.mean() - 16000) < 600


@pytest.mark.gpu
@pytest.mark.parametrize("typ", [0, 1, 2, 8, 12, 13, 14])
def test_device_generator_matches_host_bytes(gpu, typ):
    import ctypes as C
    from leafcutterllm_b200 import synth
    lib = gpu.load()
    n = 256 * 2048 + (0 if typ else 5)
    host = synth.host_tensor(typ, 1234, "blk.3.ffn_down.weight", n)
    p = C.c_void_p()
    gpu._capi.check(lib.lc_dev_alloc(host.size, C.byref(p)))
    gpu._capi.check(lib.lc_synth_tensor_dev(typ, 1234, b"blk.3.ffn_down.weight", 0.02, n, p))
    dev = np.empty_like(host)
    gpu._capi.check(lib.lc_dev_download(dev.ctypes.data_as(C.c_void_p), p, host.size))
    lib.lc_dev_free(p)
    assert np.array_equal(dev, host)


def test_oracle_side_generator_makes_the_same_bytes(lc, oracle):
    """The CPU arm of the benchmark builds its inputs inside the oracle library (so that it never loads the CUDA library);
    its generator must make the bytes the CUDA library's host generator makes."""
    import numpy as np
    from leafcutterllm_b200 import synth
    for typ, n in [(12, 256 * 40), (13, 256 * 40), (14, 256 * 40), (2, 32 * 70), (8, 32 * 70), (0, 1000), (1, 1000)]:
        a = synth.host_tensor(typ, 1234, "blk.3.ffn_up.weight", n)
        b = oracle.synth_tensor(typ, 1234, "blk.3.ffn_up.weight", synth.SIGMA, n)
        assert np.array_equal(a, b), typ
    assert np.array_equal(synth.prompt_tokens(50, 32000, 3), oracle.synth_tokens(synth.PROMPT_SEED + 3, 50, 32000))


def test_q4_k_m_type_mix(lc):
    """The "Q4_K_M" spec keeps q, k, o, gate, up and the embedding in Q4_K, and puts the head and -- in the first and last
    eighth of the layers and every third layer between -- attn_v and ffn_down in Q6_K."""
    from leafcutterllm_b200 import synth
    spec = synth.LLAMA7B_Q4KM
    types = {name: typ for name, typ, _, _ in spec.tensors()}
    assert types["output.weight"] == 14 and types["token_embd.weight"] == 12
    q6_layers = [l for l in range(32) if types[f"blk.{l}.ffn_down.weight"] == 14]
    assert q6_layers == [0, 1, 2, 3, 6, 9, 12, 15, 18, 21, 24, 27, 28, 29, 30, 31]
    assert all(types[f"blk.{l}.attn_v.weight"] == types[f"blk.{l}.ffn_down.weight"] for l in range(32))
    assert all(types[f"blk.{l}.{t}.weight"] == 12 for l in range(32) for t in ("attn_q", "attn_k", "attn_output", "ffn_gate", "ffn_up"))
    assert all(typ == 12 for name, typ, _, _ in synth.LLAMA7B.tensors() if not name.endswith("norm.weight"))
