"""Model-level parity on the GPU: Engine::forward / generate through the C ABI against the CPU oracle,
on identical synthetic weights."""
import numpy as np
import pytest

from conftest import assert_close, make_pair

pytestmark = pytest.mark.gpu

LOGIT_ABS, LOGIT_REL = 1e-2, 1e-3  # the stated bar for logits


def small_spec(layer_type, embed_type, head_type, layers=2, hidden=256, heads=8, kv=2, ffn=512, vocab=1000):
    from leafcutterllm_b200.synth import ModelSpec
    return ModelSpec("small", layers, hidden, heads, kv, ffn, vocab, 10000.0, layer_type, embed_type, head_type)


@pytest.mark.parametrize("types", [(12, 12, 12), (2, 8, 8), (8, 8, 8)])
def test_forward_and_generate_small(gpu, oracle, types):
    from leafcutterllm_b200 import synth
    spec = small_spec(*types)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=128)
    prompt = synth.prompt_tokens(17, spec.vocab_size)
    got = eng.forward(prompt)
    want = om.forward(prompt)
    assert_close(got, want, LOGIT_ABS, LOGIT_REL, "prefill logits")
    assert eng.kv_length() == 17
    assert eng.kv_memory_bytes() == om.kv_memory_bytes()  # rust/src/cache/mod.rs:80-84
    nxt = int(np.argmax(want))
    assert_close(eng.forward([nxt]), om.forward([nxt]), LOGIT_ABS, LOGIT_REL, "decode logits")
    toks = eng.generate(prompt, 24, stop_on_eos=False)
    ref, margins = om.generate(prompt, 24, stop_on_eos=False, want_margins=True)
    assert toks == ref, f"greedy tokens differ; oracle top-2 margins {margins}"
    # per-token callback path and the device-resident loop give the same tokens
    seen = []
    assert eng.generate(prompt, 24, stop_on_eos=False, on_token=seen.append) == ref and seen == ref
    eng.close()


@pytest.mark.parametrize("on_device", [False, True])
def test_q4_k_m_mix_with_generated_weights(gpu, oracle, on_device):
    """Eight layers with the type mix of a "Q4_K_M" file (Q6_K head; Q6_K attn_v and ffn_down in layers 0, 3, 6, 7), weights
    from the generator's own Q4_K and Q6_K quantisers on the host and on the device: prefill logits, a decode step and
    greedy tokens against the oracle."""
    from leafcutterllm_b200 import synth
    from leafcutterllm_b200.synth import ModelSpec
    spec = ModelSpec("small-q4_k_m", 8, 256, 8, 2, 768, 1008, 10000.0, 12, 12, 12, mix="q4_k_m")
    assert [l for l in range(8) if spec.mixed_type(l, "down") == 14] == [0, 3, 6, 7]
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=96, on_device=on_device)
    prompt = synth.prompt_tokens(21, spec.vocab_size, 5)
    want = om.forward(prompt)
    assert_close(eng.forward(prompt), want, LOGIT_ABS, LOGIT_REL, "prefill logits")
    nxt = int(np.argmax(want))
    assert_close(eng.forward([nxt]), om.forward([nxt]), LOGIT_ABS, LOGIT_REL, "decode logits")
    ref, margins = om.generate(prompt, 20, stop_on_eos=False, want_margins=True)
    assert eng.generate(prompt, 20, stop_on_eos=False) == ref, margins
    eng.close()


def test_layer_probes(gpu, oracle):
    spec = small_spec(12, 12, 12, layers=1, hidden=512, heads=8, kv=4, ffn=768)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=64)
    r = np.random.default_rng(0)
    x = r.standard_normal((5, 512)).astype(np.float32)
    assert_close(eng.probe_ffn(0, x), om.ffn(0, x), 1e-5, 1e-4, "ffn")
    assert_close(eng.probe_attention(0, x), om.attention(0, x), 1e-4, 1e-3, "attention (5 tokens)")
    x1 = r.standard_normal((1, 512)).astype(np.float32)
    assert_close(eng.probe_attention(0, x1), om.attention(0, x1), 1e-4, 1e-3, "attention (next token over the cache)")
    eng.close()


@pytest.mark.parametrize("kw", [dict(kv_dtype="f32"), dict(rope_mode="absolute"), dict(kv_page_tokens=4)])
def test_switches(gpu, oracle, kw):
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=96, **kw)
    prompt = synth.prompt_tokens(33, spec.vocab_size, 3)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, f"prefill {kw}")
    assert eng.generate(prompt, 12, stop_on_eos=False) == om.generate(prompt, 12, stop_on_eos=False)
    eng.close()


def test_chunked_prefill_matches(gpu, oracle):
    """A prompt longer than the engine's prefill chunk (512 tokens) keeps call-relative RoPE indices."""
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=1, hidden=256, heads=4, kv=4, ffn=256, vocab=500)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=800)
    prompt = synth.prompt_tokens(700, spec.vocab_size, 1)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "700-token prefill")
    eng.close()


def test_batched_sequences_match_single(gpu, oracle):
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=64, max_seqs=5)
    prompts = [synth.prompt_tokens(n, spec.vocab_size, i).tolist() for i, n in enumerate([3, 20, 1, 9, 16])]
    logits, nxt = eng.forward_batch([0, 1, 2, 3, 4], prompts)
    for i, p in enumerate(prompts):
        om.kv_clear()
        want = om.forward(p)
        assert_close(logits[i], want, LOGIT_ABS, LOGIT_REL, f"sequence {i}")
        assert nxt[i] == oracle.argmax(want)
    # four decode steps for all five sequences on the device == four oracle steps each
    toks, _ms = eng.decode_loop([0, 1, 2, 3, 4], nxt, 4)
    for i, p in enumerate(prompts):
        ref = om.generate(p, 5, stop_on_eos=False)
        assert [int(nxt[i])] + toks[:, i].tolist() == ref
    assert eng.counters()["kv_pages_in_use"] == sum((len(p) + 4 + 15) // 16 for p in prompts)
    eng.kv_clear(1)
    assert eng.kv_length(1) == 0 and eng.kv_length(0) == 3 + 4
    eng.close()


def test_many_sequences_decode_through_the_tensor_core_gemm(gpu, oracle):
    """Twelve sequences: the ragged prefill (49 tokens in one call) and every decode step (12 tokens) go through the
    many-token tcgen05 product instead of the matrix-vector kernels; tokens must still equal the oracle's, sequence by
    sequence, and a second engine must reproduce the first bit for bit (one issuing order, no atomics)."""
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=2, hidden=512, heads=4, kv=2, ffn=768, vocab=640)
    lens = [3, 7, 1, 9, 2, 5, 4, 6, 1, 3, 2, 6]
    ids = list(range(12))
    prompts = [synth.prompt_tokens(n, spec.vocab_size, 40 + i).tolist() for i, n in enumerate(lens)]
    runs = []
    for _ in range(2):
        eng, om = make_pair(gpu, oracle, spec, max_seq_len=48, max_seqs=12)
        logits, nxt = eng.forward_batch(ids, prompts)
        toks, _ms = eng.decode_loop(ids, nxt, 6)
        runs.append((logits.copy(), nxt.copy(), toks.copy()))
        if len(runs) == 1:
            for i, p in enumerate(prompts):
                om.kv_clear()
                assert_close(logits[i], om.forward(p), LOGIT_ABS, LOGIT_REL, f"sequence {i}")
                ref, margins = om.generate(p, 7, stop_on_eos=False, want_margins=True)
                assert [int(nxt[i])] + toks[:, i].tolist() == ref, (i, margins)
        eng.close()
    assert np.array_equal(runs[0][0].view(np.uint32), runs[1][0].view(np.uint32))
    assert np.array_equal(runs[0][2], runs[1][2])


def test_batched_decode_attention_over_several_context_pieces(gpu, oracle):
    """80 sequences x 8 heads of 128 dims = 640 (token, head) pairs: past four per SM, so the batched decode step runs
    the split-context attention kernel with the context cut into 1024-key pieces and the pieces merged through the
    scratch partials.  Contexts sit on both sides of the piece edges (1023 / 1024 / 1025, 2047 / 2049, 4090) and most are
    short, so many (pair, piece) CTAs have no key at all and leave at once.  Prefill logits and four decode steps are
    compared with the oracle sequence by sequence."""
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=1, hidden=1024, heads=8, kv=2, ffn=512, vocab=512)
    special = [5, 1023, 1024, 1025, 2047, 2049, 2500, 4090]
    r = np.random.default_rng(5)
    lens = special + [int(v) for v in r.integers(1, 200, 80 - len(special))]
    ids = list(range(80))
    steps = 4
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=4096, max_seqs=80, kv_pool_tokens=sum((n + steps + 15) // 16 * 16 for n in lens))
    prompts = [synth.prompt_tokens(n, spec.vocab_size, 100 + i).tolist() for i, n in enumerate(lens)]
    logits, nxt = eng.forward_batch(ids, prompts)
    step_logits, cur = [], nxt.copy()
    for _ in range(steps):  # every sequence advances by one token per call: the 80-token batched decode step
        lg, cur = eng.forward_batch(ids, [[int(t)] for t in cur])
        step_logits.append(lg.copy())
    for i, p in enumerate(prompts):
        if i >= len(special) and i % 6:  # every special context and a sample of the short ones go through the oracle
            continue
        om.kv_clear()
        want = om.forward(p)
        assert_close(logits[i], want, LOGIT_ABS, LOGIT_REL, f"prefill of sequence {i} ({lens[i]} tokens)")
        for s_ in range(steps):
            tok = int(oracle.argmax(want))
            want = om.forward([tok])
            assert_close(step_logits[s_][i], want, LOGIT_ABS, LOGIT_REL, f"sequence {i} (context {lens[i]}), decode step {s_}")
    eng.close()


def test_prefill_attention_on_tensor_cores_ragged(gpu, oracle):
    """head_dim 128, f16 cache: calls of 16 tokens and more run the tiled tensor-core prefill attention.  Four sequences of
    70, 16, 129 and 33 tokens in ONE call (tiles end where a sequence ends; 129 = two full tiles and a one-token tile), then a
    second call that appends 20 to 40 tokens to each cache (tiles that start in the middle of a page and attend to keys of
    the earlier call), grouped-query heads (4 query heads over 2 kv heads).  Logits per sequence against the oracle."""
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=2, hidden=512, heads=4, kv=2, ffn=512, vocab=600)
    lens, more = [70, 16, 129, 33], [20, 40, 25, 31]
    ids = [0, 1, 2, 3]
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=192, max_seqs=4)
    p1 = [synth.prompt_tokens(n, spec.vocab_size, 200 + i).tolist() for i, n in enumerate(lens)]
    p2 = [synth.prompt_tokens(n, spec.vocab_size, 300 + i).tolist() for i, n in enumerate(more)]
    l1, _ = eng.forward_batch(ids, p1)
    l2, _ = eng.forward_batch(ids, p2)
    for i in ids:
        om.kv_clear()
        assert_close(l1[i], om.forward(p1[i]), LOGIT_ABS, LOGIT_REL, f"sequence {i}, first call")
        assert_close(l2[i], om.forward(p2[i]), LOGIT_ABS, LOGIT_REL, f"sequence {i}, second call over the cache of the first")
    eng.close()


def test_a_second_model_does_not_disturb_a_captured_decode_step(gpu, oracle):
    """Scratch that a captured decode graph points at belongs to its model: a small model captures its step, then a
    model with more heads is created on the same device (which used to regrow a shared buffer), and the small model
    must keep decoding the oracle's tokens."""
    from leafcutterllm_b200 import synth
    small = small_spec(12, 12, 12, layers=2, hidden=256, heads=2, kv=2, ffn=512, vocab=900)
    big = small_spec(12, 12, 12, layers=1, hidden=2048, heads=16, kv=16, ffn=512, vocab=600)
    eng, om = make_pair(gpu, oracle, small, max_seq_len=96)
    prompt = synth.prompt_tokens(20, small.vocab_size, 3)
    ref, margins = om.generate(prompt, 30, stop_on_eos=False, want_margins=True)
    assert eng.generate(prompt, 10, stop_on_eos=False) == ref[:10], margins   # captures the one-sequence step
    eng2 = synth.build_engine(big, 64, on_device=True)
    assert len(eng2.generate(synth.prompt_tokens(9, big.vocab_size, 4), 6, stop_on_eos=False)) == 6
    assert eng.generate(prompt, 30, stop_on_eos=False) == ref, margins         # replays the graph captured before eng2 existed
    eng2.close()
    assert eng.generate(prompt, 30, stop_on_eos=False) == ref, margins
    eng.close()


@pytest.mark.parametrize("other", [12, 13, 14])
def test_mixed_quant_types_like_q4_k_m(gpu, oracle, other):
    """A "Q4_K_M" file keeps attn_v and ffn_down in Q6_K while q, k, o, gate and up are Q4_K: the three projections of a
    layer then cannot be one matrix (three products per layer); the Q6_K matrices run through the int8 tensor-core kernel
    (fused norm, residual epilogue), the 8-token tiles of the prefill as two passes of it.
    other = 14: every matrix is Q6_K (one fused q/k/v matrix, SiLU(gate) * up epilogue on Q6_K); other = 13: the Q5_K + Q6_K
    mix of a "Q5_K_M" file (Q5_K through the Q4_K kernel's fifth-bit variant).
    Prefill (17 tokens: the unfused parts are interleaved into the q/k/v rows), decode and greedy tokens against the oracle."""
    from leafcutterllm_b200 import Engine, synth
    H, Fd, V, nh, nkv, L = 256, 512, 384, 2, 1, 2
    r = np.random.default_rng(8)

    def q6k(rows, cols):  # random blocks with small scales (no host quantiser for Q6_K): |w| stays below ~0.3
        raw = r.integers(0, 256, (rows * cols // 256, 210), dtype=np.uint8)
        raw[:, 192:208] = r.integers(-40, 41, (raw.shape[0], 16)).astype(np.int8).view(np.uint8)
        d = np.float16(r.uniform(2e-5, 2e-4, raw.shape[0])).view(np.uint16)
        raw[:, 208] = d & 0xFF
        raw[:, 209] = d >> 8
        return raw.ravel()

    def q5k(rows, cols):  # random blocks: 6-bit scales and mins as they come, small d and dmin
        raw = r.integers(0, 256, (rows * cols // 256, 176), dtype=np.uint8)
        for at in (0, 2):
            d = np.float16(r.uniform(2e-5, 2e-4, raw.shape[0])).view(np.uint16)
            raw[:, at] = d & 0xFF
            raw[:, at + 1] = d >> 8
        return raw.ravel()

    eng = Engine(H, L, nh, nkv, Fd, V, max_seq_len=64)
    om = oracle.OracleModel(H, L, nh, nkv, Fd, V, max_seq_len=64)
    hd = H // nh
    tensors = [("token_embd.weight", 12, (H, V)), ("output_norm.weight", 0, (H,)), ("output.weight", 14, (H, V))]
    for l in range(L):
        p = f"blk.{l}."
        tensors += [(p + "attn_norm.weight", 0, (H,)), (p + "attn_q.weight", other, (H, nh * hd)), (p + "attn_k.weight", other, (H, nkv * hd)),
                    (p + "attn_v.weight", 14, (H, nkv * hd)), (p + "attn_output.weight", other, (nh * hd, H)), (p + "ffn_norm.weight", 0, (H,)),
                    (p + "ffn_gate.weight", other, (H, Fd)), (p + "ffn_up.weight", other, (H, Fd)), (p + "ffn_down.weight", 14, (Fd, H))]
    for name, typ, dims in tensors:
        n = int(np.prod(dims))
        data = np.ones(n, np.float32).view(np.uint8) if typ == 0 else (q6k(dims[1], dims[0]) if typ == 14 else (q5k(dims[1], dims[0]) if typ == 13 else synth.host_tensor(typ, 21, name, n)))
        eng.set_tensor(name, typ, dims, data)
        om.set_tensor(name, typ, list(dims), data)
    eng.finalize()
    prompt = synth.prompt_tokens(17, V, 2)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill logits, mixed types")
    nxt = 5
    assert_close(eng.forward([nxt]), om.forward([nxt]), LOGIT_ABS, LOGIT_REL, "decode logits, mixed types")
    ref, margins = om.generate(prompt, 10, stop_on_eos=False, want_margins=True)
    assert eng.generate(prompt, 10, stop_on_eos=False) == ref, margins
    eng.close()


def test_error_paths(gpu):
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=1)
    eng = gpu.Engine(spec.hidden_size, 1, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=32)
    with pytest.raises(gpu.LeafcutterError) as e:
        eng.forward([1])
    assert e.value.status == -7  # not finalized
    with pytest.raises(gpu.LeafcutterError) as e:
        eng.finalize()
    assert e.value.status == -6  # missing tensors (the reference panics: engine.rs:84,97,101)
    eng.close()
    eng = synth.build_engine(spec, 32, on_device=True)
    with pytest.raises(gpu.LeafcutterError) as e:
        eng.forward(list(range(33)))
    assert e.value.status == -5  # KV capacity
    with pytest.raises(gpu.LeafcutterError) as e:
        eng.generate([1, 2], 4, temperature=0.7)
    assert e.value.status == -2
    out = eng.forward([10 ** 6])  # engine.rs:137-141: out-of-range id -> zero embedding row, still finite
    assert np.isfinite(out).all()
    eng.close()


def test_tiny_shape_reduced_depth(gpu, oracle):
    """TinyLlama-1.1B dims (hidden 2048, 32 q / 4 kv heads, FFN 5632, vocab 32000, Q4_0 + Q8_0), 3 layers."""
    from leafcutterllm_b200 import synth
    spec = synth.TINY.with_layers(3)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=64, on_device=True)
    prompt = synth.prompt_tokens(32, spec.vocab_size)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill")
    toks = eng.generate(prompt, 16, stop_on_eos=False)
    ref, margins = om.generate(prompt, 16, stop_on_eos=False, want_margins=True)
    assert toks == ref, margins
    eng.close()


@pytest.mark.parametrize("layers,heads,kv", [(2, 4, 2), (3, 2, 2), (3, 4, 4), (3, 8, 2)])
def test_single_sequence_decode_head_dim_128(gpu, oracle, layers, heads, kv):
    """head_dim 128 + Q4_K + f16 cache: single-sequence decode steps run the streaming attention kernel and the
    tensor-core matrix-vector kernel from a captured graph.  Same tokens as the oracle through the device-resident
    loop, and the oracle's logits step by step through the host API."""
    from leafcutterllm_b200 import synth
    spec = small_spec(12, 12, 12, layers=layers, hidden=128 * heads, heads=heads, kv=kv, ffn=768, vocab=1500)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=160)
    prompt = synth.prompt_tokens(40, spec.vocab_size, 5)
    ref, margins = om.generate(prompt, 48, stop_on_eos=False, want_margins=True)
    toks = eng.generate(prompt, 48, stop_on_eos=False)
    assert toks == ref, margins
    eng.kv_clear()
    om.kv_clear()
    got = eng.forward(prompt)
    want = om.forward(prompt)
    for step in range(6):
        nxt = int(np.argmax(want))
        got, want = eng.forward([nxt]), om.forward([nxt])
        assert_close(got, want, LOGIT_ABS, LOGIT_REL, f"step {step}")
    eng.close()


def test_decode_ignores_unwritten_cache_rows(gpu, oracle):
    """The rows of a KV page beyond the current position hold whatever the pool's memory held before (the pools are
    not cleared).  Their softmax weight is zero, but 0 * NaN is NaN: kernels must not touch them.  Device memory is
    poisoned with f16 NaNs and released just before the model is built, and decoding crosses page boundaries."""
    import ctypes as C
    from leafcutterllm_b200 import synth, _capi
    lib = _capi.load()
    bufs = []
    poison = np.full(64 << 20, 0xFF, np.uint8)
    for _ in range(6):
        p = C.c_void_p()
        _capi.check(lib.lc_dev_alloc(poison.nbytes, C.byref(p)))
        _capi.check(lib.lc_dev_upload(p, poison.ctypes.data_as(C.c_void_p), poison.nbytes))
        bufs.append(p)
    for p in bufs:
        lib.lc_dev_free(p)
    spec = small_spec(12, 12, 12, layers=2, hidden=256, heads=2, kv=2, ffn=768, vocab=1500)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=160)
    prompt = synth.prompt_tokens(30, spec.vocab_size, 9)
    ref, margins = om.generate(prompt, 40, stop_on_eos=False, want_margins=True)
    toks = eng.generate(prompt, 40, stop_on_eos=False)
    assert toks == ref, margins
    eng.close()
