"""The benchmark configurations at their real shapes: config 1 (TinyLlama shape, Q4_0 + Q8_0) against the committed
oracle fixture, config 2 (7B shape, Q4_K) at reduced depth against the oracle and at full depth through properties
that do not need the oracle."""
import json
import os

import numpy as np
import pytest

from conftest import assert_close, make_pair

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
LOGIT_ABS, LOGIT_REL = 1e-2, 1e-3


def test_config1_full_depth_matches_the_oracle_fixture(gpu):
    """22 layers, 32-token prompt, 128 greedy steps: token-identical to the CPU oracle (tests/golden/make_cfg1_golden.py)."""
    from leafcutterllm_b200 import synth
    path = os.path.join(HERE, "golden", "cfg1_tinyllama_q4_0.json")
    if not os.path.exists(path):
        pytest.skip("fixture not generated")
    gold = json.load(open(path))
    eng = synth.build_engine(synth.TINY, 256, on_device=True)
    prompt = np.array(gold["prompt"], np.int64)
    assert np.array_equal(prompt, synth.prompt_tokens(32, synth.TINY.vocab_size, 0))
    logits = eng.forward(prompt)
    assert_close(logits[:16], gold["prefill_logits_first16"], LOGIT_ABS, LOGIT_REL, "prefill logits")
    assert abs(np.sqrt((logits.astype(np.float64) ** 2).sum()) - gold["prefill_logits_l2"]) < 1e-3 * gold["prefill_logits_l2"]
    toks = eng.generate(prompt, 129, stop_on_eos=False)
    bad = [i for i, (a, b) in enumerate(zip(toks, gold["tokens"])) if a != b]
    assert not bad, f"first divergence at step {bad[0]}, oracle top-2 margin there {gold['top2_margins'][bad[0]]}"
    assert eng.kv_length() == 32 + 128
    assert eng.kv_memory_bytes() == (32 + 128) * 22 * 2 * 4 * 64 * 2  # 22 KiB per token, f16
    eng.close()


def test_config2_two_layers_matches_the_oracle_fixture(gpu):
    """7B shape at two layers, 2048-token prompt, 32 decode steps at contexts 2048 .. 2079 (tests/golden/make_cfg2_golden.py):
    the single-sequence decode step at the benchmark's context length -- the streaming attention kernel with ~28 pages per
    CTA and every head merged across several CTAs, the 4096- and 11008-wide Q4_K matrix-vector products -- against the
    CPU oracle, logits step by step through the host API and tokens through the device-resident loop."""
    from leafcutterllm_b200 import synth
    path = os.path.join(HERE, "golden", "cfg2_llama7b_q4_k_2layers.json")
    gold = json.load(open(path))
    spec = synth.LLAMA7B.with_layers(2)
    n, steps = gold["prompt_len"], len(gold["tokens"]) - 1
    eng = synth.build_engine(spec, n + steps + 16, on_device=True)
    prompt = synth.prompt_tokens(n, spec.vocab_size, 0)
    assert prompt[:8].tolist() == gold["prompt_head"]

    def check(logits, g, what):
        assert_close(logits[:16], g["first16"], LOGIT_ABS, LOGIT_REL, what)
        assert abs(np.sqrt((logits.astype(np.float64) ** 2).sum()) - g["l2"]) < 1e-3 * g["l2"], what
        assert int(np.argmax(logits)) == g["argmax"] or g["margin"] < 1e-3, (what, g["margin"])

    check(eng.forward(prompt), gold["steps"][0], "prefill")
    for i in range(1, steps + 1):
        check(eng.forward([gold["tokens"][i - 1]]), gold["steps"][i], f"decode step {i} (context {n + i - 1})")
    assert eng.kv_length() == n + steps
    toks = eng.generate(prompt, steps + 1, stop_on_eos=False)  # prefill again, then the steps as graph replays on the device
    bad = [i for i, (a, b) in enumerate(zip(toks, gold["tokens"])) if a != b]
    assert not bad, f"first divergence at step {bad[0]}, oracle top-2 margin there {gold['steps'][bad[0]]['margin']}"
    eng.close()


def test_7b_shape_two_layers_against_the_oracle(gpu, oracle):
    from leafcutterllm_b200 import synth
    spec = synth.LLAMA7B.with_layers(2)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=96, on_device=True)
    prompt = synth.prompt_tokens(24, spec.vocab_size, 2)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill")
    ref, margins = om.generate(prompt, 12, stop_on_eos=False, want_margins=True)
    assert eng.generate(prompt, 12, stop_on_eos=False) == ref, margins
    eng.close()


def test_7b_full_depth_paths_agree(gpu):
    """32 layers, 3.8 GB of Q4_K weights synthesised on the device.  Without an oracle at this size: the device-resident
    loop and the per-step host API must produce the same greedy tokens and finite logits."""
    from leafcutterllm_b200 import synth
    spec = synth.LLAMA7B
    prompt = synth.prompt_tokens(300, spec.vocab_size, 9)
    eng = synth.build_engine(spec, 512, on_device=True)
    c = eng.counters()
    assert c["sanitize_hits"] == 0 and abs(c["weight_bytes"] - 3.79e9) < 0.05e9
    a = eng.generate(prompt, 24, stop_on_eos=False)               # device loop
    seen = []
    b = eng.generate(prompt, 24, stop_on_eos=False, on_token=seen.append)  # one host round trip per token
    assert a == b == seen
    logits = eng.forward([a[-1]])
    assert np.isfinite(logits).all() and logits.std() > 0
    assert eng.kv_length() == 300 + 23 + 1
    assert eng.counters()["kv_pages_in_use"] == (324 + 15) // 16
    step_bytes = eng.counters()["algo_bytes_last_step"]
    assert abs(step_bytes - (3.7165e9 + 324 * 512 * 1024)) < 0.02e9  # weights once + 512 KiB of f16 KV per cached token
    eng.close()
