"""sampler::sample_top_p (rust/src/inference/sampler.rs:6-50): greedy and, with the uniform draw handed in, the stochastic
branch -- the GPU pick against the CPU restatement, and seeded generation through the engine."""
import numpy as np
import pytest


def test_oracle_sampler_known_answers(oracle):
    # the reference's own tests (sampler.rs:56-68): greedy picks index 1; any draw gives a valid index
    assert oracle.sample_top_p([0.1, 0.5, 0.3], 0.0, 0.9) == 1
    assert oracle.sample_top_p([1.0, 2.0, 3.0], 1.0, 1.0, 0.5) < 3
    # softmax of (1, 2, 3) = (0.0900, 0.2447, 0.6652); sorted: index 2, 1, 0
    assert [oracle.sample_top_p([1.0, 2.0, 3.0], 1.0, 1.0, u) for u in (0.0, 0.66, 0.67, 0.90, 0.92, 0.999)] == [2, 2, 1, 1, 0, 0]
    # top_p = 0.5: the first probability already exceeds it, only index 2 is kept
    assert {oracle.sample_top_p([1.0, 2.0, 3.0], 1.0, 0.5, u) for u in (0.0, 0.5, 0.999)} == {2}
    # top_p = 0.7: 0.6652 does not exceed it, 0.9099 does: two kept, renormalised over 0.9099
    assert [oracle.sample_top_p([1.0, 2.0, 3.0], 1.0, 0.7, u) for u in (0.0, 0.72, 0.74, 0.999)] == [2, 2, 1, 1]
    # a low temperature sharpens: (1, 2, 3) / 0.1 -> nearly all mass on index 2
    assert oracle.sample_top_p([1.0, 2.0, 3.0], 0.1, 1.0, 0.9999) == 2
    # equal probabilities keep index order (stable sort, :23-25)
    assert [oracle.sample_top_p([0.0] * 4, 1.0, 1.0, u) for u in (0.1, 0.3, 0.6, 0.9)] == [0, 1, 2, 3]
    # greedy: ties go to the last maximum (max_by keeps the last of equal elements, :9)
    assert oracle.sample_top_p([1.0, 3.0, 3.0, 2.0], 0.0, 1.0) == 2


def _cases(rng, n):
    yield rng.normal(0.0, 2.0, n).astype(np.float32)                      # spread like decoder logits
    yield (rng.normal(0.0, 6.0, n)).astype(np.float32)                    # peaked
    yield np.round(rng.normal(0.0, 1.5, n) * 2).astype(np.float32) / 2    # many exact ties
    yield np.zeros(n, np.float32)                                         # all equal


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 3, 1000, 8192, 8193, 32000, 50257, 151936])
def test_sample_top_p_equals_the_oracle(gpu, oracle, n):
    from leafcutterllm_b200 import sample_top_p
    rng = np.random.default_rng(n)
    checked = 0
    for logits in _cases(rng, n):
        for temperature, top_p in ((1.0, 1.0), (0.8, 0.9), (0.3, 0.5), (1.7, 0.95), (1.0, 0.0), (1.0, 2.0)):
            for u in (0.0, float(rng.random()), float(rng.random()), 1.0 - 2.0 ** -24):
                want = oracle.sample_top_p(logits, temperature, top_p, u)
                got = sample_top_p(logits, temperature, top_p, u)
                assert got == want, (n, temperature, top_p, u)
                checked += 1
    assert checked == 4 * 6 * 4
    assert sample_top_p(np.array([0.1, 0.5, 0.3], np.float32), 0.0, 0.9) == 1          # sampler.rs:56-60
    assert sample_top_p(np.array([1.0, 3.0, 3.0, 2.0], np.float32), -1.0, 1.0) == 2    # greedy for temperature <= 0


@pytest.mark.gpu
def test_sampling_distribution_follows_the_probabilities(gpu):
    """A sweep of draws over [0, 1) returns each kept token in proportion to its renormalised probability."""
    from leafcutterllm_b200 import sample_top_p
    logits = np.array([2.0, 0.0, 1.0, -1.0, 3.0], np.float32)
    p = np.exp(logits - logits.max())
    p /= p.sum()
    draws = (np.arange(400) + 0.5) / 400
    counts = np.bincount([sample_top_p(logits, 1.0, 1.0, float(u)) for u in draws], minlength=5)
    assert np.abs(counts / 400 - p).max() < 0.006
    kept = np.bincount([sample_top_p(logits, 1.0, 0.8, float(u)) for u in draws], minlength=5)   # 0.636 + 0.234 > 0.8
    assert kept[[1, 2, 3]].sum() == 0 and abs(kept[4] / 400 - p[4] / (p[4] + p[0])) < 0.006


@pytest.mark.gpu
def test_sample_top_p_rejects_bad_arguments(gpu):
    from leafcutterllm_b200 import LeafcutterError, sample_top_p
    with pytest.raises(ValueError):
        sample_top_p(np.zeros(4, np.float32), 1.0, 0.9)           # no draw given
    with pytest.raises(LeafcutterError):
        sample_top_p(np.zeros(0, np.float32), 1.0, 0.9, 0.5)      # the reference panics on an empty slice


@pytest.mark.gpu
def test_seeded_generation_uses_the_documented_draws(gpu, oracle):
    """generate(temperature > 0, seed) = forward, sample_top_p with seeded_uniform(seed, i), forward, ... (engine.rs:51-76)."""
    from conftest import make_pair
    from leafcutterllm_b200 import LeafcutterError, seeded_uniform, synth
    spec = synth.TINY.with_layers(2)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=64)
    prompt = synth.prompt_tokens(9, spec.vocab_size).tolist()
    with pytest.raises(LeafcutterError, match="LC_ERR_UNSUPPORTED"):
        eng.generate(prompt, 4, temperature=0.8, top_p=0.9)      # no seed yet: the reference's unseeded branch is not reproduced
    got = eng.generate(prompt, 10, temperature=0.9, top_p=0.95, stop_on_eos=False, seed=42)
    again = eng.generate(prompt, 10, temperature=0.9, top_p=0.95, stop_on_eos=False, seed=42)
    other = eng.generate(prompt, 10, temperature=0.9, top_p=0.95, stop_on_eos=False, seed=43)
    assert got == again and got != other and len(got) == 10
    draws = [seeded_uniform(42, i) for i in range(10)]
    assert all(0.0 <= u < 1.0 for u in draws) and len(set(draws)) == 10
    eng.kv_clear()
    want, feed = [], list(prompt)
    for i in range(10):
        logits = eng.forward(feed)
        tok = oracle.sample_top_p(logits, 0.9, 0.95, draws[i])
        want.append(tok)
        feed = [tok]
    assert got == want
    assert got != eng.generate(prompt, 10, stop_on_eos=False)     # and it is not the greedy sequence
    # the callback sees the sampled tokens one by one
    seen = []
    assert eng.generate(prompt, 5, temperature=0.9, top_p=0.95, stop_on_eos=False, on_token=seen.append, seed=42) == got[:5] == seen
    eng.close()
