"""Mixture-of-experts FFN (BASELINE config 4's layer type) on the GPU against the CPU oracle.

The reference has no mixture-of-experts code, so the oracle's `moe_forward` is this project's own definition (router
logits in f32, top-k with equal logits going to the higher expert index, softmax over the chosen logits, chosen experts
summed in ascending index): parity here is unpinned by the reference.  What the tests pin is that the CUDA path -- the
router kernel, the one-launch grouped expert products, the every-expert path of long calls, the weighted sum -- computes
that definition on the same bytes."""
import numpy as np
import pytest

from conftest import assert_close, make_pair

pytestmark = pytest.mark.gpu
LOGIT_ABS, LOGIT_REL = 1e-2, 1e-3


def moe_spec(layer_type=12, layers=2, hidden=256, heads=2, kv=2, ffn=512, vocab=700, n_experts=4, top_k=2):
    from leafcutterllm_b200.synth import ModelSpec
    return ModelSpec("moe", layers, hidden, heads, kv, ffn, vocab, 10000.0, layer_type, 12 if layer_type == 12 else 8, 12 if layer_type == 12 else 8,
                     n_experts=n_experts, top_k=top_k)


@pytest.mark.parametrize("n_experts,top_k", [(4, 2), (8, 2), (8, 1), (5, 3)])
def test_moe_prefill_decode_and_tokens(gpu, oracle, n_experts, top_k):
    """17-token prefill (grouped launch, several passes per weight tile where an expert received more slots than the token
    tile), single-token decode steps (grouped launch, one token) and greedy tokens."""
    from leafcutterllm_b200 import synth
    spec = moe_spec(n_experts=n_experts, top_k=top_k)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=96)
    prompt = synth.prompt_tokens(17, spec.vocab_size, 3)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill logits")
    for step in range(3):
        tok = 11 + step
        assert_close(eng.forward([tok]), om.forward([tok]), LOGIT_ABS, LOGIT_REL, f"decode step {step}")
    ref, margins = om.generate(prompt, 20, stop_on_eos=False, want_margins=True)
    assert eng.generate(prompt, 20, stop_on_eos=False) == ref, margins
    eng.close()


def test_moe_long_call_runs_every_expert(gpu, oracle):
    """A 150-token prefill is past the grouped launch's 64 tokens: every expert runs on every token through the
    many-token product and the sum keeps the chosen ones."""
    from leafcutterllm_b200 import synth
    spec = moe_spec(layers=1, n_experts=4, top_k=2)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=192)
    prompt = synth.prompt_tokens(150, spec.vocab_size, 5)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "150-token prefill")
    assert_close(eng.forward([9]), om.forward([9]), LOGIT_ABS, LOGIT_REL, "decode after it")
    eng.close()


def test_moe_batched_decode(gpu, oracle):
    """Twelve sequences decode together: the grouped launch runs two passes per expert where an expert received more than
    eight tokens; tokens must equal the oracle's sequence by sequence."""
    from leafcutterllm_b200 import synth
    spec = moe_spec(layers=2, n_experts=4, top_k=2)
    lens = [3, 7, 1, 9, 2, 5, 4, 6, 1, 3, 2, 6]
    ids = list(range(12))
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=48, max_seqs=12)
    prompts = [synth.prompt_tokens(n, spec.vocab_size, 60 + i).tolist() for i, n in enumerate(lens)]
    logits, nxt = eng.forward_batch(ids, prompts)
    toks, _ms = eng.decode_loop(ids, nxt, 5)
    for i, p in enumerate(prompts):
        om.kv_clear()
        assert_close(logits[i], om.forward(p), LOGIT_ABS, LOGIT_REL, f"sequence {i}")
        ref, margins = om.generate(p, 6, stop_on_eos=False, want_margins=True)
        assert [int(nxt[i])] + toks[:, i].tolist() == ref, (i, margins)
    eng.close()


def test_moe_other_quant_types(gpu, oracle):
    """Q4_0 experts have no grouped kernel: every call runs every expert through the ordinary products."""
    from leafcutterllm_b200 import synth
    spec = moe_spec(layer_type=2, layers=1, n_experts=3, top_k=2)
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=64)
    prompt = synth.prompt_tokens(9, spec.vocab_size, 1)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill")
    assert_close(eng.forward([4]), om.forward([4]), LOGIT_ABS, LOGIT_REL, "decode")
    eng.close()


@pytest.mark.parametrize("top_k", [1, 2])
def test_moe_router_ties_go_to_the_higher_expert(gpu, oracle, top_k):
    """Experts 1, 2 and 3 get the same router row, scaled up so that they lead for most tokens: their logits are equal
    bit for bit, and the pick must be expert 3 (then 2), as the oracle's rule says.  The experts' weights differ, so a
    different pick changes the logits."""
    from leafcutterllm_b200 import Engine, synth
    spec = moe_spec(layers=1, n_experts=4, top_k=top_k)
    H, E = spec.hidden_size, spec.n_experts
    r = np.random.default_rng(3)
    router = (0.02 * r.standard_normal((E, H))).astype(np.float32)
    router[1] = router[2] = router[3] = 4.0 * router[3]
    eng = Engine(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=64,
                 n_experts=E, top_k=top_k)
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                            max_seq_len=64, n_experts=E, top_k=top_k)
    for name, typ, dims, kind in spec.tensors():
        data = router.view(np.uint8).ravel() if name.endswith("ffn_gate_inp.weight") else synth.tensor_bytes(spec, name, typ, dims, kind)
        eng.set_tensor(name, typ, dims, data)
        om.set_tensor(name, typ, dims, data)
    eng.finalize()
    prompt = synth.prompt_tokens(12, spec.vocab_size, 2)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill with tied router rows")
    assert_close(eng.forward([5]), om.forward([5]), LOGIT_ABS, LOGIT_REL, "decode with tied router rows")
    eng.close()


def test_moe_stacked_expert_tensors(gpu, oracle):
    """GGUF files of mixture models carry one three-dimensional tensor per projection (blk.N.ffn_gate_exps.weight, ...):
    expert e is rows [e * n, (e + 1) * n).  Same bytes, same logits as the one-tensor-per-expert form the oracle takes."""
    from leafcutterllm_b200 import Engine, synth
    spec = moe_spec(layers=1, n_experts=4, top_k=2)
    E, H, F = spec.n_experts, spec.hidden_size, spec.intermediate_size
    eng = Engine(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=64,
                 n_experts=E, top_k=2)
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                            max_seq_len=64, n_experts=E, top_k=2)
    stacks = {}
    for name, typ, dims, kind in spec.tensors():
        data = synth.tensor_bytes(spec, name, typ, dims, kind)
        om.set_tensor(name, typ, dims, data)
        if ".expert." in name:
            which = name.split(".")[-2]                    # ffn_gate / ffn_up / ffn_down
            stacks.setdefault(which, []).append((typ, dims, data))
        else:
            eng.set_tensor(name, typ, dims, data)
    for which, parts in stacks.items():
        typ, dims = parts[0][0], parts[0][1]
        eng.set_tensor(f"blk.0.{which}_exps.weight", typ, (dims[0], dims[1], E), np.concatenate([p[2] for p in parts]))
    eng.finalize()
    prompt = synth.prompt_tokens(10, spec.vocab_size, 4)
    assert_close(eng.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill, stacked expert tensors")
    eng.close()


def test_moe_config_errors(gpu):
    with pytest.raises(gpu.LeafcutterError) as e:
        gpu.Engine(256, 1, 2, 2, 512, 100, max_seq_len=16, n_experts=4, top_k=5)
    assert e.value.status == -1
    with pytest.raises(gpu.LeafcutterError) as e:
        gpu.Engine(256, 1, 2, 2, 512, 100, max_seq_len=16, n_experts=65, top_k=2)
    assert e.value.status == -1


def test_moe_long_expert_rows(gpu, oracle):
    """Experts whose down projection reads 8192-element rows (32 units per row, two per warp): the grouped launch reads the
    fixed-point planes of each unit from global memory job by job, so the row length does not limit the token tile."""
    from leafcutterllm_b200 import synth
    spec = moe_spec(layers=1, hidden=256, ffn=8192, n_experts=4, top_k=2)
    lens = [3, 7, 1, 9, 2, 5, 4, 6, 1, 3, 2, 6]
    ids = list(range(12))
    eng, om = make_pair(gpu, oracle, spec, max_seq_len=48, max_seqs=12)
    prompts = [synth.prompt_tokens(n, spec.vocab_size, 90 + i).tolist() for i, n in enumerate(lens)]
    logits, nxt = eng.forward_batch(ids, prompts)
    toks, _ms = eng.decode_loop(ids, nxt, 3)
    for i, p in enumerate(prompts):
        om.kv_clear()
        assert_close(logits[i], om.forward(p), LOGIT_ABS, LOGIT_REL, f"sequence {i}")
        ref, margins = om.generate(p, 4, stop_on_eos=False, want_margins=True)
        assert [int(nxt[i])] + toks[:, i].tolist() == ref, (i, margins)
    eng.close()
