"""A model cut across ranks (tensor-parallel attention and FFN, expert-parallel mixture layers), all ranks held by ONE
process on ONE GPU: the same cut kernels and rank-ordered sums a multi-GPU run uses, with the sums taken by one kernel
over all ranks' rows.  Everything is compared with the CPU oracle of the WHOLE model: cutting changes the grouping of
the k-sums, so logits are held to the usual tolerance and greedy tokens must still be identical."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu
LOGIT_ABS, LOGIT_REL = 1e-2, 1e-3


def build_cut(gpu, oracle, spec, tp, max_seq_len, on_device=False, **kw):
    """tp engines (ranks 0 .. tp-1, each handed the whole tensors and keeping its part), grouped; and the oracle."""
    from leafcutterllm_b200 import Engine, synth
    engines = []
    for r in range(tp):
        eng = Engine(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                     max_seq_len=max_seq_len, rope_theta=spec.rope_theta, n_experts=spec.n_experts, top_k=spec.top_k, tp_size=tp, tp_rank=r, **kw)
        for name, typ, dims, kind in spec.tensors():
            if kind == "ones" or not on_device:
                eng.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
            else:
                eng.synth_tensor(name, typ, dims, synth.WEIGHT_SEED, synth.SIGMA)
        eng.finalize()
        engines.append(eng)
    lead = Engine.group(engines)
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                            max_seq_len=max_seq_len, rope_theta=spec.rope_theta, n_experts=spec.n_experts, top_k=spec.top_k)
    for name, typ, dims, kind in spec.tensors():
        om.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    return lead, engines, om


def dense_spec(layers=2, heads=8, kv=4, ffn=1024, vocab=800, typ=12):
    from leafcutterllm_b200.synth import ModelSpec
    return ModelSpec("cut", layers, 128 * heads, heads, kv, ffn, vocab, 10000.0, typ, typ, typ)


@pytest.mark.parametrize("tp,on_device", [(2, False), (4, False), (2, True)])
def test_cut_dense_model_matches_the_whole_oracle(gpu, oracle, tp, on_device):
    from leafcutterllm_b200 import synth
    spec = dense_spec()
    lead, engines, om = build_cut(gpu, oracle, spec, tp, 96, on_device=on_device)
    prompt = synth.prompt_tokens(19, spec.vocab_size, 2)
    assert_close(lead.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, f"prefill logits, {tp} ranks")
    for step in range(3):
        assert_close(lead.forward([7 + step]), om.forward([7 + step]), LOGIT_ABS, LOGIT_REL, f"decode step {step}, {tp} ranks")
    ref, margins = om.generate(prompt, 24, stop_on_eos=False, want_margins=True)
    assert lead.generate(prompt, 24, stop_on_eos=False) == ref, margins      # device loop: one graph holds every rank's kernels
    assert lead.kv_memory_bytes() == om.kv_memory_bytes()
    for e in engines:
        e.close()


def test_cut_model_batched_decode(gpu, oracle):
    """Nine sequences: the step runs the many-token tensor-core product on every rank's part."""
    from leafcutterllm_b200 import synth
    spec = dense_spec(layers=2)
    lens = [3, 7, 1, 9, 2, 5, 4, 6, 2]
    ids = list(range(len(lens)))
    lead, engines, om = build_cut(gpu, oracle, spec, 2, 48, max_seqs=len(lens))
    prompts = [synth.prompt_tokens(n, spec.vocab_size, 70 + i).tolist() for i, n in enumerate(lens)]
    logits, nxt = lead.forward_batch(ids, prompts)
    toks, _ms = lead.decode_loop(ids, nxt, 5)
    for i, p in enumerate(prompts):
        om.kv_clear()
        assert_close(logits[i], om.forward(p), LOGIT_ABS, LOGIT_REL, f"sequence {i}")
        ref, margins = om.generate(p, 6, stop_on_eos=False, want_margins=True)
        assert [int(nxt[i])] + toks[:, i].tolist() == ref, (i, margins)
    for e in engines:
        e.close()


def test_cut_model_tied_head_and_other_types(gpu, oracle):
    """Q8_0 layers (column parts on 32-element blocks) and a head tied to the embedding: every rank reads its vocabulary
    rows of the one embedding table."""
    from leafcutterllm_b200.synth import ModelSpec
    from leafcutterllm_b200 import synth
    spec = ModelSpec("cut-tied", 1, 256, 4, 2, 384, 600, 10000.0, 8, 8, 8, tied_head=True)
    lead, engines, om = build_cut(gpu, oracle, spec, 2, 64)
    prompt = synth.prompt_tokens(11, spec.vocab_size, 6)
    assert_close(lead.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill")
    assert_close(lead.forward([3]), om.forward([3]), LOGIT_ABS, LOGIT_REL, "decode")
    for e in engines:
        e.close()


@pytest.mark.parametrize("tp", [2, 4])
def test_expert_parallel_mixture_model(gpu, oracle, tp):
    """Attention cut by heads, experts dealt whole to the ranks (four experts over two or four ranks): the router runs on
    every rank on identical rows, each rank adds the chosen experts it holds, the sum over the ranks completes the layer."""
    from leafcutterllm_b200.synth import ModelSpec
    from leafcutterllm_b200 import synth
    spec = ModelSpec("cut-moe", 2, 1024, 8, 4, 512, 800, 10000.0, 12, 12, 12, n_experts=4, top_k=2)
    lead, engines, om = build_cut(gpu, oracle, spec, tp, 200)
    prompt = synth.prompt_tokens(21, spec.vocab_size, 8)
    assert_close(lead.forward(prompt), om.forward(prompt), LOGIT_ABS, LOGIT_REL, "prefill (grouped expert launch)")
    assert_close(lead.forward([5]), om.forward([5]), LOGIT_ABS, LOGIT_REL, "decode")
    ref, margins = om.generate(prompt, 16, stop_on_eos=False, want_margins=True)
    assert lead.generate(prompt, 16, stop_on_eos=False) == ref, margins
    lead.kv_clear()
    om.kv_clear()
    long_prompt = synth.prompt_tokens(130, spec.vocab_size, 9)
    assert_close(lead.forward(long_prompt), om.forward(long_prompt), LOGIT_ABS, LOGIT_REL, "130-token prefill (every local expert on every token)")
    for e in engines:
        e.close()


def test_cut_model_call_order_errors(gpu):
    from leafcutterllm_b200 import Engine, synth
    spec = dense_spec(layers=1)
    with pytest.raises(gpu.LeafcutterError) as e:   # 8 heads cannot go to 3 ranks
        Engine(spec.hidden_size, 1, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=32, tp_size=3, tp_rank=0)
    assert e.value.status == -1
    eng = Engine(spec.hidden_size, 1, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=32, tp_size=2, tp_rank=1)
    for name, typ, dims, kind in spec.tensors():
        eng.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    eng.finalize()
    with pytest.raises(gpu.LeafcutterError) as e:   # a lone rank has nobody to sum with
        eng.forward([1, 2, 3])
    assert e.value.status == -7
    eng.close()
