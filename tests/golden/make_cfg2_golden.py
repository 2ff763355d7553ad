"""Generates tests/golden/cfg2_llama7b_q4_k_2layers.json: the CPU oracle's results for BASELINE config 2 (Llama-2-7B
shape, Q4_K throughout) at TWO of its 32 layers: a 2048-token seeded prompt is prefilled, then 32 greedy decode steps
run one token at a time over the growing cache (contexts 2048 .. 2079, so the steps cross two page boundaries of the
16-token KV pages), f16 KV cache, call-relative RoPE.  Kept per step: the token, the top-2 margin, the first 16 logits
and the L2 norm of the logits.  The depth is cut so that the CPU finishes in minutes; every per-layer code path of the
single-sequence decode step (32 heads of 128 dims over ~2050 cached keys, 4096 / 11008-wide Q4_K products) runs at its
full size.  The GPU test compares against the committed file, so the oracle never has to run this on the GPU box.

    python tests/golden/make_cfg2_golden.py
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from leafcutterllm_b200 import synth  # noqa: E402

PROMPT_LEN, STEPS, LAYERS = 2048, 32, 2


def main():
    spec = synth.LLAMA7B.with_layers(LAYERS)
    t0 = time.time()
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size,
                            spec.vocab_size, max_seq_len=PROMPT_LEN + STEPS + 16, rope_theta=spec.rope_theta)
    for name, typ, dims, kind in spec.tensors():
        om.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    print(f"weights ready in {time.time() - t0:.1f}s", flush=True)
    prompt = synth.prompt_tokens(PROMPT_LEN, spec.vocab_size, 0)
    t0 = time.time()
    logits = om.forward(prompt)
    print(f"prefill of {PROMPT_LEN} tokens in {time.time() - t0:.1f}s", flush=True)

    def summary(v):
        order = np.argsort(v.astype(np.float64), kind="stable")
        return {"first16": [float(x) for x in v[:16]], "l2": float(np.sqrt((v.astype(np.float64) ** 2).sum())),
                "argmax": int(oracle.argmax(v)), "margin": float(v[order[-1]] - v[order[-2]])}

    steps = [summary(logits)]
    tokens = [steps[0]["argmax"]]
    t0 = time.time()
    for _ in range(STEPS):
        logits = om.forward([tokens[-1]])
        steps.append(summary(logits))
        tokens.append(steps[-1]["argmax"])
    print(f"{STEPS} decode steps in {time.time() - t0:.1f}s", flush=True)
    out = {
        "config": f"Llama-2-7B shape cut to {LAYERS} layers: hidden 4096, 32 heads MHA (head_dim 128), FFN 11008, vocab 32000, theta 10000, "
                  f"eps 1e-5; Q4_K throughout; weights N(0,0.02) seed 1234; prompt {PROMPT_LEN} ids seed 4321; {STEPS} greedy decode steps",
        "prompt_len": PROMPT_LEN,
        "prompt_head": prompt[:8].tolist(),
        "tokens": tokens,                  # tokens[0] from the prefill logits, tokens[i] from the logits of decode step i
        "steps": steps,                    # steps[0] = prefill, steps[i] = decode step i (input tokens[i-1], context PROMPT_LEN + i - 1 cached keys)
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cfg2_llama7b_q4_k_2layers.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path, "min margin", min(s["margin"] for s in steps))


if __name__ == "__main__":
    main()
