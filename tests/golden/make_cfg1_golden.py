"""Generates tests/golden/cfg1_tinyllama_q4_0.json: the CPU oracle's greedy tokens, top-2 margins and a few logits for
BASELINE config 1 (TinyLlama-1.1B shape, 22 layers, Q4_0 weights with Q8_0 embedding and head, 32-token seeded prompt,
128 greedy steps, f16 KV cache, call-relative RoPE).  Takes a few minutes and ~6 GB of RAM on 8 cores; the GPU test
compares against the committed file so that the full-size oracle never has to run on the GPU box.

    python tests/golden/make_cfg1_golden.py
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


def main():
    spec = synth.TINY
    t0 = time.time()
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size,
                            spec.vocab_size, max_seq_len=256, rope_theta=spec.rope_theta)
    for name, typ, dims, kind in spec.tensors():
        om.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    print(f"weights ready in {time.time() - t0:.1f}s", flush=True)
    prompt = synth.prompt_tokens(32, spec.vocab_size, 0)
    logits = om.forward(prompt)
    om.kv_clear()
    t0 = time.time()
    toks, margins = om.generate(prompt, 129, stop_on_eos=False, want_margins=True)
    print(f"generated {len(toks)} tokens in {time.time() - t0:.1f}s", flush=True)
    out = {
        "config": "TinyLlama-1.1B shape: 22 layers, hidden 2048, 32 q / 4 kv heads, FFN 5632, vocab 32000, theta 10000, eps 1e-5; "
                  "layers Q4_0, embedding and head Q8_0; weights N(0,0.02) seed 1234; prompt 32 ids seed 4321",
        "prompt": prompt.tolist(),
        "tokens": [int(t) for t in toks],          # first token from the prefill, then 128 decode steps (engine.rs:51-76 without the EOS stop)
        "top2_margins": [float(m) for m in margins],
        "prefill_logits_first16": [float(v) for v in logits[:16]],
        "prefill_logits_argmax": int(oracle.argmax(logits)),
        "prefill_logits_l2": float(np.sqrt((logits.astype(np.float64) ** 2).sum())),
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cfg1_tinyllama_q4_0.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path, "min margin", min(out["top2_margins"]))


if __name__ == "__main__":
    main()
