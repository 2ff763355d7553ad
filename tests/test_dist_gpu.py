"""A model cut across TWO GPUs, one process per GPU: the sums over the ranks taken by NCCL and by the peer-memory kernel.
Needs two devices; on a one-GPU box the in-process rank groups of test_tp_gpu.py cover the same cut kernels."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, os, sys, time
sys.path.insert(0, {root!r})
import numpy as np
import leafcutterllm_b200 as lc
from leafcutterllm_b200 import synth, dist, Engine
from leafcutterllm_b200.synth import ModelSpec
from leafcutterllm_b200._capi import check

rank, world, peer = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["PEER"] == "1"
idfile = os.environ["IDFILE"]
check(lc.load().lc_set_device(rank))
if rank == 0:
    ident = dist.unique_id()
    with open(idfile + ".tmp", "wb") as f:
        f.write(ident)
    os.replace(idfile + ".tmp", idfile)
else:
    t0 = time.time()
    while not os.path.exists(idfile):
        if time.time() - t0 > 120: raise SystemExit("no identifier from rank 0")
        time.sleep(0.05)
    ident = open(idfile, "rb").read()
dist.init(rank, world, ident, peer_memory=peer)
out = {{"rank": rank}}
out["allreduce_us_32k"] = dist.time_allreduce(8192, 50)
out["allreduce_us_1m"] = dist.time_allreduce(262144, 50)
out["peer_memory"] = dist.info()["peer_memory"]
moe = os.environ["MOE"] == "1"
spec = ModelSpec("cut", 2, 1024, 8, 4, 512 if moe else 1024, 800, 10000.0, 12, 12, 12, n_experts=4 if moe else 0, top_k=2 if moe else 0)
eng = Engine(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size, max_seq_len=96,
             n_experts=spec.n_experts, top_k=spec.top_k, device=rank, max_seqs=6)
for name, typ, dims, kind in spec.tensors():
    if kind == "ones":
        eng.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    else:
        eng.synth_tensor(name, typ, dims, synth.WEIGHT_SEED, synth.SIGMA)
eng.finalize()
prompt = synth.prompt_tokens(19, spec.vocab_size, 2)
try:
    logits = eng.forward(prompt)
    step = eng.forward([7])
except Exception as ex:
    print("rank", rank, "failed:", ex, "wait record", dist.debug(), file=sys.stderr, flush=True)
    raise
toks = eng.generate(prompt, 24, stop_on_eos=False)
lens = [3, 7, 1, 9, 2, 5]
prompts = [synth.prompt_tokens(n, spec.vocab_size, 70 + i).tolist() for i, n in enumerate(lens)]
eng.kv_clear(-1)
blog, nxt = eng.forward_batch(list(range(6)), prompts)
btoks, _ = eng.decode_loop(list(range(6)), nxt, 5)
if rank == 0:
    import oracle
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                            max_seq_len=96, n_experts=spec.n_experts, top_k=spec.top_k)
    for name, typ, dims, kind in spec.tensors():
        om.set_tensor(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind))
    w0, w1 = om.forward(prompt), om.forward([7])
    def worst(a, b): return float((np.abs(a - b) - 1e-3 * np.abs(b)).max())
    out["prefill_excess"] = worst(logits, w0)
    out["decode_excess"] = worst(step, w1)
    om.kv_clear()
    ref = om.generate(prompt, 24, stop_on_eos=False)
    out["tokens_equal"] = toks == ref
    out["first_bad_token"] = next((i for i, (a, b) in enumerate(zip(toks, ref)) if a != b), -1)
    ok, bad = True, []
    for i, p in enumerate(prompts):
        om.kv_clear()
        a_ok = worst(blog[i], om.forward(p)) <= 1e-2
        r6 = om.generate(p, 6, stop_on_eos=False)
        b_ok = [int(nxt[i])] + btoks[:, i].tolist() == r6
        if not (a_ok and b_ok): bad.append((i, bool(a_ok), bool(b_ok)))
        ok = ok and a_ok and b_ok
    out["batch_ok"] = bool(ok)
    out["batch_bad"] = bad
out["tokens"] = toks[:6]
eng.close()
dist.finalize()
print(json.dumps(out))
"""


@pytest.mark.parametrize("peer,moe", [(0, 0), (1, 0), (1, 1)])
def test_two_processes_two_gpus(gpu, tmp_path, peer, moe):
    if gpu.load().lc_device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT))
    idfile = str(tmp_path / f"id_{peer}_{moe}")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", PEER=str(peer), MOE=str(moe), IDFILE=idfile, NCCL_NVLS_ENABLE="0",
                   LC_DIST_TIMEOUT_MS="2000")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs, results = [], []
    for p in procs:
        try:
            results.append(p.communicate(timeout=240))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
    for p, (out, err) in zip(procs, results):
        assert p.returncode == 0, "\n---- other rank ----\n".join(e[-1500:] for _o, e in results)
        outs.append(json.loads(out.strip().splitlines()[-1]))
    r0 = [o for o in outs if o["rank"] == 0][0]
    assert r0["prefill_excess"] <= 1e-2 and r0["decode_excess"] <= 1e-2
    assert r0["tokens_equal"] and r0["batch_ok"], (r0["first_bad_token"], r0["batch_bad"])
    assert outs[0]["tokens"] == outs[1]["tokens"]          # every rank ends up with the same picks
    assert all(o["peer_memory"] == bool(peer) for o in outs)   # the requested way of summing is the one that ran
    print("sum over the ranks, 32 KiB / 1 MiB:", [(round(o["allreduce_us_32k"], 1), round(o["allreduce_us_1m"], 1)) for o in outs], "us",
          "peer memory" if peer else "NCCL")
