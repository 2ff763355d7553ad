"""How a model is cut across ranks: the plan the library applies to every tensor (pure host arithmetic, no GPU), and --
with two gloo ranks on the CPU -- that computing on the parts and combining them the way the GPU path does (concatenate
row parts, sum column parts in rank order, take the largest (logit, index) key) reproduces the whole computation of the
CPU oracle."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plan(lc, cfg_kwargs, name, dims):
    from leafcutterllm_b200._capi import ModelConfig, check
    cfg = ModelConfig()
    for k, v in cfg_kwargs.items():
        setattr(cfg, k, v)
    d = (C.c_uint64 * len(dims))(*dims)
    kind, first, count = C.c_int32(), C.c_uint64(), C.c_uint64()
    check(lc.load().lc_shard_plan(C.byref(cfg), name.encode(), d, len(dims), C.byref(kind), C.byref(first), C.byref(count)))
    return kind.value, first.value, count.value


def test_plan_of_the_70b_shape(lc):
    base = dict(hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8, intermediate_size=28672, vocab_size=128256, tp_size=8)
    for r in range(8):
        c = dict(base, tp_rank=r)
        assert plan(lc, c, "blk.3.attn_q.weight", (8192, 8192)) == (1, 1024 * r, 1024)          # 8 of 64 heads
        assert plan(lc, c, "blk.3.attn_k.weight", (8192, 1024)) == (1, 128 * r, 128)            # one kv head
        assert plan(lc, c, "blk.3.attn_output.weight", (8192, 8192)) == (2, 1024 * r, 1024)     # columns: 4 super-blocks
        assert plan(lc, c, "blk.3.ffn_up.weight", (8192, 28672)) == (1, 3584 * r, 3584)
        assert plan(lc, c, "blk.3.ffn_down.weight", (28672, 8192)) == (2, 3584 * r, 3584)       # 14 super-blocks
        assert plan(lc, c, "output.weight", (8192, 128256)) == (1, 16032 * r, 16032)
        assert plan(lc, c, "token_embd.weight", (8192, 128256))[0] == 0
        assert plan(lc, c, "blk.3.attn_norm.weight", (8192,))[0] == 0
        assert plan(lc, c, "model.norm.weight", (8192,))[0] == 0
        # engine-side names map to the same parts (rust/src/model/arch.rs:83-96)
        assert plan(lc, c, "blk.3.self_attn.o_proj.weight", (8192, 8192)) == (2, 1024 * r, 1024)
    assert plan(lc, dict(base, tp_size=1), "blk.3.attn_q.weight", (8192, 8192))[0] == 0


def test_plan_of_the_mixture_shape(lc):
    base = dict(hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, intermediate_size=14336, vocab_size=32000, n_experts=8, top_k=2, tp_size=4)
    for r in range(4):
        c = dict(base, tp_rank=r)
        for e in range(8):
            kind = plan(lc, c, f"blk.0.expert.{e}.ffn_down.weight", (14336, 4096))[0]
            assert kind == (0 if e // 2 == r else 3)                                             # two whole experts per rank
        assert plan(lc, c, "blk.0.ffn_gate_exps.weight", (4096, 14336, 8)) == (1, 2 * 14336 * r, 2 * 14336)
        assert plan(lc, c, "blk.0.ffn_down_exps.weight", (14336, 4096, 8)) == (1, 2 * 4096 * r, 2 * 4096)
        assert plan(lc, c, "blk.0.ffn_gate_inp.weight", (4096, 8))[0] == 0
        assert plan(lc, c, "blk.0.attn_v.weight", (4096, 1024)) == (1, 256 * r, 256)


def test_plan_rejects_what_cannot_be_cut(lc):
    from leafcutterllm_b200 import LeafcutterError
    with pytest.raises(LeafcutterError):
        plan(lc, dict(hidden_size=4096, num_heads=32, num_kv_heads=32, intermediate_size=11008, vocab_size=32000, tp_size=3, tp_rank=0),
             "blk.0.ffn_up.weight", (4096, 11008))
    with pytest.raises(LeafcutterError):
        plan(lc, dict(n_experts=8, tp_size=3, tp_rank=0), "blk.0.expert.1.ffn_up.weight", (4096, 14336))


CHILD = r"""
import ctypes as C, json, os, sys
sys.path.insert(0, {root!r})
import numpy as np
import torch, torch.distributed as dist
import oracle
import leafcutterllm_b200 as lc
from leafcutterllm_b200 import synth
from leafcutterllm_b200._capi import ModelConfig, check, QUANT_GEOMETRY

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
H, NQ, F, V, T = 512, 512, 1024, 640, 3
cfg = ModelConfig()
cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, cfg.vocab_size, cfg.tp_size, cfg.tp_rank = H, 4, 4, F, V, world, rank

def part(name, typ, dims, data):
    # this rank's bytes of a whole tensor, cut as lc_shard_plan says
    d = (C.c_uint64 * len(dims))(*dims)
    kind, first, count = C.c_int32(), C.c_uint64(), C.c_uint64()
    check(lc.load().lc_shard_plan(C.byref(cfg), name.encode(), d, len(dims), C.byref(kind), C.byref(first), C.byref(count)))
    be, bb = QUANT_GEOMETRY[typ]
    row_bytes = dims[0] // be * bb
    rows = data.reshape(-1, row_bytes)
    if kind.value == 1:
        return rows[first.value:first.value + count.value].copy().ravel(), kind.value, first.value, count.value
    if kind.value == 2:
        return rows[:, first.value // be * bb:(first.value + count.value) // be * bb].copy().ravel(), kind.value, first.value, count.value
    return data, kind.value, first.value, count.value

r = np.random.default_rng(5)   # same draws on every rank
x = r.standard_normal((T, H)).astype(np.float32)
out = {{}}
# a row-cut product (the q projection): the parts side by side are the whole product, bit for bit
wq = synth.host_tensor(12, 77, "blk.0.attn_q.weight", NQ * H)
mine, kind, first, count = part("blk.0.attn_q.weight", 12, (H, NQ), wq)
y_part = oracle.qmatmul(12, x, mine, T, H, count).reshape(T, count)
gathered = [torch.empty(T, count) for _ in range(world)]
dist.all_gather(gathered, torch.from_numpy(y_part.copy()))
y_whole = oracle.qmatmul(12, x, wq, T, H, NQ).reshape(T, NQ)
out["rows_exact"] = bool(np.array_equal(torch.cat(gathered, 1).numpy(), y_whole)) and kind == 1
# a column-cut product (the down projection): the parts' results summed in rank order are the whole product to rounding
h = r.standard_normal((T, F)).astype(np.float32)
wd = synth.host_tensor(12, 77, "blk.0.ffn_down.weight", H * F)
mine, kind, first, count = part("blk.0.ffn_down.weight", 12, (F, H), wd)
p = oracle.qmatmul(12, np.ascontiguousarray(h[:, first:first + count]), mine, T, count, H).reshape(T, H)
parts = [torch.empty(T, H) for _ in range(world)]
dist.all_gather(parts, torch.from_numpy(p.copy()))
total = parts[0].numpy().copy()
for q in parts[1:]:
    total = total + q.numpy()          # rank order, as the GPU sum
whole = oracle.qmatmul(12, h, wd, T, F, H).reshape(T, H)
out["cols_err"] = float(np.abs(total - whole).max() / np.abs(whole).max())
out["cols_kind"] = kind
# the greedy pick over vocabulary slices: largest (total-order key, global index)
logits = r.standard_normal(V).astype(np.float32)
logits[[17, 400, 639]] = logits.max() + 1.0     # three equal maxima: the last index must win
lo, n = rank * (V // world), V // world
local = logits[lo:lo + n]
def key(v, i):
    b = int(np.float32(v).view(np.int32))
    k = b ^ ((b >> 31) & 0x7fffffff)
    return (k << 32) | i
best = max(key(local[i], lo + i) for i in range(n))
t = torch.tensor([best], dtype=torch.int64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
out["pick"] = int(t.item() & 0xffffffff)
out["want_pick"] = int(oracle.argmax(logits))
print(json.dumps(out))
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reproduce_the_whole_computation(tmp_path, lc, oracle):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, err[-3000:]
        o = json.loads(out.strip().splitlines()[-1])
        assert o["rows_exact"]
        assert o["cols_kind"] == 2 and o["cols_err"] < 1e-5
        assert o["pick"] == o["want_pick"] == 639
