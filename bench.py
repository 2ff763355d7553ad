#!/usr/bin/env python
"""Decode throughput of the 7B-shape Q4_K model on B200 through the C ABI.

  python bench.py --gpus N --steps K --warmup W        this library (one process per GPU)
  python bench.py --impl reference ...                 the reference's CPU path (oracle port) on the host cores

One "step" = one greedy decode step of one sequence per GPU over a 2048-token context (Llama-2-7B
shape, random-init N(0,0.02) weights quantised to Q4_K, synthetic prompt).  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tok/s, 7B-shape Q4_K, batch 1 per GPU, 2048-token context"
PROMPT_LEN = 2048


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class Ranks:
    """Replicas only: the ranks never exchange data on the decode path.  They meet at a barrier before and after the
    timed region and agree on the slowest rank's time (max over ranks)."""

    def __init__(self, rank: int, world: int, local: int, backend: str):
        self.rank, self.world, self.dist, self.cuda = rank, world, None, backend == "nccl"
        if world > 1:
            import torch
            import torch.distributed as dist
            if self.cuda:
                torch.cuda.set_device(local)
                dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            else:
                dist.init_process_group(backend)
            self.dist = dist

    def barrier_max(self, v: float) -> float:
        if self.dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device="cuda" if self.cuda else "cpu")
        if self.cuda:
            torch.cuda.synchronize()
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        if self.cuda:
            torch.cuda.synchronize()
        return float(t.item())

    def aggregate_rate(self, units_per_rank: float, seconds_this_rank: float) -> float:
        """Whole-job rate: every rank did `units_per_rank` (weak scaling), the job took as long as its slowest rank."""
        return self.world * units_per_rank / self.barrier_max(seconds_this_rank)

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def oracle_tensor(oracle, synth, spec, name, typ, dims, kind):
    """A synthetic tensor's bytes from the generator inside the oracle library (the CPU arm never loads the CUDA library)."""
    import numpy as np
    n = int(np.prod(dims))
    if kind == "ones":
        return np.ones(n, np.float32).view(np.uint8)
    return oracle.synth_tensor(typ, synth.WEIGHT_SEED, name, synth.SIGMA, n)


def cpu_baseline(spec, steps: int = 4, layers: int = 2, prompt: int = 64, threads: int | None = None) -> dict:
    """The oracle (CPU restatement of the reference) on a bounded sample: `layers` of the 32 layers plus the head,
    a short prompt, `steps` decode steps, dequantised weights cached, OpenMP over output columns on every host
    thread; the per-token time is scaled to the full depth.  Also times the reference-faithful mode (per-call
    re-dequantise + transpose of every tensor, rust/src/inference/engine.rs:95-97)."""
    import oracle
    from leafcutterllm_b200 import synth   # the model description only (pure Python); the library itself is not loaded
    oracle.build()
    if not threads:
        # every host core this process may run on, set explicitly: a launcher may export OMP_NUM_THREADS=1 to its ranks
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.lib().orc_set_num_threads(threads)
    cores = oracle.lib().orc_num_threads()
    sub = spec.with_layers(layers)

    def make():
        om = oracle.OracleModel(sub.hidden_size, sub.num_layers, sub.num_heads, sub.num_kv_heads, sub.intermediate_size,
                                sub.vocab_size, max_seq_len=prompt + steps + 8, rope_theta=sub.rope_theta)
        for name, typ, dims, kind in sub.tensors():
            om.set_tensor(name, typ, dims, oracle_tensor(oracle, synth, sub, name, typ, dims, kind))
        return om

    toks = oracle.synth_tokens(synth.PROMPT_SEED, prompt, sub.vocab_size)
    om = make()
    om.forward(toks)          # also fills the dequantised-weight cache
    t0 = time.perf_counter()
    for s in range(steps):
        om.forward([int(toks[s])])
    t_cached = (time.perf_counter() - t0) / steps
    om.timers(reset=True)
    om.forward([1])
    tm = om.timers()
    om.close()
    # head cost measured separately: one-layer model minus ... simpler: matmul time splits by weight count
    w_layer = 4 * sub.hidden_size * sub.hidden_size + 3 * sub.hidden_size * sub.intermediate_size
    w_head = sub.hidden_size * sub.vocab_size
    per_weight = tm["matmul_s"] / (layers * w_layer + w_head)
    other = max(t_cached - tm["matmul_s"], 0.0) / layers
    full = spec.num_layers * (w_layer * per_weight + other) + w_head * per_weight
    om = make()
    om.set_mode(True)
    om.forward(toks[:8])
    t0 = time.perf_counter()
    om.forward([1])
    t_faithful = time.perf_counter() - t0
    om.close()
    full_faithful = t_faithful * (spec.num_layers * w_layer + w_head) / (layers * w_layer + w_head)
    return {"value": 1.0 / full, "unit": "tok/s", "cores": cores, "kind": "port", "steps_run": steps, "layers_run": layers, "context": prompt,
            "sample": f"{layers} of {spec.num_layers} layers + head of the same shape, {prompt}-token context, {steps} decode steps, "
                      f"dequantised f32 weights cached, OpenMP over output columns; per-token time scaled to {spec.num_layers} layers",
            "reference_faithful_tok_s": 1.0 / full_faithful,
            "reference_faithful_note": "per-call re-dequantise + transpose of every tensor as engine.rs:95-97, same sample and scaling"}


def tiny_cpu(steps: int = 32) -> dict:
    """BASELINE.json configs[0] (TinyLlama-1.1B shape, Q4_0 layers, Q8_0 embedding and head) in FULL on the host cores through
    the oracle: 32-token prompt prefilled, then `steps` decode steps, weights cached as f32, OpenMP on every core.  The one
    workload where the CPU number is the same configuration as the GPU number."""
    import oracle
    from leafcutterllm_b200 import synth
    oracle.build()
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.lib().orc_set_num_threads(threads)
    spec = synth.TINY
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size, spec.vocab_size,
                            max_seq_len=32 + steps + 8, rope_theta=spec.rope_theta)
    for name, typ, dims, kind in spec.tensors():
        om.set_tensor(name, typ, dims, oracle_tensor(oracle, synth, spec, name, typ, dims, kind))
    prompt = oracle.synth_tokens(synth.PROMPT_SEED, 32, spec.vocab_size)
    logits = om.forward(prompt)
    tok = int(oracle.argmax(logits))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = int(oracle.argmax(om.forward([tok])))
    dt = time.perf_counter() - t0
    om.close()
    return {"value": round(steps / dt, 3), "unit": "tok/s", "cores": oracle.lib().orc_num_threads(), "kind": "port", "steps_run": steps,
            "sample": f"the whole configuration: 22 layers, 32-token prompt, {steps} greedy decode steps, f32 weights cached, OpenMP"}


def tiny_decode(lc, synth, local: int, steps: int = 128, warm: int = 3) -> dict:
    """BASELINE.json configs[0] on the GPU: TinyLlama-1.1B shape (22 layers, hidden 2048, 32 q / 4 kv heads of 64 dims, FFN 5632,
    vocabulary 32000), Q4_0 layers with Q8_0 embedding and head, 32-token seeded prompt, then greedy decode steps (CUDA events
    around the graph replays)."""
    spec = synth.TINY
    eng = synth.build_engine(spec, 32 + warm + steps + 16, on_device=True, device=local)
    prompt = synth.prompt_tokens(32, spec.vocab_size, 0)
    _, nxt = eng.forward_batch([0], [prompt.tolist()], want_logits=False)
    toks, _ = eng.decode_loop([0], nxt, warm)
    eng.reset_counters()
    toks, ms = eng.decode_loop([0], toks[-1].tolist(), steps)
    ctr = eng.counters()
    eng.close()
    peak, which = measured_peaks()
    algo = ctr["algo_bytes_last_step"]
    per_step = ms / steps
    return {"workload": "configs[0]: TinyLlama-1.1B shape, Q4_0 layers + Q8_0 embedding/head, batch 1, 32-token prompt, greedy decode; "
                        "0.62 GB per step, so after the first step the weights stay in the 126 MB L2 only in small part",
            "value": round(steps / (ms * 1e-3), 1), "unit": "tok/s", "ms_per_step": round(per_step, 4), "steps": steps,
            "algorithmic_bytes_per_step": int(algo), "achieved_gbs": round(algo / (per_step * 1e-3) / 1e9, 1), "peak_gbs": peak,
            "frac": round(algo / (per_step * 1e-3) / 1e9 / peak, 4), "peak_source": which, "gpu_launches": int(ctr["kernel_launches"])}


def q4km_decode(lc, synth, local: int, prompt_len: int = PROMPT_LEN, steps: int = 64, warm: int = 3, layers: int = 0) -> dict:
    """The bench workload with the type mix of a "Q4_K_M" file instead of Q4_K throughout: Q6_K head, Q6_K attn_v and ffn_down
    in 16 of the 32 layers (synth.ModelSpec.mixed_type), so q/k/v run as three products in those layers.  Batch 1,
    2048-token seeded prompt, greedy decode steps (CUDA events around the graph replays)."""
    spec = synth.LLAMA7B_Q4KM if layers <= 0 else synth.LLAMA7B_Q4KM.with_layers(layers)
    eng = synth.build_engine(spec, prompt_len + warm + steps + 16, on_device=True, device=local, max_seqs=2)
    # a first prefill on the second sequence pays for what a process pays once (kernel images loaded at their first launch)
    eng.forward_batch([1], [synth.prompt_tokens(prompt_len, spec.vocab_size, 1).tolist()], want_logits=False)
    prompt = synth.prompt_tokens(prompt_len, spec.vocab_size, 0)
    t0 = time.perf_counter()
    _, nxt = eng.forward_batch([0], [prompt.tolist()], want_logits=False)
    t_prefill = time.perf_counter() - t0
    toks, _ = eng.decode_loop([0], nxt, warm)
    eng.reset_counters()
    toks, ms = eng.decode_loop([0], toks[-1].tolist(), steps)
    ctr = eng.counters()
    eng.close()
    peak, which = measured_peaks()
    algo = ctr["algo_bytes_last_step"]
    per_step = ms / steps
    n_q6 = sum(1 for l in range(spec.num_layers) if spec.mixed_type(l, "down") == 14)
    return {"workload": f"Llama-2-7B shape with the Q4_K_M type mix (Q6_K head, Q6_K attn_v and ffn_down in {n_q6} of {spec.num_layers} layers, Q4_K "
                        f"elsewhere), batch 1, {prompt_len}-token seeded prompt, greedy decode",
            "value": round(steps / (ms * 1e-3), 1), "unit": "tok/s", "ms_per_step": round(per_step, 4), "steps": steps, "prefill_s": round(t_prefill, 3),
            "algorithmic_bytes_per_step": int(algo), "achieved_gbs": round(algo / (per_step * 1e-3) / 1e9, 1), "peak_gbs": peak,
            "frac": round(algo / (per_step * 1e-3) / 1e9 / peak, 4), "peak_source": which, "gpu_launches": int(ctr["kernel_launches"])}


def moe_decode(lc, synth, local: int, n_seqs: int = 16, prompt_len: int = 1024, steps: int = 64, warm: int = 3, layers: int = 0) -> dict:
    """BASELINE.json configs[3] on ONE GPU: Mixtral-8x7B shape (32 layers, hidden 4096, 32 q / 8 kv heads, 8 experts of FFN 14336,
    two per token, vocabulary 32000), experts and attention Q4_K, f32 router; 16 sequences with 1024-token seeded prompts, then
    greedy decode steps.  Bytes per step = attention and head weights + the experts that received a token (counted on the
    device) + every sequence's KV."""
    spec = synth.MIXTRAL if layers <= 0 else synth.MIXTRAL.with_layers(layers)
    t0 = time.perf_counter()
    eng = synth.build_engine(spec, prompt_len + warm + steps + 16, on_device=True, device=local, max_seqs=n_seqs)
    t_build = time.perf_counter() - t0
    t0 = time.perf_counter()
    first = []
    for s_ in range(n_seqs):
        prompt = synth.prompt_tokens(prompt_len, spec.vocab_size, 2000 + s_)
        _, nxt = eng.forward_batch([s_], [prompt], want_logits=False)
        first.append(int(nxt[0]))
    t_prefill = time.perf_counter() - t0
    ids = list(range(n_seqs))
    toks, _ = eng.decode_loop(ids, first, warm)
    eng.reset_counters()
    toks, ms = eng.decode_loop(ids, toks[-1].tolist(), steps)
    ctr = eng.counters()
    eng.close()
    peak, which = measured_peaks()
    algo = ctr["algo_bytes_last_step"]
    per_step = ms / steps
    out = {"workload": "configs[3] on one GPU: Mixtral-8x7B shape, Q4_K experts and attention, f32 router, 16 sequences x 1024-token prompts, greedy decode",
           "value": round(n_seqs * steps / (ms * 1e-3), 1), "unit": "tok/s", "ms_per_step": round(per_step, 3), "steps": steps, "sequences": n_seqs,
           "model_build_s": round(t_build, 2), "prefill_s": round(t_prefill, 2), "algorithmic_bytes_per_step": int(algo),
           "achieved_gbs": round(algo / (per_step * 1e-3) / 1e9, 1), "peak_gbs": peak, "frac": round(algo / (per_step * 1e-3) / 1e9 / peak, 4),
           "peak_source": which, "gpu_launches": int(ctr["kernel_launches"])}
    if layers > 0:
        out["not_the_metric"] = f"profiling case: {layers} of 32 layers"
    return out


def gemv_sweep(lc) -> dict:
    """Q4_K GEMV (one token) timed alone for a range of row counts: back-to-back launches over >= 600 MB of distinct
    weights per shape, CUDA events on the library's stream.  Shows the streaming rate and the fixed cost per launch."""
    import ctypes as C
    lib = lc.load()
    chk = lc._capi.check
    rows = []
    for (k, n) in [(4096, 4096), (4096, 12288), (4096, 32768), (4096, 131072), (11008, 4096)]:
        nb = lib.lc_tensor_bytes(12, k * n)
        copies = max(2, int(600e6 // nb))
        x = C.c_void_p(); y = C.c_void_p()
        chk(lib.lc_dev_alloc(4 * k, C.byref(x))); chk(lib.lc_dev_alloc(4 * n, C.byref(y)))
        chk(lib.lc_synth_tensor_dev(0, 1, b"x", 1.0, k, x))
        ws = []
        for c in range(copies):
            p = C.c_void_p()
            chk(lib.lc_dev_alloc(nb, C.byref(p)))
            chk(lib.lc_synth_tensor_dev(12, 7, f"w{c}".encode(), 0.02, k * n, p))
            ws.append(p)
        for p in ws:
            chk(lib.lc_qmatmul_dev(12, x, p, 1, k, n, y))
        chk(lib.lc_dev_sync()); chk(lib.lc_timer_begin())
        reps = 5
        for _ in range(reps):
            for p in ws:
                chk(lib.lc_qmatmul_dev(12, x, p, 1, k, n, y))
        ms = C.c_float(); chk(lib.lc_timer_end(C.byref(ms)))
        for p in ws:
            lib.lc_dev_free(p)
        lib.lc_dev_free(x); lib.lc_dev_free(y)
        us = ms.value * 1e3 / (reps * copies)
        rows.append({"k": k, "n": n, "MB": round(nb / 1e6, 2), "us_per_launch": round(us, 2), "GBps": round(nb / us / 1e3, 1)})
    return {"kernel": "Q4_K GEMV, one token" + (" (tcgen05 variant)" if os.environ.get("LC_GEMV_UMMA") else ""), "sweep": rows}


def gemv_types(lc) -> dict:
    """One-token matrix-vector product per ggml type on two 7B shapes, timed alone over >= 300 MB of distinct weights (any
    bytes do for timing: the buffers are filled by the f32 generator and read as blocks of the type)."""
    import ctypes as C
    lib = lc.load()
    chk = lc._capi.check
    rows = []
    for typ, name in [(12, "Q4_K"), (13, "Q5_K"), (14, "Q6_K"), (2, "Q4_0"), (8, "Q8_0"), (20, "IQ4_NL"), (1, "F16")]:
        for (k, n) in [(4096, 4096), (11008, 4096)]:
            nb = lib.lc_tensor_bytes(typ, k * n)
            copies = max(2, int(300e6 // nb))
            x = C.c_void_p(); y = C.c_void_p()
            chk(lib.lc_dev_alloc(4 * k, C.byref(x))); chk(lib.lc_dev_alloc(4 * n, C.byref(y)))
            chk(lib.lc_synth_tensor_dev(0, 1, b"x", 1.0, k, x))
            ws = []
            for c in range(copies):
                p = C.c_void_p(); chk(lib.lc_dev_alloc(nb + 16, C.byref(p)))
                chk(lib.lc_synth_tensor_dev(0, 7, f"t{c}".encode(), 0.02, nb // 4, p)); ws.append(p)
            for p in ws:
                chk(lib.lc_qmatmul_dev(typ, x, p, 1, k, n, y))
            chk(lib.lc_dev_sync()); chk(lib.lc_timer_begin())
            for _ in range(3):
                for p in ws:
                    chk(lib.lc_qmatmul_dev(typ, x, p, 1, k, n, y))
            ms = C.c_float(); chk(lib.lc_timer_end(C.byref(ms)))
            us = ms.value * 1e3 / (3 * copies)
            rows.append({"type": name, "k": k, "n": n, "MB": round(nb / 1e6, 2), "us_per_launch": round(us, 1), "GBps": round(nb / us / 1e3, 1)})
            for p in ws:
                lib.lc_dev_free(p)
            lib.lc_dev_free(x); lib.lc_dev_free(y)
    return {"kernel": "matrix-vector product, one token, per ggml type", "rows": rows}


def gemm_microbench(lc, tokens=(64, 512), small: bool = False, shapes=None) -> dict:
    """The many-token tensor-core product (Q4_K weights dequantised on the fly, tcgen05) timed alone on the 7B shapes:
    per shape and token count the time of one launch pair (activation split + product) over distinct weight copies
    larger than L2, CUDA events on the library's stream."""
    import ctypes as C
    lib = lc.load()
    chk = lc._capi.check
    rows = []
    if shapes is None:
        shapes = [(4096, 12288), (4096, 4096), (11008, 4096)] if not small else [(4096, 4096)]
    for m in tokens:
        for (k, n) in shapes:
            nb = lib.lc_tensor_bytes(12, k * n)
            copies = max(2, int((200e6 if small else 600e6) // nb))
            x = C.c_void_p(); y = C.c_void_p()
            chk(lib.lc_dev_alloc(4 * k * m, C.byref(x))); chk(lib.lc_dev_alloc(4 * n * m, C.byref(y)))
            chk(lib.lc_synth_tensor_dev(0, 1, b"x", 1.0, k * m, x))
            ws = []
            for c in range(copies):
                p = C.c_void_p()
                chk(lib.lc_dev_alloc(nb, C.byref(p)))
                chk(lib.lc_synth_tensor_dev(12, 7, f"g{c}".encode(), 0.02, k * n, p))
                ws.append(p)
            for p in ws[:2]:
                chk(lib.lc_qmatmul_dev(12, x, p, m, k, n, y))
            chk(lib.lc_dev_sync()); chk(lib.lc_timer_begin())
            reps = 1 if small else 3
            for _ in range(reps):
                for p in ws:
                    chk(lib.lc_qmatmul_dev(12, x, p, m, k, n, y))
            ms = C.c_float(); chk(lib.lc_timer_end(C.byref(ms)))
            for p in ws:
                lib.lc_dev_free(p)
            lib.lc_dev_free(x); lib.lc_dev_free(y)
            us = ms.value * 1e3 / (reps * copies)
            rows.append({"tokens": m, "k": k, "n": n, "weight_MB": round(nb / 1e6, 2), "us_per_launch": round(us, 1),
                         "weight_GBps": round(nb / us / 1e3, 1), "TFLOPs": round(2.0 * m * k * n / us / 1e6, 1)})
    return {"kernel": "qgemm_umma_q4k_kernel (tcgen05 kind::f16, %s products per k step)" % os.environ.get("LC_GEMM_TERMS", "3"),
            "rows": rows}


def gemv_roofline(lc, spec, reps: int = 3, copies: int = 8, warm: int = 3) -> dict:
    """The dominant kernel (quantised GEMV, one launch per weight matrix) timed alone with CUDA events on the
    library's stream over 8 distinct copies of a layer's matrices (0.9 GB, larger than L2)."""
    import ctypes as C
    lib = lc.load()
    H, F = spec.hidden_size, spec.intermediate_size
    shapes = [(H, 3 * H), (H, H), (H, F), (H, F), (F, H)]  # (k, n)
    bufs, total_bytes = [], 0
    x = C.c_void_p(); y = C.c_void_p()
    lc._capi.check(lib.lc_dev_alloc(4 * max(H, F), C.byref(x)))
    lc._capi.check(lib.lc_dev_alloc(4 * 3 * max(H, F), C.byref(y)))
    lc._capi.check(lib.lc_synth_tensor_dev(0, 1, b"x", 1.0, max(H, F), x))
    for c in range(copies):
        for i, (k, n) in enumerate(shapes):
            nb = lib.lc_tensor_bytes(12, k * n)
            p = C.c_void_p()
            lc._capi.check(lib.lc_dev_alloc(nb, C.byref(p)))
            lc._capi.check(lib.lc_synth_tensor_dev(12, 77, f"rf{c}_{i}".encode(), 0.02, k * n, p))
            bufs.append((p, k, n, nb))
            total_bytes += nb

    def sweep():
        for (p, k, n, _nb) in bufs:
            lc._capi.check(lib.lc_qmatmul_dev(12, x, p, 1, k, n, y))

    for _ in range(warm):
        sweep()
    lc._capi.check(lib.lc_dev_sync())
    lc._capi.check(lib.lc_timer_begin())
    for _ in range(reps):
        sweep()
    ms = C.c_float()
    lc._capi.check(lib.lc_timer_end(C.byref(ms)))
    for (p, *_r) in bufs:
        lib.lc_dev_free(p)
    lib.lc_dev_free(x); lib.lc_dev_free(y)
    launches = reps * len(bufs)
    peak, which = measured_peaks()
    achieved = total_bytes * reps / (ms.value * 1e-3) / 1e9
    traffic = None
    tp = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if os.path.exists(tp):
        traffic = json.load(open(tp)).get("qgemv_tma_q4k_bytes_per_launch_avg")
    return {"bound": "hbm", "kernel": "qgemv_mma_q4k_kernel<m=1> (int8 MMA, TMA-staged)", "achieved": round(achieved, 1), "peak": peak,
            "peak_source": which + " (MEASURED_PEAKS.json hbm_gbs, burst)" if which == "measured" else which,
            "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": traffic,
            "algorithmic_bytes_per_launch_avg": total_bytes / len(bufs), "avg_launch_us": round(ms.value * 1e3 / launches, 3),
            "launches_timed": launches}


def attention_microbench(lc, n_heads=32, n_kv=32, hd=128, ctx=2100, layers=8, reps=5) -> dict:
    """Decode attention of one token (7B shape: 32 heads of 128 dims, f16 cache, 16-token pages) through
    lc_attention_decode_dev over `layers` distinct caches (0.28 GB, larger than L2); CUDA events on the library's stream.
    Every call also queues an 8-byte host-to-device copy and a counter clear, so the figure is an upper bound."""
    import ctypes as C
    import numpy as np
    lib, chk = lc.load(), lc._capi.check
    pt = 16
    n_pages = (ctx + pt - 1) // pt
    pool_bytes = n_pages * n_kv * pt * hd * 2

    def dev(nbytes):
        p = C.c_void_p()
        chk(lib.lc_dev_alloc(nbytes, C.byref(p)))
        return p

    ks = [dev(pool_bytes) for _ in range(layers)]
    vs = [dev(pool_bytes) for _ in range(layers)]
    for i, p in enumerate(ks + vs):
        chk(lib.lc_synth_tensor_dev(1, 5, f"kv{i}".encode(), 1.0, pool_bytes // 2, p))
    table = np.arange(n_pages, dtype=np.int32)
    td = dev(table.nbytes)
    chk(lib.lc_dev_upload(td, table.ctypes.data_as(C.c_void_p), table.nbytes))
    q = np.random.default_rng(0).standard_normal(n_heads * hd).astype(np.float32)
    qd = dev(q.nbytes)
    chk(lib.lc_dev_upload(qd, q.ctypes.data_as(C.c_void_p), q.nbytes))
    out = dev(n_heads * hd * 4)

    def sweep():
        for k, v in zip(ks, vs):
            chk(lib.lc_attention_decode_dev(qd, k, v, td, n_pages, ctx, n_heads, n_kv, hd, pt, 0, out))

    sweep()
    chk(lib.lc_dev_sync())
    chk(lib.lc_timer_begin())
    for _ in range(reps):
        sweep()
    ms = C.c_float()
    chk(lib.lc_timer_end(C.byref(ms)))
    for p in ks + vs + [td, qd, out]:
        lib.lc_dev_free(p)
    us = ms.value * 1e3 / (reps * layers)
    byt = 2 * ctx * n_kv * hd * 2
    return {"kernel": "decode attention, 1 token", "heads": n_heads, "kv_heads": n_kv, "head_dim": hd, "context": ctx,
            "us_per_call": round(us, 2), "kv_bytes": byt, "achieved_gbs": round(byt / us / 1e3, 1)}


def batched_decode(lc, synth, spec, local: int, n_seqs: int = 64, steps: int = 128, warm: int = 3, profile_range: bool = False,
                   check_tokens: bool = True) -> dict:
    """BASELINE.json configs[2]: the same model under continuous batching -- 64 sequences whose context lengths are
    uniform in [128, 4096] from seed 777, paged f16 KV cache (16-token pages), greedy decode.  Every sequence is
    prefilled with its own seeded prompt (through the many-token tensor-core product), then `steps` decode steps are
    timed on the device (CUDA events around the graph replays).  Bytes per step = weights once + every sequence's KV."""
    import numpy as np
    rng = np.random.default_rng(777)
    ctx = rng.integers(128, 4097, n_seqs)
    pool = int(sum((int(c) + warm + steps + 2 + 15) // 16 * 16 for c in ctx))
    t0 = time.perf_counter()
    eng = synth.build_engine(spec, 4096 + warm + steps + 16, on_device=True, device=local, max_seqs=n_seqs, kv_pool_tokens=pool)
    first = []
    for s_ in range(n_seqs):
        prompt = synth.prompt_tokens(int(ctx[s_]), spec.vocab_size, 1000 + s_)
        _, nxt = eng.forward_batch([s_], [prompt], want_logits=False)
        first.append(int(nxt[0]))
    t_prefill = time.perf_counter() - t0
    ids = list(range(n_seqs))
    warm_toks, _ = eng.decode_loop(ids, first, warm)
    eng.reset_counters()
    if profile_range:  # a profiler started with --profile-from-start off sees the timed steps only, not the prefill
        import torch
        torch.cuda.cudart().cudaProfilerStart()
    toks, ms = eng.decode_loop(ids, warm_toks[-1].tolist(), steps)
    if profile_range:
        torch.cuda.cudart().cudaProfilerStop()
    ctr = eng.counters()
    eng.close()
    checked = []
    if check_tokens:
        # two of the sequences again, each ALONE (single-sequence kernels: streaming attention, matrix-vector products): the
        # batched run must have produced the same greedy tokens for them
        for s_ in (int(np.argmin(ctx)), int(np.argmax(ctx))):
            solo = synth.build_engine(spec, int(ctx[s_]) + warm + steps + 16, on_device=True, device=local)
            got = solo.generate(synth.prompt_tokens(int(ctx[s_]), spec.vocab_size, 1000 + s_), 1 + warm + steps, stop_on_eos=False)
            solo.close()
            want = [first[s_]] + warm_toks[:, s_].tolist() + toks[:, s_].tolist()
            same = sum(1 for a, b in zip(got, want) if a == b)
            if got != want:
                # a greedy pick can legitimately differ where two logits are closer than the kernels' rounding; report, do not hide
                first_bad = next(i for i, (a, b) in enumerate(zip(got, want)) if a != b)
                checked.append({"sequence": s_, "context": int(ctx[s_]), "identical": False, "first_difference_at": first_bad, "equal_tokens": same})
            else:
                checked.append({"sequence": s_, "context": int(ctx[s_]), "identical": True, "tokens": len(want)})
    peak, which = measured_peaks()
    # bytes of the last step, minus what the contexts grew since the middle step: the mean over the timed steps
    kv_per_token = spec.num_layers * 2 * spec.num_kv_heads * spec.head_dim * 2
    algo = ctr["algo_bytes_last_step"] - int((steps - 1) / 2 * n_seqs * kv_per_token)
    per_step = ms / steps
    return {"workload": "configs[2]: 64 sequences, context lengths drawn once from numpy default_rng(777).integers(128, 4097) (mean of this draw "
                        f"{float(ctx.mean()):.0f}, the distribution's mean is 2112), paged f16 KV cache, greedy decode; bytes per step are the mean over the timed steps",
            "token_check": checked,
            "value": round(n_seqs * steps / (ms * 1e-3), 1), "unit": "tok/s", "ms_per_step": round(per_step, 3), "steps": steps,
            "sequences": n_seqs, "mean_context": round(float(ctx.mean()), 1), "tokens_prefilled": int(ctx.sum()),
            "build_and_prefill_s": round(t_prefill, 2), "algorithmic_bytes_per_step": int(algo),
            "achieved_gbs": round(algo / (per_step * 1e-3) / 1e9, 1), "peak_gbs": peak, "frac": round(algo / (per_step * 1e-3) / 1e9 / peak, 4),
            "peak_source": which, "gpu_launches": int(ctr["kernel_launches"])}


def cut_model_legs(lc, synth, ranks, rank: int, world: int, local: int) -> dict:
    """The configurations BASELINE.json partitions across the GPUs of the box, run by ALL ranks together after the replicas metric:
    configs[4] (Llama-3-70B shape, tensor parallel over the world) and configs[3] (Mixtral shape, attention tensor parallel, experts
    dealt to the ranks).  Every figure is device time from CUDA events, the maximum over the ranks."""
    import numpy as np
    import torch
    from leafcutterllm_b200 import dist as lcd
    ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        ident = torch.tensor(list(lcd.unique_id()), dtype=torch.uint8, device="cuda")
    ranks.dist.broadcast(ident, 0)
    torch.cuda.synchronize()
    lcd.init(rank, world, bytes(ident.cpu().numpy().tobytes()))
    out = {}
    peak, which = measured_peaks()
    try:
        sums = {"32 KiB (one token of hidden 8192)": round(ranks.barrier_max(lcd.time_allreduce(8192, 100)), 2),
                "1 MiB (32 tokens)": round(ranks.barrier_max(lcd.time_allreduce(262144, 50)), 2)}
        out["rank_sums"] = {"us_per_sum": sums, "path_up_to_256KiB": "peer memory: tagged words written into every rank's buffer over NVLink, summed in rank order"
                            if lcd.info()["peer_memory"] else "NCCL all-reduce", "larger": "NCCL all-reduce"}

        def decode_leg(eng, spec, n_seqs, prompt_len, steps, warm, seed0):
            ids = list(range(n_seqs))
            t0 = time.perf_counter()
            first = []
            for s_ in ids:
                _, nxt = eng.forward_batch([s_], [synth.prompt_tokens(prompt_len, spec.vocab_size, seed0 + s_)], want_logits=False)
                first.append(int(nxt[0]))
            t_prefill = ranks.barrier_max(time.perf_counter() - t0)
            toks, _ = eng.decode_loop(ids, first, warm)
            eng.reset_counters()
            ranks.barrier_max(0.0)
            toks, ms = eng.decode_loop(ids, toks[-1].tolist(), steps)
            ms = ranks.barrier_max(ms)
            ctr = eng.counters()
            per_step = ms / steps
            algo = ctr["algo_bytes_last_step"]
            return {"value": round(n_seqs * steps / (ms * 1e-3), 1), "unit": "tok/s (whole job)", "ms_per_step": round(per_step, 4), "steps": steps,
                    "sequences": n_seqs, "context": prompt_len, "prefill_s": round(t_prefill, 2), "bytes_per_gpu_per_step": int(algo),
                    "per_gpu_gbs": round(algo / (per_step * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(algo / (per_step * 1e-3) / 1e9 / peak, 4),
                    "gpu_launches_per_rank": int(ctr["kernel_launches"])}

        spec = synth.LLAMA70B
        if spec.num_heads % world == 0 and spec.num_kv_heads % world == 0 and (spec.intermediate_size // world) % 256 == 0 and spec.vocab_size % world == 0:
            steps, warm = 128, 3
            big = world >= 8   # the 32-sequence case prefills 131072 tokens: only where eight GPUs share that work
            t0 = time.perf_counter()
            eng = synth.build_engine(spec, 4096 + warm + steps + 16, on_device=True, device=local, max_seqs=32 if big else 1)
            leg = {"workload": f"configs[4]: Llama-3-70B shape, Q4_K, tensor parallel over {world} GPUs (heads, FFN rows and vocabulary cut; two sums over "
                               "the ranks per layer), 4096-token seeded prompts, greedy decode", "model_build_s": round(ranks.barrier_max(time.perf_counter() - t0), 2)}
            leg["bs1"] = decode_leg(eng, spec, 1, 4096, steps, warm, 3000)
            if big:
                eng.kv_clear()
                leg["bs32"] = decode_leg(eng, spec, 32, 4096, steps, warm, 3100)
            eng.close()
            out["tp70b"] = leg
        spec = synth.MIXTRAL
        if spec.num_heads % world == 0 and spec.num_kv_heads % world == 0 and spec.n_experts % world == 0 and spec.vocab_size % world == 0:
            t0 = time.perf_counter()
            eng = synth.build_engine(spec, 1024 + 3 + 64 + 16, on_device=True, device=local, max_seqs=16)
            leg = {"workload": f"configs[3]: Mixtral-8x7B shape, Q4_K, attention tensor parallel and {spec.n_experts // world} expert(s) per GPU over {world} GPUs "
                               "(every rank routes the same rows, adds the chosen experts it holds, one sum over the ranks completes the layer), "
                               "16 sequences x 1024-token prompts, greedy decode", "model_build_s": round(ranks.barrier_max(time.perf_counter() - t0), 2)}
            leg.update(decode_leg(eng, spec, 16, 1024, 64, 3, 2000))
            eng.close()
            out["ep_moe"] = leg
    finally:
        lcd.finalize()
    return out


def tp_ranks_one_gpu(lc, synth, tp: int, layers: int, ctx: int, steps: int) -> dict:
    """The ranks of the Llama-3-70B shape cut over `tp` GPUs, all in this process on ONE GPU (an in-process group: the same
    kernels with the same per-rank shapes, the sums over the ranks by a local kernel instead of over NVLink).  A profiling
    case: a launch list of this run shows what each rank executes; the time printed is all ranks' kernels one after the other."""
    from leafcutterllm_b200.engine import Engine
    lc._capi.check(lc.load().lc_set_device(0))
    spec = synth.LLAMA70B.with_layers(layers)
    engs = [synth.build_engine(spec, ctx + 64, on_device=True, device=0, tp_size=tp, tp_rank=r) for r in range(tp)]
    lead = Engine.group(engs)
    _, nxt = lead.forward_batch([0], [synth.prompt_tokens(ctx, spec.vocab_size, 5)], want_logits=False)
    toks, _ = lead.decode_loop([0], [int(nxt[0])], 3)
    toks, ms = lead.decode_loop([0], toks[-1].tolist(), steps)
    for e in engs:
        e.close()
    return {"workload": f"Llama-3-70B shape, {layers} layers, cut over {tp} ranks that all run on one GPU, batch 1, context {ctx}",
            "ms_per_step_all_ranks_in_turn": round(ms / steps, 4), "steps": steps, "not_the_metric": "profiling case"}


def run_ours(args):
    rank, world, local = dist_env()
    import leafcutterllm_b200 as lc
    from leafcutterllm_b200 import synth
    lib = lc.load()
    if lib.lc_device_count() <= 0:
        raise SystemExit("bench.py needs a CUDA device: " + lib.lc_last_error().decode())
    lc._capi.check(lib.lc_set_device(local))
    ranks = Ranks(rank, world, local, "nccl")
    barrier_max = ranks.barrier_max

    spec = synth.LLAMA7B if args.layers <= 0 else synth.LLAMA7B.with_layers(args.layers)
    e2e_steps = min(args.steps, 64)
    plen = args.prompt_len
    cap = plen + args.warmup + args.steps + e2e_steps + 3 + 64
    t0 = time.perf_counter()
    eng = synth.build_engine(spec, cap, on_device=True, device=local)
    t_build = time.perf_counter() - t0
    prompt = synth.prompt_tokens(plen, spec.vocab_size, seq_index=rank)
    t0 = time.perf_counter()
    _, nxt = eng.forward_batch([0], [prompt.tolist()], want_logits=False)
    t_prefill = time.perf_counter() - t0
    toks, _ = eng.decode_loop([0], nxt, max(args.warmup, 3))
    nxt = toks[-1]
    barrier_max(0.0)
    sampler = ClockSampler(local)
    sampler.start()
    eng.reset_counters()
    if args.profile_range:
        import torch
        torch.cuda.cudart().cudaProfilerStart()
    toks, ms = eng.decode_loop([0], nxt, args.steps)
    if args.profile_range:
        torch.cuda.cudart().cudaProfilerStop()
    ctr = eng.counters()
    ms_max = barrier_max(ms)
    clocks = sampler.stop()
    nxt = toks[-1]
    ctx_mid = plen + max(args.warmup, 3) + args.steps // 2

    # end to end: host token in (pinned staging inside the library), logits + pick out, every step, through the C ABI's
    # lc_forward_batch with host buffers that live across the steps (what a binding of the reference's Engine::forward would hold)
    import ctypes as C
    import numpy as np
    e_seq = np.zeros(1, np.int32); e_cnt = np.ones(1, np.int32)
    e_tok = np.array([int(nxt[0])], np.int64); e_next = np.zeros(1, np.int64)
    e_logits = np.empty((1, spec.vocab_size), np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    def e2e_step():
        lc._capi.check(lib.lc_forward_batch(eng._h, 1, vp(e_seq), vp(e_tok), vp(e_cnt), vp(e_logits), vp(e_next)))
        e_tok[0] = e_next[0]
    for _ in range(3):
        e2e_step()
    barrier_max(0.0)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = barrier_max(time.perf_counter() - t0)
    assert int(np.argmax(e_logits[0][::-1])) == spec.vocab_size - 1 - int(e_next[0]), "the pick is not the last maximum of the logits that came back"
    h2d = 8
    d2h = spec.vocab_size * 4 + 8

    value = world * args.steps / (ms_max * 1e-3)
    peak, which = measured_peaks()
    algo = ctr["algo_bytes_last_step"]
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_max / args.steps, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: Llama-2-7B-shape decoder (32 layers, hidden 4096, 32 heads, FFN 11008, vocab 32000), "
                               "Q4_K weights, batch 1 per GPU, 2048-token seeded prompt prefilled, then greedy decode steps; f16 KV cache",
                   "parallelism": "replicas only (one independent sequence per GPU, no exchange)" if world > 1 else "single GPU",
                   "l2": "inputs larger than L2: every step streams 3.7 GB of weights + 1.1 GB of KV through a 126 MB L2",
                   "context_at_midpoint": ctx_mid, "prefill_s": round(t_prefill, 3), "model_build_s": round(t_build, 3)},
        "e2e": {"value": round(world * e2e_steps / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "path": "lc_forward_batch: host token id -> pinned -> device, CUDA-graph step, logits + greedy pick -> pinned -> host"},
        "gpu_launches": int(ctr["kernel_launches"]),
        "clocks": clocks,
        "step_roofline": {"algorithmic_bytes_per_step": int(algo), "achieved_gbs": round(algo / (ms_max / args.steps * 1e-3) / 1e9, 1),
                          "peak_gbs": peak, "frac": round(algo / (ms_max / args.steps * 1e-3) / 1e9 / peak, 4), "peak_source": which},
    }
    if args.layers > 0:
        line["not_the_metric"] = f"profiling case: {args.layers} of 32 layers"
    if rank == 0:
        line["roofline"] = gemv_roofline(lc, spec)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(spec)
    eng.close()
    try:
        if rank == 0 and world == 1 and not args.no_bs64 and args.layers <= 0:
            line["bs64"] = batched_decode(lc, synth, spec, local, steps=min(max(args.steps, 32), 128))
        if rank == 0 and world == 1 and not args.no_extra and args.layers <= 0:
            line["tiny"] = tiny_decode(lc, synth, local)
            if not args.no_cpu:
                line["tiny"]["cpu_baseline"] = tiny_cpu()
            line["moe"] = moe_decode(lc, synth, local)
            line["q4km"] = q4km_decode(lc, synth, local)
        if world > 1 and not args.no_extra and args.layers <= 0:
            extra = cut_model_legs(lc, synth, ranks, rank, world, local)
            if rank == 0:
                line.update(extra)
    except Exception as ex:  # the legs after the metric must not cost the metric line
        line["extra_legs_error"] = f"{type(ex).__name__}: {ex}"[:400]
    ranks.close()
    if rank == 0:
        print(json.dumps(line))


def run_reference(args):
    rank, world, _local = dist_env()
    if rank != 0:
        return
    from leafcutterllm_b200 import synth   # model description only; nothing of the CUDA library is loaded or run in this arm
    spec = synth.LLAMA7B
    steps = max(1, min(args.steps, 4))
    ctx = max(8, min(args.ref_context, args.prompt_len))
    t0 = time.perf_counter()
    cb = cpu_baseline(spec, steps=steps, prompt=ctx)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(cb["value"], 4), "unit": "tok/s", "n_gpus": world, "steps": steps,
        "steps_requested": args.steps, "warmup": 0, "ms_per_step": round(1e3 / cb["value"], 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"configs[1] SAMPLED, not run in full: 2 of the 32 layers + the head of the Llama-2-7B shape, Q4_K weights, batch 1, "
                               f"a {ctx}-token context (the GPU arm decodes over 2048), {steps} greedy decode steps timed, the per-token time "
                               "extrapolated to 32 layers.  The reference cannot be compiled here (no Rust toolchain), so its CPU path is the C++ "
                               "restatement in oracle/ in its FASTEST mode (weights dequantised once, OpenMP on every host core); the reference's own "
                               "per-token re-dequantisation is the reference_faithful figure",
                   "same_config_as_gpu_arm": False, "wall_s": None},
        "cpu_baseline": cb,
        "e2e": {"value": round(cb["value"], 4), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line["config"]["wall_s"] = round(time.perf_counter() - t0, 1)
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-bs64", action="store_true", help="skip the 64-sequence continuous-batching leg (configs[2])")
    ap.add_argument("--no-extra", action="store_true", help="skip the legs after the metric: configs[0], configs[3] (one GPU), the cut 70B / mixture models (several GPUs)")
    ap.add_argument("--ref-context", type=int, default=64, help="--impl reference: context of the sampled CPU run (the oracle's prefill is slow)")
    ap.add_argument("--only", default="", choices=["", "gemv", "attn", "gemv-sweep", "gemv-types", "gemm", "gemm-small", "bs64", "moe", "tiny", "q4km", "tp-ranks", "tcgen05-probe"], help="gemv / attn: run just the isolated GEMV or decode-attention loop (small cases for profilers); gemv-sweep: GEMV time against row count; tp-ranks: the ranks of a cut 70B-shape model as one in-process group on one GPU (what each rank's kernels cost)")
    ap.add_argument("--gemm-shapes", default="", help="--only gemm: k x n pairs instead of the 7B layer shapes, e.g. 1024x12288,8192x12288")
    ap.add_argument("--gemm-tokens", default="", help="--only gemm: token counts instead of 64,512")
    ap.add_argument("--tp", type=int, default=8, help="--only tp-ranks: ranks the model is cut over")
    ap.add_argument("--profile-range", action="store_true", help="bracket the timed decode loop with cudaProfilerStart/Stop")
    ap.add_argument("--layers", type=int, default=0, help="profiling only: keep this many of the 32 layers (the printed number is then not the metric)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="context prefilled before decoding (default: the 2048 of the workload)")
    args = ap.parse_args()
    if args.only == "attn":
        import leafcutterllm_b200 as lc
        print(json.dumps(attention_microbench(lc)))
    elif args.only == "gemv-sweep":
        import leafcutterllm_b200 as lc
        print(json.dumps(gemv_sweep(lc)))
    elif args.only == "gemv-types":
        import leafcutterllm_b200 as lc
        print(json.dumps(gemv_types(lc)))
    elif args.only == "bs64":
        import leafcutterllm_b200 as lc
        from leafcutterllm_b200 import synth
        spec = synth.LLAMA7B if args.layers <= 0 else synth.LLAMA7B.with_layers(args.layers)
        out = batched_decode(lc, synth, spec, 0, steps=min(args.steps, 128), profile_range=args.profile_range)
        if args.layers > 0:
            out["not_the_metric"] = f"profiling case: {args.layers} of 32 layers"
        print(json.dumps(out))
    elif args.only == "q4km":
        import leafcutterllm_b200 as lc
        from leafcutterllm_b200 import synth
        lc._capi.check(lc.load().lc_set_device(0))
        print(json.dumps(q4km_decode(lc, synth, 0, prompt_len=args.prompt_len, steps=min(args.steps, 64), layers=args.layers)))
    elif args.only in ("moe", "tiny"):
        import leafcutterllm_b200 as lc
        from leafcutterllm_b200 import synth
        lc._capi.check(lc.load().lc_set_device(0))
        print(json.dumps(moe_decode(lc, synth, 0, steps=min(args.steps, 64), layers=args.layers) if args.only == "moe" else tiny_decode(lc, synth, 0)))
    elif args.only in ("gemm", "gemm-small"):
        import leafcutterllm_b200 as lc
        shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.gemm_shapes.split(",")] if args.gemm_shapes else None
        tokens = tuple(int(v) for v in args.gemm_tokens.split(",")) if args.gemm_tokens else ((64,) if args.only == "gemm-small" else (64, 512))
        print(json.dumps(gemm_microbench(lc, tokens=tokens, small=args.only == "gemm-small", shapes=shapes)))
    elif args.only == "tcgen05-probe":
        import ctypes as C
        import leafcutterllm_b200 as lc
        out = (C.c_double * 16)()
        lc._capi.check(lc.load().lc_tcgen05_probe(out))
        names = ["mma_n128_one_issuer", "mma_n256_one_issuer", "mma_n128_two_issuers_each", "commit", "st16_wait", "st16_wait_fence_arrive128",
                 "ld16_wait", "fence_before", "fence_after", "barrier_probe_vote", "arrive_to_waiter_returns", "unpack_chunk_4_warps",
                 "unpack_chunk_8_warps", "unpack_chunk_16_warps"]
        print(json.dumps({"unit": "SM cycles per operation", **{n: round(out[i], 1) for i, n in enumerate(names)}}))
    elif args.only == "tp-ranks":
        import leafcutterllm_b200 as lc
        from leafcutterllm_b200 import synth
        print(json.dumps(tp_ranks_one_gpu(lc, synth, args.tp, args.layers if args.layers > 0 else 2, args.prompt_len if args.prompt_len != PROMPT_LEN else 4096,
                                          min(args.steps, 16))))
    elif args.only == "gemv":
        import leafcutterllm_b200 as lc
        from leafcutterllm_b200 import synth
        print(json.dumps(gemv_roofline(lc, synth.LLAMA7B, reps=1, copies=2, warm=1)))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
