"""Pins the CPU oracle on the known-answer values of the reference's own unit tests
(tests/golden/reference_kat.json, each with its file:line citation) and on independent numpy
restatements of the block formats."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
KAT = json.load(open(os.path.join(HERE, "golden", "reference_kat.json")))["cases"]


def shard_q8(k, n):  # rust/src/kernels/int8_gemm.rs:377-392
    bpr = n // 32
    scales = np.array([[0.01 * (row + 1)] * bpr for row in range(k)], np.float32)
    qs = np.array([[b * 32 + jj - 16 for b in range(bpr) for jj in range(32)] for _ in range(k)], np.int8)
    return scales, qs


def shard_q4(k, n):  # rust/src/kernels/int8_gemm.rs:455-472
    bpr = n // 32
    scales = np.array([[0.01 * (row + 1)] * bpr for row in range(k)], np.float32)
    qs = np.zeros((k, n // 2), np.uint8)
    for row in range(k):
        for b in range(bpr):
            for jj in range(16):
                low = min(8 + (b * 32 + jj * 2) % 8, 15)
                high = min(8 + (b * 32 + jj * 2 + 1) % 8, 15)
                qs[row, b * 16 + jj] = (high << 4) | low
    return scales, qs


@pytest.mark.parametrize("case", KAT, ids=[c["id"] for c in KAT])
def test_reference_known_answers(oracle, case):
    op = case["op"]
    if op == "dequantize":
        out = oracle.dequantize(case["type"], np.frombuffer(bytes.fromhex(case["bytes_hex"]), np.uint8), case["n"])
        for i, v in case["expect_at"].items():
            assert abs(out[int(i)] - v) < case["tol"]
    elif op == "dequantize_zeros":
        out = oracle.dequantize(case["type"], np.zeros(case["nbytes"], np.uint8), case["n"])
        assert (out == 0.0).all()
    elif op == "q8_0_block_iota":
        raw = np.zeros(34, np.uint8)
        raw[:2] = np.frombuffer(np.float16(case["scale"]).tobytes(), np.uint8)
        raw[2:] = np.arange(32, dtype=np.int8).view(np.uint8)
        out = oracle.dequantize(8, raw, 32)
        for i, v in case["expect_at"].items():
            assert abs(out[int(i)] - v) < case["tol"]
    elif op == "q4_0_shard_block":
        qs = np.array([[((min(8 + 2 * i + 1, 15) << 4) | (8 + 2 * i)) & 0xFF for i in range(16)]], np.uint8)
        out = oracle.q4_0_matmul_shard(np.ones(1, np.float32), np.array([case["scale"]], np.float32), qs, 1, 1, 32).ravel()
        for i, v in case["expect_at"].items():
            assert abs(out[int(i)] - v) < case["tol"]
    elif op == "quant_roundtrip_q8_0":
        data = ((np.arange(case["n"], dtype=np.float32) - 32.0) * np.float32(0.1)).astype(np.float32)
        out = oracle.dequantize(8, oracle.quantize_q8_0_ref(data), case["n"])
        assert np.abs(out - data).max() < case["tol"]
    elif op == "quant_roundtrip_q4_0":
        data = ((np.arange(case["n"], dtype=np.float32) - 32.0) * np.float32(0.1)).astype(np.float32)
        raw = oracle.quantize_q4_0_ref(data).reshape(-1, 18)
        for b in range(raw.shape[0]):  # shard order: byte i -> elements 2i, 2i+1 (q4_0.rs:36-46)
            scale = np.frombuffer(raw[b, :2].tobytes(), np.float16)[0].astype(np.float32)
            out = oracle.q4_0_matmul_shard(np.ones(1, np.float32), np.array([scale], np.float32), raw[b:b + 1, 2:], 1, 1, 32).ravel()
            assert np.abs(out - data[32 * b:32 * b + 32]).max() < case["tol"]
    elif op == "matmul":
        out = oracle.matmul(case["a"], case["b"], case["m"], case["k"], case["n"])
        assert out.tolist() == case["expect"]
    elif op == "matmul_ramp":
        m, k, n = case["m"], case["k"], case["n"]
        a = np.arange(m * k, dtype=np.float32) * np.float32(case["step"])
        b = np.arange(k * n, dtype=np.float32) * np.float32(case["step"])
        out = oracle.matmul(a, b, m, k, n)
        ref = (a.reshape(m, k).astype(np.float64) @ b.reshape(k, n).astype(np.float64)).ravel()
        # the reference compares against an f32 sequential loop at 1e-4; products here reach ~400, so allow its rounding
        assert np.abs(out - ref).max() < case["tol"] + 1e-6 * np.abs(ref).max()
    elif op == "vec_add":
        assert oracle.vec_add(case["a"], case["b"]).tolist() == case["expect"]
    elif op == "sum_sq":
        assert abs(oracle.sum_sq(case["a"]) - case["expect"]) < case["tol"]
    elif op == "rms_norm_finite":
        assert np.isfinite(oracle.rms_norm(case["x"], case["w"], case["eps"], 3)).all()
    elif op == "softmax_sum":
        assert abs(oracle.softmax(case["x"], 3).sum() - 1.0) < case["tol"]
    elif op == "argmax":
        assert oracle.argmax(case["v"]) == case["expect"]
    elif op == "f16_roundtrip_exact":
        assert oracle.f16_roundtrip(case["v"]).tolist() == case["v"]
    elif op == "tensor_bytes":
        for typ, count, want in case["cases"]:
            assert oracle.lib().orc_tensor_bytes(typ, count) == want
    elif op in ("shard_gemm_q8", "shard_gemm_q4"):
        m, k, n = case["m"], case["k"], case["n"]
        a = (np.arange(m * k, dtype=np.float32) * np.float32(case["a_step"]) + np.float32(case["a_off"])).astype(np.float32)
        if op == "shard_gemm_q8":
            scales, qs = shard_q8(k, n)
            got = oracle.q8_0_matmul_shard(a, scales, qs, m, k, n)
            deq = qs.astype(np.float32) * np.repeat(scales, 32, axis=1)
        else:
            scales, qs = shard_q4(k, n)
            got = oracle.q4_0_matmul_shard(a, scales, qs, m, k, n)
            nib = np.stack([qs & 0x0F, qs >> 4], axis=-1).reshape(k, n).astype(np.float32)
            deq = (nib - np.float32(8.0)) * np.repeat(scales, 32, axis=1)
        want = oracle.matmul(a, deq.astype(np.float32), m, k, n).reshape(m, n)
        assert np.abs(got - want).max() < case["tol"]
        assert np.array_equal(got, want)  # same FMA chain over k: bit-identical, as the reference's AVX2 path is
    else:
        raise AssertionError("unknown op " + op)


# ---- independent numpy restatements of the GGUF block formats (rust/src/kernels/mod.rs) ----
def np_f16(raw2):
    return np.ascontiguousarray(raw2).view(np.float16).astype(np.float32).ravel()


def np_dequant_q4_0(raw):
    b = raw.reshape(-1, 18)
    s = np_f16(b[:, :2])[:, None]
    lo = (b[:, 2:] & 0x0F).astype(np.float32) - np.float32(8)
    hi = (b[:, 2:] >> 4).astype(np.float32) - np.float32(8)
    return (np.concatenate([lo, hi], axis=1) * s).astype(np.float32).ravel()


def np_dequant_q8_0(raw):
    b = raw.reshape(-1, 34)
    s = np_f16(b[:, :2])[:, None]
    return (b[:, 2:].view(np.int8).astype(np.float32) * s).astype(np.float32).ravel()


def np_dequant_q4_k(raw):
    b = raw.reshape(-1, 144)
    d = np_f16(b[:, 0:2])[:, None]
    dmin = np_f16(b[:, 2:4])[:, None]
    q = b[:, 4:16].astype(np.uint32)
    sc = np.zeros((b.shape[0], 8), np.uint32)
    mn = np.zeros((b.shape[0], 8), np.uint32)
    for j in range(8):
        if j < 4:
            sc[:, j] = q[:, j] & 63
            mn[:, j] = q[:, j + 4] & 63
        else:
            sc[:, j] = (q[:, j + 4] & 0x0F) | ((q[:, j - 4] >> 6) << 4)
            mn[:, j] = (q[:, j + 4] >> 4) | ((q[:, j] >> 6) << 4)
    out = np.zeros((b.shape[0], 256), np.float32)
    qs = b[:, 16:]
    for g in range(4):
        byts = qs[:, 32 * g:32 * g + 32]
        dl1 = (d * sc[:, 2 * g:2 * g + 1].astype(np.float32)).astype(np.float32)
        dl2 = (d * sc[:, 2 * g + 1:2 * g + 2].astype(np.float32)).astype(np.float32)
        m1 = (dmin * mn[:, 2 * g:2 * g + 1].astype(np.float32)).astype(np.float32)
        m2 = (dmin * mn[:, 2 * g + 1:2 * g + 2].astype(np.float32)).astype(np.float32)
        out[:, 64 * g:64 * g + 32] = (dl1 * (byts & 0x0F).astype(np.float32)).astype(np.float32) - m1
        out[:, 64 * g + 32:64 * g + 64] = (dl2 * (byts >> 4).astype(np.float32)).astype(np.float32) - m2
    return out.ravel()


@pytest.mark.parametrize("typ,fn,bb,be", [(2, np_dequant_q4_0, 18, 32), (8, np_dequant_q8_0, 34, 32), (12, np_dequant_q4_k, 144, 256)])
def test_dequant_matches_independent_numpy(oracle, lc, typ, fn, bb, be):
    from leafcutterllm_b200 import synth
    raw = synth.host_tensor(typ, 11, "kat", be * 512)
    with np.errstate(all="ignore"):
        assert np.array_equal(oracle.dequantize(typ, raw, be * 512).view(np.uint32), fn(raw).view(np.uint32))
    r = np.random.default_rng(typ)
    raw = r.integers(0, 256, bb * 300, dtype=np.uint8)
    raw.reshape(-1, bb)[:, 1] &= 0x3B  # keep the f16 scales finite
    if typ == 12:
        raw.reshape(-1, bb)[:, 3] &= 0x3B
    with np.errstate(all="ignore"):
        assert np.array_equal(oracle.dequantize(typ, raw, be * 300).view(np.uint32), fn(raw).view(np.uint32))


def test_f16_conversion_matches_ieee(oracle):
    r = np.random.default_rng(0)
    x = np.concatenate([r.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** r.integers(-9, 6, 20000).astype(np.float32),
                        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 6.1e-5, np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(oracle.f16_roundtrip(x).view(np.uint32), want.view(np.uint32))
    for h in [0, 1, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x8001, 0xFBFF]:
        assert oracle.lib().orc_f16_to_f32(h) == np.array([h], np.uint16).view(np.float16).astype(np.float32)[0]


def test_matmul_layouts_agree_and_tail_rule(oracle):
    r = np.random.default_rng(5)
    m, k, n = 3, 70, 21  # 16 fused columns + 5 unfused tail columns (simd.rs:238-246)
    a = r.standard_normal(m * k).astype(np.float32)
    b = r.standard_normal(k * n).astype(np.float32)
    got = oracle.matmul(a, b, m, k, n).reshape(m, n)
    wt = np.ascontiguousarray(b.reshape(k, n).T)
    out2 = np.empty(m * n, np.float32)
    oracle.lib().orc_matmul_nk(a.ctypes.data, wt.ctypes.data, m, k, n, out2.ctypes.data)
    assert np.array_equal(got.ravel(), out2)
    tail = np.zeros(m, np.float32)
    for i in range(m):  # unfused: round the product, then the sum
        s = np.float32(0)
        for l in range(k):
            s = np.float32(s + np.float32(a[i * k + l] * b[l * n + 20]))
        tail[i] = s
    assert np.array_equal(got[:, 20], tail)


def test_rope_is_call_relative_and_half_split(oracle):
    x = np.arange(2 * 1 * 8, dtype=np.float32) + 1
    y = oracle.rope(x, 2, 1, 8, 10000.0)
    assert np.array_equal(y[:8], x[:8])  # position 0 of the call is the identity (attention.rs:13-21)
    d = 1
    ang = np.float32(1.0) * np.float32(1.0 / np.float32(10000.0) ** np.float32(2.0 * d / 8))
    assert abs(y[8 + d] - (x[8 + d] * np.cos(ang) - x[8 + d + 4] * np.sin(ang))) < 1e-5  # pairs (d, d + hd/2)


def test_argmax_takes_last_maximum(oracle):
    assert oracle.argmax([1.0, 3.0, 3.0, 2.0]) == 2  # sampler.rs:9: max_by keeps the last of equal maxima
    assert oracle.argmax([-0.0, 0.0]) == 1 and oracle.argmax([0.0, -0.0]) == 0  # total_cmp orders -0 < +0
