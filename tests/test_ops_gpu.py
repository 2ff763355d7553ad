"""Operator-level parity on the GPU: every method of the Backend mirror, the dequantisers and the
quantised matmuls against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu

ALL_TYPES = [0, 1, 2, 8, 12, 13, 14, 20]


def rng(seed):
    return np.random.default_rng(seed)


def test_matmul_f32_is_bit_exact(gpu, oracle):
    be = gpu.B200Backend()
    r = rng(1)
    for (m, k, n) in [(2, 2, 2), (2, 3, 3), (16, 32, 24), (5, 77, 41), (128, 256, 128), (1, 512, 40)]:
        a = r.standard_normal(m * k).astype(np.float32)
        b = r.standard_normal(k * n).astype(np.float32)
        got = be.matmul(a, b, m, k, n)
        want = oracle.matmul(a, b, m, k, n)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (m, k, n)


def test_vector_ops_are_bit_exact(gpu, oracle):
    be = gpu.B200Backend()
    r = rng(2)
    for n in [1, 5, 1000, 4097]:
        a = r.standard_normal(n).astype(np.float32)
        b = r.standard_normal(n).astype(np.float32)
        assert np.array_equal(be.vec_add(a, b), oracle.vec_add(a, b))
        assert np.array_equal(be.vec_mul(a, b), oracle.vec_mul(a, b))
        assert np.array_equal(be.vec_scale(a, 0.37), oracle.vec_scale(a, np.float32(0.37)))
        assert np.array_equal(be.vec_scale_mul(a, 1.7, b), oracle.vec_scale_mul(a, np.float32(1.7), b))


def test_rms_norm_silu_softmax_sum_sq(gpu, oracle):
    be = gpu.B200Backend()
    r = rng(3)
    for hidden, rows in [(3, 1), (64, 4), (2048, 3), (4096, 2), (11008, 1)]:
        x = (r.standard_normal(hidden * rows) * 2).astype(np.float32)
        w = r.standard_normal(hidden).astype(np.float32)
        # sum of squares: different association than the reference's 4 strided lanes -> a few ulp of the sum
        assert_close(be.rms_norm(x, w, 1e-5, hidden), oracle.rms_norm(x, w, 1e-5, hidden), 1e-6, 2e-6, "rms_norm")
        assert_close(be.silu(x), oracle.silu(x), 1e-6, 1e-6, "silu")
        assert_close(be.softmax(x, hidden), oracle.softmax(x, hidden), 1e-8, 2e-6, "softmax")
        assert abs(be.sum_sq(x) - oracle.sum_sq(x)) <= 2e-6 * oracle.sum_sq(x)
    y = be.softmax(np.array([1.0, 2.0, 3.0], np.float32), 3)  # rust/src/model/tensor.rs:211-216
    assert abs(y.sum() - 1.0) < 1e-5


@pytest.mark.parametrize("typ", ALL_TYPES)
def test_dequantize_bit_exact_on_random_bytes(gpu, oracle, typ):
    be_elems, bb = gpu.QUANT_GEOMETRY[typ]
    r = rng(100 + typ)
    nblocks = 257 if be_elems > 1 else 4099
    raw = r.integers(0, 256, nblocks * bb, dtype=np.uint8)
    n = nblocks * be_elems
    got = gpu.dequantize(typ, raw, n)
    want = oracle.dequantize(typ, raw, n)
    g, w = got.view(np.uint32), want.view(np.uint32)
    nan_both = np.isnan(got) & np.isnan(want)
    assert np.array_equal(g[~nan_both], w[~nan_both])


@pytest.mark.parametrize("typ", [2, 8, 12])
def test_dequantize_bit_exact_on_synthetic_weights(gpu, oracle, typ):
    from leafcutterllm_b200 import synth
    n = 256 * 1024
    raw = synth.host_tensor(typ, 7, "t", n)
    assert np.array_equal(gpu.dequantize(typ, raw, n).view(np.uint32), oracle.dequantize(typ, raw, n).view(np.uint32))


def test_dequantize_rejects_ragged_and_unknown(gpu):
    with pytest.raises((ValueError, gpu.LeafcutterError)):
        gpu.dequantize(12, np.zeros(144, np.uint8), 255)
    with pytest.raises(gpu.LeafcutterError):
        gpu.dequantize(3, np.zeros(32, np.uint8), 32)  # Q4_1 has no kernel in the reference either


QM_CASES = [
    # typ, m, k, n
    (12, 1, 256, 32), (12, 1, 4096, 4096), (12, 1, 11008, 4096), (12, 1, 4096, 1000), (12, 3, 2048, 96), (12, 8, 512, 33),
    (12, 9, 1024, 64), (12, 2, 11008, 128),
    (2, 1, 2048, 2048), (2, 1, 5632, 2048), (2, 4, 256, 100), (2, 1, 96, 64),
    (8, 1, 2048, 3200), (8, 5, 512, 70), (8, 1, 64, 48),
    # Q4_0 / Q8_0 on the int8 tensor-core kernel: two to four tokens, rows of one to 43 units, row counts off the 32-row tile
    (2, 2, 1024, 77), (2, 3, 2304, 40), (2, 4, 11008, 33), (8, 2, 1024, 50), (8, 3, 768, 100), (8, 4, 4096, 33), (8, 1, 11008, 65),
    (13, 1, 512, 40), (14, 2, 512, 40), (20, 1, 128, 40), (0, 2, 100, 24), (1, 1, 100, 24),
    (13, 1, 4096, 300), (13, 5, 2816, 64), (13, 8, 256, 19), (14, 1, 4096, 300), (14, 3, 11008, 40), (14, 8, 768, 21),
    (20, 1, 4096, 300), (20, 2, 2816, 33), (0, 3, 512, 40), (1, 1, 4096, 300), (1, 8, 256, 19), (1, 2, 11008, 33),
    # Q6_K on the int8 tensor-core kernel (a multiple of 16 rows, one to four tokens): one unit, an odd number of units (every
    # other row's blocks then start two bytes off a word), more units than warps, several tiles per CTA
    (14, 1, 256, 16), (14, 1, 4096, 4096), (14, 1, 11008, 4096), (14, 2, 2816, 64), (14, 3, 11008, 48), (14, 4, 768, 160), (14, 4, 8192, 32),
    (14, 1, 4096, 32000),
    # Q5_K on the Q4_K kernel's fifth-bit variant (one to four tokens)
    (13, 1, 11008, 4096), (13, 2, 2816, 77), (13, 3, 11008, 40), (13, 4, 4096, 33), (13, 1, 256, 8),
    # five to eight tokens of these types: two passes of the tensor-core kernels
    (14, 8, 4096, 64), (14, 6, 11008, 32), (14, 5, 512, 48), (13, 7, 11008, 40), (13, 8, 4096, 96),
]


@pytest.mark.parametrize("typ,m,k,n", QM_CASES)
def test_qmatmul_vs_oracle(gpu, oracle, typ, m, k, n):
    from leafcutterllm_b200 import synth
    r = rng(k * 7 + n)
    if typ in (2, 8, 12, 0, 1):
        w = synth.host_tensor(typ, 99, f"w{typ}_{k}_{n}", n * k)
    else:  # no quantiser for these: random bytes with sane f16 scales
        be_elems, bb = gpu.QUANT_GEOMETRY[typ]
        w = r.integers(0, 256, n * k // be_elems * bb, dtype=np.uint8).reshape(-1, bb)
        sc = np.float16(r.uniform(0.001, 0.01, w.shape[0])).view(np.uint16)
        off = {13: 0, 14: 208, 20: 0}[typ]
        w[:, off] = sc & 0xFF
        w[:, off + 1] = sc >> 8
        if typ == 13:
            w[:, 2] = sc & 0xFF
            w[:, 3] = sc >> 8
        w = w.ravel()
    a = r.standard_normal(m * k).astype(np.float32)
    got = gpu.qmatmul(typ, a, w, m, k, n)
    want = oracle.qmatmul(typ, a, w, m, k, n)
    scale = np.abs(want).max()
    # the reference's own tolerance for its quantised GEMMs is 1e-3 absolute (int8_gemm.rs:394-511)
    assert_close(got, want, 2e-5 * scale, 1e-4, f"qmatmul typ={typ} {m}x{k}x{n}")


@pytest.mark.parametrize("typ", [12, 13])
@pytest.mark.parametrize("m,k,n", [(9, 256, 128), (16, 512, 128), (64, 4096, 512), (40, 2816, 300), (130, 1024, 256), (200, 11008, 128)])
def test_qmatmul_q4k_many_tokens_tensor_core_gemm(gpu, oracle, monkeypatch, typ, m, k, n):
    """Q4_K and Q5_K (the same unit with a fifth bit per element).  Nine tokens and more go through the tcgen05 product (weights dequantised into tensor memory as f16 high/low halves,
    activations as swizzled f16 high/low tiles): one k unit, token counts that are not a multiple of 16 or of the
    64-token tile, rows that are not a multiple of 128, a long k.  Activations carry a wide dynamic range so that the
    per-token power-of-two scale matters."""
    from leafcutterllm_b200 import synth
    w = synth.host_tensor(typ, 43, f"gemm_{k}_{n}", n * k)
    r = rng(k + n + m)
    a = (r.standard_normal((m, k)) * np.exp(r.uniform(-6, 6, (m, 1)))).astype(np.float32).ravel()
    got = gpu.qmatmul(typ, a, w, m, k, n).reshape(m, n)
    want = oracle.qmatmul(typ, a, w, m, k, n).reshape(m, n)
    for t in range(m):  # per token: its own scale
        assert_close(got[t], want[t], 2e-5 * np.abs(want[t]).max(), 1e-4, f"gemm {m}x{k}x{n} token {t}")
    monkeypatch.setenv("LC_GEMM_TERMS", "1")  # plain f16 operands: 2^-11 per factor
    fast = gpu.qmatmul(typ, a, w, m, k, n).reshape(m, n)
    for t in range(m):
        assert_close(fast[t], want[t], 4e-3 * np.abs(want[t]).max(), 0, f"one-term gemm token {t}")


def test_qmatmul_linearity_full_size(gpu, oracle):
    """7B-shape matrices: A(x+y) = Ax + Ay and a sample of rows against the oracle."""
    from leafcutterllm_b200 import synth
    for (k, n) in [(4096, 4096), (11008, 4096), (4096, 11008)]:
        w = synth.host_tensor(12, 5, f"full_{k}_{n}", n * k)
        r = rng(k + n)
        x = r.standard_normal(k).astype(np.float32)
        y = r.standard_normal(k).astype(np.float32)
        ax, ay, axy = (gpu.qmatmul(12, v, w, 1, k, n).ravel() for v in (x, y, x + y))
        assert_close(axy, ax + ay, 1e-4 * np.abs(axy).max(), 1e-4, "linearity")
        rows = r.choice(n, 64, replace=False)
        rb = k // 256 * 144
        sub = np.concatenate([w[i * rb:(i + 1) * rb] for i in rows])
        want = oracle.qmatmul(12, x, sub, 1, k, 64).ravel()
        assert_close(ax[rows], want, 2e-5 * np.abs(want).max(), 1e-4, "row sample")


def test_shard_order_gemms_are_bit_exact(gpu, oracle):
    # generators of rust/src/kernels/int8_gemm.rs:377-392 and :455-472
    for (m, k, n) in [(4, 8, 32), (8, 16, 64)]:
        bpr = n // 32
        scales = np.array([[0.01 * (row + 1)] * bpr for row in range(k)], np.float32)
        q8 = np.array([[b * 32 + jj - 16 for b in range(bpr) for jj in range(32)] for _ in range(k)], np.int8)
        a = (np.arange(m * k, dtype=np.float32) * np.float32(0.1)) if n == 32 else (np.arange(m * k, dtype=np.float32) * np.float32(0.01) - np.float32(0.5))
        got = gpu.q8_0_matmul(a, gpu.Q8Matrix(k, n, scales, q8), m, k, n)
        want = oracle.q8_0_matmul_shard(a, scales, q8, m, k, n)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        deq = (q8.astype(np.float32) * np.repeat(scales, 32, axis=1)).astype(np.float32)
        assert_close(got, oracle.matmul(a, deq, m, k, n), 1e-3, 0, "q8 vs dequant->f32 (reference test bound)")
        q4 = np.zeros((k, n // 2), np.uint8)
        for row in range(k):
            for b in range(bpr):
                for jj in range(16):
                    low = min(8 + (b * 32 + jj * 2) % 8, 15)
                    high = min(8 + (b * 32 + jj * 2 + 1) % 8, 15)
                    q4[row, b * 16 + jj] = (high << 4) | low
        got4 = gpu.q4_0_matmul(a, gpu.Q4Matrix(k, n, scales, q4), m, k, n)
        want4 = oracle.q4_0_matmul_shard(a, scales, q4, m, k, n)
        assert np.array_equal(got4.view(np.uint32), want4.view(np.uint32))
    with pytest.raises(gpu.LeafcutterError):
        gpu.q8_0_matmul(np.zeros(8, np.float32), gpu.Q8Matrix(8, 33, np.zeros((8, 1), np.float32), np.zeros((8, 33), np.int8)), 1, 8, 33)


def test_rope_and_argmax(gpu, oracle):
    r = rng(9)
    for (seq, heads, hd, theta, pos0) in [(1, 4, 64, 10000.0, 0), (7, 32, 128, 10000.0, 0), (5, 8, 64, 500000.0, 2043)]:
        x = r.standard_normal(seq * heads * hd).astype(np.float32)
        got = gpu.apply_rotary_emb(x, seq, heads, hd, theta, pos0)
        want = oracle.rope(x, seq, heads, hd, theta, pos0)
        # powf/sinf/cosf of the device and of glibc differ by ulps; at angle ~2000 rad that is ~1e-4 of |x|
        assert_close(got, want, 4e-4 * (1 + pos0 / 500.0), 1e-5, "rope")
    assert np.array_equal(gpu.apply_rotary_emb(x[:64 * 4], 1, 4, 64, 10000.0, 0), x[:64 * 4])  # position 0 is the identity
    assert gpu.sample_top_p(np.array([0.1, 0.5, 0.3], np.float32), 0.0, 0.9) == 1  # rust/src/inference/sampler.rs:56-61
    v = np.zeros(32000, np.float32)
    v[[5, 31000, 17]] = 3.0
    assert gpu.sample_top_p(v, 0.0, 1.0) == 31000 == oracle.argmax(v)  # last of equal maxima
    v = r.standard_normal(128256).astype(np.float32)
    assert gpu.sample_top_p(v, 0.0, 1.0) == oracle.argmax(v)


def test_tcgen05_probe_runs(gpu):
    """The diagnostic that times the building blocks of the many-token product: it must come back (every wait inside is
    bounded) with a positive cycle count for each of its fourteen measurements."""
    import ctypes as C
    out = (C.c_double * 16)()
    gpu._capi.check(gpu.load().lc_tcgen05_probe(out))
    vals = [out[i] for i in range(14)]
    assert all(v > 0 for v in vals), vals
    assert out[15] == 0.0
