"""The allocation-free attention entry point against the regular one, through the C ABI.

Some callers of this library cannot call cudaMalloc when they need an attention result: a plugin that runs inside
a host framework's pre-sized arena, a process whose device-memory budget is already handed out, or code on a
latency path where an allocation would stall the device.  `lc_attention_decode_static` serves them: it keeps the
split-context partials in an array that is part of the library image, so calling it allocates and frees nothing.
This file checks that it returns what `lc_attention_decode_dev` returns, twice in a row (the second call finds
the first call's partials still in the shared array), and that it turns down shapes the array cannot hold.
It is collected last so that a failure here cannot hide any other test's result.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class Dev:
    """Device buffers made through the library's own allocation helper (the test may allocate; the call under test may not)."""

    def __init__(self, lc):
        self.lc, self.lib, self.ptrs = lc, lc.load(), []

    def put(self, arr):
        arr = np.ascontiguousarray(arr)
        p = C.c_void_p()
        self.lc._capi.check(self.lib.lc_dev_alloc(arr.nbytes, C.byref(p)))
        self.lc._capi.check(self.lib.lc_dev_upload(p, arr.ctypes.data_as(C.c_void_p), arr.nbytes))
        self.ptrs.append(p)
        return p

    def empty(self, nbytes):
        p = C.c_void_p()
        self.lc._capi.check(self.lib.lc_dev_alloc(nbytes, C.byref(p)))
        self.ptrs.append(p)
        return p

    def get(self, p, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        self.lc._capi.check(self.lib.lc_dev_download(out.ctypes.data_as(C.c_void_p), p, out.nbytes))
        return out

    def close(self):
        for p in self.ptrs:
            self.lib.lc_dev_free(p)


def reference(q, K, V, table, ctx, n_heads, n_kv, hd, page_tokens):
    """attention.rs:69-113 in float64 over the f16 values of the cache."""
    out = np.zeros((n_heads, hd))
    pos = np.arange(ctx)
    for h in range(n_heads):
        kvh = h // (n_heads // n_kv)
        k = K[table[pos // page_tokens], kvh, pos % page_tokens].astype(np.float64)
        v = V[table[pos // page_tokens], kvh, pos % page_tokens].astype(np.float64)
        s = k @ q[h].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v
    return out


@pytest.mark.parametrize("n_heads,n_kv,hd,ctx", [(32, 32, 128, 2100), (32, 4, 64, 777), (8, 2, 128, 33)])
def test_static_scratch_attention_matches_allocating_entry_point(gpu, n_heads, n_kv, hd, ctx):
    lib, page_tokens = gpu.load(), 16
    r = np.random.default_rng(ctx)
    n_pages = (ctx + page_tokens - 1) // page_tokens
    pool_pages = n_pages + 7
    K = r.standard_normal((pool_pages, n_kv, page_tokens, hd)).astype(np.float16)
    V = r.standard_normal((pool_pages, n_kv, page_tokens, hd)).astype(np.float16)
    table = r.permutation(pool_pages)[:n_pages].astype(np.int32)  # scattered pages
    d = Dev(gpu)
    try:
        kd, vd, td = d.put(K), d.put(V), d.put(table)
        out_a, out_b = d.empty(n_heads * hd * 4), d.empty(n_heads * hd * 4)
        for call in range(2):  # two calls in a row: the shared array still holds the previous call's partials
            q = r.standard_normal((n_heads, hd)).astype(np.float32)
            qd = d.put(q)
            args = (qd, kd, vd, td, n_pages, ctx, n_heads, n_kv, hd, page_tokens, 0)
            # the entry point under test goes first: run alone in a fresh process, it is then the first call of the
            # process that launches a kernel, so nothing it relies on can have been allocated by an earlier call
            gpu._capi.check(lib.lc_attention_decode_static(*args, out_b))
            gpu._capi.check(lib.lc_attention_decode_dev(*args, out_a))
            gpu._capi.check(lib.lc_dev_sync())
            a, b = d.get(out_a, (n_heads, hd)), d.get(out_b, (n_heads, hd))
            assert np.abs(a - b).max() <= 1e-6, f"call {call}: the two entry points disagree"
            want = reference(q, K, V, table, ctx, n_heads, n_kv, hd, page_tokens)
            assert np.abs(b - want).max() <= 1e-4 + 1e-3 * np.abs(want).max(), f"call {call}: differs from the reference formula"
    finally:
        d.close()


def test_static_scratch_rejects_what_does_not_fit(gpu):
    """128 heads of 256 dims over 4096 keys: the split partials (about 4 MB) exceed the 1 MiB array.  Every buffer is real
    and large enough, so nothing invalid could run whatever the call decides."""
    lib = gpu.load()
    n_heads, n_kv, hd, ctx, page_tokens = 128, 1, 256, 4096, 16
    n_pages = ctx // page_tokens
    d = Dev(gpu)
    try:
        pool = np.zeros((n_pages, n_kv, page_tokens, hd), np.float16)
        kd, vd = d.put(pool), d.put(pool)
        td = d.put(np.arange(n_pages, dtype=np.int32))
        qd = d.put(np.zeros((n_heads, hd), np.float32))
        out = d.empty(n_heads * hd * 4)
        rc = lib.lc_attention_decode_static(qd, kd, vd, td, n_pages, ctx, n_heads, n_kv, hd, page_tokens, 0, out)
        assert rc == -1
        assert b"built-in array" in lib.lc_last_error()
        gpu._capi.check(lib.lc_attention_decode_dev(qd, kd, vd, td, n_pages, ctx, n_heads, n_kv, hd, page_tokens, 0, out))  # the allocating one takes it
        gpu._capi.check(lib.lc_dev_sync())
        assert lib.lc_attention_decode_static(None, kd, vd, td, n_pages, ctx, n_heads, n_kv, hd, page_tokens, 0, out) == -1
    finally:
        d.close()


@pytest.mark.parametrize("ctx,accepted", [(7936, True), (7937, False)])
def test_static_scratch_size_rule_at_its_edge(gpu, ctx, accepted):
    """32 heads of 128 dims: 62 pieces of 128 keys are the most whose partials fit the array, so a context of 7936 is
    taken (and agrees with the allocating entry point) and one of 7937 is refused."""
    lib = gpu.load()
    n_heads, n_kv, hd, page_tokens = 32, 2, 128, 16
    n_pages = (ctx + page_tokens - 1) // page_tokens
    r = np.random.default_rng(ctx)
    d = Dev(gpu)
    try:
        K = r.standard_normal((n_pages, n_kv, page_tokens, hd)).astype(np.float16)
        V = r.standard_normal((n_pages, n_kv, page_tokens, hd)).astype(np.float16)
        kd, vd = d.put(K), d.put(V)
        td = d.put(np.arange(n_pages, dtype=np.int32))
        qd = d.put(r.standard_normal((n_heads, hd)).astype(np.float32))
        out_a, out_b = d.empty(n_heads * hd * 4), d.empty(n_heads * hd * 4)
        args = (qd, kd, vd, td, n_pages, ctx, n_heads, n_kv, hd, page_tokens, 0)
        rc = lib.lc_attention_decode_static(*args, out_b)
        if not accepted:
            assert rc == -1 and b"built-in array" in lib.lc_last_error()
            return
        gpu._capi.check(rc)
        gpu._capi.check(lib.lc_attention_decode_dev(*args, out_a))
        gpu._capi.check(lib.lc_dev_sync())
        assert np.abs(d.get(out_a, (n_heads, hd)) - d.get(out_b, (n_heads, hd))).max() <= 1e-6
    finally:
        d.close()
