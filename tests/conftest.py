import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc
    orc.build()
    orc.lib()
    return orc


@pytest.fixture(scope="session")
def lc():
    import leafcutterllm_b200 as m
    m.load()
    return m


@pytest.fixture(scope="session")
def gpu(lc):
    if lc.load().lc_device_count() <= 0:
        pytest.fail("a test marked gpu ran without a CUDA device")
    return lc


def make_pair(lc, oracle, spec, max_seq_len=256, seed=1234, on_device=False, oracle_kwargs=None, **engine_kwargs):
    """The same synthetic model in the CUDA engine and in the CPU oracle (identical bytes)."""
    from leafcutterllm_b200 import synth
    eng = synth.build_engine(spec, max_seq_len, seed=seed, on_device=on_device, **engine_kwargs)
    okw = dict(oracle_kwargs or {})
    if engine_kwargs.get("kv_dtype") == "f32":
        okw["kv_f32"] = True
    if engine_kwargs.get("rope_mode") == "absolute":
        okw["rope_absolute"] = True
    om = oracle.OracleModel(spec.hidden_size, spec.num_layers, spec.num_heads, spec.num_kv_heads, spec.intermediate_size,
                            spec.vocab_size, max_seq_len=max_seq_len, rope_theta=spec.rope_theta, n_experts=spec.n_experts, top_k=spec.top_k, **okw)
    for name, typ, dims, kind in spec.tensors():
        if on_device and kind != "ones":
            data = eng.get_tensor(name, typ, dims)
        else:
            data = synth.tensor_bytes(spec, name, typ, dims, kind, seed)
        om.set_tensor(name, typ, dims, data)
    return eng, om


def assert_close(got, want, abs_tol, rel_tol, what=""):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape, what
    err = np.abs(got - want)
    bound = abs_tol + rel_tol * np.abs(want)
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance; worst abs err {err.max():.3e} at {err.argmax()}"
