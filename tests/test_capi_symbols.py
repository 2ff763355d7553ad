"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "leafcutter_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(lc_[a-z0-9_]+)\s*\(", text))
    names.discard("lc_token_cb")
    return sorted(names)


def test_header_declares_the_interface():
    names = declared_symbols()
    for must in ["lc_matmul_f32", "lc_rms_norm", "lc_qmatmul", "lc_dequantize", "lc_forward", "lc_generate", "lc_kv_clear",
                 "lc_q8_0_matmul_shard", "lc_q4_0_matmul_shard", "lc_forward_batch", "lc_model_set_tensor"]:
        assert must in names


def test_library_exports_every_declared_symbol(lc):
    from leafcutterllm_b200 import _capi
    lib = ctypes.CDLL(_capi.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    unbound = [n for n in declared_symbols() if n not in _capi.SIGNATURES]
    assert not unbound, f"declared in the header but not bound in _capi.py: {unbound}"


def test_no_device_is_a_loud_error_not_a_fallback(lc):
    import numpy as np
    lib = lc.load()
    if lib.lc_device_count() > 0:
        pytest.skip("a device is present")
    with pytest.raises(lc.LeafcutterError) as e:
        lc.B200Backend().vec_add(np.ones(4, np.float32), np.ones(4, np.float32))
    assert "no CPU fallback" in str(e.value)
    with pytest.raises(lc.LeafcutterError):
        lc.Engine(64, 1, 2, 2, 128, 100)


def test_tensor_bytes_matches_reference_size_table(lc):
    # rust/src/model/gguf.rs:339-346 and rust/src/model/quant.rs:314-335
    lib = lc.load()
    for typ, want in [(12, 144), (13, 176), (14, 210), (2, 144), (8, 272)]:
        assert lib.lc_tensor_bytes(typ, 256) == want
    assert lib.lc_tensor_bytes(20, 16_777_216) == 9_437_184
    assert lib.lc_tensor_bytes(0, 100) == 400
