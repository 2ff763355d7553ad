"""Pre-flight checks of a GGUF file: scan_for_corruption (rust/src/model/loader.rs:301-422) as a GPU block-scale scan and
GGUFModel::capability_report (loader.rs:54-104)."""
import numpy as np
import pytest

from gguf_util import spec_metadata, write_gguf

# (type code, elements per block, bytes per block): rust/src/model/quant.rs:71-100, 160-238
BLOCK_TYPES = [(2, 32, 18), (3, 32, 20), (6, 32, 22), (7, 32, 24), (8, 32, 34), (9, 32, 36), (10, 256, 84), (11, 256, 110),
               (12, 256, 144), (13, 256, 176), (14, 256, 210), (15, 256, 292), (16, 256, 66), (17, 256, 74), (18, 256, 98),
               (19, 256, 110), (20, 32, 18), (21, 256, 136), (22, 256, 136), (23, 256, 162), (24, 256, 162), (25, 256, 176)]

F16_INF, F16_NAN, F16_MAX, F16_1E4_UP, F16_1E4 = 0x7C00, 0x7E00, 0x7BFF, 0x70E3, 0x70E2  # 0x70E2 = 10000.0, 0x70E3 = 10008.0


def _put16(buf, at, v):
    buf[at], buf[at + 1] = v & 0xFF, v >> 8


def test_oracle_scan_known_answers(oracle):
    """The reading rules of loader.rs:338-392, one by one."""
    # Q4_K: d at 0, dmin at 2; the limit is |v| > 1e4, not >=
    b = np.zeros(144 * 6, np.uint8)
    _put16(b, 0 * 144, F16_1E4)         # exactly 1e4: good
    _put16(b, 1 * 144, F16_1E4_UP)      # above: bad
    _put16(b, 2 * 144 + 2, F16_INF)     # dmin infinite: bad
    _put16(b, 3 * 144 + 2, F16_NAN | 0x8000)  # dmin NaN (sign set): bad
    _put16(b, 4 * 144, 0xF0E3)          # -10008: bad
    _put16(b, 5 * 144 + 4, F16_INF)     # byte 4 is not a scale: good
    assert oracle.scan_blocks(12, b, 6 * 256) == (6, 4)
    # Q6_K: only the f16 at byte 208
    b = np.zeros(210 * 3, np.uint8)
    _put16(b, 0, F16_INF)               # ql bytes: not looked at
    _put16(b, 210 + 208, F16_NAN)
    assert oracle.scan_blocks(14, b, 3 * 256) == (3, 1)
    # Q8_K: f32 at 0; Q8_1: f32 at 0 and at 4
    b = np.zeros(292 * 2, np.uint8)
    b[292:296] = np.frombuffer(np.float32(1.0e4 + 1).tobytes(), np.uint8)
    assert oracle.scan_blocks(15, b, 512) == (2, 1)
    b = np.zeros(36 * 3, np.uint8)
    b[36 + 4:36 + 8] = np.frombuffer(np.float32(-np.inf).tobytes(), np.uint8)
    b[72:76] = np.frombuffer(np.float32(9999.0).tobytes(), np.uint8)
    assert oracle.scan_blocks(9, b, 96) == (3, 1)
    # Q4_0 / Q8_0 / IQ4_NL: the reference reads bytes 2..3 (quantised data) as a second scale (loader.rs:372-377)
    for typ, bb in ((2, 18), (8, 34), (20, 18)):
        b = np.zeros(bb * 2, np.uint8)
        _put16(b, bb + 2, F16_MAX)
        assert oracle.scan_blocks(typ, b, 64) == (2, 1)
    # a ragged element count rounds the block count up (loader.rs:325); types without blocks are skipped (:309-322)
    assert oracle.scan_blocks(12, np.zeros(288, np.uint8), 257) == (2, 0)
    for typ in (0, 1, 30, 4, 5, 26, 99):
        assert oracle.scan_blocks(typ, np.zeros(64, np.uint8), 16) == (0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("typ,be,bb", BLOCK_TYPES)
def test_scan_equals_the_oracle_on_random_bytes(gpu, oracle, typ, be, bb):
    """Random bytes make every kind of scale: about 1 in 6 half-words is NaN, infinite or above 1e4."""
    from leafcutterllm_b200 import scan_blocks
    rng = np.random.default_rng(1000 + typ)
    for n_blocks, ragged in ((1, 0), (7, 3), (1000, 0), (40_001, be - 1)):
        raw = rng.integers(0, 256, n_blocks * bb, dtype=np.uint8)
        n_elems = n_blocks * be - ragged
        want = oracle.scan_blocks(typ, raw, n_elems)
        assert want[0] == n_blocks and want[1] <= n_blocks and (n_blocks < 1000 or want[1] > 0)
        assert scan_blocks(typ, raw, n_elems) == want


@pytest.mark.gpu
def test_scan_edge_cases(gpu, oracle):
    from leafcutterllm_b200 import scan_blocks
    assert scan_blocks(12, np.zeros(0, np.uint8), 0) == (0, 0)          # empty tensor
    assert scan_blocks(0, np.zeros(64, np.uint8), 16) == (0, 0)         # F32: nothing to scan
    assert scan_blocks(30, np.zeros(64, np.uint8), 32) == (0, 0)        # BF16
    assert scan_blocks(77, np.zeros(64, np.uint8), 32) == (0, 0)        # unknown code
    clean = np.zeros(144 * 5000, np.uint8)
    assert scan_blocks(12, clean, 5000 * 256) == (5000, 0)
    clean[144 * 4999 + 1] = 0x7C                                         # the last block only
    assert scan_blocks(12, clean, 5000 * 256) == oracle.scan_blocks(12, clean, 5000 * 256) == (5000, 1)
    all_bad = np.full(34 * 3000, 0xFF, np.uint8)                         # every scale NaN
    assert scan_blocks(8, all_bad, 3000 * 32) == (3000, 3000)


@pytest.mark.gpu
def test_scan_of_a_7b_sized_matrix(gpu, oracle):
    """One 11008 x 4096 Q4_K matrix (25 MB) of synthetic weights with a handful of damaged blocks."""
    from leafcutterllm_b200 import scan_blocks, synth
    raw = synth.tensor_bytes(synth.LLAMA7B, "blk.0.ffn_down.weight", 12, (11008, 4096), "normal", 1234).copy()
    n = 11008 * 4096
    assert scan_blocks(12, raw, n) == (n // 256, 0)
    rng = np.random.default_rng(5)
    hit = rng.choice(n // 256, 37, replace=False)
    for i, blk in enumerate(hit):
        _put16(raw, int(blk) * 144 + (2 if i % 2 else 0), (F16_INF, F16_NAN, F16_1E4_UP)[i % 3])
    assert scan_blocks(12, raw, n) == oracle.scan_blocks(12, raw, n) == (n // 256, 37)


def _tensors(spec, seed=1234):
    from leafcutterllm_b200 import synth
    return [(name, typ, dims, synth.tensor_bytes(spec, name, typ, dims, kind, seed)) for name, typ, dims, kind in spec.tensors()]


def test_capability_report_needs_no_gpu(tmp_path):
    """scan = 0: the file is only parsed (loader.rs:54-104)."""
    from leafcutterllm_b200 import inspect_gguf, synth
    spec = synth.TINY.with_layers(2)
    path = tmp_path / "ok.gguf"
    write_gguf(path, spec_metadata(spec), _tensors(spec))
    rep = inspect_gguf(path, scan=False)
    assert rep["architecture"] == "Llama" and rep["arch_supported"] and rep["can_run"]
    assert rep["missing_tensors"] == [] and rep["extra_tensors"] == []
    n = len(list(spec.tensors()))
    assert rep["quant_summary"]["total_tensors"] == n and rep["quant_summary"]["unsupported"] == []
    assert rep["quant_summary"]["types"] == {0: 5, 2: 14, 8: 2}        # 2 x 2 + 1 gains, 2 x 7 matrices, embedding + head
    assert rep["config"]["hidden_size"] == spec.hidden_size and rep["config"]["num_hidden_layers"] == 2
    assert rep["config"]["num_key_value_heads"] == spec.num_kv_heads and rep["config"]["vocab_size"] == spec.vocab_size
    assert "corruption" not in rep


def test_capability_report_findings(tmp_path):
    from leafcutterllm_b200 import inspect_gguf, synth
    spec = synth.TINY.with_layers(6)
    tensors = [t for t in _tensors(spec) if t[0] not in ("blk.1.ffn_up.weight", "blk.3.attn_k.weight", "blk.5.attn_q.weight")]
    tensors += [("blk.0.attn_qkv.weight", 0, (4,), np.zeros(4, np.float32)),      # unmapped suffix: extra
                ("blk.2.ffn_gate_inp.weight", 10, (256,), np.zeros(84, np.uint8)),  # Q2_K: no dequantiser
                ("blk.0.attn_norm.bias", 0, (4,), np.zeros(4, np.float32)),       # not *.weight: not looked at
                ("blk.4.weight", 0, (4,), np.zeros(4, np.float32)),               # no suffix after the second dot: extra
                ("odd.weight", 27, (4,), np.zeros(4, np.uint8))]                  # a type code the table does not know
    path = tmp_path / "findings.gguf"
    write_gguf(path, spec_metadata(spec, arch="qwen35"), tensors)
    rep = inspect_gguf(path, scan=False)
    assert rep["architecture"] == "Qwen3.5" and not rep["arch_supported"] and not rep["can_run"]
    # only the first four layers are sampled (loader.rs:63): blk.5 is not reported
    assert rep["missing_tensors"] == ["blk.1.ffn_up.weight", "blk.3.attn_k.weight"]
    # attn_qkv.weight is a known extra of this architecture (arch.rs:100-108)
    assert rep["extra_tensors"] == ["blk.2.ffn_gate_inp.weight", "blk.4.weight"]
    assert rep["quant_summary"]["unsupported"] == [10]
    assert rep["quant_summary"]["total_tensors"] == len(tensors)
    assert sum(rep["quant_summary"]["types"].values()) == len(tensors) - 1         # the unknown code is not counted (gguf.rs:321)
    # the same file as a Llama: attn_qkv.weight is unknown there, and only the type blocks the run
    write_gguf(path, spec_metadata(spec, arch="llama"), [t for t in tensors if t[0] != "blk.2.ffn_gate_inp.weight"] +
               [t for t in _tensors(spec) if t[0] in ("blk.1.ffn_up.weight", "blk.3.attn_k.weight")])
    rep = inspect_gguf(path, scan=False)
    assert rep["arch_supported"] and rep["missing_tensors"] == [] and rep["can_run"]
    assert rep["extra_tensors"] == ["blk.0.attn_qkv.weight", "blk.4.weight"]


def _q4k_spec(layers):
    import dataclasses
    from leafcutterllm_b200 import synth
    return dataclasses.replace(synth.TINY.with_layers(layers), layer_type=12, embed_type=12, head_type=12)


@pytest.mark.gpu
def test_corruption_report_of_a_file(gpu, oracle, tmp_path):
    from leafcutterllm_b200 import inspect_gguf
    spec = _q4k_spec(2)
    tensors = [(n, t, d, np.array(raw, copy=True).view(np.uint8).ravel()) for n, t, d, raw in _tensors(spec)]
    damaged = {"blk.0.attn_v.weight": [0, 5, 77], "blk.1.ffn_down.weight": [123], "token_embd.weight": [31999 * 8 + 7]}
    for name, typ, dims, raw in tensors:
        for i, blk in enumerate(damaged.get(name, [])):
            _put16(raw, blk * 144 + 2 * (i % 2), F16_INF)
    tensors.append(("blk.0.odd.weight", 13, (512,), np.full(2 * 176, 0xFF, np.uint8)))   # Q5_K, both blocks NaN
    path = tmp_path / "damaged.gguf"
    write_gguf(path, spec_metadata(spec), tensors)
    rep = inspect_gguf(path, scan=True)
    cor = rep["corruption"]
    want = []
    for name, typ, dims, raw in tensors:
        total, bad = oracle.scan_blocks(typ, raw, int(np.prod(dims)))
        if bad:
            want.append((name, typ, total, bad))
    got = [(r["name"], r["quant_type"], r["blocks_total"], r["blocks_bad"]) for r in cor["corrupted_tensors"]]
    assert got == want and len(want) == 4
    assert {n: b for n, _, _, b in want} == {"blk.0.attn_v.weight": 3, "blk.1.ffn_down.weight": 1, "token_embd.weight": 1,
                                             "blk.0.odd.weight": 2}
    # only the tensors with a bad block count towards total_blocks_checked (loader.rs:404-406)
    assert cor["total_blocks_checked"] == sum(t for _, _, t, _ in want) and cor["total_bad_blocks"] == 7
    assert cor["n_corrupt_tensors"] == 4
    few = inspect_gguf(path, scan=True, max_corrupt=2)["corruption"]
    assert few["n_corrupt_tensors"] == 4 and len(few["corrupted_tensors"]) == 2 and few["total_bad_blocks"] == 7
    # the synthetic model itself is clean
    clean = tmp_path / "clean.gguf"
    write_gguf(clean, spec_metadata(spec), _tensors(spec))
    assert inspect_gguf(clean)["corruption"] == {"corrupted_tensors": [], "n_corrupt_tensors": 0, "total_blocks_checked": 0,
                                                  "total_bad_blocks": 0}


@pytest.mark.gpu
def test_q4_0_files_are_reported_as_the_reference_reports_them(gpu, oracle, tmp_path):
    """For Q4_0 / Q8_0 the reference reads bytes 2..3 of a block -- quantised data -- as a second scale (loader.rs:372-377),
    so an undamaged file of these types comes back with about one block in seven marked.  The scan keeps that reading:
    the report of a file equals the reference's, finding by finding."""
    from leafcutterllm_b200 import inspect_gguf, synth
    spec = synth.TINY.with_layers(1)
    tensors = _tensors(spec)
    path = tmp_path / "q4_0.gguf"
    write_gguf(path, spec_metadata(spec), tensors)
    cor = inspect_gguf(path)["corruption"]
    want = []
    for name, typ, dims, raw in tensors:
        total, bad = oracle.scan_blocks(typ, np.ascontiguousarray(raw).view(np.uint8).ravel(), int(np.prod(dims)))
        if bad:
            want.append((name, typ, total, bad))
    assert [(r["name"], r["quant_type"], r["blocks_total"], r["blocks_bad"]) for r in cor["corrupted_tensors"]] == want
    assert len(want) == 9 and cor["total_bad_blocks"] == sum(b for *_, b in want) > 0
