"""The oracle's mixture-of-experts FFN against an independent numpy restatement of its definition (the reference has no
mixture-of-experts code, so there is no reference value to pin it on): router logits from the f32 router, the top_k
experts with equal logits going to the higher index, softmax over the chosen logits, chosen experts added in ascending
index."""
import numpy as np
import pytest


def numpy_moe(x, router, experts, top_k):
    out = np.zeros_like(x, dtype=np.float64)
    picks = []
    for s in range(x.shape[0]):
        logits = (router.astype(np.float64) @ x[s].astype(np.float64)).astype(np.float32)
        order = sorted(range(len(logits)), key=lambda e: (logits[e], e), reverse=True)[:top_k]   # ties: higher index first
        chosen = sorted(order)
        w = np.exp(logits[chosen].astype(np.float64) - logits[chosen].max())
        w /= w.sum()
        picks.append(chosen)
        for e, we in zip(chosen, w):
            g, u, d = experts[e]
            h = g.astype(np.float64) @ x[s]
            h = h / (1.0 + np.exp(-h)) * (u.astype(np.float64) @ x[s])
            out[s] += we * (d.astype(np.float64) @ h)
    return out, picks


@pytest.mark.parametrize("top_k,tie", [(2, False), (1, False), (2, True), (1, True)])
def test_oracle_moe_matches_numpy(oracle, top_k, tie):
    from leafcutterllm_b200 import synth
    from leafcutterllm_b200.synth import ModelSpec
    H, F, E = 256, 512, 4
    spec = ModelSpec("moe", 1, H, 2, 2, F, 300, 10000.0, 12, 12, 12, n_experts=E, top_k=top_k)
    om = oracle.OracleModel(H, 1, 2, 2, F, 300, max_seq_len=16, n_experts=E, top_k=top_k)
    r = np.random.default_rng(1)
    router = (0.02 * r.standard_normal((E, H))).astype(np.float32)
    if tie:
        router[1] = router[2] = router[3] = 4.0 * router[3]
    experts = {}
    for name, typ, dims, kind in spec.tensors():
        data = router.view(np.uint8).ravel() if name.endswith("ffn_gate_inp.weight") else synth.tensor_bytes(spec, name, typ, dims, kind)
        om.set_tensor(name, typ, dims, data)
        if ".expert." in name:
            e, which = int(name.split(".")[3]), name.split(".")[-2]
            experts.setdefault(e, {})[which] = oracle.dequantize(typ, data, int(np.prod(dims))).reshape(dims[1], dims[0])
    ex = {e: (v["ffn_gate"], v["ffn_up"], v["ffn_down"]) for e, v in experts.items()}
    x = r.standard_normal((6, H)).astype(np.float32)
    want, picks = numpy_moe(x, router, ex, top_k)
    got = om.ffn(0, x)
    assert np.abs(got - want).max() <= 1e-5 + 1e-4 * np.abs(want).max()
    if tie:  # the three equal rows lead (their row is four times larger): the pick among them must be the highest indices
        lead = [p for p in picks if 0 not in p]
        assert lead and all(p == ([3] if top_k == 1 else [2, 3]) for p in lead)
