"""The CPU oracle against the golden fixtures produced by the reference's own Python code."""
import numpy as np
import pytest

from oracle import nvfp4_oracle as o
from conftest import load_golden

MOE_CASES = ["balanced", "skew_clamp", "situ", "masked", "empty", "zero", "hotspot"]


def test_e4m3_roundtrip_all_codes():
    codes = np.arange(0, 0x7F, dtype=np.uint8)
    assert np.array_equal(o.e4m3_encode(o.e4m3_decode(codes)), codes)


def test_e4m3_matches_torch_cast():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.uniform(0, 448, 20000), rng.uniform(0, 0.05, 20000),
                        (o.E4M3_LUT[:0x7E] + o.E4M3_LUT[1:0x7F]) / 2]).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(o.e4m3_encode(x), ref)


def test_quantize_matches_reference_bytes():
    g = load_golden("quantize")
    for xk, pk, sk in (("x", "payload", "scale"), ("special", "special_payload", "special_scale"),
                       ("ties", "ties_payload", "ties_scale")):
        q, s = o.quantize(o.bf16_from_bits(g[xk]))
        assert np.array_equal(q, g[pk]), xk
        assert np.array_equal(s, g[sk]), xk
    q, s = o.quantize(o.bf16_from_bits(g["x"]), 16, float(g["global_scale"]))
    assert np.array_equal(q, g["payload_gs"])
    assert np.array_equal(s, g["scale_gs"])


def test_activation_qdq_matches_reference():
    g = load_golden("qdq")
    assert np.array_equal(o.nvfp4_qdq(g["value"]), g["qdq"])
    code = o.e2m1_code(g["e2m1_in"])
    assert np.array_equal(o.E2M1_LUT[code], g["e2m1_out"])


def test_router_matches_reference():
    g = load_golden("routes")
    for i in range(int(g["n"])):
        t, e, k, empty, masked = g[f"meta{i}"]
        ids, w = o.route_topk(g[f"logits{i}"], int(k))
        ids, w = o.apply_route_masks(ids, w, empty=bool(empty), masked_routes=bool(masked))
        assert np.array_equal(ids, g[f"ids{i}"]), i
        ref = g[f"w{i}"]
        ulp = np.abs(w.view(np.int32).astype(np.int64) - ref.view(np.int32).astype(np.int64))
        assert ulp.max() <= 4, (i, ulp.max())   # torch fp32 softmax vs correctly rounded


def test_weight_layout_matches_reference():
    g = load_golden("layout")
    for tag, gated in (("g", True), ("n", False)):
        pq, ps = o.prepare_weights(g["q"], g["sf"], gated)
        assert np.array_equal(pq, g["pq_" + tag])
        assert np.array_equal(ps, g["ps_" + tag])
        for e in range(pq.shape[0]):
            assert np.array_equal(o.weight_decode(pq[e], ps[e], gated), g["logical"][e])


def _moe_params(g):
    e, k, i, act = (int(v) for v in g["scalars"])
    p = dict(topk_ids=(g["ids"], g["scores"]), hidden_states=g["hidden_states"],
             hidden_states_scale=g["hidden_states_scale"], gemm1_weights=g["gemm1_weights"],
             gemm1_weights_scale=g["gemm1_weights_scale"], gemm2_weights=g["gemm2_weights"],
             gemm2_weights_scale=g["gemm2_weights_scale"], gemm1_alpha=g["gemm1_alpha"], gemm1_beta=g["gemm1_beta"],
             gemm1_clamp_limit=g.get("gemm1_clamp_limit"), num_experts=e, top_k=k, intermediate_size=i,
             activation_type=act)
    return p


def compare_outputs(got, ref, atol=0.01, rtol=0.05):
    """The reference contract's tolerance (metadata.json:40-45) plus the max-abs / rms bound."""
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    bad = np.abs(ref - got) > atol + rtol * np.abs(got)
    denom = np.sqrt((ref ** 2).sum())
    rel_l2 = 0.0 if denom == 0 else np.sqrt(((ref - got) ** 2).sum()) / denom
    rms = np.sqrt((ref ** 2).mean())
    max_abs = np.abs(ref - got).max() if ref.size else 0.0
    return dict(mismatch=bad.mean() if ref.size else 0.0, rel_l2=rel_l2, rms=rms, max_abs=max_abs)


@pytest.mark.parametrize("name", MOE_CASES)
def test_moe_layer_matches_reference(name):
    g = load_golden("moe_" + name)
    out = o.moe_expected(_moe_params(g))
    ref = o.bf16_from_bits(g["out"])
    r = compare_outputs(out, ref)
    # both sides are fp32 with different summation orders: allow a bf16 ulp on a few elements only
    assert r["max_abs"] <= 2e-2 * max(r["rms"], 1e-30) or r["rms"] == 0, r
    assert r["rel_l2"] <= 2e-3, r
    assert (o.bf16_bits(out) != g["out"]).mean() <= 0.02, (o.bf16_bits(out) != g["out"]).mean()


def test_moe_c1_shape_matches_reference_output():
    """The small benchmark shape (T=256, H=1024, I=512, E=8, top-2, seed 0): inputs regenerated with the same torch CPU
    generator calls and the oracle quantiser, pinned by the digests stored beside the reference's own output."""
    import hashlib
    torch = pytest.importorskip("torch")
    g = load_golden("moe_c1")
    t, h, i, e, k = 256, 1024, 512, 8, 2
    torch.manual_seed(0)
    x = torch.randn(t, h).to(torch.bfloat16)
    torch.randn(e, h)                                  # the gate matrix: drawn to keep the generator in step
    w1 = (torch.randn(e, 2 * i, h) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(e, h, i) * 0.02).to(torch.bfloat16)
    hq, hs = o.quantize(x.float().numpy())
    q1, s1 = o.prepare_weights(*o.quantize(w1.float().numpy()), True)
    q2, s2 = o.prepare_weights(*o.quantize(w2.float().numpy()), False)
    made = dict(hidden_states=hq, hidden_states_scale=hs, gemm1_weights=q1, gemm1_weights_scale=s1, gemm2_weights=q2,
                gemm2_weights_scale=s2)
    want = dict(zip(g["digest_names"].tolist(), g["digest_values"].tolist()))
    for name, arr in made.items():
        assert hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest() == want[name], name
    ids, scores = o.route_topk(g["logits"], k)
    assert np.array_equal(ids, g["ids"])
    assert np.abs(scores - g["scores"]).max() <= 4 * np.finfo(np.float32).eps
    p = dict(made, topk_ids=(g["ids"], g["scores"]), gemm1_alpha=np.ones(e, np.float32), gemm1_beta=np.zeros(e, np.float32),
             gemm1_clamp_limit=None, num_experts=e, top_k=k, intermediate_size=i, activation_type=3)
    out = o.moe_expected(p)
    r = compare_outputs(out, o.bf16_from_bits(g["out"]))
    assert r["max_abs"] <= 2e-2 * r["rms"] and r["rel_l2"] <= 2e-3, r
    assert (o.bf16_bits(out) != g["out"]).mean() <= 0.02


def test_dense_matches_reference():
    g = load_golden("dense")
    out = o.dense_expected(o.bf16_from_bits(g["a"]), g["b"], g["b_descale"], float(g["alpha"][0]))
    ref = o.bf16_from_bits(g["out"])
    r = compare_outputs(out, ref)
    assert r["rel_l2"] <= 1e-3 and r["mismatch"] == 0, r


def test_route_map_is_a_stable_partition():
    rng = np.random.default_rng(3)
    ids = rng.integers(-1, 8, size=(300, 4)).astype(np.int32)
    m = o.route_map(ids, 8, 128)
    assert m["seg_start"][-1] % 128 == 0 and np.all(m["seg_start"] % 128 == 0)
    for e in range(8):
        tok, slot = np.nonzero(ids == e)
        rows = m["row_of"][tok, slot]
        assert np.array_equal(rows, m["seg_start"][e] + np.arange(len(tok)))
        assert np.array_equal(m["tok_of_row"][rows], tok)
    assert np.all(m["row_of"][ids < 0] == -1)
    assert m["tile_rows"].sum() == (ids >= 0).sum()
