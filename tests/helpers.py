"""Helpers shared by the parity tests: fixture unpacking, seeded case generation, tolerance checks."""
import numpy as np

from oracle import nvfp4_oracle as o


def moe_params_from_golden(g):
    e, k, i, act = (int(v) for v in g["scalars"])
    return dict(topk_ids=(g["ids"], g["scores"]), hidden_states=g["hidden_states"],
                hidden_states_scale=g["hidden_states_scale"], gemm1_weights=g["gemm1_weights"],
                gemm1_weights_scale=g["gemm1_weights_scale"], gemm2_weights=g["gemm2_weights"],
                gemm2_weights_scale=g["gemm2_weights_scale"], gemm1_alpha=g["gemm1_alpha"], gemm1_beta=g["gemm1_beta"],
                gemm1_clamp_limit=g.get("gemm1_clamp_limit"), num_experts=e, top_k=k, intermediate_size=i,
                activation_type=act)


def compare_outputs(got, ref, atol=0.01, rtol=0.05):
    """Metrics of the reference contract (problem/metadata.json:34-46) and of the max-abs / rms bound."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if ref.size == 0:
        return dict(mismatch=0.0, rel_l2=0.0, rms=0.0, max_abs=0.0)
    bad = np.abs(ref - got) > atol + rtol * np.abs(got)
    denom = np.sqrt((ref ** 2).sum())
    rel_l2 = 0.0 if denom == 0 else float(np.sqrt(((ref - got) ** 2).sum()) / denom)
    return dict(mismatch=float(bad.mean()), rel_l2=rel_l2, rms=float(np.sqrt((ref ** 2).mean())),
                max_abs=float(np.abs(ref - got).max()))


def assert_layer_parity(got, ref, what="", extra_bf16_roundings=0):
    """Both acceptance rules: the reference's (atol .01, rtol .05, <=0.1% mismatches, rel-L2 <= .01) and
    max-abs-error <= 2e-2 * rms(output). `extra_bf16_roundings` widens the max-abs bound by that many bf16 ulps of the
    largest output magnitude: the expert-parallel path rounds one partial row per visited rank to bf16 before the
    final sum, which the single-GPU layer (and the reference) do not."""
    r = compare_outputs(got, ref)
    assert np.all(np.isfinite(got)), what
    if r["rms"] == 0.0:
        assert r["max_abs"] == 0.0, (what, r)
        return r
    assert r["mismatch"] <= 1e-3, (what, r)
    assert r["rel_l2"] <= 1e-2, (what, r)
    slack = 0.0
    if extra_bf16_roundings:
        peak = float(np.abs(np.asarray(ref, dtype=np.float64)).max())
        slack = extra_bf16_roundings * 2.0 ** (np.floor(np.log2(max(peak, 1e-30))) - 7)
    assert r["max_abs"] <= 2e-2 * r["rms"] + slack + 1e-6, (what, r)
    return r


def make_moe_case(seed, t, h, i, e, k, *, shared=0, global_scales=False, w_std=0.02, routing="uniform", masked=False):
    """Seeded synthetic layer inputs in the reference's storage formats (numpy), weights prepared with the oracle."""
    rng = np.random.default_rng(seed)
    x = o.bf16_round(rng.standard_normal((t, h), dtype=np.float32))
    hq, hs = o.quantize(x)
    etot = e + shared
    w1 = o.bf16_round((rng.standard_normal((etot, 2 * i, h), dtype=np.float32) * w_std))
    w2 = o.bf16_round((rng.standard_normal((etot, h, i), dtype=np.float32) * w_std))
    p = {}
    if global_scales:
        g1 = np.abs(w1).reshape(etot, -1).max(1) / (6.0 * 448.0)
        g2 = np.abs(w2).reshape(etot, -1).max(1) / (6.0 * 448.0)
        q1 = [o.quantize(w1[j], 16, float(g1[j])) for j in range(etot)]
        q2 = [o.quantize(w2[j], 16, float(g2[j])) for j in range(etot)]
        p["output1_scale_scalar"] = g1.astype(np.float32)
        p["output1_scale_gate_scalar"] = g1.astype(np.float32)
        p["output2_scale_scalar"] = g2.astype(np.float32)
    else:
        q1 = [o.quantize(w1[j]) for j in range(etot)]
        q2 = [o.quantize(w2[j]) for j in range(etot)]
    w1q, w1s = o.prepare_weights(np.stack([a for a, _ in q1]), np.stack([b for _, b in q1]), True)
    w2q, w2s = o.prepare_weights(np.stack([a for a, _ in q2]), np.stack([b for _, b in q2]), False)
    logits = rng.standard_normal((t, e), dtype=np.float32)
    if routing == "zipf":
        ranks = rng.permutation(e) + 1
        logits = logits + np.log(1.0 / ranks ** 1.2).astype(np.float32)
    ids, w = o.route_topk(logits, k)
    ids, w = o.apply_route_masks(ids, w, masked_routes=masked)
    p.update(topk_ids=(ids, w), hidden_states=hq, hidden_states_scale=hs, gemm1_weights=w1q, gemm1_weights_scale=w1s,
             gemm2_weights=w2q, gemm2_weights_scale=w2s, gemm1_alpha=np.ones(etot, np.float32),
             gemm1_beta=np.zeros(etot, np.float32), gemm1_clamp_limit=None, num_experts=e, top_k=k, intermediate_size=i,
             activation_type=3, num_fused_shared_experts=shared or None)
    return p
