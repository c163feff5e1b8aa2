"""GPU parity of the whole layer through the drop-in Model (C ABI underneath) against the reference's outputs
(golden fixtures) and the oracle."""
import hashlib

import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import assert_layer_parity, make_moe_case, moe_params_from_golden
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu

MOE_CASES = ["balanced", "skew_clamp", "situ", "masked", "empty", "zero", "hotspot"]


@pytest.mark.parametrize("name", MOE_CASES)
def test_layer_matches_reference_golden(name):
    from gpu_util import run_model
    g = load_golden("moe_" + name)
    p = moe_params_from_golden(g)
    got, _, _ = run_model(p)
    assert_layer_parity(got, o.bf16_from_bits(g["out"]), name)


def test_intermediates_match_oracle():
    """Every stage against the oracle on one fixture: permuted rows, requantised activations, per-route FC2 rows."""
    from gpu_util import run_model
    g = load_golden("moe_hotspot")
    p = moe_params_from_golden(g)
    got, kw, model = run_model(p)
    layer = next(iter(model._layers.values()))
    ws = layer.workspace()
    ids = p["topk_ids"][0]
    m = o.route_map(ids, p["num_experts"], 128)
    rows = int(m["seg_start"][-1])
    live = np.nonzero(m["tok_of_row"] >= 0)[0]
    assert np.array_equal(ws["tok_of_row"][:rows].cpu().numpy()[live], m["tok_of_row"][live])
    tok = m["tok_of_row"][live]
    assert np.array_equal(ws["a_q"][:rows].cpu().numpy()[live], p["hidden_states"][tok])
    a_sf = o.unblock_scales(ws["a_sf"][: rows // 128].cpu().numpy()[None].reshape(1, rows // 128, -1, 32, 16), rows,
                            p["hidden_states_scale"].shape[1])[0]
    assert np.array_equal(a_sf[live], p["hidden_states_scale"][tok])
    _, inter = o.moe_expected(p, return_intermediates=True)
    i_sz = p["intermediate_size"]
    act_sf = o.unblock_scales(ws["act_sf"][: rows // 128].cpu().numpy().reshape(1, rows // 128, -1, 32, 16), rows, i_sz // 16)[0]
    act_q = ws["act_q"][:rows].cpu().numpy()
    rout = ws["rout"][:rows].float().cpu().numpy()
    for e, d in inter.items():
        r = m["row_of"][d["tok"], d["slot"]]
        code, stored = o.nvfp4_qdq_parts(d["act"])
        # the device uses fast exp / reciprocal in the activation: allow rare one-step differences
        assert (act_sf[r] != stored).mean() <= 0.02
        assert (act_q[r] != o.pack_codes(code)).mean() <= 0.05
        dev_act = o.decode(act_q[r], act_sf[r])
        ref_act = o.nvfp4_qdq(d["act"])
        assert np.abs(dev_act - ref_act).max() <= 0.26 * np.abs(ref_act).max() + 1e-6
        ref_rout = o.bf16_round(d["fc2"].astype(np.float32))
        assert np.sqrt(((rout[r] - ref_rout) ** 2).sum()) <= 2e-2 * np.sqrt((ref_rout ** 2).sum()) + 1e-6


def test_c1_shape_against_reference_output():
    """T=256, H=1024, I=512, E=8, top-2, seed 0: inputs are regenerated with the same torch CPU generator calls and the
    oracle quantiser, pinned by the digests stored with the reference's output."""
    from gpu_util import run_model
    g = load_golden("moe_c1")
    t, h, i, e, k = 256, 1024, 512, 8, 2
    torch.manual_seed(0)
    x = torch.randn(t, h).to(torch.bfloat16)
    gate_w = (torch.randn(e, h) * 0.02).to(torch.bfloat16)
    w1 = (torch.randn(e, 2 * i, h) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(e, h, i) * 0.02).to(torch.bfloat16)
    hq, hs = o.quantize(x.float().numpy())
    q1, s1 = o.quantize(w1.float().numpy())
    q2, s2 = o.quantize(w2.float().numpy())
    q1, s1 = o.prepare_weights(q1, s1, True)
    q2, s2 = o.prepare_weights(q2, s2, False)
    made = dict(hidden_states=hq, hidden_states_scale=hs, gemm1_weights=q1, gemm1_weights_scale=s1, gemm2_weights=q2,
                gemm2_weights_scale=s2)
    want = dict(zip(g["digest_names"].tolist(), g["digest_values"].tolist()))
    for name, arr in made.items():
        assert hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest() == want[name], name
    # router on the device from the stored logits, then the layer
    import kernelschema_b200 as ks
    ids, w = ks.route_topk(torch.from_numpy(g["logits"]).cuda(), k)
    assert np.array_equal(ids.cpu().numpy(), g["ids"])
    dev_logits = ks.router_logits(x.cuda(), gate_w.cuda()).cpu().numpy()
    assert np.abs(dev_logits - g["logits"]).max() <= 1e-5
    p = dict(made, topk_ids=(ids.cpu().numpy(), w.cpu().numpy()), gemm1_alpha=np.ones(e, np.float32),
             gemm1_beta=np.zeros(e, np.float32), gemm1_clamp_limit=None, num_experts=e, top_k=k, intermediate_size=i,
             activation_type=3)
    got, _, _ = run_model(p)
    assert_layer_parity(got, o.bf16_from_bits(g["out"]), "c1")


@pytest.mark.parametrize("kw", [
    dict(t=300, h=512, i=256, e=16, k=4),
    dict(t=64, h=256, i=512, e=8, k=2, shared=1),
    dict(t=500, h=512, i=512, e=32, k=8, global_scales=True, shared=1, routing="zipf"),
    dict(t=1, h=256, i=256, e=8, k=8),
    dict(t=129, h=256, i=256, e=4, k=4, masked=True),
])
def test_layer_matches_oracle_extensions(kw):
    """Seeded cases incl. the extensions the reference does not pin: shared experts and per-expert global scales."""
    from gpu_util import run_model
    kw = dict(kw)
    p = make_moe_case(11, kw.pop("t"), kw.pop("h"), kw.pop("i"), kw.pop("e"), kw.pop("k"), **kw)
    got, _, _ = run_model(p)
    assert_layer_parity(got, o.moe_expected(p), str(kw))


def test_tile_variants_agree():
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    p = make_moe_case(5, 400, 512, 256, 8, 2)
    ref = o.moe_expected(p)
    ids, w = p["topk_ids"]
    for bn in (128, 256, 512):
        layer = ks.MoELayer(512, 256, 8, 2, 400, tile_n=bn)
        out = torch.empty(400, 512, dtype=torch.bfloat16, device="cuda")
        layer.run(to_dev(ids), to_dev(w), to_dev(p["hidden_states"]), to_dev(p["hidden_states_scale"]),
                  to_dev(p["gemm1_weights"]), to_dev(p["gemm1_weights_scale"]), to_dev(p["gemm2_weights"]),
                  to_dev(p["gemm2_weights_scale"]), out)
        torch.cuda.synchronize()
        assert layer.status() == 0
        assert_layer_parity(out.float().cpu().numpy(), ref, f"tile_n={bn}")
        layer.close()


def test_expert_offset_selects_local_experts_only():
    """local_expert_offset: only ids in [offset, offset+E) contribute (the expert-parallel building block)."""
    from gpu_util import run_model
    p = make_moe_case(9, 200, 256, 256, 8, 4)
    full = o.moe_expected(p)
    parts = []
    for off in (0, 4):
        q = dict(p)
        for name in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "gemm1_alpha", "gemm1_beta"):
            q[name] = p[name][off:off + 4]
        q["num_experts"] = 4
        q["local_expert_offset"] = off
        got, _, _ = run_model(q)
        assert_layer_parity(got, o.moe_expected(q), f"offset {off}")
        parts.append(got)
    # the two halves sum to the full layer (up to the extra bf16 rounding of each half)
    assert np.abs(parts[0] + parts[1] - full).max() <= 5e-2 * np.sqrt((full ** 2).mean())


def test_model_rejects_bad_shapes():
    import kernelschema_b200 as ks
    from gpu_util import run_model
    p = make_moe_case(1, 8, 256, 256, 4, 2)
    bad = dict(p)
    bad["hidden_states_scale"] = p["hidden_states_scale"][:, :-1]
    with pytest.raises(ValueError):
        run_model(bad)
    with pytest.raises(ValueError):
        ks.MoELayer(100, 256, 4, 2, 8)


def test_direct_rows_mode_writes_per_route_results():
    """direct_rows: top-1 routing, FC2 stores bf16(fc2) of the token's route straight into the output (no combine pass)."""
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    p = make_moe_case(17, 300, 256, 256, 8, 1)
    ids, w = p["topk_ids"]
    ids = ids.copy()
    ids[::7] = -1                                    # tokens without a route stay untouched
    q = dict(p, topk_ids=(ids, np.ones_like(w)))
    ref = o.moe_expected(q)
    layer = ks.MoELayer(256, 256, 8, 1, 300)
    out = torch.full((300, 256), -17.0, dtype=torch.bfloat16, device="cuda")
    layer.run(to_dev(ids), to_dev(np.ones_like(w)), to_dev(p["hidden_states"]), to_dev(p["hidden_states_scale"]),
              to_dev(p["gemm1_weights"]), to_dev(p["gemm1_weights_scale"]), to_dev(p["gemm2_weights"]),
              to_dev(p["gemm2_weights_scale"]), out, direct_rows=True)
    torch.cuda.synchronize()
    assert layer.status() == 0
    got = out.float().cpu().numpy()
    routed = ids[:, 0] >= 0
    assert np.all(got[~routed] == -17.0)
    assert_layer_parity(got[routed], ref[routed], "direct_rows")
    layer.close()


def test_layer_is_cuda_graph_capturable():
    """The forward allocates nothing and never synchronises after warm-up, so a caller can capture it in a CUDA graph."""
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    p = make_moe_case(23, 64, 512, 256, 8, 2, shared=1)
    ids, w = p["topk_ids"]
    args = [to_dev(ids), to_dev(w), to_dev(p["hidden_states"]), to_dev(p["hidden_states_scale"]), to_dev(p["gemm1_weights"]),
            to_dev(p["gemm1_weights_scale"]), to_dev(p["gemm2_weights"]), to_dev(p["gemm2_weights_scale"])]
    layer = ks.MoELayer(512, 256, 8, 2, 64, num_shared_experts=1)
    out = torch.zeros(64, 512, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        layer.run(*args, out)                      # warm-up: tensor maps, kernel attributes
        side.synchronize()
        eager = out.clone()
        out.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            layer.run(*args, out)
        out.zero_()
        graph.replay()
        side.synchronize()
    assert layer.status() == 0
    assert torch.equal(out, eager)
    assert_layer_parity(out.float().cpu().numpy(), o.moe_expected(p), "graph replay")
    layer.close()


def test_library_graph_cache_and_hot_call():
    """b200moe_config.graph_cache: the second call with an identical argument block captures the launch chain, later ones
    replay it; routing and activations are read from memory at replay time, another argument block misses. The drop-in
    Model's repeat-call path (same tensor objects) goes through the same cache."""
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    p = make_moe_case(21, 200, 512, 256, 16, 4, shared=1, global_scales=True)
    ids, scores = p["topk_ids"]
    dev = dict(ids=to_dev(ids.astype(np.int32)), w=to_dev(scores.astype(np.float32)), hq=to_dev(p["hidden_states"]),
               hs=to_dev(p["hidden_states_scale"]), w1=to_dev(p["gemm1_weights"]), s1=to_dev(p["gemm1_weights_scale"]),
               w2=to_dev(p["gemm2_weights"]), s2=to_dev(p["gemm2_weights_scale"]))
    kw = dict(scale_up=to_dev(p["output1_scale_scalar"]), scale_gate=to_dev(p["output1_scale_gate_scalar"]),
              scale_out=to_dev(p["output2_scale_scalar"]))
    eager = ks.MoELayer(512, 256, 16, 4, 200, num_shared_experts=1)
    cached = ks.MoELayer(512, 256, 16, 4, 200, num_shared_experts=1, graph_cache=True)
    out_e = torch.empty((200, 512), dtype=torch.bfloat16, device="cuda")
    out_c = torch.empty_like(out_e)
    run = lambda layer, out: layer.run(dev["ids"], dev["w"], dev["hq"], dev["hs"], dev["w1"], dev["s1"], dev["w2"], dev["s2"], out, **kw)
    run(eager, out_e)
    for _ in range(4):
        out_c.fill_(-3)
        run(cached, out_c)
        assert torch.equal(out_c, out_e)
    st = cached.stats()
    assert (st["runs"], st["graph_captures"], st["graph_replays"]) == (4, 1, 2), st
    # new routing and activations in the same buffers: the replayed graph reads them
    p2 = make_moe_case(22, 200, 512, 256, 16, 4, shared=1, global_scales=True)
    dev["ids"].copy_(to_dev(p2["topk_ids"][0].astype(np.int32)))
    dev["w"].copy_(to_dev(p2["topk_ids"][1].astype(np.float32)))
    dev["hq"].copy_(to_dev(p2["hidden_states"]))
    dev["hs"].copy_(to_dev(p2["hidden_states_scale"]))
    run(eager, out_e)
    run(cached, out_c)
    assert torch.equal(out_c, out_e) and cached.stats()["graph_replays"] == 3
    # another output buffer is another argument block: eager first, then its own graph
    out_d = torch.empty_like(out_e)
    for _ in range(3):
        run(cached, out_d)
    assert torch.equal(out_d, out_e)
    st = cached.stats()
    assert st["graph_captures"] == 2 and st["graph_replays"] == 4 and st["graph_evictions"] == 0, st
    # inside the caller's own stream capture the library launches into that capture instead of nesting one
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        run(cached, out_c)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(g):
        run(cached, out_c)
    out_c.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_c, out_e) and cached.stats()["eager_in_capture"] >= 1
    assert cached.status() == 0
    # the drop-in Model: three calls with the same objects -> validation once, then the cached argument block
    from gpu_util import run_model
    model = ks.Model()
    got, kwm, model = run_model(p2, model)
    ref = got.copy()
    for _ in range(3):
        kwm["output"].zero_()
        res = model(**kwm)
        torch.cuda.synchronize()
        assert res[0] is kwm["output"]
        assert np.array_equal(kwm["output"].float().cpu().numpy(), ref)
    layer = next(iter(model._layers.values()))
    assert layer.stats()["graph_replays"] >= 2
    eager.close()
    cached.close()


@pytest.mark.parametrize("t,graph", [(200, False), (200, True), (1, True), (16, True), (2500, False), (2500, True)])
def test_whole_step_entry_equals_separate_calls(t, graph):
    """b200moe_step (bf16 tokens -> quantiser -> router logits -> top-k -> layer in one library call) against the same
    kernels called one by one; with the graph cache the second call captures and the later ones replay. From 2048 tokens
    on the quantiser runs on the library's side stream beside the router kernels (fork and join by events, captured too)."""
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    h, i, e, k, s = 512, 256, 16, 4, 1
    p = make_moe_case(31, t, h, i, e, k, shared=s, global_scales=True)
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((t, h), device="cuda", generator=gen).to(torch.bfloat16)
    gate = (torch.randn((e, h), device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    bias = torch.randn(e, device="cuda", generator=gen) * 0.1
    gs = 0.0021
    w = dict(w1=to_dev(p["gemm1_weights"]), s1=to_dev(p["gemm1_weights_scale"]), w2=to_dev(p["gemm2_weights"]),
             s2=to_dev(p["gemm2_weights_scale"]))
    kw = dict(scale_up=to_dev(p["output1_scale_scalar"]), scale_gate=to_dev(p["output1_scale_gate_scalar"]),
              scale_out=to_dev(p["output2_scale_scalar"]))
    ref_layer = ks.MoELayer(h, i, e, k, t, num_shared_experts=s)
    hq, hs = ks.nvfp4_quantize(x, gs)
    ids, wt = ks.route_topk(ks.router_logits(x, gate), k, bias)
    want = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ref_layer.run(ids, wt, hq, hs.view(torch.uint8), w["w1"], w["s1"], w["w2"], w["s2"], want, **kw)
    layer = ks.MoELayer(h, i, e, k, t, num_shared_experts=s, graph_cache=graph)
    out = torch.empty_like(want)
    for _ in range(4):
        out.fill_(-5)
        layer.step(x, gate, bias, gs, w["w1"], w["s1"], w["w2"], w["s2"], out, **kw)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    got = layer.step_outputs(t)
    assert torch.equal(got["ids"], ids) and torch.equal(got["weights"], wt)
    st = layer.stats()
    assert st["runs"] == 4 and st["graph_replays"] == (2 if graph else 0) and st["graph_captures"] == (1 if graph else 0), st
    # new tokens in the same buffer: the replayed chain re-quantises and re-routes them
    x.copy_(torch.randn((t, h), device="cuda", generator=gen).to(torch.bfloat16))
    hq, hs = ks.nvfp4_quantize(x, gs)
    ids, wt = ks.route_topk(ks.router_logits(x, gate), k, bias)
    ref_layer.run(ids, wt, hq, hs.view(torch.uint8), w["w1"], w["s1"], w["w2"], w["s2"], want, **kw)
    layer.step(x, gate, bias, gs, w["w1"], w["s1"], w["w2"], w["s2"], out, **kw)
    torch.cuda.synchronize()
    assert torch.equal(out, want) and layer.status() == 0
    ref_layer.close()
    layer.close()
