"""The reference's own acceptance run against the drop-in, and whole-output parity at the full benchmark sizes.

`oracle/build_ref.py` stages (unchanged, outside version control) the operator's problem files, its check harness
and its own host. Where that staging exists:

* `check_correctness` of the harness (eval/correctness.py:558-572) is called exactly as the reference's runner calls
  it, with `reference.py` as the truth and a two-line candidate `solution.py` that imports this package's `Model`,
  for all ten fixed shapes (problem/shape_cases.json) and both recorded seeds (problem/metadata.json:28-31). That run
  includes the harness' input-storage snapshot, its guard-band check and its alias check.
* the Qwen3-30B (T=16384) and DeepSeek-V3 (T=8192, shared expert, per-expert global scales, Zipf routing) layers of
  the benchmark are compared over the WHOLE output with the reference's `decode` / `weight` / `nvfp4` functions
  evaluated on the GPU one expert at a time (the stock `expected` materialises every expert in fp32: 45 GB for the
  DeepSeek-V3 geometry), with the two rules: the reference's tolerance, and max-abs-error <= 2e-2 * rms(output) in the
  form that a whole output of 1e7+ elements allows (see the comment at the assertion).
  Global scales and the shared expert are extensions the reference never evaluates (decode x scale; one more
  always-routed expert with weight 1).

The dense NVFP4 GEMM at its two largest benchmark sizes is compared with an fp32 matmul (TF32 off) of the decoded
operands; that needs no staging.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "oracle", "_ref")
STAGED = all(os.path.exists(os.path.join(REF, p)) for p in
             ("problem/reference.py", "problem/input.py", "problem/shapes.json", "problem/metadata.json",
              "harness/atrex_bench/eval/correctness.py"))

pytestmark = pytest.mark.gpu
needs_staging = pytest.mark.skipif(not STAGED, reason="oracle/_ref staging absent (python oracle/build_ref.py needs the reference checkout)")


def _reference_module():
    spec = importlib.util.spec_from_file_location("staged_reference", os.path.join(REF, "problem", "reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def candidate_path(tmp_path_factory):
    d = tmp_path_factory.mktemp("candidate")
    (d / "solution.py").write_text(f"import sys\nsys.path.insert(0, {ROOT!r})\nfrom kernelschema_b200.solution import Model\n")
    return d / "solution.py"


@needs_staging
@pytest.mark.parametrize("shape_id", [str(i) for i in range(10)])
def test_reference_check_correctness_fixed_shapes(shape_id, candidate_path):
    sys.path.insert(0, os.path.join(REF, "harness"))
    from atrex_bench.eval.correctness import check_correctness
    res = check_correctness(Path(REF) / "problem" / "reference.py", candidate_path, shape_id=shape_id, num_correctness_cases=2,
                            device="cuda")
    detail = [(c.error, [(o.name, o.passed, o.relative_l2, o.mismatched_elements, o.error) for o in (c.outputs or []) + (c.mutated_inputs or [])
                         + (c.unexpected_mutations or [])]) for c in res.cases]
    assert res.status == "passed", (res.reason, detail)
    assert len(res.cases) == 2 and all(c.error is None for c in res.cases), detail
    print(f"shape {shape_id}: " + "; ".join(f"seed {c.input_artifact['seed']} rel_l2 {c.outputs[0].relative_l2:.2e} "
                                            f"mismatch {c.outputs[0].mismatched_elements}/{c.outputs[0].total_elements}" for c in res.cases))


def _expected_streaming(ref, wl, L, ids, w, hq, hs):
    """reference.py::expected (lines 69-92) with one expert decoded at a time, the per-expert accumulator scales and
    the shared experts (every token, weight 1) added; fp32 on the GPU, TF32 off."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    e_routed, s = wl["e"], wl["s"]
    a = ref.decode(hq, hs.view(torch.uint8), "nvfp4")
    y = torch.zeros_like(a)
    f8 = torch.float8_e4m3fn
    for e in range(e_routed + s):
        if e < e_routed:
            tok, slot = (ids == e).nonzero(as_tuple=True)
            score = w[tok, slot]
        else:
            tok = torch.arange(a.shape[0], device=a.device)
            score = torch.ones(a.shape[0], device=a.device)
        if tok.numel() == 0:
            continue
        w1 = ref.weight(L["w1q"][e:e + 1], L["w1s"][e:e + 1].view(f8), True)[0]
        w2 = ref.weight(L["w2q"][e:e + 1], L["w2s"][e:e + 1].view(f8), False)[0]
        for off in range(0, tok.numel(), 4096):
            rows = tok[off:off + 4096]
            up, gate = (torch.einsum("th,ih->ti", a[rows], w1) * L["scale_fc1"][e]).chunk(2, -1)
            act = ref.nvfp4(gate * torch.sigmoid(gate) * up)
            part = (torch.einsum("ti,hi->th", act, w2) * L["scale_fc2"][e]).to(torch.bfloat16).float()
            y.index_add_(0, rows, part * score[off:off + 4096, None])
        del w1, w2
    return y


@needs_staging
@pytest.mark.parametrize("name", ["qwen3", "dsv3"])
def test_whole_output_parity_full_size(name):
    import bench
    import kernelschema_b200 as ks
    from helpers import compare_outputs
    ref = _reference_module()
    wl = dict(bench.WORKLOADS[name])
    dev = torch.device("cuda", 0)
    L = bench.build_layer(wl, 0, 1, dev)
    t, h, k = wl["t"], wl["h"], wl["k"]
    x = torch.randn((t, h), device=dev, generator=torch.Generator(device=dev).manual_seed(77)).to(torch.bfloat16)
    hq, hs = ks.nvfp4_quantize(x, bench.ACT_GLOBAL_SCALE)
    ids, w = ks.route_topk(ks.router_logits(x, L["gate_w"]), k, L["bias"])
    layer = ks.MoELayer(h, wl["i"], wl["e"], k, t, num_shared_experts=wl["s"])
    out = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
    layer.run(ids, w, hq, hs.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], out, scale_up=L["scale_fc1"],
              scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
    torch.cuda.synchronize()
    assert layer.status() == 0
    want32 = _expected_streaming(ref, wl, L, ids, w, hq, hs)          # the reference's fp32 sum, before its bf16 rounding
    got, exp = out.float(), want32.to(torch.bfloat16).float()
    diff = (got - exp).abs()
    rms = float(exp.pow(2).mean().sqrt())
    rel_l2 = float((got - exp).norm() / exp.norm())
    mismatch = float((diff > 0.01 + 0.05 * got.abs()).float().mean())
    # Where the max-abs rule can and cannot hold over a whole output of 3e7 .. 6e7 elements: both sides accumulate FC1 in
    # fp32 in different orders (relative noise ~1e-6), so a handful of the ~1e8 requantised activations fall on the other
    # side of an E2M1 threshold (or a block's E4M3 scale byte does), and such a flip moves every output of that route by
    # one code step x its weight: up to a few % of the rms on the largest weights. No implementation with another
    # summation order escapes that, the reference's own kernel included. Asserted: no element beyond 6 % of the rms, at
    # most one element per million beyond 2 % of the rms plus one bf16 step of the element (the final rounding to bf16 is
    # common to both sides: over 1e7+ elements some outputs lie 6-10 rms out, where a bf16 step alone is 2-4 % of the rms).
    ulp = torch.exp2(torch.floor(torch.log2(want32.abs().clamp_min(1e-30))) - 7)
    beyond = float((diff > 2e-2 * rms + ulp).float().mean())
    max_abs = float(diff.max())
    print(f"{name}: rms {rms:.4e} rel_l2 {rel_l2:.3e} mismatch {mismatch:.2e} max_abs/rms {max_abs / rms:.4f} "
          f"fraction beyond 2e-2 rms + 1 bf16 step {beyond:.2e}, bf16-identical {float((diff == 0).float().mean()):.4f}")
    assert bool(torch.isfinite(got).all())
    assert mismatch <= 1e-3 and rel_l2 <= 1e-2, (mismatch, rel_l2)
    assert beyond <= 1e-6 and max_abs <= 6e-2 * rms, (beyond, max_abs, rms)
    layer.close()


@pytest.mark.parametrize("m,n,k", [(8192, 8192, 8192), (16384, 7168, 2048)])
def test_dense_gemm_full_size_against_fp32_matmul(m, n, k):
    import kernelschema_b200 as ks
    torch.backends.cuda.matmul.allow_tf32 = False
    gen = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    gs_a = float(a.float().abs().max()) / (6.0 * 448.0)
    gs_b = float(b.float().abs().max()) / (6.0 * 448.0)
    aq, asf = ks.nvfp4_quantize(a, gs_a)
    bq, bsf = ks.nvfp4_quantize(b, gs_b)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = ks.mm_nvfp4(aq, ks.scales_to_tiles(asf), bq, ks.scales_to_tiles(bsf), alpha=gs_a * gs_b, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device="cuda")

    def dec(q, sf):
        codes = torch.stack((q & 15, q >> 4), -1).long().reshape(q.shape[0], -1)
        return lut[codes] * sf.float().repeat_interleave(16, -1)

    bd = dec(bq, bsf)
    worst_rel, worst_max = 0.0, 0.0
    for r0 in range(0, m, 2048):                       # row slabs keep the fp32 temporaries small
        want = (dec(aq[r0:r0 + 2048], asf[r0:r0 + 2048]) @ bd.t()) * (gs_a * gs_b)
        got = out[r0:r0 + 2048].float()
        rms = float(want.pow(2).mean().sqrt())
        worst_rel = max(worst_rel, float((got - want).norm() / want.norm()))
        worst_max = max(worst_max, float((got - want).abs().max()) / rms)
    print(f"dense {m}x{n}x{k}: rel_l2 {worst_rel:.3e} max_abs/rms {worst_max:.4f}")
    # exact products, fp32 accumulation, one bf16 rounding: rel-L2 of a bf16 rounding is ~1.7e-3
    assert worst_rel <= 2.5e-3 and worst_max <= 2e-2, (worst_rel, worst_max)
