"""Generate the golden fixtures under tests/golden/ from the reference's own Python code.

Run once, in a container that has the reference checkout (its location is
taken from ``KERNELSCHEMA_REFERENCE``):

    python tests/golden/make_golden.py

It imports, *by path*, the reference operator's ``problem/input.py`` and
``problem/reference.py`` (NVFP4 fused MoE) and the dense GEMM problem's
``input.py`` / ``reference.py``, runs them with torch on the CPU on seeded
inputs and stores inputs and outputs as ``.npz`` files.  Nothing here is used
at test time; the tests only read the ``.npz`` files.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

REF = os.environ.get("KERNELSCHEMA_REFERENCE", "/root/reference")
OPS = os.path.join(REF, "kernel_wiki/aka-cuda-operators-20261030/operators")
NV = os.path.join(OPS, "moe/nvfp4_fused_moe/problem")
DG = os.path.join(OPS, "gemm/dense/bf16_nvfp4_gemm/problem")
OUT = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


moe_in = _load(os.path.join(NV, "input.py"), "ref_moe_input")
moe_ref = _load(os.path.join(NV, "reference.py"), "ref_moe_reference")
dg_in = _load(os.path.join(DG, "input.py"), "ref_dense_input")
dg_ref = _load(os.path.join(DG, "reference.py"), "ref_dense_reference")


def u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def save(name, **arrays):
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


# ----------------------------------------------------------------------------- quantiser
def special_values():
    """Rows that sit on the rounding boundaries of both casts."""
    rows = []
    base = torch.tensor([0.0, -0.0, 0.25, -0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -6.0, 0.5, 1.0, 1.5, 3.0])
    for peak in (6.0, 3.0, 1.0, 0.4375, 448.0 * 6, 3000.0, 2.0 ** -10, 2.0 ** -22, 6.375, 0.0117):
        rows.append(base * (peak / 6.0))
    rows.append(torch.zeros(16))
    rows.append(-torch.zeros(16))
    rows.append(torch.full((16,), 1e-30))
    rows.append(torch.tensor([(-1.0) ** i * 2.0 ** (-i) for i in range(16)]))
    blk = torch.stack(rows)                       # [n, 16]
    n = blk.shape[0]
    pad = (-n) % 4
    if pad:
        blk = torch.cat([blk, torch.zeros(pad, 16)])
    return blk.reshape(-1, 64).to(torch.bfloat16)


def gen_quantize():
    torch.manual_seed(1234)
    x = torch.randn(96, 256).to(torch.bfloat16)
    x[5] *= 40.0
    x[6] *= 1e-3
    x[7] = 0
    sp = special_values()
    q, s = moe_in.quantize(x.float(), 16)
    qs, ss = moe_in.quantize(sp.float(), 16)
    # every e4m3 scale as a divisor x every e2m1 midpoint: x = mid * scale is exact in bf16
    # for the scales whose mantissa product fits; the reference result pins ties either way.
    sc = torch.arange(1, 127, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0])
    tie = torch.zeros(126, 16)
    tie[:, :8] = sc[:, None] * mids[None, :]
    tie[:, 8:] = -tie[:, :8]
    tie[:, 7] = sc * 6.0
    tie = tie.to(torch.bfloat16)
    pad = torch.zeros(2, 16, dtype=torch.bfloat16)
    tie = torch.cat([tie, pad]).reshape(-1, 64)
    qt, st = moe_in.quantize(tie.float(), 16)
    gs = float(x.float().abs().max() / (6.0 * 448.0))
    qg, sg = dg_in.quantize(x.float(), "nvfp4", 16, gs)
    save("quantize",
         x=bf16_bits(x), payload=u8(q), scale=u8(s),
         special=bf16_bits(sp), special_payload=u8(qs), special_scale=u8(ss),
         ties=bf16_bits(tie), ties_payload=u8(qt), ties_scale=u8(st),
         global_scale=np.float32(gs), payload_gs=u8(qg), scale_gs=u8(sg))


def gen_qdq():
    torch.manual_seed(99)
    v = torch.randn(64, 128) * torch.logspace(-4, 2, 64)[:, None]
    v[3] = 0
    v[4, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    out = moe_ref.nvfp4(v)
    e = moe_ref.e2m1(torch.linspace(-7, 7, 1121))
    save("qdq", value=v.numpy(), qdq=out.numpy(), e2m1_in=torch.linspace(-7, 7, 1121).numpy(), e2m1_out=e.numpy())


# ----------------------------------------------------------------------------- router
def gen_routes():
    arrays = {}
    real_topk = torch.Tensor.topk
    for i, (mode, masked, t, e, k) in enumerate([("balanced", False, 40, 16, 4), ("skewed", False, 33, 32, 8),
                                                 ("hotspot", False, 24, 16, 4), ("empty", False, 16, 8, 2),
                                                 ("balanced", True, 50, 128, 8), ("balanced", False, 257, 256, 8)]):
        captured = {}

        def spy(self, *a, **kw):
            captured["logits"] = self.clone()
            return real_topk(self, *a, **kw)

        torch.manual_seed(7 + i)
        torch.Tensor.topk = spy
        try:
            ids, w = moe_in.routes({"routing": mode, "masked_routes": masked}, t, e, k, "cpu")
        finally:
            torch.Tensor.topk = real_topk
        arrays[f"logits{i}"] = captured["logits"].numpy()
        arrays[f"ids{i}"] = ids.to(torch.int32).numpy()
        arrays[f"w{i}"] = w.numpy()
        arrays[f"meta{i}"] = np.array([t, e, k, int(mode == "empty"), int(masked)], dtype=np.int32)
    arrays["n"] = np.int32(6)
    save("routes", **arrays)


# ----------------------------------------------------------------------------- weight layout
def gen_layout():
    torch.manual_seed(5)
    e, n, k = 2, 256, 128
    q = torch.randint(0, 256, (e, n, k // 2), dtype=torch.uint8)
    sf = torch.randint(1, 0x78, (e, n, k // 16), dtype=torch.uint8).view(torch.float8_e4m3fn)
    out = {}
    for gated in (True, False):
        pq, ps = moe_in.prepare_weights(q, sf, gated)
        dec = moe_ref.weight(pq, ps, gated)
        logical = moe_ref.decode(q, sf, "nvfp4")
        assert torch.equal(dec, logical), "reference prepare/weight are not inverses?"
        tag = "g" if gated else "n"
        out["pq_" + tag] = u8(pq)
        out["ps_" + tag] = u8(ps)
    save("layout", q=u8(q), sf=u8(sf), logical=moe_ref.decode(q, sf, "nvfp4").numpy(), **out)


# ----------------------------------------------------------------------------- whole layer
def pack_inputs(p):
    ids, scores = p["topk_ids"]
    d = dict(ids=ids.numpy(), scores=scores.numpy(), hidden_states=u8(p["hidden_states"]),
             hidden_states_scale=u8(p["hidden_states_scale"]), gemm1_weights=u8(p["gemm1_weights"]),
             gemm1_weights_scale=u8(p["gemm1_weights_scale"]), gemm2_weights=u8(p["gemm2_weights"]),
             gemm2_weights_scale=u8(p["gemm2_weights_scale"]), gemm1_alpha=p["gemm1_alpha"].numpy(),
             gemm1_beta=p["gemm1_beta"].numpy(),
             scalars=np.array([p["num_experts"], p["top_k"], p["intermediate_size"], p["activation_type"]], dtype=np.int32))
    if p["gemm1_clamp_limit"] is not None:
        d["gemm1_clamp_limit"] = p["gemm1_clamp_limit"].numpy()
    return d


def gen_moe_small():
    cases = {
        "balanced": dict(hidden=256, intermediate=256, local_experts=4, tokens=48, topk=2),
        "skew_clamp": dict(hidden=256, intermediate=256, local_experts=8, tokens=70, topk=4, routing="skewed",
                           activation_alpha=1.702, activation_beta=1.0, activation_limit=7.0),
        "situ": dict(hidden=256, intermediate=256, local_experts=4, tokens=33, topk=2, activation="situ"),
        "masked": dict(hidden=256, intermediate=256, local_experts=8, tokens=30, topk=8, masked_routes=True),
        "empty": dict(hidden=256, intermediate=256, local_experts=4, tokens=16, topk=2, routing="empty"),
        "zero": dict(hidden=256, intermediate=256, local_experts=4, tokens=16, topk=2, distribution="zero", routing="skewed"),
        "hotspot": dict(hidden=256, intermediate=256, local_experts=8, tokens=200, topk=2, routing="hotspot"),
    }
    model = moe_ref.Model()
    for name, kw in cases.items():
        torch.manual_seed(2026101501)
        p = moe_in._make_inputs(**kw, device="cpu")
        out = model(**p)[0]
        save("moe_" + name, out=bf16_bits(out), **pack_inputs(p))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def gen_moe_c1():
    """T=256, H=1024, I=512, E=8, top-2, seed 0, unit global scales so the reference compute applies.

    Inputs are NOT stored (6 MB): the test regenerates them with the same torch CPU
    generator calls plus the oracle's quantiser and checks these digests first.
    """
    t, h, i, e, k = 256, 1024, 512, 8, 2
    torch.manual_seed(0)
    x = torch.randn(t, h).to(torch.bfloat16)
    gate_w = (torch.randn(e, h) * 0.02).to(torch.bfloat16)
    w1 = (torch.randn(e, 2 * i, h) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(e, h, i) * 0.02).to(torch.bfloat16)
    a, sa = moe_in.quantize(x.float(), 16)
    q1, s1 = moe_in.quantize(w1.float(), 16)
    q2, s2 = moe_in.quantize(w2.float(), 16)
    q1, s1 = moe_in.prepare_weights(q1, s1, True)
    q2, s2 = moe_in.prepare_weights(q2, s2, False)
    logits = x.float() @ gate_w.float().T
    sel, ids = logits.topk(k, dim=-1)
    scores = sel.softmax(-1)
    ids = ids.to(torch.int32)
    out = moe_in.guarded((t, h), torch.bfloat16, "cpu")
    ones = torch.ones(e)
    p = dict(topk_ids=(ids, scores), routing_bias=None, hidden_states=a, hidden_states_scale=sa, gemm1_weights=q1,
             gemm1_weights_scale=s1, gemm1_bias=None, gemm1_alpha=ones.clone(), gemm1_beta=torch.zeros(e),
             gemm1_clamp_limit=None, gemm2_weights=q2, gemm2_weights_scale=s2, gemm2_bias=None,
             output1_scale_scalar=ones, output1_scale_gate_scalar=ones, output2_scale_scalar=ones, num_experts=e,
             top_k=k, n_group=None, topk_group=None, intermediate_size=i, local_expert_offset=0, local_num_experts=e,
             routed_scaling_factor=1.0, routing_method_type=0, do_finalize=True, enable_pdl=False, activation_type=3,
             output=out, hidden_states_scale_layout=2)
    res = moe_ref.Model()(**p)[0]
    digests = {n: sha(u8(v)) for n, v in dict(hidden_states=a, hidden_states_scale=sa, gemm1_weights=q1,
                                               gemm1_weights_scale=s1, gemm2_weights=q2, gemm2_weights_scale=s2).items()}
    save("moe_c1", out=bf16_bits(res), logits=logits.numpy(), ids=ids.numpy(), scores=scores.numpy(),
         digest_names=np.array(list(digests.keys())), digest_values=np.array(list(digests.values())))


# ----------------------------------------------------------------------------- dense GEMM
def gen_dense():
    torch.manual_seed(2026)
    p = dg_in._make_inputs(192, 256, 512, alpha=0.75, device="cpu")
    out = dg_ref.Model()(**p)
    save("dense", a=bf16_bits(p["a"]), b=u8(p["b"]), b_descale=u8(p["b_descale"]), alpha=p["alpha"].numpy(),
         out=bf16_bits(out))


if __name__ == "__main__":
    torch.set_num_threads(8)
    gen_quantize()
    gen_qdq()
    gen_routes()
    gen_layout()
    gen_moe_small()
    gen_moe_c1()
    gen_dense()
    print("done", file=sys.stderr)
