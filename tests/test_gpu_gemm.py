"""GPU parity of the tcgen05 NVFP4 GEMM (dense entry point) against the oracle's dequantise-then-matmul."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import compare_outputs
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def _dense_case(m, n, k, seed, tile_n, alpha=1.0, a_scale=1.0):
    import kernelschema_b200 as ks
    rng = np.random.default_rng(seed)
    a = o.bf16_round(rng.standard_normal((m, k), dtype=np.float32) * a_scale)
    b = o.bf16_round(rng.standard_normal((n, k), dtype=np.float32) * 0.02)
    bq, bs = o.quantize(b)
    a_dev = torch.from_numpy(o.bf16_bits(a).view(np.int16)).cuda().view(torch.bfloat16)
    aq, asf = ks.nvfp4_quantize(a_dev, 1.0, tiled_scales=True)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    bsf_t = ks.scales_to_tiles(torch.from_numpy(bs).cuda())
    out = ks.mm_nvfp4(aq, asf, torch.from_numpy(bq).cuda(), bsf_t, alpha=alpha, tile_n=tile_n, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, f"bounded device wait expired: code {int(status[0])}"
    oq, os_ = o.quantize(a)
    assert np.array_equal(aq.cpu().numpy(), oq)
    ref = o.dense_expected(o.decode(oq, os_), bq, bs, alpha)
    return out.float().cpu().numpy(), ref


@pytest.mark.parametrize("m,n,k,tile_n", [(128, 128, 256, 128), (128, 256, 256, 256), (192, 256, 512, 128),
                                          (192, 256, 512, 256), (1000, 1024, 2048, 128), (1000, 1024, 2048, 256),
                                          (5, 128, 7168, 128), (2048, 2048, 2048, 256), (256, 256, 256, 512),
                                          (192, 256, 512, 512), (1000, 1024, 2048, 512), (5, 256, 7168, 512),
                                          (2048, 2048, 2048, 512), (4096 + 128, 512, 1024, 512)])
def test_dense_gemm_matches_oracle(m, n, k, tile_n):
    got, ref = _dense_case(m, n, k, seed=m + n + k, tile_n=tile_n, alpha=0.75)
    r = compare_outputs(got, ref)
    # exact products, fp32 accumulation in a different order: at most a bf16 ulp on a few elements
    assert r["rel_l2"] <= 2e-3, r
    ulp_off = (o.bf16_bits(got) != o.bf16_bits(ref)).mean()
    assert ulp_off <= 0.05, ulp_off
    assert r["max_abs"] <= 2e-2 * r["rms"], r


@pytest.mark.parametrize("m,n,k,tile_n", [(128 * 600, 128, 256, 128), (128 * 400, 256, 512, 256), (256 * 300, 256, 512, 512),
                                          (128 * 330, 512, 768, 256)])
def test_dense_gemm_many_items_per_cta(m, n, k, tile_n):
    """Short K and several work items per CTA (or CTA pair): the stage ring and the per-stage scale-factor buffers wrap
    across tiles, the accumulator phases flip and the tile-table entries are prefetched one item ahead."""
    got, ref = _dense_case(m, n, k, seed=7 + tile_n, tile_n=tile_n)
    r = compare_outputs(got, ref)
    assert r["rel_l2"] <= 2e-3 and r["max_abs"] <= 2e-2 * r["rms"], r
    assert (o.bf16_bits(got) != o.bf16_bits(ref)).mean() <= 0.05


def test_dense_gemm_golden_weights():
    """B operand and scales from the reference's dense problem generator; A quantised on the device."""
    import kernelschema_b200 as ks
    g = load_golden("dense")
    a = o.bf16_from_bits(g["a"])
    aq, asf = ks.nvfp4_quantize(torch.from_numpy(g["a"].view(np.int16)).cuda().view(torch.bfloat16), 1.0, tiled_scales=True)
    out = ks.mm_nvfp4(aq, asf, torch.from_numpy(g["b"]).cuda(), ks.scales_to_tiles(torch.from_numpy(g["b_descale"]).cuda()),
                      alpha=float(g["alpha"][0]))
    oq, os_ = o.quantize(a)
    ref = o.dense_expected(o.decode(oq, os_), g["b"], g["b_descale"], float(g["alpha"][0]))
    r = compare_outputs(out.float().cpu().numpy(), ref)
    assert r["rel_l2"] <= 2e-3 and r["max_abs"] <= 2e-2 * r["rms"], r
    # against the reference's own output (bf16 A, not quantised): only the A quantisation error remains
    r2 = compare_outputs(out.float().cpu().numpy(), o.bf16_from_bits(g["out"]))
    assert r2["rel_l2"] <= 0.12, r2


def test_dense_gemm_linearity_full_size():
    """Size-independent property at a benchmark size: scaling A by 2 (exact in bf16 and in the block scales) doubles the output."""
    import kernelschema_b200 as ks
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(4096, 4096, device="cuda", generator=gen).to(torch.bfloat16)
    b = (torch.randn(4096, 4096, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    bq, bsf = ks.nvfp4_quantize(b, 1.0, tiled_scales=True)
    outs = []
    for s in (1.0, 2.0):
        aq, asf = ks.nvfp4_quantize((a * s).to(torch.bfloat16), 1.0, tiled_scales=True)
        outs.append(ks.mm_nvfp4(aq, asf, bq, bsf, tile_n=256).float())
    assert torch.equal(outs[0] * 2, outs[1])
    # spot-check 64 rows against the oracle
    rows = torch.arange(0, 4096, 64)
    aq, asf = ks.nvfp4_quantize(a, 1.0)
    bq_r, bs_r = ks.nvfp4_quantize(b, 1.0)
    ref = o.dense_expected(o.decode(aq[rows].cpu().numpy(), asf.view(torch.uint8)[rows].cpu().numpy()), bq_r.cpu().numpy(),
                           bs_r.view(torch.uint8).cpu().numpy())
    r = compare_outputs(outs[0][rows].cpu().numpy(), ref)
    assert r["rel_l2"] <= 2e-3 and r["max_abs"] <= 2e-2 * r["rms"], r


# ----------------------------------------------------------------------------- bf16 x NVFP4 (A not quantised)
def _w4a16_case(m, n, k, seed, outliers=False):
    rng = np.random.default_rng(seed)
    a = o.bf16_round(rng.standard_normal((m, k), dtype=np.float32) * np.linspace(0.65, 1.35, k, dtype=np.float32))
    if outliers:
        a[:, ::64] = o.bf16_round(a[:, ::64] * 8.0)
    w = o.bf16_round(rng.standard_normal((n, k), dtype=np.float32) * np.float32(k ** -0.5))
    bq, bsf = o.quantize(w)
    return a, bq, bsf


def _bf16_dev(a):
    return torch.from_numpy(o.bf16_bits(a).view(np.int16)).cuda().view(torch.bfloat16)


def test_w4a16_matches_reference_output_bits():
    """The reference's own dense problem (bf16 A, its generator's B, scales and alpha) and its own output: the weights
    are expanded exactly, so only the order of the fp32 additions differs (a bf16 ulp on a few elements)."""
    import kernelschema_b200 as ks
    g = load_golden("dense")
    a = torch.from_numpy(g["a"].view(np.int16)).cuda().view(torch.bfloat16)
    backing = torch.full((192 * 256 + 128,), -17, dtype=torch.bfloat16, device="cuda")
    out = backing[64:-64].view(192, 256)
    inputs = [a.clone(), torch.from_numpy(g["b"]).cuda(), torch.from_numpy(g["b_descale"]).cuda(), torch.from_numpy(g["alpha"]).cuda()]
    snap = [t.clone() for t in inputs]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = ks.DenseModel()(inputs[0], inputs[1], inputs[2].view(torch.float8_e4m3fn), inputs[3], backend="blackwell-native",
                          out_dtype=torch.bfloat16, out=out, block_size=16, enable_pdl=False)
    torch.cuda.synchronize()
    assert res is out and int(status.item()) == 0
    assert all(torch.equal(x, y) for x, y in zip(inputs, snap))                  # inputs preserved
    assert (backing[:64] == -17).all() and (backing[-64:] == -17).all()          # nothing written outside `out`
    got, ref = out.float().cpu().numpy(), o.bf16_from_bits(g["out"])
    r = compare_outputs(got, ref)
    assert r["rel_l2"] <= 1e-3 and r["max_abs"] <= 2e-2 * r["rms"], r
    # the reference's own acceptance rule (metadata.json: atol 0.01, rtol 0.05, no mismatch allowed)
    assert (np.abs(got - ref) <= 0.01 + 0.05 * np.abs(ref)).all()
    assert (o.bf16_bits(got) != o.bf16_bits(ref)).mean() <= 0.05


@pytest.mark.parametrize("m,n,k,outliers", [(1, 128, 256, False), (100, 256, 512, False), (129, 384, 768, True), (256, 128, 2048, False),
                                            (300, 1536, 1024, False), (1000, 512, 256, True), (300, 384, 512, False),
                                            (513, 768, 1024, False)])
def test_w4a16_matches_oracle(m, n, k, outliers):
    import kernelschema_b200 as ks
    a, bq, bsf = _w4a16_case(m, n, k, 100 + m, outliers)
    alpha = torch.tensor([0.75], dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ks.mm_bf16_nvfp4(_bf16_dev(a), torch.from_numpy(bq).cuda(), torch.from_numpy(bsf).cuda(), alpha, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = o.dense_expected(a, bq, bsf, 0.75)
    got = out.float().cpu().numpy()
    r = compare_outputs(got, ref)
    assert r["rel_l2"] <= 1e-3 and r["max_abs"] <= 2e-2 * r["rms"], r
    assert (np.abs(got - ref) <= 0.01 + 0.05 * np.abs(ref)).all()
    assert (o.bf16_bits(got) != o.bf16_bits(ref)).mean() <= 0.05


def test_w4a16_strided_a_and_no_alpha():
    import kernelschema_b200 as ks
    a, bq, bsf = _w4a16_case(64, 128, 512, 7)
    wide = torch.zeros((64, 512 + 64), dtype=torch.bfloat16, device="cuda")
    wide[:, :512] = _bf16_dev(a)
    out = ks.mm_bf16_nvfp4(wide[:, :512], torch.from_numpy(bq).cuda(), torch.from_numpy(bsf).cuda())
    ref = o.dense_expected(a, bq, bsf, 1.0)
    r = compare_outputs(out.float().cpu().numpy(), ref)
    assert r["rel_l2"] <= 1e-3, r


def test_w4a16_linearity_full_size():
    """Size-independent properties at a reference shape (M 8192, N 4096, K 2048): doubling A doubles the output exactly,
    and a row of A gives the same output row whatever tile it sits in."""
    import kernelschema_b200 as ks
    gen = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(8192, 2048, device="cuda", generator=gen).to(torch.bfloat16)
    w = (torch.randn(4096, 2048, device="cuda", generator=gen) * 2048 ** -0.5).to(torch.bfloat16)
    bq, bsf = ks.nvfp4_quantize(w, 1.0)
    y1 = ks.mm_bf16_nvfp4(a, bq, bsf.view(torch.uint8))
    y2 = ks.mm_bf16_nvfp4((a * 2).to(torch.bfloat16), bq, bsf.view(torch.uint8))
    assert torch.equal(y1.float() * 2, y2.float())
    perm = torch.randperm(8192, device="cuda", generator=gen)
    y3 = ks.mm_bf16_nvfp4(a[perm].contiguous(), bq, bsf.view(torch.uint8))
    assert torch.equal(y3, y1[perm])
    assert y1.float().abs().mean() > 0.1


def test_w4a16_rejects_bad_shapes():
    import kernelschema_b200 as ks
    a = torch.zeros((8, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises((ValueError, RuntimeError)):
        ks.mm_bf16_nvfp4(a, torch.zeros((128, 64), dtype=torch.uint8, device="cuda"), torch.zeros((128, 8), dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("m,n,k", [(16, 4096, 3072), (128, 1024, 2048), (1, 256, 1024), (100, 7168, 2048)])
def test_w4a16_split_k_small_m(m, n, k):
    """Small M: several CTAs share one output tile through fp32 partial sums added in a fixed order. Same result as the
    one-CTA-per-tile form up to the order of the fp32 additions, and identical from run to run."""
    import kernelschema_b200 as ks
    a, bq, bsf = _w4a16_case(m, n, k, 300 + m)
    args = (_bf16_dev(a), torch.from_numpy(bq).cuda(), torch.from_numpy(bsf).cuda(), torch.tensor([1.25], dtype=torch.float32, device="cuda"))
    y_split = ks.mm_bf16_nvfp4(*args, split_k=True)
    y_again = ks.mm_bf16_nvfp4(*args, split_k=True)
    y_plain = ks.mm_bf16_nvfp4(*args, split_k=False)
    torch.cuda.synchronize()
    assert torch.equal(y_split, y_again)
    ref = o.dense_expected(a, bq, bsf, 1.25)
    for y in (y_split, y_plain):
        got = y.float().cpu().numpy()
        r = compare_outputs(got, ref)
        assert r["rel_l2"] <= 1e-3 and r["max_abs"] <= 2e-2 * r["rms"], r
        assert (np.abs(got - ref) <= 0.01 + 0.05 * np.abs(ref)).all()
