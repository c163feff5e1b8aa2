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
    """Size-independent property at a BASELINE size: scaling A by 2 (exact in bf16 and in the block scales) doubles the output."""
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
