"""GPU parity of the front-end kernels (quantiser, router, route map) through the C ABI: bit-exact."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def _bf16_dev(bits):
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def test_quantize_golden_bytes():
    import kernelschema_b200 as ks
    g = load_golden("quantize")
    for xk, pk, sk in (("x", "payload", "scale"), ("special", "special_payload", "special_scale"),
                       ("ties", "ties_payload", "ties_scale")):
        q, s = ks.nvfp4_quantize(_bf16_dev(g[xk]))
        assert np.array_equal(q.cpu().numpy(), g[pk]), xk
        assert np.array_equal(s.view(torch.uint8).cpu().numpy(), g[sk]), xk
    q, s = ks.nvfp4_quantize(_bf16_dev(g["x"]), float(g["global_scale"]))
    assert np.array_equal(q.cpu().numpy(), g["payload_gs"])
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), g["scale_gs"])


@pytest.mark.parametrize("rows,cols,scale", [(1000, 7168, 1.0), (257, 2048, 37.0), (64, 64, 1e-3), (0, 256, 1.0)])
def test_quantize_matches_oracle(rows, cols, scale):
    import kernelschema_b200 as ks
    gen = torch.Generator(device="cpu").manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=gen) * scale).to(torch.bfloat16)
    q, s = ks.nvfp4_quantize(x.cuda())
    oq, os_ = o.quantize(x.float().numpy())
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_)
    if rows:
        for gs in (float(x.float().abs().max() / (6 * 448)), 2.0 ** -9, 4.0):      # general, and exact power-of-two scales
            q, s = ks.nvfp4_quantize(x.cuda(), gs)
            oq, os_ = o.quantize(x.float().numpy(), 16, gs)
            assert np.array_equal(q.cpu().numpy(), oq), gs
            assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_), gs
        # tiled scale layout = block_scales() of the row-major bytes
        q2, st = ks.nvfp4_quantize(x.cuda(), 1.0, tiled_scales=True)
        ref_t = o.block_scales(o.quantize(x.float().numpy())[1][None])[0]
        assert np.array_equal(st.cpu().numpy(), ref_t)
        assert np.array_equal(ks.scales_to_tiles(ks.nvfp4_quantize(x.cuda())[1]).cpu().numpy(), ref_t)


def _torch_quantize_true_division(x, gs):
    """The reference quantize() (gemm/dense/bf16_nvfp4_gemm/problem/input.py:40-64) in torch ops on the device with
    tensor / tensor divisions only (IEEE round-to-nearest; tensor / python-scalar would multiply by a reciprocal)."""
    dev = x.device
    groups = x.float().view(-1, 16)
    t = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)
    peak = groups.abs().amax(-1).clamp_min(2.0 ** -20)
    scale = torch.div(torch.div(peak, t(6.0)), t(gs)) if gs != 1.0 else torch.div(peak, t(6.0))
    stored = scale.clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn)
    d = stored.float() * t(gs)
    q = torch.div(groups, d[:, None])
    mag = q.abs()
    code = torch.zeros_like(mag, dtype=torch.int32)
    for i, mid in enumerate((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)):
        code += (mag > mid if i % 2 == 0 else mag >= mid).int()
    code |= torch.signbit(q).int() << 3
    code = code.view(-1, 8, 2)
    return (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8), stored.view(torch.uint8)


@pytest.mark.parametrize("gs", [1.0, 2.0 ** -9, 3.0, 0.7431, 1.0 / (6 * 448) * 5.3, 1.9999999, 1.0000001, 12.375e-3, 6.1e-5, 977.25])
def test_quantize_reciprocal_path_equals_true_division_all_bf16(gs):
    """Every finite bf16 value as a numerator against every E4M3 block scale (the block's first element sets the scale)
    x a set of global scales incl. mantissas of all ones and 1 + ulp: the residual-corrected reciprocal multiply of the
    kernel must give the codes of IEEE division."""
    import kernelschema_b200 as ks
    dev = "cuda"
    bits = torch.arange(0, 65536, dtype=torch.int32, device=dev).to(torch.int16)
    vals = bits.view(torch.bfloat16).float()
    finite = torch.isfinite(vals)
    codes = torch.arange(1, 127, dtype=torch.uint8, device=dev)
    peaks = (codes.view(torch.float8_e4m3fn).float() * 6.0 * gs).to(torch.bfloat16)
    peaks = peaks[torch.isfinite(peaks.float()) & (peaks.float() > 0)]
    rows = []
    for pk in peaks.unique():
        cand = vals[finite & (vals.abs() <= pk.float())].to(torch.bfloat16)
        pad = (-cand.numel()) % 15
        cand = torch.cat([cand, cand.new_zeros(pad)]).view(-1, 15)
        rows.append(torch.cat([pk.expand(cand.shape[0], 1), cand], 1))
    x = torch.cat(rows).reshape(-1)
    x = torch.cat([x, x.new_zeros((-x.numel()) % 1024)]).view(-1, 1024)
    q, s = ks.nvfp4_quantize(x, gs)
    rq, rs = _torch_quantize_true_division(x, gs)
    assert torch.equal(s.view(torch.uint8).reshape(-1), rs)
    assert torch.equal(q.reshape(-1, 8), rq), int((q.reshape(-1, 8) != rq).sum())
    # the torch formulation itself against the numpy oracle (pinned by the reference's fixtures) on a slice
    sub = x[:: max(1, x.shape[0] // 64)]
    oq, os_ = o.quantize(sub.float().cpu().numpy(), 16, gs)
    sq, ss = _torch_quantize_true_division(sub.contiguous(), gs)
    assert np.array_equal(sq.reshape(sub.shape[0], -1).cpu().numpy(), oq) and np.array_equal(ss.reshape(sub.shape[0], -1).cpu().numpy(), os_)


def test_quantize_tiny_global_scale_and_tiny_blocks():
    """Blocks below the 2^-20 peak floor (all-zero, |x| < 1e-6) with small power-of-two and general global scales: the
    floor applies to the unscaled peak (problem/input.py of the dense operator, lines 40-64)."""
    import kernelschema_b200 as ks
    x = torch.zeros(4, 64, dtype=torch.float32)
    x[0, 16:32] = torch.linspace(-9e-7, 9e-7, 16)
    x[1, :16] = torch.linspace(-3e-7, 5e-7, 16)
    x[2] = torch.randn(64, generator=torch.Generator().manual_seed(1)) * 1e-5
    x[3, 48:] = 2.0 ** -21
    xb = x.to(torch.bfloat16)
    for gs in (2.0 ** -16, 2.0 ** -14, 2.0 ** -20, 3.3e-5, 1.0):
        q, s = ks.nvfp4_quantize(xb.cuda(), gs)
        oq, os_ = o.quantize(xb.float().numpy(), 16, gs)
        assert np.array_equal(s.view(torch.uint8).cpu().numpy(), os_), gs
        assert np.array_equal(q.cpu().numpy(), oq), gs


def test_quantize_strided_rows():
    import kernelschema_b200 as ks
    x = torch.randn(50, 512, device="cuda").to(torch.bfloat16)
    view = x[:, :256]
    q, s = ks.nvfp4_quantize(view)
    oq, os_ = o.quantize(view.float().cpu().numpy())
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.view(torch.uint8).cpu().numpy(), os_)


def test_router_golden():
    import kernelschema_b200 as ks
    g = load_golden("routes")
    for i in range(int(g["n"])):
        t, e, k, empty, masked = g[f"meta{i}"]
        lg = g[f"logits{i}"]
        ids, w = ks.route_topk(torch.from_numpy(lg).cuda(), int(k))
        ids, w = ids.cpu().numpy(), w.cpu().numpy()
        oi, ow = o.route_topk(lg, int(k))
        assert np.array_equal(ids, oi), i
        ulp = np.abs(w.view(np.int32).astype(np.int64) - ow.view(np.int32).astype(np.int64))
        assert ulp.max() <= 1, (i, ulp.max())          # against the correctly rounded oracle
        ids, w = o.apply_route_masks(ids, w, empty=bool(empty), masked_routes=bool(masked))
        assert np.array_equal(ids, g[f"ids{i}"]), i     # against the reference
        ulp = np.abs(w.view(np.int32).astype(np.int64) - g[f"w{i}"].view(np.int32).astype(np.int64))
        assert ulp.max() <= 4, (i, ulp.max())           # torch's fp32 softmax


@pytest.mark.parametrize("t,e,k", [(1, 8, 2), (333, 256, 8), (4096, 128, 8), (100, 1024, 32), (7, 5, 5)])
def test_router_random_with_bias_and_ties(t, e, k):
    import kernelschema_b200 as ks
    rng = np.random.default_rng(t + e)
    lg = rng.standard_normal((t, e), dtype=np.float32)
    lg[::5] = np.round(lg[::5] * 2) / 2            # many exact ties: lowest index must win
    bias = rng.standard_normal(e).astype(np.float32)
    ids, w = ks.route_topk(torch.from_numpy(lg).cuda(), k, torch.from_numpy(bias).cuda())
    oi, ow = o.route_topk(lg, k, bias)
    assert np.array_equal(ids.cpu().numpy(), oi)
    ulp = np.abs(w.cpu().numpy().view(np.int32).astype(np.int64) - ow.view(np.int32).astype(np.int64))
    assert ulp.max() <= 1


@pytest.mark.parametrize("t,h,e", [(300, 2048, 130), (300, 7168, 256), (1000, 2048, 128), (129, 1024, 8), (5, 256, 72),
                                   (1, 7168, 256), (8, 2048, 128), (9, 2048, 127), (16, 7168, 256), (17, 2048, 128),
                                   (8, 7168, 256), (12, 2048, 128), (64, 7168, 256), (128, 2048, 40), (200, 1088, 64), (1024, 4096, 24), (1025, 2048, 128),
                                   (2000, 7168, 256), (8192, 2048, 256)])
def test_router_logits(t, h, e):
    """A handful of tokens (T <= 8 and T x H <= 32768, or shapes the tensor-core kernels do not take) run the SIMT decode kernel; above, e=130 takes the SIMT kernel, the others the tcgen05 bf16 kernels:
    while token tiles x 64-expert slices fit one wave, clusters of 8, 4, 2 or 1 blocks that split the k-steps (1088 = 17
    k-steps cannot be split), above that one or two blocks per token tile."""
    import kernelschema_b200 as ks
    x = torch.randn(t, h).to(torch.bfloat16)
    w = (torch.randn(e, h) * 0.02).to(torch.bfloat16)
    got = ks.router_logits(x.cuda(), w.cuda()).cpu().numpy()
    ref = o.router_logits(x.float().numpy(), w.float().numpy())
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max() + 1e-6    # fp32 accumulation vs fp64


@pytest.mark.parametrize("t,k,e,shared,offset", [(1, 8, 128, 0, 0), (300, 4, 8, 0, 0), (4096, 8, 256, 1, 0),
                                                 (1000, 8, 32, 0, 64), (50, 2, 4, 2, 0), (2049, 1, 3, 0, 0), (600, 8, 512, 0, 0), (1500, 8, 128, 1, 0),
                                                 (300, 8, 1000, 1, 0), (5000, 8, 1000, 0, 0)])
def test_route_map_matches_oracle(t, k, e, shared, offset):
    import kernelschema_b200 as ks
    rng = np.random.default_rng(t * 7 + e)
    span = e * 4 if offset else e
    ids = np.stack([rng.permutation(span)[:k] for _ in range(t)]).astype(np.int32)
    ids[rng.random(ids.shape) < 0.1] = -1
    w = rng.random(ids.shape, dtype=np.float32)
    layer = ks.MoELayer(256, 256, e, k, t, num_shared_experts=shared)
    layer.route_map(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), offset)
    torch.cuda.synchronize()
    ws = layer.workspace()
    m = o.route_map(ids, e, 128, expert_offset=offset, shared_experts=shared)
    n_tiles, rows, valid, n_pairs = (int(v) for v in ws["totals"].cpu())
    # 256-row pair items: consecutive tile pairs of one expert
    pe, pr0, prw = [], [], []
    for e_ in range(e + shared):
        c = int(m["counts"][e_])
        for j in range(0, c, 256):
            pe.append(e_); pr0.append(int(m["seg_start"][e_]) + j); prw.append(min(256, c - j))
    assert n_pairs == len(pe)
    assert ws["pair_expert"][:n_pairs].cpu().tolist() == pe
    assert ws["pair_row0"][:n_pairs].cpu().tolist() == pr0
    assert ws["pair_rows"][:n_pairs].cpu().tolist() == prw
    assert n_tiles == len(m["tile_expert"]) and rows == m["seg_start"][-1] and valid == (m["row_of"] >= 0).sum()
    assert np.array_equal(ws["counts"].cpu().numpy(), m["counts"])
    assert np.array_equal(ws["seg_start"].cpu().numpy(), m["seg_start"])
    for name in ("tile_expert", "tile_row0", "tile_rows"):
        assert np.array_equal(ws[name][:n_tiles].cpu().numpy(), m[name]), name
    assert np.array_equal(ws["row_of"][:t].cpu().numpy(), m["row_of"])
    live = m["tok_of_row"] >= 0                      # padding rows of a tile carry no defined token
    assert np.array_equal(ws["tok_of_row"][:rows].cpu().numpy()[live], m["tok_of_row"][live])
    wr = ws["weight_of_row"][:rows].cpu().numpy()
    full_w = np.concatenate([w, np.ones((t, shared), np.float32)], 1)
    assert np.array_equal(wr[live], full_w[m["tok_of_row"][live], m["slot_of_row"][live]])
    layer.close()


def test_route_map_all_invalid():
    import kernelschema_b200 as ks
    ids = torch.full((64, 8), -1, dtype=torch.int32, device="cuda")
    layer = ks.MoELayer(256, 256, 16, 8, 64)
    layer.route_map(ids, torch.zeros(64, 8, device="cuda"))
    torch.cuda.synchronize()
    ws = layer.workspace()
    assert ws["totals"].cpu().tolist() == [0, 0, 0, 0]
    assert bool((ws["row_of"][:64] == -1).all())
    layer.close()
