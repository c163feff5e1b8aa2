"""The allocation-free route-map entry point (b200moe_route_map_noalloc) against the regular one.

Some callers cannot allocate device memory while they run: code that lives inside a memory pool owned by
someone else, plugins of serving frameworks whose allocator forbids raw cudaMalloc, or latency-critical
sections where an allocation would synchronise the whole device. For them the library offers one entry point
whose only scratch is a fixed array inside the library image. This test drives it through the C ABI with
caller-owned output arrays and checks that it produces exactly the integers (and weights) of
b200moe_route_map, on two consecutive calls with different inputs so that whatever the first call left in the
shared scratch is shown not to matter. The file name sorts last on purpose: a run that stops at the first
failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, ids, w, t, k, shared, e, offset, cap, tiles):
    dev = "cuda"
    out = dict(counts=torch.empty(e + shared, dtype=torch.int32, device=dev),
               seg_start=torch.empty(e + shared + 1, dtype=torch.int32, device=dev),
               tile_expert=torch.empty(tiles, dtype=torch.int32, device=dev),
               tile_row0=torch.empty(tiles, dtype=torch.int32, device=dev),
               tile_rows=torch.empty(tiles, dtype=torch.int32, device=dev),
               totals=torch.empty(4, dtype=torch.int32, device=dev),
               row_of=torch.empty((t, k + shared), dtype=torch.int32, device=dev),
               tok_of_row=torch.empty(cap, dtype=torch.int32, device=dev),
               weight_of_row=torch.zeros(cap, dtype=torch.float32, device=dev))
    rc = lib.b200moe_route_map_noalloc(ids.data_ptr(), w.data_ptr(), t, k, shared, e, offset, out["counts"].data_ptr(),
                                       out["seg_start"].data_ptr(), out["tile_expert"].data_ptr(), out["tile_row0"].data_ptr(),
                                       out["tile_rows"].data_ptr(), out["totals"].data_ptr(), out["row_of"].data_ptr(),
                                       out["tok_of_row"].data_ptr(), out["weight_of_row"].data_ptr(), cap,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.b200moe_last_error()
    torch.cuda.synchronize()
    return out


def test_noalloc_route_map_equals_regular_entry_point_twice():
    import kernelschema_b200 as ks
    from kernelschema_b200 import _lib
    lib = _lib.load()
    t, k, shared, e, offset = 3000, 8, 1, 256, 0
    layer = ks.MoELayer(256, 256, e, k, t, num_shared_experts=shared)
    ws = layer.workspace()
    cap, tiles = ws["row_capacity"], ws["tile_capacity"]
    for call, seed in enumerate((1, 2)):
        rng = np.random.default_rng(seed)
        tt = t if call == 0 else t - 777              # second call: fewer tokens, other routing
        ids = np.stack([rng.permutation(e)[:k] for _ in range(tt)]).astype(np.int32)
        ids[rng.random(ids.shape) < 0.05] = -1
        ids_d = torch.from_numpy(ids).cuda()
        w_d = torch.rand(tt, k, device="cuda")
        layer.route_map(ids_d, w_d, offset)
        torch.cuda.synchronize()
        got = _call_noalloc(lib, ids_d, w_d, tt, k, shared, e, offset, cap, tiles)
        n_tiles, rows, _, _ = (int(v) for v in ws["totals"].cpu())
        assert got["totals"].cpu().tolist() == ws["totals"].cpu().tolist()
        for name in ("counts", "seg_start"):
            assert torch.equal(got[name], ws[name]), name
        for name in ("tile_expert", "tile_row0", "tile_rows"):
            assert torch.equal(got[name][:n_tiles], ws[name][:n_tiles]), name
        assert torch.equal(got["row_of"], ws["row_of"][:tt])
        live = torch.zeros(rows, dtype=torch.bool, device="cuda")
        live[ws["row_of"][:tt][ws["row_of"][:tt] >= 0].long()] = True
        assert torch.equal(got["tok_of_row"][:rows][live], ws["tok_of_row"][:rows][live])
        assert torch.equal(got["weight_of_row"][:rows][live], ws["weight_of_row"][:rows][live])   # exact: copied values
        # and directly against the CPU oracle's route map (shared experts: one extra always-routed id per token)
        from oracle import nvfp4_oracle as o
        ref = o.route_map(ids, e, 128, expert_offset=offset, shared_experts=shared)
        assert np.array_equal(got["counts"].cpu().numpy(), ref["counts"])
        assert np.array_equal(got["seg_start"].cpu().numpy(), ref["seg_start"])
        assert np.array_equal(got["row_of"].cpu().numpy(), ref["row_of"])
        assert np.array_equal(got["tile_rows"][:n_tiles].cpu().numpy(), ref["tile_rows"])
        assert np.array_equal(got["tile_expert"][:n_tiles].cpu().numpy(), ref["tile_expert"])
        live_rows = ref["row_of"][ref["row_of"] >= 0]
        assert np.array_equal(got["tok_of_row"].cpu().numpy()[live_rows], ref["tok_of_row"][live_rows])
    layer.close()


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from kernelschema_b200 import _lib
    lib = _lib.load()
    one = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = one.data_ptr()
    rc = lib.b200moe_route_map_noalloc(p, p, 8, 8, 0, 512, 0, p, p, p, p, p, p, p, p, p, 1 << 20, None)
    assert rc == 770 and b"exceed" in lib.b200moe_last_error()
    rc = lib.b200moe_route_map_noalloc(p, p, 100000, 8, 0, 64, 0, p, p, p, p, p, p, p, p, p, 1 << 22, None)
    assert rc == 770
