"""The expert-parallel dispatch plan on ONE GPU: the library's three-launch planner against the torch-op plan of
kernelschema_b200/ep.py, and the layer run on row-strided views of a message buffer against the same run on contiguous
copies."""
import numpy as np
import pytest
import torch

from helpers import make_moe_case
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("t,h,e,k,world,shared", [(96, 512, 8, 4, 2, True), (300, 256, 16, 3, 4, False),
                                                   (4096, 1024, 64, 8, 8, True), (1, 256, 8, 2, 8, False)])
def test_cuda_planner_matches_torch_plan(t, h, e, k, world, shared):
    from kernelschema_b200.ep import CudaPlanner, message_views, plan_messages_torch
    p = make_moe_case(5, t, h, 256, e, k, routing="zipf", masked=True)
    ids, w = _dev(p["topk_ids"][0].astype(np.int32)), _dev(p["topk_ids"][1].astype(np.float32))
    hq, hs = _dev(p["hidden_states"]), _dev(p["hidden_states_scale"])
    ref_msg, ref_seg, ref_row_of = plan_messages_torch(ids, w, hq, hs, e // world, world, shared)
    planner = CudaPlanner(h, k, e // world, world, t, shared, ids.device)
    for _ in range(2):       # buffers are reused between steps
        msg, seg, row_of, w_rows = planner.plan(ids, w, hq, hs)
        torch.cuda.synchronize()
        assert planner.layer.status() == 0
        assert seg.tolist() == ref_seg
        assert torch.equal(row_of, ref_row_of)
        n = sum(ref_seg)
        got = message_views(msg[:n], h, k)
        want = message_views(ref_msg, h, k)
        live = (want[2] >= 0).any(dim=1)
        # every live pair row is byte-identical; padding rows (and rows of tokens whose routes are all masked: there are
        # none, such a token visits no rank) only promise ids = -1
        used_bytes = h // 2 + h // 16 + 8 * k     # the tail that rounds a row up to 16 bytes is never written or read
        assert torch.equal(msg[:n][live][:, :used_bytes], ref_msg[live][:, :used_bytes])
        assert torch.equal(got[2], want[2])
        used = row_of[row_of >= 0].long()
        assert (w_rows[used] == 1).all()


def test_layer_runs_on_strided_message_views():
    from kernelschema_b200.ep import message_views, plan_messages_torch
    from kernelschema_b200.ops import MoELayer
    t, h, i, e, k = 200, 512, 256, 4, 2
    p = make_moe_case(9, t, h, i, e, k, global_scales=True, masked=True)
    ids, w = _dev(p["topk_ids"][0].astype(np.int32)), _dev(p["topk_ids"][1].astype(np.float32))
    hq, hs = _dev(p["hidden_states"]), _dev(p["hidden_states_scale"])
    msg, seg, _ = plan_messages_torch(ids, w, hq, hs, e, 1)          # one rank owns every expert
    m_q, m_sf, m_ids, m_w = message_views(msg, h, k)
    wt = [_dev(p[n]) for n in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale")]
    kw = dict(scale_up=_dev(p["output1_scale_scalar"]), scale_gate=_dev(p["output1_scale_gate_scalar"]),
              scale_out=_dev(p["output2_scale_scalar"]))
    layer = MoELayer(h, i, e, k, msg.shape[0])
    out_strided = torch.empty((msg.shape[0], h), dtype=torch.bfloat16, device="cuda")
    layer.run(m_ids, m_w, m_q, m_sf, *wt, out_strided, **kw)
    out_packed = torch.empty_like(out_strided)
    layer.run(m_ids.contiguous(), m_w.contiguous(), m_q.contiguous(), m_sf.contiguous(), *wt, out_packed, **kw)
    torch.cuda.synchronize()
    assert layer.status() == 0
    assert torch.equal(out_strided, out_packed)
    assert out_strided.float().abs().sum() > 0
    # bad strides are refused before any launch
    odd = torch.zeros((msg.shape[0], h // 2 + 8), dtype=torch.uint8, device="cuda")[:, :h // 2]     # row stride not % 16
    with pytest.raises((RuntimeError, ValueError), match="stride"):
        layer.run(m_ids, m_w, odd, m_sf, *wt, out_strided, **kw)


@pytest.mark.parametrize("shared,tokens", [(1, 200), (0, 128), (1, 1)])
def test_peer_memory_exchange_single_rank_loop(shared, tokens):
    """The whole peer-memory path (dispatch kernel, flags, layer over the receive buffer with its combine pass writing
    into the return buffer, final combine) on ONE GPU: a group of one rank is its own peer. Two steps with different
    tokens, so both buffer parities and the reuse of flags and counters are exercised; against the CPU oracle."""
    import torch.distributed as dist
    from helpers import assert_layer_parity, make_moe_case
    from kernelschema_b200.ep import ExpertParallelMoE
    h, i, e, k = 512, 256, 8, 4
    own = not dist.is_initialized()
    if own:
        import socket
        with socket.socket() as sock:
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        ep = ExpertParallelMoE(h, i, e, k, 256, num_shared_experts=shared, transport="p2p")
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        for step, seed in enumerate((3, 4, 5)):
            p = make_moe_case(seed, tokens, h, i, e, k, shared=shared, global_scales=True, routing="zipf", masked=(step == 1))
            ids, scores = p["topk_ids"]
            out = ep.forward(dev(ids), dev(scores), dev(p["hidden_states"]), dev(p["hidden_states_scale"]), dev(p["gemm1_weights"]),
                             dev(p["gemm1_weights_scale"]), dev(p["gemm2_weights"]), dev(p["gemm2_weights_scale"]),
                             scale_up=dev(p["output1_scale_scalar"]), scale_gate=dev(p["output1_scale_gate_scalar"]),
                             scale_out=dev(p["output2_scale_scalar"]))
            torch.cuda.synchronize()
            assert ep.status() == 0
            assert_layer_parity(out.float().cpu().numpy(), o.moe_expected(p), f"step {step}", extra_bf16_roundings=1)
        assert ep._px.epoch == 3
        ep.close()
    finally:
        if own:
            dist.destroy_process_group()


def test_ep_wait_is_bounded_and_reports():
    """A flag that nobody sets: the device-side wait gives up after its poll limit (a few seconds), records status code 301
    on the layer and returns; the context stays usable and a later wait on a flag that IS set succeeds."""
    import time
    import kernelschema_b200 as ks
    from kernelschema_b200 import _lib
    lib = _lib.load()
    layer = ks.MoELayer(256, 256, 2, 2, 128)
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert layer.status() == 0
    t0 = time.perf_counter()
    _lib.check(lib.b200moe_ep_wait(layer._h, flags.data_ptr(), 2, 7, stream), "b200moe_ep_wait")
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.2 < waited < 30.0, waited
    assert layer.status() == 301
    flags.fill_(7)
    t0 = time.perf_counter()
    _lib.check(lib.b200moe_ep_wait(layer._h, flags.data_ptr(), 4, 7, stream), "b200moe_ep_wait")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.2
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0
    layer.close()
