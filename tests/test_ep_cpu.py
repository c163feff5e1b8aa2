"""Expert-parallel dispatch/combine logic on 2 gloo ranks (CPU). The exchange, index plans and slot-ordered combine
are the product code of kernelschema_b200/ep.py; the three compute hooks (which run libb200moe on a GPU) are replaced
by the oracle here, so the test checks the plumbing: every rank must reproduce the single-process oracle result for
its own tokens."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_layer_parity, make_moe_case
from oracle import nvfp4_oracle as o

T, H, I, E, K, S = 24, 256, 256, 4, 2, 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(rank, world, masked):
    """Global problem (all ranks' tokens); every rank builds the same one from the seed."""
    p = make_moe_case(21, T * world, H, I, E, K, shared=S, global_scales=True, masked=masked)
    return p


def _np_params(p, w1q, w1s, w2q, w2s, extra, sl):
    q = dict(gemm1_weights=w1q[sl], gemm1_weights_scale=w1s[sl], gemm2_weights=w2q[sl], gemm2_weights_scale=w2s[sl],
             gemm1_alpha=p["gemm1_alpha"][sl], gemm1_beta=p["gemm1_beta"][sl], gemm1_clamp_limit=None,
             intermediate_size=I, activation_type=3)
    for name in ("output1_scale_scalar", "output1_scale_gate_scalar", "output2_scale_scalar"):
        q[name] = extra[name][sl]
    return q


def _worker(rank, world, port, masked, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kernelschema_b200.ep import ExpertParallelMoE
        p = _case(rank, world, masked)
        e_local = E // world
        mine = slice(rank * T, (rank + 1) * T)
        own = list(range(rank * e_local, (rank + 1) * e_local)) + list(range(E, E + S))   # local experts, then shared
        w = {n: p[n][own] for n in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale",
                                    "gemm1_alpha", "gemm1_beta", "output1_scale_scalar", "output1_scale_gate_scalar",
                                    "output2_scale_scalar")}

        def params(sl):
            return _np_params(w, w["gemm1_weights"], w["gemm1_weights_scale"], w["gemm2_weights"], w["gemm2_weights_scale"], w, sl)

        def expert_rows(rows_q, rows_sf, local_ids, weights, w1q, w1s, w2q, w2s, out_rows, kw):
            q = params(slice(0, e_local))
            q.update(topk_ids=(local_ids.numpy(), weights.numpy()), hidden_states=rows_q.numpy(),
                     hidden_states_scale=rows_sf.numpy(), num_experts=e_local, top_k=K)
            out_rows.copy_(torch.from_numpy(o.moe_expected(q)).to(torch.bfloat16))

        def shared_rows(hq, hs, w1q, w1s, w2q, w2s, out_rows, kw):
            q = params(slice(e_local, e_local + S))
            q.update(topk_ids=(np.zeros((hq.shape[0], 0), np.int32), np.zeros((hq.shape[0], 0), np.float32)),
                     hidden_states=hq.numpy(), hidden_states_scale=hs.numpy(), num_experts=0, top_k=0,
                     num_fused_shared_experts=S)
            out_rows.copy_(torch.from_numpy(o.moe_expected(q)).to(torch.bfloat16))

        def combine_rows(rows, row_of, weight_of_row, out):
            r = rows.float().numpy()
            acc = np.zeros((row_of.shape[0], r.shape[1]), np.float32)
            for s in range(row_of.shape[1]):
                idx = row_of[:, s].numpy()
                ok = idx >= 0
                acc[ok] += r[idx[ok]] * weight_of_row.numpy()[idx[ok], None]
            out.copy_(torch.from_numpy(o.bf16_round(acc)).to(torch.bfloat16))

        ep = ExpertParallelMoE(H, I, E, K, T, num_shared_experts=S, expert_rows=expert_rows, combine_rows=combine_rows,
                               shared_rows=shared_rows)
        ids, scores = p["topk_ids"]
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        out = ep.forward(t(ids[mine]), t(scores[mine]), t(p["hidden_states"][mine]), t(p["hidden_states_scale"][mine]),
                         t(w["gemm1_weights"]), t(w["gemm1_weights_scale"]), t(w["gemm2_weights"]), t(w["gemm2_weights_scale"]))
        ref = o.moe_expected(p)[mine]
        r = assert_layer_parity(out.float().numpy(), ref, f"rank {rank}", extra_bf16_roundings=world)
        results[rank] = r["rel_l2"]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("masked", [False, True])
def test_expert_parallel_two_ranks_matches_single_process(masked):
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), masked, results), nprocs=world, join=True)
        assert sorted(results.keys()) == [0, 1]
        assert all(v <= 1e-2 for v in results.values())


def test_build_dispatch_plan():
    from kernelschema_b200.ep import build_dispatch
    ids = torch.tensor([[3, 0], [-1, 2], [1, 1], [9, 0]], dtype=torch.int32)   # 9 is out of range -> dropped
    plan = build_dispatch(ids, experts_per_rank=2, world=2)
    # rank 0 owns experts 0,1; rank 1 owns 2,3. token 0 visits both ranks, token 1 rank 1, tokens 2 and 3 rank 0
    assert plan["send_counts"].tolist() == [3, 2]
    assert plan["dest"].tolist() == [0, 0, 0, 1, 1]
    assert plan["tok"].tolist() == [0, 2, 3, 0, 1]
    assert plan["local_ids"].tolist() == [[-1, 0], [1, 1], [-1, 0], [1, -1], [-1, 0]]
    assert plan["pos_of_pair"].tolist() == [[0, 3], [-1, 4], [1, -1], [2, -1]]


def test_plan_messages_torch_layout():
    from kernelschema_b200.ep import message_views, plan_messages_torch, row_bytes
    h, k = 256, 2
    ids = torch.tensor([[3, 0], [-1, 2], [1, 1], [9, 0]], dtype=torch.int32)
    w = torch.arange(8, dtype=torch.float32).reshape(4, 2)
    hq = torch.arange(4 * h // 2, dtype=torch.int64).reshape(4, h // 2).to(torch.uint8)
    hs = (torch.arange(4 * h // 16, dtype=torch.int64).reshape(4, h // 16) + 100).to(torch.uint8)
    msg, seg_rows, row_of = plan_messages_torch(ids, w, hq, hs, experts_per_rank=2, world=2, shared_slot=True)
    assert row_bytes(h, k) == 160 and msg.shape == (256, 160)
    assert seg_rows == [128, 128]                      # 3 and 2 pairs, each segment padded to 128 rows
    assert row_of.tolist() == [[0, 128, 256], [-1, 129, 257], [1, -1, 258], [2, -1, 259]]
    m_q, m_sf, m_ids, m_w = message_views(msg, h, k)
    assert torch.equal(m_q[[0, 1, 2, 128, 129]], hq[[0, 2, 3, 0, 1]])
    assert torch.equal(m_sf[[0, 1, 2, 128, 129]], hs[[0, 2, 3, 0, 1]])
    assert m_ids[[0, 1, 2, 128, 129]].tolist() == [[-1, 0], [1, 1], [-1, 0], [1, -1], [-1, 0]]
    assert torch.equal(m_w[[0, 1, 2, 128, 129]], w[[0, 2, 3, 0, 1]])
    live = torch.zeros(256, dtype=torch.bool)
    live[[0, 1, 2, 128, 129]] = True
    assert (m_ids[~live] == -1).all()                  # padding rows carry no routes
