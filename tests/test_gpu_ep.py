"""Expert-parallel layer on 2 GPUs of one box (NCCL all-to-all + libb200moe on every rank) against the single-process
oracle. Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

T, H, I, E, K, S = 96, 512, 256, 8, 4, 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results, tokens=T, micro_batches=1, transport=None):
    T = tokens
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import assert_layer_parity, make_moe_case
        from oracle import nvfp4_oracle as o
        from kernelschema_b200.ep import ExpertParallelMoE
        p = make_moe_case(33, T * world, H, I, E, K, shared=S, global_scales=True, routing="zipf")
        e_local = E // world
        mine = slice(rank * T, (rank + 1) * T)
        own = list(range(rank * e_local, (rank + 1) * e_local)) + list(range(E, E + S))
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        ep = ExpertParallelMoE(H, I, E, K, T, num_shared_experts=S, micro_batches=micro_batches, transport=transport)
        assert ep.micro_batches == micro_batches
        ids, scores = p["topk_ids"]
        out = ep.forward(dev(ids[mine]), dev(scores[mine]), dev(p["hidden_states"][mine]), dev(p["hidden_states_scale"][mine]),
                         dev(p["gemm1_weights"][own]), dev(p["gemm1_weights_scale"][own]), dev(p["gemm2_weights"][own]),
                         dev(p["gemm2_weights_scale"][own]), scale_up=dev(p["output1_scale_scalar"][own]),
                         scale_gate=dev(p["output1_scale_gate_scalar"][own]), scale_out=dev(p["output2_scale_scalar"][own]))
        out = ep.forward(dev(ids[mine]), dev(scores[mine]), dev(p["hidden_states"][mine]), dev(p["hidden_states_scale"][mine]),
                         dev(p["gemm1_weights"][own]), dev(p["gemm1_weights_scale"][own]), dev(p["gemm2_weights"][own]),
                         dev(p["gemm2_weights_scale"][own]), scale_up=dev(p["output1_scale_scalar"][own]),
                         scale_gate=dev(p["output1_scale_gate_scalar"][own]), scale_out=dev(p["output2_scale_scalar"][own]))   # buffers reused
        torch.cuda.synchronize()
        assert ep.status() == 0
        r = assert_layer_parity(out.float().cpu().numpy(), o.moe_expected(p)[mine], f"rank {rank}", extra_bf16_roundings=world)
        results[rank] = r["rel_l2"]
        dist.barrier()
        ep.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("transport", ["p2p", "collective"])
def test_expert_parallel_two_gpus(transport):
    """`p2p`: rows and results as peer stores of the library's kernels with flags; `collective`: NCCL all-to-all."""
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), results, T, 1, transport), nprocs=2, join=True)
        assert sorted(results.keys()) == [0, 1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus_pipelined():
    """Two token halves pipelined over a compute and a communication stream (optional form, off by default)."""
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), results, 384, 2, "collective"), nprocs=2, join=True)
        assert sorted(results.keys()) == [0, 1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_devices():
    """The dynamic-shared-memory opt-in of the large kernels belongs to a (kernel, device) pair: a process that runs the
    layer, the dense GEMMs and the router on cuda:0 and then on cuda:1 must succeed on both."""
    import kernelschema_b200 as ks
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import assert_layer_parity, make_moe_case
    from gpu_util import run_model
    from oracle import nvfp4_oracle as o
    p = make_moe_case(5, 200, 512, 256, 8, 2, shared=1)
    want = o.moe_expected(p)
    for dev in (0, 1):
        with torch.cuda.device(dev):
            got, _, model = run_model(p)
            assert_layer_parity(got, want, f"device {dev}")
            x = torch.randn(256, 512, device="cuda").to(torch.bfloat16)
            g = (torch.randn(64, 512, device="cuda") * 0.02).to(torch.bfloat16)
            lg = ks.router_logits(x, g)
            assert torch.allclose(lg, x.float() @ g.float().t(), atol=1e-3, rtol=1e-3)
            aq, asf = ks.nvfp4_quantize(x, 1.0, tiled_scales=True)
            bq, bsf = ks.nvfp4_quantize(g.repeat(2, 1), 1.0, tiled_scales=True)
            y = ks.mm_nvfp4(aq, asf, bq, bsf)
            y2 = ks.mm_bf16_nvfp4(x, *[t.view(torch.uint8) for t in ks.nvfp4_quantize(g.repeat(2, 1), 1.0)])
            torch.cuda.synchronize()
            assert bool(torch.isfinite(y.float()).all()) and bool(torch.isfinite(y2.float()).all())
