"""The layer at the benchmark's full sizes (Qwen3-30B-A3B T=16384; DeepSeek-V3 T=8192 + shared expert, Zipf routing),
checked through size-independent properties and a handful of sampled tokens against the oracle.

* token permutation: rows are independent, so permuting the tokens permutes the output bit for bit;
* routing-weight scaling by 2 (exact in fp32 and bf16) doubles the output bit for bit;
* tokens whose routes are all invalid produce exact zeros (plus the shared expert's row when there is one);
* sampled tokens: the oracle evaluates only the experts those tokens touch;
* decode batches: the first 1, 32, 64 and 256 tokens run alone take other kernels (one-launch route map + permute,
  narrower tiles and epilogues, batched combine) and must reproduce their rows of the full batch bit for bit.
Weights are generated and quantised on the device with the benchmark's own generator (the quantiser's bytes are
verified separately, bit for bit)."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from helpers import assert_layer_parity
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def _setup(name, tokens=None):
    import bench
    import kernelschema_b200 as ks
    wl = dict(bench.WORKLOADS[name])
    if tokens:
        wl["t"] = tokens
    dev = torch.device("cuda", 0)
    L = bench.build_layer(wl, 0, 1, dev)
    t, h, k = wl["t"], wl["h"], wl["k"]
    gen = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn((t, h), device=dev, generator=gen).to(torch.bfloat16)
    hq, hs = ks.nvfp4_quantize(x, bench.ACT_GLOBAL_SCALE)
    ids, w = ks.route_topk(ks.router_logits(x, L["gate_w"]), k, L["bias"])
    layer = ks.MoELayer(h, wl["i"], wl["e"], k, t, num_shared_experts=wl["s"])

    def run(ids_, w_, hq_, hs_):
        out = torch.empty((hq_.shape[0], h), dtype=torch.bfloat16, device=dev)
        layer.run(ids_, w_, hq_, hs_.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], out, scale_up=L["scale_fc1"],
                  scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
        torch.cuda.synchronize()
        assert layer.status() == 0
        return out

    return wl, L, (ids, w, hq, hs), run, layer


def _oracle_for_tokens(wl, L, ids, w, hq, hs, tokens):
    """Reference rows for a few tokens: only the experts they touch are brought to the host and decoded."""
    e, s, i, h = wl["e"], wl["s"], wl["i"], wl["h"]
    tok = torch.as_tensor(tokens, device=ids.device)
    sub_ids = ids[tok].cpu().numpy()
    touched = sorted(set(int(v) for v in sub_ids.reshape(-1) if v >= 0)) + list(range(e, e + s))
    remap = {g: j for j, g in enumerate(touched)}
    n_routed = len(touched) - s
    new_ids = np.vectorize(lambda g: remap[g] if g >= 0 else -1)(sub_ids).astype(np.int32)
    sel = torch.as_tensor(touched, device=ids.device)
    # the device holds scales as 128x4 tiles in a [rows, K/16] array, which is the reference's prepared layout; the
    # benchmark's random weights are "prepared" by construction (any row order of i.i.d. rows is as good as another)
    p = dict(topk_ids=(new_ids, w[tok].cpu().numpy()), hidden_states=hq[tok].cpu().numpy(),
             hidden_states_scale=hs.view(torch.uint8)[tok].cpu().numpy(), gemm1_weights=L["w1q"][sel].cpu().numpy(),
             gemm1_weights_scale=L["w1s"][sel].cpu().numpy(), gemm2_weights=L["w2q"][sel].cpu().numpy(),
             gemm2_weights_scale=L["w2s"][sel].cpu().numpy(), gemm1_alpha=np.ones(len(touched), np.float32),
             gemm1_beta=np.zeros(len(touched), np.float32), gemm1_clamp_limit=None, num_experts=n_routed, top_k=wl["k"],
             intermediate_size=i, activation_type=3, num_fused_shared_experts=s or None,
             output1_scale_scalar=L["scale_fc1"][sel].cpu().numpy(), output1_scale_gate_scalar=L["scale_fc1"][sel].cpu().numpy(),
             output2_scale_scalar=L["scale_fc2"][sel].cpu().numpy())
    return o.moe_expected(p)


@pytest.mark.parametrize("name,n_sample", [("qwen3", 24), ("dsv3", 2)])
def test_full_size_properties_and_samples(name, n_sample):
    wl, L, (ids, w, hq, hs), run, layer = _setup(name)
    t = wl["t"]
    base = run(ids, w, hq, hs)
    assert bool(torch.isfinite(base.float()).all())
    # permutation of the tokens
    perm = torch.randperm(t, device=ids.device, generator=torch.Generator(device=ids.device).manual_seed(5))
    out_p = run(ids[perm].contiguous(), w[perm].contiguous(), hq[perm].contiguous(), hs.view(torch.uint8)[perm].contiguous())
    assert torch.equal(out_p, base[perm])
    # doubling the routing weights doubles the routed part; with a shared expert (weight 1) compare through the difference
    if wl["s"] == 0:
        assert torch.equal(run(ids, (w * 2).contiguous(), hq, hs).float(), base.float() * 2)
    # tokens without routes
    ids0 = ids.clone()
    ids0[::97] = -1
    out0 = run(ids0, w, hq, hs)
    if wl["s"] == 0:
        assert bool((out0[::97] == 0).all())
    untouched = torch.ones(t, dtype=torch.bool, device=ids.device)
    untouched[::97] = False
    assert torch.equal(out0[untouched], base[untouched])
    # sampled tokens against the oracle
    rng = np.random.default_rng(1)
    tokens = sorted(rng.choice(t, size=n_sample, replace=False).tolist())
    ref = _oracle_for_tokens(wl, L, ids, w, hq, hs, tokens)
    assert_layer_parity(base[torch.as_tensor(tokens, device=ids.device)].float().cpu().numpy(), ref, f"{name} sampled tokens")
    # decode batches of the same tokens: every output element is the same sum in the same order, whatever the tile shapes
    for n in (1, 32, 64, 256):
        small = run(ids[:n].contiguous(), w[:n].contiguous(), hq[:n].contiguous(), hs.view(torch.uint8)[:n].contiguous())
        assert torch.equal(small, base[:n]), f"{name}: decode batch of {n} tokens differs from its rows of the full batch"
    layer.close()


def test_peer_memory_exchange_full_size_single_rank():
    """The expert-parallel peer-memory path at the benchmark's size on ONE GPU (a group of one rank is its own peer): 8192
    tokens, 256 + 1 experts. Its result may differ from the plain layer's only by the one extra bf16 rounding of the partial
    row that travels (exactly reproduced here: round the routed part to bf16, add the shared row, round again is NOT what
    the layer does, so compare with the parity rule instead)."""
    import socket
    import torch.distributed as dist
    from kernelschema_b200.ep import ExpertParallelMoE
    wl, L, (ids, w, hq, hs), run, layer = _setup("dsv3")
    base = run(ids, w, hq, hs)
    own = not dist.is_initialized()
    if own:
        with socket.socket() as sock:
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        ep = ExpertParallelMoE(wl["h"], wl["i"], wl["e"], wl["k"], wl["t"], num_shared_experts=wl["s"], transport="p2p")
        for _ in range(2):
            out = ep.forward(ids, w, hq, hs.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], scale_up=L["scale_fc1"],
                             scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
        torch.cuda.synchronize()
        assert ep.status() == 0
        assert_layer_parity(out.float().cpu().numpy(), base.float().cpu().numpy(), "p2p world=1 at full size", extra_bf16_roundings=1)
        ep.close()
    finally:
        if own:
            dist.destroy_process_group()
    layer.close()
