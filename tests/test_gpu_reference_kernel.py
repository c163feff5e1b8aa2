"""The reference's own Blackwell kernel (compiled by oracle/build_ref.py from the reference checkout) as a second
checker next to the CPU oracle: this library, the reference kernel and the oracle must agree on the same inputs.
Skipped when the compiled reference library is absent."""
import numpy as np
import pytest
import torch

from helpers import assert_layer_parity, make_moe_case
from oracle import nvfp4_oracle as o
from oracle import ref_kernel

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernel.available(), reason="oracle/_ref library not built")]


@pytest.mark.parametrize("t,h,i,e,k,routing", [(512, 1024, 512, 16, 8, "uniform"), (300, 512, 256, 32, 8, "zipf")])
def test_three_way_agreement(t, h, i, e, k, routing):
    import kernelschema_b200 as ks
    from gpu_util import to_dev
    p = make_moe_case(41, t, h, i, e, k, routing=routing)
    ids, w = p["topk_ids"]
    dev = dict(ids=to_dev(ids), w=to_dev(w), hq=to_dev(p["hidden_states"]), hs=to_dev(p["hidden_states_scale"]),
               w1q=to_dev(p["gemm1_weights"]), w1s=to_dev(p["gemm1_weights_scale"]), w2q=to_dev(p["gemm2_weights"]),
               w2s=to_dev(p["gemm2_weights_scale"]), alpha=to_dev(p["gemm1_alpha"]), beta=to_dev(p["gemm1_beta"]))
    ref_out = torch.zeros(t, h, dtype=torch.bfloat16, device="cuda")
    ref_kernel.ReferenceKernel().run(dev["ids"], dev["w"], dev["hq"], dev["hs"], dev["w1q"], dev["w1s"], dev["w2q"], dev["w2s"],
                                     dev["alpha"], dev["beta"], None, ref_out)
    layer = ks.MoELayer(h, i, e, k, t)
    out = torch.zeros(t, h, dtype=torch.bfloat16, device="cuda")
    layer.run(dev["ids"], dev["w"], dev["hq"], dev["hs"], dev["w1q"], dev["w1s"], dev["w2q"], dev["w2s"], out,
              alpha=dev["alpha"], beta=dev["beta"])
    torch.cuda.synchronize()
    assert layer.status() == 0
    expect = o.moe_expected(p)
    mine, theirs = out.float().cpu().numpy(), ref_out.float().cpu().numpy()
    assert_layer_parity(theirs, expect, "reference kernel vs oracle")
    assert_layer_parity(mine, expect, "this library vs oracle")
    assert_layer_parity(mine, theirs, "this library vs reference kernel")
    layer.close()
