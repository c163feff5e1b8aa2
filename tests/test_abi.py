"""CPU-only checks of the C-ABI boundary: the library loads, exports exactly what include/b200moe.h declares,
and refuses bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from kernelschema_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from kernelschema_b200 import _lib
    names = declared_symbols()
    assert names == sorted(_lib.SIGNATURES), (names, sorted(_lib.SIGNATURES))
    for n in names:
        assert hasattr(lib, n), n
    assert lib.b200moe_abi_version() == _lib.ABI_VERSION


def test_struct_sizes_match_header(lib):
    from kernelschema_b200 import _lib
    assert C.sizeof(_lib.Config) == 16 * 4
    assert C.sizeof(_lib.Args) == 8 + 8 * 4 + 8 + 8 * 10 + 8 + 16 + 24
    assert C.sizeof(_lib.WorkspaceView) == 14 * 8 + 16 + 24 + 16
    assert C.sizeof(_lib.StepArgs) == 8 + 8 * 4 + 8 + 8 * 10 + 16
    assert C.sizeof(_lib.EpPeers) == 8 + 3 * 16 * 8
    assert C.sizeof(_lib.Stats) == 6 * 8


def test_bad_config_is_refused_without_a_device(lib):
    from kernelschema_b200 import _lib
    cfg = _lib.Config(struct_size=C.sizeof(_lib.Config), hidden=100, intermediate=256, num_experts=4, top_k=2, max_tokens=8)
    assert lib.b200moe_workspace_bytes(C.byref(cfg)) == -1
    assert b"hidden" in lib.b200moe_last_error()
    h = C.c_void_p()
    assert lib.b200moe_create(C.byref(cfg), C.byref(h)) == 711 and not h
    cfg.hidden = 256
    cfg.struct_size = 3
    assert lib.b200moe_create(C.byref(cfg), C.byref(h)) == 710
    cfg.struct_size = C.sizeof(_lib.Config)
    assert lib.b200moe_workspace_bytes(C.byref(cfg)) > 0
    cfg.tma_gather = 2
    assert lib.b200moe_create(C.byref(cfg), C.byref(h)) == 707 and b"tma_gather" in lib.b200moe_last_error()
    cfg.tma_gather = 0
    cfg.graph_cache = 5
    assert lib.b200moe_create(C.byref(cfg), C.byref(h)) == 709


def test_argument_checks_precede_launches(lib):
    assert lib.b200moe_quantize_nvfp4(None, 4, 100, 100, 1.0, None, None, 0, None) == 740
    assert lib.b200moe_quantize_nvfp4(None, 4, 128, 128, 1.0, None, None, 0, None) == 742
    assert lib.b200moe_route_topk(None, None, 4, 8, 9, None, None, None) == 750
    assert lib.b200moe_gemm_nvfp4(None, None, None, None, 1.0, None, 4, 128, 100, 128, 0, None, None) == 761
    assert lib.b200moe_run(None, None, None) == 720
    # expert-parallel exchange and diagnostics
    assert lib.b200moe_run_ep(None, None, None, None, 128, None) == 720
    assert lib.b200moe_ep_wait(None, None, 2, 1, None) == 796
    assert lib.b200moe_ep_post(None, 32, 1, None) == 796
    assert lib.b200moe_ep_dispatch(None, None, None, None, None, 4, 256, 2, 2, 4096, None, 1, 0, 0, None, None) == 792
    assert lib.b200moe_ep_shared_alloc(0, None, None) == 797
    assert lib.b200moe_ep_shared_open(None, None) == 797
    assert lib.b200moe_ep_shared_close(None) == 0 and lib.b200moe_ep_shared_free(None) == 0
    assert lib.b200moe_get_stats(None, None) == 719
    assert lib.b200moe_step(None, None, None) == 720
    from kernelschema_b200 import _lib
    bad = _lib.EpPeers(world=99, rank=0)
    assert lib.b200moe_ep_post(C.byref(bad), _lib.EP_FLAG_RETURN, 1, None) == 796 and b"world" in lib.b200moe_last_error()


def test_model_refuses_cpu_tensors():
    import torch
    import kernelschema_b200 as ks
    m = ks.Model()
    z = torch.zeros(2, 128, dtype=torch.uint8)
    with pytest.raises(ValueError):
        m(topk_ids=(torch.zeros(2, 2, dtype=torch.int32), torch.zeros(2, 2)), routing_bias=None, hidden_states=z,
          hidden_states_scale=torch.zeros(2, 16, dtype=torch.uint8), gemm1_weights=z, gemm1_weights_scale=z, gemm1_bias=None,
          gemm1_alpha=None, gemm1_beta=None, gemm1_clamp_limit=None, gemm2_weights=z, gemm2_weights_scale=z, gemm2_bias=None,
          output1_scale_scalar=None, output1_scale_gate_scalar=None, output2_scale_scalar=None, num_experts=4, top_k=2,
          n_group=None, topk_group=None, intermediate_size=256, local_expert_offset=0, local_num_experts=4,
          routed_scaling_factor=1.0, output=torch.zeros(2, 256, dtype=torch.bfloat16))


def test_pybind_shim_loads_and_maps_errors(lib):
    from kernelschema_b200 import _lib
    from kernelschema_b200.ops import _shim
    shim = _shim()
    assert shim.abi_version() == _lib.ABI_VERSION
    with pytest.raises(ValueError):
        shim.create(100, 256, 4, 2, 0, 8, 0, 0)
    with pytest.raises(ValueError):
        shim.run(0, 1, *([0] * 21))


def test_dense_entry_refuses_bad_shapes_without_a_device(lib):
    """Argument checks of the bf16 x NVFP4 GEMM entry run before any CUDA call."""
    import ctypes as C
    assert lib.b200moe_gemm_bf16_nvfp4(None, 128, None, None, None, None, 8, 128, 100, 128, None, 0, None, None) == 765   # K % 256
    assert b"K % 256" in lib.b200moe_last_error()
    assert lib.b200moe_gemm_bf16_nvfp4(None, 256, None, None, None, None, 8, 100, 256, 128, None, 0, None, None) == 765   # N % 128
    assert lib.b200moe_gemm_bf16_nvfp4(None, 256, None, None, None, None, 8, 128, 256, 128, None, 0, None, None) == 766   # null pointers
    assert lib.b200moe_gemm_bf16_nvfp4(None, 256, None, None, None, None, 0, 128, 256, 128, None, 0, None, None) == 0     # M = 0: nothing to do
    assert lib.b200moe_gemm_bf16_nvfp4_workspace_bytes(8, 100, 256) == 0
