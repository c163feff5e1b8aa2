"""Torch-facing wrappers of the C ABI. Torch supplies device memory and the current stream only; every
computation runs in libb200moe.so and a missing library or a non-CUDA tensor is an error, never a fallback."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


_shim_mod = None


def _shim():
    """The pybind11 binding (built next to the library by ``python -m kernelschema_b200.build``)."""
    global _shim_mod
    if _shim_mod is None:
        _lib.load()
        try:
            from . import _b200moe_shim
        except ImportError as exc:
            raise RuntimeError("kernelschema_b200/_b200moe_shim.so is missing: run `python -m kernelschema_b200.build`") from exc
        _shim_mod = _b200moe_shim
    return _shim_mod


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("libb200moe operates on CUDA tensors only")


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def nvfp4_quantize(x: torch.Tensor, global_scale: float = 1.0, tiled_scales: bool = False, out=None):
    """bf16 [rows, cols] -> (payload uint8 [rows, cols/2], scales float8_e4m3fn).

    ``out = (payload, scales)`` reuses caller-owned buffers of those shapes (uint8; a steady-state loop then allocates
    nothing); padding rows of a tiled scale buffer are left as they are.

    Same bytes as the reference generator's ``quantize(value, 16)`` (problem/input.py:53-71) and, with a
    global scale, as the dense GEMM problem's ``quantize`` (bf16_nvfp4_gemm/problem/input.py:40-64).
    ``tiled_scales`` returns the 128x4-tiled layout (uint8, [ceil(rows/128), cols/64, 32, 16]) instead of
    row-major [rows, cols/16].
    """
    _need_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError("nvfp4_quantize expects a 2-D bfloat16 tensor")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    if out is not None:
        payload, scales = out
        _need_cuda(payload, scales)
        want = ((rows + 127) // 128 * (cols // 64) * 512) if tiled_scales else rows * (cols // 16)
        if payload.dtype != torch.uint8 or payload.numel() != rows * (cols // 2) or not payload.is_contiguous():
            raise ValueError("out[0] must be a contiguous uint8 tensor of rows * cols / 2 bytes")
        scales = scales.view(torch.uint8) if scales.dtype != torch.uint8 else scales
        if scales.numel() != want or not scales.is_contiguous():
            raise ValueError("out[1] must be a contiguous 1-byte tensor of the scale layout's size")
    else:
        payload = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
        if tiled_scales:
            scales = torch.zeros(((rows + 127) // 128, cols // 64, 32, 16), dtype=torch.uint8, device=x.device)
        else:
            scales = torch.empty((rows, cols // 16), dtype=torch.uint8, device=x.device)
    lib = _lib.load()
    _lib.check(lib.b200moe_quantize_nvfp4(x.data_ptr(), rows, cols, x.stride(0), float(global_scale), payload.data_ptr(),
                                          scales.data_ptr(), _lib.SF_TILED if tiled_scales else _lib.SF_ROW_MAJOR, _stream()),
               "b200moe_quantize_nvfp4")
    return payload, (scales if tiled_scales else scales.view(torch.float8_e4m3fn))


def scales_to_tiles(scales: torch.Tensor) -> torch.Tensor:
    """Row-major scale bytes [rows, cols/16] -> 128x4 tiles [ceil(rows/128), cols/64, 32, 16] (uint8)."""
    _need_cuda(scales)
    s = scales.contiguous().view(torch.uint8)
    rows, blocks = s.shape
    out = torch.empty(((rows + 127) // 128, blocks // 4, 32, 16), dtype=torch.uint8, device=s.device)
    _lib.check(_lib.load().b200moe_scales_to_tiles(s.data_ptr(), rows, blocks * 16, out.data_ptr(), _stream()),
               "b200moe_scales_to_tiles")
    return out


def route_topk(logits: torch.Tensor, top_k: int, bias: torch.Tensor | None = None, out=None):
    """fp32 logits [T, E] -> (ids int32 [T, K], weights fp32 [T, K]); problem/input.py:35-36.
    ``out = (ids, weights)`` reuses caller-owned contiguous buffers."""
    _need_cuda(logits, bias)
    lg = logits.contiguous().float()
    t, e = lg.shape
    if out is not None:
        ids, w = out
        _need_cuda(ids, w)
        if ids.dtype != torch.int32 or w.dtype != torch.float32 or tuple(ids.shape) != (t, top_k) or tuple(w.shape) != (t, top_k) \
                or not ids.is_contiguous() or not w.is_contiguous():
            raise ValueError("out must be (int32 [T, K], float32 [T, K]), contiguous")
    else:
        ids = torch.empty((t, top_k), dtype=torch.int32, device=lg.device)
        w = torch.empty((t, top_k), dtype=torch.float32, device=lg.device)
    b = None if bias is None else bias.contiguous().float()
    _lib.check(_lib.load().b200moe_route_topk(lg.data_ptr(), _ptr(b), t, e, top_k, ids.data_ptr(), w.data_ptr(), _stream()),
               "b200moe_route_topk")
    return ids, w


def router_logits(x: torch.Tensor, gate_weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 x [T, H] times bf16 gate [E, H]^T -> fp32 logits [T, E] (``out``: caller-owned contiguous fp32 [T, E])."""
    _need_cuda(x, gate_weight, out)
    x = x.contiguous()
    g = gate_weight.contiguous()
    if out is None:
        out = torch.empty((x.shape[0], g.shape[0]), dtype=torch.float32, device=x.device)
    elif out.dtype != torch.float32 or tuple(out.shape) != (x.shape[0], g.shape[0]) or not out.is_contiguous():
        raise ValueError("out must be a contiguous float32 [T, E] tensor")
    _lib.check(_lib.load().b200moe_router_logits(x.data_ptr(), g.data_ptr(), x.shape[0], x.shape[1], g.shape[0], out.data_ptr(),
                                                 _stream()), "b200moe_router_logits")
    return out


def mm_nvfp4(a_q, a_sf_tiled, b_q, b_sf_tiled, alpha: float = 1.0, out: torch.Tensor | None = None, tile_n: int = 0,
             status: torch.Tensor | None = None):
    """out[M, N] = bf16(alpha * A @ B^T) with both operands NVFP4 (payload uint8 [rows, K/2], tiled scales)."""
    _need_cuda(a_q, a_sf_tiled, b_q, b_sf_tiled, out)
    m, k2 = a_q.shape
    n = b_q.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a_q.device)
    _lib.check(_lib.load().b200moe_gemm_nvfp4(a_q.data_ptr(), a_sf_tiled.data_ptr(), b_q.data_ptr(), b_sf_tiled.data_ptr(),
                                              float(alpha), out.data_ptr(), m, n, k2 * 2, out.stride(0), tile_n, _ptr(status),
                                              _stream()), "b200moe_gemm_nvfp4")
    return out


_W4A16_WORKSPACE: dict = {}     # device index -> fp32 split-K scratch, grown on demand (small M only)


def mm_bf16_nvfp4(a: torch.Tensor, b: torch.Tensor, b_descale: torch.Tensor, alpha: torch.Tensor | None = None,
                  out: torch.Tensor | None = None, status: torch.Tensor | None = None, split_k: bool = True) -> torch.Tensor:
    """out[M, N] = bf16(alpha * a @ decode(b)^T): bf16 activations [M, K] (not quantised), NVFP4 weights uint8 [N, K/2] with
    row-major E4M3 scales [N, K/16], alpha a 1-element fp32 device tensor or None (the dense operator's contract,
    gemm/dense/bf16_nvfp4_gemm/problem/reference.py:10-15)."""
    _need_cuda(a, b, b_descale, out, alpha)
    if a.dtype != torch.bfloat16 or a.dim() != 2 or a.stride(1) != 1:
        raise ValueError("a must be a bf16 matrix with unit column stride")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] * 2 != k or b_descale.shape != (n, k // 16) or not b.is_contiguous() or not b_descale.is_contiguous():
        raise ValueError(f"b must be contiguous [N, K/2] and b_descale contiguous [N, K/16]; got {tuple(b.shape)}, {tuple(b_descale.shape)}")
    if alpha is not None and (alpha.dtype != torch.float32 or alpha.numel() != 1):
        raise ValueError("alpha must be one fp32 value")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if out.dtype != torch.bfloat16 or out.shape != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be bf16 [M, N] with unit column stride")
    lib = _lib.load()
    ws = None
    need = int(lib.b200moe_gemm_bf16_nvfp4_workspace_bytes(m, n, k)) if split_k else 0
    if need:
        # one scratch buffer per device, reused by later calls on the same stream order (calls on different streams
        # that may overlap should pass split_k=False or run on one stream)
        dev = a.device.index
        ws = _W4A16_WORKSPACE.get(dev)
        if ws is None or ws.numel() < need:
            ws = _W4A16_WORKSPACE[dev] = torch.empty(need, dtype=torch.uint8, device=a.device)
    _lib.check(lib.b200moe_gemm_bf16_nvfp4(a.data_ptr(), a.stride(0), b.data_ptr(), b_descale.data_ptr(), _ptr(alpha), out.data_ptr(),
                                           m, n, k, out.stride(0), _ptr(ws), need, _ptr(status), _stream()),
               "b200moe_gemm_bf16_nvfp4")
    return out


def combine(rows: torch.Tensor, row_of: torch.Tensor, weight_of_row: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = bf16(sum_s rows[row_of[t, s]] * weight_of_row[row_of[t, s]]) (reference.py:91-92), slots ascending."""
    _need_cuda(rows, row_of, weight_of_row, out)
    t, slots = row_of.shape
    _lib.check(_lib.load().b200moe_combine(rows.data_ptr(), row_of.data_ptr(), weight_of_row.data_ptr(), t, slots,
                                           rows.shape[1], out.data_ptr(), out.stride(0), _stream()), "b200moe_combine")
    return out


def ep_visits(ids: torch.Tensor, experts_per_rank: int, world: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """int32 [T, world]: column r holds r where the token has a route to an expert of rank r, else -1."""
    _need_cuda(ids)
    t, k = ids.shape
    if out is None:
        out = torch.empty((t, world), dtype=torch.int32, device=ids.device)
    _lib.check(_lib.load().b200moe_ep_visits(_ptr(ids), t, k, experts_per_rank, world, _ptr(out), _stream()), "b200moe_ep_visits")
    return out


def ep_pack(plan: "MoELayer", hidden_states, hidden_states_scale, ids, weights, experts_per_rank: int, out: torch.Tensor):
    """Fill the dispatch message rows (uint8 [rows, row_bytes]) of the (token, rank) pairs of ``plan``'s route map."""
    _need_cuda(hidden_states, hidden_states_scale, ids, weights, out)
    h = hidden_states.shape[1] * 2
    _lib.check(_lib.load().b200moe_ep_pack(plan._h, _ptr(hidden_states), _ptr(hidden_states_scale), _ptr(ids), _ptr(weights), h,
                                           ids.shape[1], experts_per_rank, out.shape[1], _ptr(out), _stream()), "b200moe_ep_pack")
    return out


class MoELayer:
    """One layer instance: owns the library workspace for a geometry (b200moe_create / b200moe_destroy)."""

    def __init__(self, hidden: int, intermediate: int, num_experts: int, top_k: int, max_tokens: int,
                 num_shared_experts: int = 0, tile_n: int = 0, sm_margin: int = 0, graph_cache: bool = False,
                 tma_gather: bool = False):
        lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("libb200moe needs a CUDA device (sm_100a); there is no CPU path")
        self.cfg = _lib.Config(struct_size=C.sizeof(_lib.Config), hidden=hidden, intermediate=intermediate,
                               num_experts=num_experts, top_k=top_k, num_shared_experts=num_shared_experts,
                               max_tokens=max_tokens, tile_n=tile_n, sm_margin=sm_margin, graph_cache=int(bool(graph_cache)),
                               tma_gather=int(bool(tma_gather)))
        self._h = C.c_void_p()
        _lib.check(lib.b200moe_create(C.byref(self.cfg), C.byref(self._h)), "b200moe_create")
        self.device = torch.cuda.current_device()
        self._keep = None

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            _lib.load().b200moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ building blocks
    def _args(self, ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, out, *, alpha=None, beta=None, limit=None,
              scale_up=None, scale_gate=None, scale_out=None, activation_type=3, expert_offset=0, scale_layout=2, direct_rows=False):
        t = hidden_states.shape[0]
        a = _lib.Args(struct_size=C.sizeof(_lib.Args), num_tokens=t, topk_ids=_ptr(ids), topk_weights=_ptr(weights),
                      hidden_states=_ptr(hidden_states), hidden_states_scale=_ptr(hidden_states_scale),
                      hidden_states_scale_layout=scale_layout, activation_type=activation_type, gemm1_weights=_ptr(w1),
                      gemm1_weights_scale=_ptr(s1), gemm2_weights=_ptr(w2), gemm2_weights_scale=_ptr(s2),
                      gemm1_alpha=_ptr(alpha), gemm1_beta=_ptr(beta), gemm1_clamp_limit=_ptr(limit),
                      output1_scale_scalar=_ptr(scale_up), output1_scale_gate_scalar=_ptr(scale_gate),
                      output2_scale_scalar=_ptr(scale_out), local_expert_offset=expert_offset, direct_rows=int(direct_rows),
                      output=_ptr(out),
                      output_stride=out.stride(0),
                      hidden_states_stride=hidden_states.stride(0) * hidden_states.element_size() if hidden_states.dim() == 2 else 0,
                      hidden_states_scale_stride=(hidden_states_scale.stride(0) * hidden_states_scale.element_size()
                                                  if (scale_layout == 2 and hidden_states_scale.dim() == 2) else 0),
                      topk_stride=0 if ids is None else ids.stride(0))
        return a

    def run(self, ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, out, *, alpha=None, beta=None, limit=None,
            scale_up=None, scale_gate=None, scale_out=None, activation_type=3, expert_offset=0, scale_layout=2, direct_rows=False):
        """Asynchronous forward on the current stream; writes ``out`` (bf16 [T, H]) in place. The hot call goes through
        the pybind11 shim (one positional C++ call, no ctypes struct marshalling). ids/weights, the payload and row-major
        scales may be row-strided views (e.g. columns of a packed message buffer); their strides are passed on."""
        _need_cuda(hidden_states, hidden_states_scale, w1, s1, w2, s2, out)
        p = lambda t: 0 if t is None else t.data_ptr()
        if ids is not None and weights is not None and ids.stride(0) != weights.stride(0):
            raise ValueError("topk_ids and topk_weights must have the same row stride")
        _shim().run(self._h.value, hidden_states.shape[0], p(ids), p(weights), p(hidden_states), p(hidden_states_scale),
                    scale_layout, activation_type, p(w1), p(s1), p(w2), p(s2), p(alpha), p(beta), p(limit), p(scale_up),
                    p(scale_gate), p(scale_out), expert_offset, int(direct_rows), p(out), out.stride(0), _stream(),
                    hidden_states.stride(0) * hidden_states.element_size() if hidden_states.dim() == 2 else 0,
                    hidden_states_scale.stride(0) * hidden_states_scale.element_size()
                    if (scale_layout == 2 and hidden_states_scale.dim() == 2) else 0,
                    0 if ids is None else ids.stride(0))
        return out

    def step(self, x, gate_weight, gate_bias, global_scale, w1, s1, w2, s2, out, *, alpha=None, beta=None, limit=None,
             scale_up=None, scale_gate=None, scale_out=None, activation_type=3):
        """The whole step from bf16 tokens in one library call (b200moe_step): quantiser, router logits, top-k / softmax,
        layer. The argument block is cached per (tensors, sizes): a repeat call only hands its address to the library,
        which replays its graph when the layer was created with ``graph_cache``."""
        key = (x.data_ptr(), x.shape[0], x.stride(0), gate_weight.data_ptr(), _ptr(gate_bias), float(global_scale), w1.data_ptr(),
               s1.data_ptr(), w2.data_ptr(), s2.data_ptr(), _ptr(alpha), _ptr(beta), _ptr(limit), _ptr(scale_up), _ptr(scale_gate),
               _ptr(scale_out), out.data_ptr(), out.stride(0), activation_type)
        cached = getattr(self, "_step_cache", None)
        if cached is None or cached[0] != key:
            _need_cuda(x, gate_weight, gate_bias, w1, s1, w2, s2, out)
            if x.dtype != torch.bfloat16 or gate_weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
                raise ValueError("x, gate_weight and out must be bfloat16")
            if x.stride(1) != 1 or not gate_weight.is_contiguous() or out.stride(1) != 1:
                raise ValueError("x and out need unit inner stride, gate_weight must be contiguous")
            a = _lib.StepArgs(struct_size=C.sizeof(_lib.StepArgs), num_tokens=x.shape[0], x=x.data_ptr(), x_stride=x.stride(0),
                              gate_weight=gate_weight.data_ptr(), gate_bias=_ptr(gate_bias), activation_global_scale=float(global_scale),
                              activation_type=activation_type, gemm1_weights=w1.data_ptr(), gemm1_weights_scale=s1.data_ptr(),
                              gemm2_weights=w2.data_ptr(), gemm2_weights_scale=s2.data_ptr(), gemm1_alpha=_ptr(alpha),
                              gemm1_beta=_ptr(beta), gemm1_clamp_limit=_ptr(limit), output1_scale_scalar=_ptr(scale_up),
                              output1_scale_gate_scalar=_ptr(scale_gate), output2_scale_scalar=_ptr(scale_out), output=out.data_ptr(),
                              output_stride=out.stride(0))
            cached = self._step_cache = (key, a)
        _lib.check(_lib.load().b200moe_step(self._h, C.byref(cached[1]), _stream()), "b200moe_step")
        return out

    def step_outputs(self, num_tokens: int) -> dict:
        """Views of what the last `step` left in the workspace: ids int32 [T, K], weights fp32 [T, K] (for accounting)."""
        v = _lib.WorkspaceView()
        _lib.check(_lib.load().b200moe_workspace(self._h, C.byref(v)), "b200moe_workspace")
        k = max(1, self.cfg.top_k)
        return dict(ids=_from_device_ptr(v.step_ids, 4 * num_tokens * k, torch.int32, (num_tokens, k), self.device),
                    weights=_from_device_ptr(v.step_weights, 4 * num_tokens * k, torch.float32, (num_tokens, k), self.device))

    def run_ep(self, peers, ctrl_ptr: int, seg_len: int, ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, scratch_out,
               **kw):
        """The layer over the token slots of an expert-parallel receive buffer (b200moe_run_ep): `peers` is a
        ``_lib.EpPeers`` of the step's parity, `ctrl_ptr` the device address of this rank's control block. The combine
        pass writes into the source ranks' return buffers; `scratch_out` only satisfies the argument checks."""
        _need_cuda(hidden_states, hidden_states_scale, w1, s1, w2, s2)
        a = self._args(ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, scratch_out, **kw)
        _lib.check(_lib.load().b200moe_run_ep(self._h, C.byref(a), C.byref(peers), ctrl_ptr, seg_len, _stream()), "b200moe_run_ep")

    def run_profiled(self, ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, out, **kw):
        a = self._args(ids, weights, hidden_states, hidden_states_scale, w1, s1, w2, s2, out, **kw)
        ms = (C.c_float * 5)()
        _lib.check(_lib.load().b200moe_run_profiled(self._h, C.byref(a), _stream(), ms), "b200moe_run_profiled")
        return dict(zip(("route_map", "permute", "fc1", "fc2", "combine"), (float(v) for v in ms)))

    def route_map(self, ids, weights, expert_offset: int = 0):
        t = ids.shape[0]
        _lib.check(_lib.load().b200moe_route_map(self._h, _ptr(ids), _ptr(weights), t, expert_offset, _stream()),
                   "b200moe_route_map")

    def stats(self) -> dict:
        """Host-side counters of the layer (calls, graph replays / captures / evictions)."""
        st = _lib.Stats()
        _lib.check(_lib.load().b200moe_get_stats(self._h, C.byref(st)), "b200moe_get_stats")
        return {name: int(getattr(st, name)) for name, _ in _lib.Stats._fields_}

    def status(self) -> int:
        code = C.c_int32(0)
        _lib.check(_lib.load().b200moe_status(self._h, _stream(), C.byref(code)), "b200moe_status")
        return int(code.value)

    def workspace(self) -> dict:
        """Torch views (no copies) of the library-owned intermediates, for tests and the expert-parallel wrapper."""
        v = _lib.WorkspaceView()
        _lib.check(_lib.load().b200moe_workspace(self._h, C.byref(v)), "b200moe_workspace")
        c = self.cfg
        etot, kk = c.num_experts + c.num_shared_experts, c.top_k + c.num_shared_experts
        rows, tiles = int(v.row_capacity), int(v.tile_capacity)

        def view(ptr, nbytes, dtype, shape):
            return _from_device_ptr(ptr, nbytes, dtype, shape, self.device)

        return dict(
            counts=view(v.counts, 4 * etot, torch.int32, (etot,)),
            seg_start=view(v.seg_start, 4 * (etot + 1), torch.int32, (etot + 1,)),
            tile_expert=view(v.tile_expert, 4 * tiles, torch.int32, (tiles,)),
            tile_row0=view(v.tile_row0, 4 * tiles, torch.int32, (tiles,)),
            tile_rows=view(v.tile_rows, 4 * tiles, torch.int32, (tiles,)),
            totals=view(v.totals, 16, torch.int32, (4,)),
            pair_expert=view(v.pair_expert, 4 * tiles, torch.int32, (tiles,)),
            pair_row0=view(v.pair_row0, 4 * tiles, torch.int32, (tiles,)),
            pair_rows=view(v.pair_rows, 4 * tiles, torch.int32, (tiles,)),
            row_of=view(v.row_of, 4 * c.max_tokens * kk, torch.int32, (c.max_tokens, kk)),
            tok_of_row=view(v.tok_of_row, 4 * rows, torch.int32, (rows,)),
            weight_of_row=view(v.weight_of_row, 4 * rows, torch.float32, (rows,)),
            a_q=view(v.a_q, rows * c.hidden // 2, torch.uint8, (rows, c.hidden // 2)),
            a_sf=view(v.a_sf, rows * c.hidden // 16, torch.uint8, (rows // 128, c.hidden // 64, 32, 16)),
            act_q=view(v.act_q, rows * c.intermediate // 2, torch.uint8, (rows, c.intermediate // 2)),
            act_sf=view(v.act_sf, rows * c.intermediate // 16, torch.uint8, (rows // 128, c.intermediate // 64, 32, 16)),
            rout=view(v.rout, rows * c.hidden * 2, torch.bfloat16, (rows, c.hidden)),
            row_capacity=rows, tile_capacity=tiles)


class _DevMem:
    """Minimal __cuda_array_interface__ carrier so torch can alias library-owned device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _from_device_ptr(ptr: int, nbytes: int, dtype, shape, device):
    raw = torch.as_tensor(_DevMem(ptr, nbytes), device=f"cuda:{device}")
    return raw.view(dtype).view(shape)
