"""CPU oracle for the NVFP4 mixture-of-experts path.  TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of the reference operator's fp32
"dequantise then matmul" compute and of its input generator.  It is the
checker for the CUDA library, never a product path: only the tests, the
smoke check and the CPU-baseline leg of the benchmark import it.

Every function cites the reference file:line it follows.  Reference paths are
relative to
``kernel_wiki/aka-cuda-operators-20261030/operators/`` of bcacdwk/KernelSchema:

* ``moe/nvfp4_fused_moe/problem/reference.py``  (fp32 compute)
* ``moe/nvfp4_fused_moe/problem/input.py``      (quantiser, router, weight layout)
* ``gemm/dense/bf16_nvfp4_gemm/problem/{input,reference}.py`` (global-scale
  quantiser and the dense GEMM contract)

Parity pin: ``tests/golden/make_golden.py`` imports those reference modules,
runs them on seeded inputs and stores inputs + outputs; ``tests/test_oracle.py``
replays the fixtures through this file.  Three extensions have no counterpart
in the reference and are therefore *unpinned* (defined here as the obvious
extension of the reference math): per-expert output scale scalars different
from 1, fused shared experts, and the router-logits matmul.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------- formats

#: E2M1 magnitudes, code 0..7 (reference.py:29, input.py:46)
E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
#: signed decode table indexed by the 4-bit code (reference.py:47)
E2M1_LUT = np.concatenate([E2M1_LEVELS, -E2M1_LEVELS]).astype(np.float32)


def _e4m3_table() -> np.ndarray:
    """All 256 E4M3 (fn variant: no inf, 0x7f/0xff NaN) values as fp32."""
    out = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = s * v
    return out


E4M3_LUT = _e4m3_table()


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    """uint8 E4M3 bytes -> fp32 (what ``.view(float8_e4m3fn).float()`` does)."""
    return E4M3_LUT[np.asarray(b, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> E4M3 byte, round-to-nearest-even, for finite 0 <= x <= 448.

    Restates the ``.to(torch.float8_e4m3fn)`` cast the reference applies to
    already-clamped, non-negative scales (input.py:60, reference.py:41).
    """
    x = np.asarray(x, dtype=np.float32)
    assert np.all(np.isfinite(x)) and np.all(x >= 0) and np.all(x <= 448.0)
    pos = E4M3_LUT[:0x7F].astype(np.float64)          # 0 .. 448, ascending
    xd = x.astype(np.float64)
    hi = np.searchsorted(pos, xd, side="left")        # first code with value >= x
    hi = np.clip(hi, 0, 0x7E)
    lo = np.clip(hi - 1, 0, 0x7E)
    d_hi = pos[hi] - xd
    d_lo = xd - pos[lo]
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((hi & 1) == 0))
    exact = pos[hi] == xd
    code = np.where(exact | pick_hi, hi, lo)
    return code.astype(np.uint8)


def e2m1_code(normalized: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit signed E2M1 code (input.py:62-69).

    Magnitude code = number of midpoints crossed, with ``>`` at even midpoint
    index and ``>=`` at odd index (nearest, ties to even); sign bit 3 is the
    IEEE sign bit, so -0.0 and tiny negatives encode as 8.
    """
    n = np.asarray(normalized, dtype=np.float32)
    mag = np.abs(n)
    code = np.zeros(n.shape, dtype=np.uint8)
    for j in range(7):
        mid = np.float32((E2M1_LEVELS[j] + E2M1_LEVELS[j + 1]) / 2)
        code += (mag > mid if j % 2 == 0 else mag >= mid).astype(np.uint8)
    code |= np.signbit(n).astype(np.uint8) << 3
    return code


def pack_codes(code: np.ndarray) -> np.ndarray:
    """Even element in the low nibble (input.py:70)."""
    return (code[..., 0::2] | (code[..., 1::2] << 4)).astype(np.uint8)


def unpack_codes(q: np.ndarray) -> np.ndarray:
    q = np.asarray(q, dtype=np.uint8)
    return np.stack((q & 15, q >> 4), -1).reshape(*q.shape[:-1], q.shape[-1] * 2)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round-to-nearest-even) -> fp32, the ``.to(bfloat16).float()`` round trip."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).astype(np.uint32)
    nan = np.isnan(x)
    out = np.where(nan, np.uint32(0x7FC00000), out)
    return out.view(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 (already bf16-representable or not) -> uint16 bf16 bit pattern, RNE."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- quantiser

def quantize(value: np.ndarray, block: int = 16, global_scale: float = 1.0):
    """bf16/fp32 values -> (payload uint8 [.., k/2], scale bytes uint8 [.., k/block]).

    ``global_scale == 1``: moe/nvfp4_fused_moe/problem/input.py:53-71.
    otherwise: gemm/dense/bf16_nvfp4_gemm/problem/input.py:40-64
    (``scale = peak / 6 / gs``; ``normalized = x / (stored * gs)``), all in
    fp32 with IEEE division, as torch computes it on the CPU.
    """
    v = np.asarray(value, dtype=np.float32)
    k = v.shape[-1]
    assert k % block == 0
    groups = v.reshape(*v.shape[:-1], k // block, block)
    peak = np.maximum(np.abs(groups).max(-1), np.float32(2.0 ** -20))
    scale = peak / np.float32(6.0)
    gs = np.float32(global_scale)
    if global_scale != 1.0:
        scale = scale / gs
    stored = e4m3_encode(np.clip(scale, np.float32(2.0 ** -9), np.float32(448.0)))
    sf = e4m3_decode(stored)
    denom = sf[..., None] if global_scale == 1.0 else (sf[..., None] * gs).astype(np.float32)
    normalized = (groups / denom).astype(np.float32).reshape(v.shape)
    return pack_codes(e2m1_code(normalized)), stored


def decode(q: np.ndarray, sf: np.ndarray) -> np.ndarray:
    """payload + row-major E4M3 scale bytes -> fp32 (reference.py:45-50)."""
    val = E2M1_LUT[unpack_codes(q)]
    return val * np.repeat(e4m3_decode(sf), 16, axis=-1)


def nvfp4_qdq_parts(value: np.ndarray):
    """Activation quantise step of reference.py:38-43, returning codes and scale bytes.

    ``sf = e4m3(clamp(amax * (1/6), 0, 448))``; a zero scale gives an all-zero
    block; otherwise ``q = e2m1(x / sf)``.
    """
    v = np.asarray(value, dtype=np.float32)
    blocks = v.reshape(*v.shape[:-1], -1, 16)
    sf = np.abs(blocks).max(-1) * np.float32(1.0 / 6.0)
    stored = e4m3_encode(np.clip(sf, np.float32(0.0), np.float32(448.0)))
    sff = e4m3_decode(stored)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        normalized = np.where(sff > 0, blocks / sff, np.float32(0.0)).astype(np.float32)
    code = e2m1_code(normalized)
    return code.reshape(v.shape), stored


def nvfp4_qdq(value: np.ndarray) -> np.ndarray:
    """reference.py:38-43 ``nvfp4``: quantise-dequantise to the values FC2 consumes."""
    code, stored = nvfp4_qdq_parts(value)
    return (E2M1_LUT[code].reshape(*stored.shape, 16) * e4m3_decode(stored)[..., None]).reshape(code.shape)


# --------------------------------------------------------------------------- weight layout

def prepared_row_source(n: int, gated: bool) -> np.ndarray:
    """src[p] = logical row stored at prepared row p (input.py:88-92)."""
    row = np.arange(n)
    row = (row // 32) * 32 + (row % 8) * 4 + (row % 32) // 8
    if gated:
        row = row // 2 + (row % 2) * (n // 2)
    return row


def block_scales(scale_u8: np.ndarray) -> np.ndarray:
    """[e, n, k] row-major scale bytes -> 128x4 tiles [e, n/128, k/4, 32, 16] (input.py:82-87)."""
    e, n, k = scale_u8.shape
    pn, pk = (n + 127) // 128 * 128, (k + 3) // 4 * 4
    raw = np.zeros((e, pn, pk), dtype=np.uint8)
    raw[:, :n, :k] = scale_u8
    return np.ascontiguousarray(
        raw.reshape(e, pn // 128, 4, 32, pk // 4, 4).transpose(0, 1, 4, 3, 2, 5)
    ).reshape(e, pn // 128, pk // 4, 32, 16)


def unblock_scales(tiled: np.ndarray, n: int, k: int) -> np.ndarray:
    """Inverse of :func:`block_scales` (reference.py:60)."""
    e = tiled.shape[0]
    t = np.asarray(tiled, dtype=np.uint8).reshape(e, n // 128, k // 4, 32, 4, 4)
    return np.ascontiguousarray(t.transpose(0, 1, 4, 3, 2, 5)).reshape(e, n, k)


def prepare_weights(q: np.ndarray, sf: np.ndarray, gated: bool):
    """Logical [e, n, k/2] payload + [e, n, k/16] scales -> frozen weight ABI (input.py:88-99).

    Rows are 32-row shuffled (and up/gate interleaved when ``gated``); scales
    follow the same row map and are then tiled 128x4.  The returned scale array
    keeps the logical shape [e, n, k/16] like the reference's ``reshape_as``.
    """
    n = q.shape[1]
    row = prepared_row_source(n, gated)
    payload = np.ascontiguousarray(q[:, row])
    scales = block_scales(np.asarray(sf, dtype=np.uint8)[:, row]).reshape(sf.shape)
    return payload, scales


def weight_decode(q_e: np.ndarray, sf_e: np.ndarray, gated: bool) -> np.ndarray:
    """One expert of the frozen ABI -> logical fp32 [n, k] (reference.py:52-67, one ``e``)."""
    n, c = sf_e.shape
    linear = unblock_scales(np.asarray(sf_e, dtype=np.uint8)[None], n, c)[0]
    rows = np.arange(n)
    if gated:
        rows = np.where(rows < n // 2, rows * 2, (rows - n // 2) * 2 + 1)
    source = rows // 32 * 32 + rows % 4 * 8 + rows % 32 // 4
    return decode(q_e[source], linear[source])


# --------------------------------------------------------------------------- router

def route_topk(logits: np.ndarray, topk: int, bias: np.ndarray | None = None):
    """Top-k by logit then softmax over the selected logits (input.py:35-36).

    ``bias`` (an extension, used for the skewed benchmark routing) is added to
    the logits before selection *and* softmax, exactly like the reference's
    ``logits += ...`` profiles (input.py:30-33).  Ties resolve to the lowest
    expert index.  The softmax is evaluated in float64 and rounded once to
    fp32 (the reference's fp32 softmax agrees to within 4 ulp).
    Returns (ids int32 [T,K] in descending-logit order, weights fp32 [T,K]).
    """
    lg = np.asarray(logits, dtype=np.float32)
    if bias is not None:
        lg = (lg + np.asarray(bias, dtype=np.float32)[None, :]).astype(np.float32)
    order = np.argsort(-lg, axis=-1, kind="stable")[:, :topk]
    sel = np.take_along_axis(lg, order, axis=-1).astype(np.float64)
    ex = np.exp(sel - sel[:, :1])
    w = (ex / ex.sum(-1, keepdims=True)).astype(np.float32)
    return order.astype(np.int32), w


def apply_route_masks(ids: np.ndarray, weights: np.ndarray, *, empty=False, masked_routes=False):
    """input.py:37-41: invalid routes carry id -1 and weight 0."""
    ids = ids.copy()
    weights = weights.copy()
    if empty:
        ids[:] = -1
    if masked_routes:
        ids[::3, -1] = -1
    weights[ids < 0] = 0.0
    return ids, weights


def router_logits(x_bf16_as_f32: np.ndarray, gate_w_bf16_as_f32: np.ndarray) -> np.ndarray:
    """fp32 matmul of bf16 operands (no reference counterpart: the reference synthesises logits)."""
    return (x_bf16_as_f32.astype(np.float64) @ gate_w_bf16_as_f32.astype(np.float64).T).astype(np.float32)


# --------------------------------------------------------------------------- route map

def route_map(ids: np.ndarray, num_experts: int, tile_m: int = 128, *, expert_offset: int = 0,
              shared_experts: int = 0):
    """Expert-permutation index build.

    Semantics of the reference's route-map kernels (candidate ``k_count`` /
    ``k_scan_tiles`` / ``k_scatter_agg``, described in
    schema_wiki .../nvfp4_fused_moe/root.yaml:172-197), with one tightening:
    positions inside an expert are assigned in ascending flat route index
    ``t*K + k`` (the reference leaves that order arbitrary), which is also the
    order ``(ids == e).nonzero()`` yields in reference.py:76.

    Each expert segment starts on a ``tile_m`` boundary of the permuted buffer.
    ``shared_experts`` appends that many always-selected experts (ids
    ``num_experts + s``), one extra slot per token each.

    Returns dict with counts[E'], seg_start[E'+1] (padded), tile_expert,
    tile_row0, tile_rows, row_of[T, K'] (-1 invalid), tok_of_row[R_pad] (-1 pad),
    slot_of_row[R_pad].
    """
    ids = np.asarray(ids, dtype=np.int64)
    t, k = ids.shape
    e_tot = num_experts + shared_experts
    if shared_experts:
        extra = np.broadcast_to(np.arange(num_experts, e_tot)[None, :] + expert_offset, (t, shared_experts))
        ids = np.concatenate([ids, extra], axis=1)
    kk = ids.shape[1]
    local = ids - expert_offset
    valid = (local >= 0) & (local < e_tot)
    flat = np.where(valid, local, -1).reshape(-1)
    counts = np.bincount(flat[flat >= 0], minlength=e_tot).astype(np.int32)
    padded = (counts + tile_m - 1) // tile_m * tile_m
    seg_start = np.concatenate([[0], np.cumsum(padded)]).astype(np.int32)
    r_pad = int(seg_start[-1])
    row_of = np.full(t * kk, -1, dtype=np.int32)
    tok_of_row = np.full(r_pad, -1, dtype=np.int32)
    slot_of_row = np.full(r_pad, -1, dtype=np.int32)
    order = np.argsort(np.where(flat >= 0, flat, e_tot), kind="stable")
    nvalid = int(valid.sum())
    order = order[:nvalid]
    exp_sorted = flat[order]
    first = np.concatenate([[0], np.cumsum(counts)])[exp_sorted]
    pos = np.arange(nvalid) - first
    rows = seg_start[exp_sorted] + pos
    row_of[order] = rows
    tok_of_row[rows] = order // kk
    slot_of_row[rows] = order % kk
    tile_expert, tile_row0, tile_rows = [], [], []
    for e in range(e_tot):
        for m0 in range(0, int(counts[e]), tile_m):
            tile_expert.append(e)
            tile_row0.append(int(seg_start[e]) + m0)
            tile_rows.append(min(tile_m, int(counts[e]) - m0))
    return dict(counts=counts, seg_start=seg_start,
                tile_expert=np.array(tile_expert, dtype=np.int32),
                tile_row0=np.array(tile_row0, dtype=np.int32),
                tile_rows=np.array(tile_rows, dtype=np.int32),
                row_of=row_of.reshape(t, kk), tok_of_row=tok_of_row, slot_of_row=slot_of_row)


# --------------------------------------------------------------------------- MoE layer

def _activation(up, gate, alpha, beta, limit, activation_type):
    """reference.py:81-89."""
    if limit is not None:
        up = np.clip(up, -limit, limit)
        gate = np.minimum(gate, limit)
    if activation_type == 10:
        sig = 1.0 / (1.0 + np.exp(-gate.astype(np.float32)))
        return (alpha * np.tanh(gate / alpha) * sig * (beta * np.tanh(up / beta))).astype(np.float32)
    sig = (1.0 / (1.0 + np.exp(-(alpha * gate).astype(np.float32)))).astype(np.float32)
    return (gate * sig * (up + beta)).astype(np.float32)


def moe_expected(p: dict, *, return_intermediates: bool = False):
    """fp32 reference of the whole layer (reference.py:69-92), one expert at a time.

    ``p`` uses the reference's argument names with numpy arrays
    (``hidden_states`` uint8 [T,H/2], ``hidden_states_scale`` uint8 [T,H/16],
    prepared weights, ``topk_ids = (ids, scores)``).  Extensions beyond the
    reference (unpinned): ``output1_scale_scalar`` / ``output1_scale_gate_scalar``
    multiply the up / gate accumulators and ``output2_scale_scalar`` the FC2
    accumulator per expert (the reference never reads them and always passes
    ones); ``num_fused_shared_experts = S`` routes every token to experts
    ``E .. E+S-1`` with weight 1.

    Returns the fp32 values of the bf16 output [T, H].
    """
    a = decode(p["hidden_states"], p["hidden_states_scale"])
    ids, scores = p["topk_ids"]
    ids = np.asarray(ids)
    scores = np.asarray(scores, dtype=np.float32)
    e_routed = int(p["num_experts"])
    shared = int(p.get("num_fused_shared_experts") or 0)
    off = int(p.get("local_expert_offset") or 0)
    t = a.shape[0]
    if shared:
        ids = np.concatenate([ids, np.broadcast_to(np.arange(e_routed, e_routed + shared)[None] + off, (t, shared))], 1)
        scores = np.concatenate([scores, np.ones((t, shared), dtype=np.float32)], 1)
    w1q, w1s = p["gemm1_weights"], p["gemm1_weights_scale"]
    w2q, w2s = p["gemm2_weights"], p["gemm2_weights_scale"]
    n_e = w1q.shape[0]
    s1 = p.get("output1_scale_scalar")
    s1g = p.get("output1_scale_gate_scalar")
    s2 = p.get("output2_scale_scalar")
    limit = p.get("gemm1_clamp_limit")
    act_type = int(p.get("activation_type", 3))
    y = np.zeros_like(a)
    inter = {}
    for e in range(n_e):
        tok, slot = np.nonzero(ids == e + off)
        if len(tok) == 0:
            continue
        w1 = weight_decode(w1q[e], np.asarray(w1s[e]).view(np.uint8), True)
        w2 = weight_decode(w2q[e], np.asarray(w2s[e]).view(np.uint8), False)
        fc1 = a[tok] @ w1.T
        half = fc1.shape[1] // 2
        up, gate = fc1[:, :half], fc1[:, half:]
        if s1 is not None:
            up = up * np.float32(s1[e])
        if s1g is not None:
            gate = gate * np.float32(s1g[e])
        act = _activation(up, gate, np.float32(p["gemm1_alpha"][e]), np.float32(p["gemm1_beta"][e]),
                          None if limit is None else np.float32(limit[e]), act_type)
        actq = nvfp4_qdq(act)
        fc2 = actq @ w2.T
        if s2 is not None:
            fc2 = fc2 * np.float32(s2[e])
        contrib = bf16_round(fc2.astype(np.float32)) * scores[tok, slot, None]
        np.add.at(y, tok, contrib.astype(np.float32))
        if return_intermediates:
            inter[e] = dict(tok=tok, slot=slot, act=act, fc2=fc2)
    out = bf16_round(y)
    return (out, inter) if return_intermediates else out


def dense_expected(a_f32: np.ndarray, b_q: np.ndarray, b_sf: np.ndarray, alpha: float = 1.0) -> np.ndarray:
    """gemm/dense/bf16_nvfp4_gemm/problem/reference.py:10-15: bf16(alpha * A @ decode(B)^T).

    ``a_f32`` holds the values of the A operand (bf16 values, or dequantised
    NVFP4 values when A was quantised on the device); ``b_sf`` is row-major.
    """
    b = decode(b_q, b_sf)
    y = a_f32.astype(np.float32) @ b.T
    return bf16_round((y * np.float32(alpha)).astype(np.float32))


# --------------------------------------------------------------------------- input generation (numpy side)

def matrix_values_from_normal(z: np.ndarray, std: float, role: str) -> np.ndarray:
    """input.py:4-13 applied to an already-drawn standard-normal array ``z``."""
    x = np.asarray(z, dtype=np.float32).copy()
    x *= np.linspace(0.65, 1.35, x.shape[-1], dtype=np.float32)
    if role == "weight":
        x *= np.linspace(0.7, 1.3, x.shape[-2], dtype=np.float32)[:, None]
    x *= np.float32(std)
    return x
