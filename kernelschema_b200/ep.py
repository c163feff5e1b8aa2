"""Expert-parallel wrapper: experts sharded contiguously over the ranks of one box, tokens data-parallel.

Per step and rank:
  1. plan: a token goes ONCE to every rank that owns at least one of its experts (not once per route). The
     (token, rank) pairs are ordered by rank, then token; every rank's segment is padded to a multiple of 128 rows;
  2. pack: one message row per pair, `row_bytes(H, K)` bytes: NVFP4 payload | scale bytes | the token's K expert ids
     relative to the destination rank (-1 for experts that live elsewhere, and for padding rows) | its K weights;
  3. ONE dispatch all-to-all of the message rows;
  4. the receiving rank runs the ordinary layer directly on the message buffer (row-strided views of its columns:
     no unpacking copy), i.e. it already applies the routing weights and sums over its own experts: one bf16
     partial row per (token, rank);
  5. combine all-to-all of those partial rows back to the source, received in place;
  6. the source adds the partial rows (and the shared experts' row, computed locally on a side stream under the
     exchange) in rank order with `b200moe_combine` and rounds once to bf16.
On CUDA steps 1-2 are three launches of the library (`b200moe_ep_visits`, the route map of a "plan" layer whose
experts are the ranks, `b200moe_ep_pack`); `plan_messages_torch` is the same plan in torch ops for the CPU tests and as
the checker of the kernels. One host synchronisation per step: the segment sizes for the uneven all-to-all.

A token that visits r ranks costs r rows in each direction instead of top_k: 5.25 instead of 8 on average at
8 ranks with uniform top-8 routing, at most 2 at 2 ranks. The partial rows are rounded to bf16 before they travel, so
the result differs from the single-GPU layer by one extra bf16 rounding per visited rank (well inside the
operator's tolerance). The reference has no multi-GPU path for this operator; its result is defined as the
single-GPU result. The exchange is `torch.distributed.all_to_all_single` (NCCL over NVLink on GPUs; the same code
runs on gloo for the CPU tests, where the compute hooks are replaced by a checker).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

SEGMENT_ROWS = 128


def row_bytes(hidden: int, top_k: int) -> int:
    """Bytes of one dispatch message row (multiple of 16)."""
    return (hidden // 2 + hidden // 16 + 8 * top_k + 15) // 16 * 16


def message_views(msg: torch.Tensor, hidden: int, top_k: int):
    """Column views (no copies) of a message buffer uint8 [n, row_bytes]: payload, scales, local ids, weights."""
    q, sf = hidden // 2, hidden // 16
    words = msg.view(torch.int32)
    c0 = (q + sf) // 4
    return msg[:, :q], msg[:, q:q + sf], words[:, c0:c0 + top_k], words[:, c0 + top_k:c0 + 2 * top_k].view(torch.float32)


def build_dispatch(ids: torch.Tensor, experts_per_rank: int, world: int):
    """Index plan of one rank. ids int32 [T, K] hold global expert ids (-1 = no route).

    Returns dict: tok (token of every (rank, token) pair to send, sorted by rank then token), dest (its rank),
    send_counts [world] (int64, on the ids' device), local_ids int32 [n, K] (the token's expert ids relative to the
    destination rank, -1 for experts that live elsewhere), pos_of_pair int32 [T, world] (position of the pair in
    send order, -1 if the token does not visit that rank).
    """
    t, k = ids.shape
    idl = ids.to(torch.int64)
    valid = (idl >= 0) & (idl < experts_per_rank * world)
    dest_of_route = torch.where(valid, idl // experts_per_rank, torch.full_like(idl, -1))          # [T, K]
    ranks = torch.arange(world, device=ids.device)
    visits = (dest_of_route.unsqueeze(-1) == ranks).any(dim=1)                                     # [T, world]
    pairs = visits.t().nonzero()                                                                   # sorted by rank, then token
    dest, tok = pairs[:, 0], pairs[:, 1]
    send_counts = visits.sum(0)
    on_dest = dest_of_route[tok] == dest.unsqueeze(-1)
    local_ids = torch.where(on_dest, idl[tok] % experts_per_rank, torch.full_like(idl[tok], -1)).to(torch.int32)
    pos = torch.full((world, t), -1, dtype=torch.int32, device=ids.device)
    pos[dest, tok] = torch.arange(tok.numel(), dtype=torch.int32, device=ids.device)
    return dict(tok=tok, dest=dest, send_counts=send_counts, local_ids=local_ids, pos_of_pair=pos.t().contiguous())


def plan_messages_torch(ids, weights, hq, hs, experts_per_rank: int, world: int, shared_slot: bool = False):
    """The dispatch plan and message buffer of one rank in torch ops (any device). Returns (msg uint8 [n_send,
    row_bytes], seg_rows list[int] per destination rank, row_of int32 [T, world (+1)]); with ``shared_slot`` the last
    column of row_of points at row n_send + t, where the caller puts the shared experts' row of token t."""
    t, k = ids.shape
    h = hq.shape[1] * 2
    plan = build_dispatch(ids, experts_per_rank, world)
    counts = plan["send_counts"]
    padded = (counts + SEGMENT_ROWS - 1) // SEGMENT_ROWS * SEGMENT_ROWS
    seg_start = torch.cumsum(padded, 0) - padded
    first_pair = torch.cumsum(counts, 0) - counts
    dest, tok = plan["dest"], plan["tok"]
    position = seg_start[dest] + torch.arange(tok.numel(), device=ids.device) - first_pair[dest]
    seg_rows = [int(v) for v in padded.tolist()]
    n_send = sum(seg_rows)
    msg = torch.zeros((n_send, row_bytes(h, k)), dtype=torch.uint8, device=ids.device)
    m_q, m_sf, m_ids, m_w = message_views(msg, h, k)
    m_ids.fill_(-1)
    m_q[position] = hq.view(torch.uint8)[tok]
    m_sf[position] = hs.view(torch.uint8)[tok]
    m_ids[position] = plan["local_ids"]
    m_w[position] = weights[tok].to(torch.float32)
    row_of = torch.full((t, world + int(shared_slot)), -1, dtype=torch.int32, device=ids.device)
    row_of[tok, dest] = position.to(torch.int32)
    if shared_slot:
        row_of[:, world] = n_send + torch.arange(t, dtype=torch.int32, device=ids.device)
    return msg, seg_rows, row_of


def exchange(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> torch.Tensor:
    """Uneven all-to-all of rows: send is [sum(send_counts), ...] in destination order."""
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(out, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


class CudaPlanner:
    """`plan_messages_torch` in three launches of the library: `b200moe_ep_visits`, the route map of a "plan" layer
    whose experts are the ranks (plus one shared slot), `b200moe_ep_pack`. Buffers are allocated once."""

    def __init__(self, hidden, top_k, experts_per_rank, world, max_tokens, shared_slot, device, message_buffer=True):
        from .ops import MoELayer
        self.h, self.k, self.e_local, self.world = hidden, top_k, experts_per_rank, world
        # the plan layer's GEMM operands are never used, so it gets the smallest legal sizes
        self.layer = MoELayer(256, 256, world, world, max_tokens, num_shared_experts=1 if shared_slot else 0)
        self.ws = self.layer.workspace()
        self.slots = torch.empty((max_tokens, world), dtype=torch.int32, device=device)
        self.msg = (torch.empty((self.ws["row_capacity"], row_bytes(hidden, top_k)), dtype=torch.uint8, device=device)
                    if message_buffer else None)     # the peer-memory transport packs straight into the destinations' buffers

    def plan(self, ids, weights, hq, hs):
        """Returns (msg buffer, segment rows per rank as a device tensor, row_of [T, world (+1)], row weights (all 1) for
        `b200moe_combine`); the first sum(segment rows) rows of msg are the messages."""
        from .ops import ep_pack, ep_visits
        t = ids.shape[0]
        slots = self.slots[:t]
        ep_visits(ids, self.e_local, self.world, slots)
        self.layer.route_map(slots, None)
        ep_pack(self.layer, hq, hs, ids, weights, self.e_local, self.msg)
        seg_start = self.ws["seg_start"]
        return self.msg, seg_start[1:self.world + 1] - seg_start[:self.world], self.ws["row_of"][:t], self.ws["weight_of_row"]


class PeerExchange:
    """Buffers of the peer-memory exchange of one rank (see csrc/ep_exchange.cu) and the address tables of its peers.

    One allocation per rank, the same layout everywhere, every region twice (step parity): control block | receive buffer
    of world regions x seg_len message rows | return buffer of world * seg_len (+ tokens_per_rank shared-expert) bf16 rows.
    The 64-byte handles travel once through `torch.distributed.all_gather_object`; a group of one rank uses its own
    buffer as its only peer (the whole device path on a single GPU)."""

    def __init__(self, hidden, top_k, tokens_per_rank, shared_rows, group, device):
        import ctypes as C
        from . import _lib
        from .ops import _from_device_ptr
        self.lib = _lib.load()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _lib.EP_MAX_RANKS:
            raise ValueError(f"at most {_lib.EP_MAX_RANKS} ranks")
        self.h, self.k = hidden, top_k
        self.seg_len = (tokens_per_rank + SEGMENT_ROWS - 1) // SEGMENT_ROWS * SEGMENT_ROWS
        self.row_bytes = row_bytes(hidden, top_k)
        self.slots = self.world * self.seg_len
        self.shared_base = self.slots
        self.ret_rows = self.slots + (tokens_per_rank if shared_rows else 0)
        al = lambda n: (n + 1023) // 1024 * 1024
        ctrl_b, recv_b, ret_b = al(_lib.EP_CTRL_INTS * 4), al(self.slots * self.row_bytes), al(self.ret_rows * hidden * 2)
        self.off_ctrl = [0, ctrl_b]
        self.off_counter = 2 * ctrl_b
        self.off_recv = [2 * ctrl_b + 1024, 2 * ctrl_b + 1024 + recv_b]
        self.off_ret = [self.off_recv[1] + recv_b, self.off_recv[1] + recv_b + ret_b]
        self.bytes = self.off_ret[1] + ret_b
        base, handle = C.c_void_p(), C.create_string_buffer(64)
        _lib.check(self.lib.b200moe_ep_shared_alloc(self.bytes, C.byref(base), handle), "b200moe_ep_shared_alloc")
        self.base = base.value
        handles = [None] * self.world
        dist.all_gather_object(handles, (self.rank, handle.raw), group=group)
        self.peer_base, self._opened = [None] * self.world, []
        for r, raw in handles:
            if r == self.rank:
                self.peer_base[r] = self.base
            else:
                ptr = C.c_void_p()
                _lib.check(self.lib.b200moe_ep_shared_open(C.create_string_buffer(raw, 64), C.byref(ptr)), "b200moe_ep_shared_open")
                self.peer_base[r] = ptr.value
                self._opened.append(ptr.value)
        self.peers = []
        for p in (0, 1):
            pe = _lib.EpPeers(world=self.world, rank=self.rank)
            for r in range(self.world):
                pe.recv[r] = self.peer_base[r] + self.off_recv[p] + self.rank * self.seg_len * self.row_bytes
                pe.ctrl[r] = self.peer_base[r] + self.off_ctrl[p]
                pe.ret[r] = self.peer_base[r] + self.off_ret[p]
            self.peers.append(pe)
        dev = device.index if device.index is not None else torch.cuda.current_device()
        self.recv = [_from_device_ptr(self.base + self.off_recv[p], self.slots * self.row_bytes, torch.uint8, (self.slots, self.row_bytes), dev)
                     for p in (0, 1)]
        self.ret = [_from_device_ptr(self.base + self.off_ret[p], self.ret_rows * hidden * 2, torch.bfloat16, (self.ret_rows, hidden), dev)
                    for p in (0, 1)]
        self.ctrl_ptr = [self.base + self.off_ctrl[p] for p in (0, 1)]
        self.counter_ptr = self.base + self.off_counter
        self.epoch = 0
        dist.barrier(group=group)          # nobody writes a peer before every rank has mapped every buffer

    def close(self):
        for ptr in self._opened:
            self.lib.b200moe_ep_shared_close(ptr)
        self._opened = []
        if self.base:
            self.lib.b200moe_ep_shared_free(self.base)
            self.base = None


class ExpertParallelMoE:
    """Layer instance on one rank. `expert_rows`, `shared_rows` and `combine_rows` are the compute hooks; by default
    they run libb200moe on the current CUDA device. `planner` is "cuda" (library kernels; default on a GPU) or
    "torch" (`plan_messages_torch`; the only choice on CPU)."""

    def __init__(self, hidden, intermediate, num_experts, top_k, tokens_per_rank, num_shared_experts=0, group=None,
                 expert_rows=None, combine_rows=None, shared_rows=None, recv_capacity=None, planner=None, micro_batches=None,
                 sm_margin=None, transport=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("num_experts must be a multiple of the number of ranks")
        self.h, self.i, self.k, self.s = hidden, intermediate, top_k, num_shared_experts
        self.e_local = num_experts // self.world
        self.t = tokens_per_rank
        seg = lambda n: (n + SEGMENT_ROWS - 1) // SEGMENT_ROWS * SEGMENT_ROWS
        # every token of every rank, at worst (each source's segment padded to 128 rows)
        self.recv_capacity = recv_capacity or self.world * seg(tokens_per_rank)
        self._expert_rows = expert_rows or self._cuda_expert_rows
        self._combine_rows = combine_rows or self._cuda_combine_rows
        self._shared_rows = shared_rows or self._cuda_shared_rows
        self.planner = planner
        # Optional: two micro-batches (token halves) pipeline the exchanges under the expert GEMMs (dispatch of the second
        # half beside the experts of the first, the return of the first beside the experts of the second); the persistent
        # GEMM grids then stay off `sm_margin` SMs so that the collective's kernels find room next to them. Measured on
        # B200s it does not pay (2 ranks: 3.78 against 3.22 ms; 8 ranks: 5.37 against 5.16 ms per step): every half re-reads
        # this rank's expert weights and the GEMMs lose the SMs they leave free. Off unless asked for.
        self.micro_batches = micro_batches or 1
        # "p2p": rows and results travel as peer stores of this library's kernels, flags instead of host synchronisation
        # (CUDA only; the default there when no hook replaces the compute). "collective": torch.distributed all-to-all
        # (NCCL, or gloo on CPU).
        self.transport = transport
        self._px = None
        self.sm_margin = (sm_margin if sm_margin is not None else 16) if self.micro_batches > 1 else 0
        self._routed = self._shared = self._plan = None
        self._plans = {}
        self.profile = False
        # quantise/route launches are the caller's; here: plan (visits + route map + pack), then (route map + permute +
        # FC1 + FC2 + combine) for the received tokens, the same for the shared experts, and the final combine
        # (peer-memory transport: visits + route map + dispatch, two flag waits and one flag post instead of the pack)
        self.launches_per_step = 3 + 5 * (2 if num_shared_experts else 1) + 1 + 3

    # ------------------------------------------------------------------ CUDA hooks
    def _cuda_expert_rows(self, rows_q, rows_sf, local_ids, weights, w1q, w1s, w2q, w2s, out_rows, kw):
        from .ops import MoELayer
        n = rows_q.shape[0]
        if self._routed is None or self._routed.cfg.max_tokens < n:
            if self._routed is not None:
                self._routed.close()
            self._routed = MoELayer(self.h, self.i, self.e_local, self.k, max(n, self.recv_capacity), sm_margin=self.sm_margin)
        e = self.e_local
        self._routed.run(local_ids, weights, rows_q, rows_sf, w1q[:e], w1s[:e], w2q[:e], w2s[:e], out_rows,
                         **{k: (None if v is None else v[:e]) for k, v in kw.items()})

    def _cuda_shared_layer(self):
        from .ops import MoELayer
        if self._shared is None:
            self._shared = MoELayer(self.h, self.i, 0, 0, self.t, num_shared_experts=self.s, sm_margin=self.sm_margin)
        return self._shared

    def _cuda_shared_rows(self, hq, hs, w1q, w1s, w2q, w2s, out_rows, kw):
        self._cuda_shared_layer()
        e = self.e_local
        self._shared.run(None, None, hq, hs, w1q[e:], w1s[e:], w2q[e:], w2s[e:], out_rows,
                         **{k: (None if v is None else v[e:]) for k, v in kw.items()})

    def _cuda_combine_rows(self, rows, row_of, weight_of_row, out):
        from .ops import combine
        combine(rows, row_of, weight_of_row, out)

    def _side_stream(self, dev):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=dev)
        return self._side

    def close(self):
        """Frees the peer-exchange buffers (every rank must have finished its last step: barrier first)."""
        if self._px is not None:
            self._px.close()
            self._px = None

    def status(self) -> int:
        code = 0
        for layer in [self._routed, self._shared, self._plan.layer if self._plan else None] + [p.layer for p in self._plans.values()]:
            if layer is not None:
                code = code or layer.status()
        return code

    # ------------------------------------------------------------------ forward
    def forward(self, ids, weights, hq, hs, w1q, w1s, w2q, w2s, out=None, **kw):
        """ids/weights [T, K] with global expert ids; hq uint8 [T, H/2]; hs uint8 [T, H/16]; the weight tensors hold
        this rank's experts followed by the shared experts. kw: per-expert fp32 vectors (alpha, beta, limit, scale_up,
        scale_gate, scale_out) for the same experts. Returns bf16 [T, H]."""
        dev = hq.device
        t = hq.shape[0]
        transport = self.transport or ("p2p" if dev.type == "cuda" and self.micro_batches == 1 else "collective")
        if transport == "p2p":
            return self._forward_p2p(ids, weights, hq, hs, w1q, w1s, w2q, w2s, out, kw)
        if self.micro_batches > 1 and dev.type == "cuda" and t >= 2 * SEGMENT_ROWS:
            return self._forward_pipelined(ids, weights, hq, hs, w1q, w1s, w2q, w2s, out, kw)
        marks = []

        def mark(name):
            if self.profile and dev.type == "cuda":
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        planner = self.planner or ("cuda" if dev.type == "cuda" else "torch")
        if planner == "cuda":
            if self._plan is None or self._plan.layer.cfg.max_tokens < t:
                self._plan = CudaPlanner(self.h, self.k, self.e_local, self.world, max(t, self.t), bool(self.s), dev)
            msg, seg_rows_t, row_of, w_rows = self._plan.plan(ids, weights, hq, hs)
            seg_rows_t = seg_rows_t.to(torch.int64)
        else:
            msg, seg_rows, row_of = plan_messages_torch(ids, weights, hq, hs, self.e_local, self.world, bool(self.s))
            seg_rows_t = torch.tensor(seg_rows, dtype=torch.int64, device=dev)
            w_rows = None
        recv_rows_t = torch.empty_like(seg_rows_t)
        dist.all_to_all_single(recv_rows_t, seg_rows_t, group=self.group)
        sizes = torch.cat([seg_rows_t, recv_rows_t]).tolist()      # the step's one host copy: split sizes
        send_counts, recv_counts = sizes[:self.world], sizes[self.world:]
        n_send, n_recv = sum(send_counts), sum(recv_counts)
        if n_recv > self.recv_capacity:
            raise RuntimeError(f"rank {self.rank} received {n_recv} rows, capacity is {self.recv_capacity}")
        mark("plan+counts")
        shared_slot = 1 if self.s else 0
        rows_all = torch.empty((n_send + t * shared_slot, self.h), dtype=torch.bfloat16, device=dev)
        side = None
        if self.s:
            # the shared experts only need this rank's own tokens: run them on a side stream under the exchange
            if dev.type == "cuda":
                side = self._side_stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    self._shared_rows(hq, hs, w1q, w1s, w2q, w2s, rows_all[n_send:], kw)
            else:
                self._shared_rows(hq, hs, w1q, w1s, w2q, w2s, rows_all[n_send:], kw)
        got = exchange(msg[:n_send], send_counts, recv_counts, self.group)
        mark("dispatch")
        # one partial row per row received: routing-weighted sum over this rank's experts, rounded to bf16
        res = torch.empty((n_recv, self.h), dtype=torch.bfloat16, device=dev)
        if n_recv:
            rows_q, rows_sf, ids_recv, w_recv = message_views(got, self.h, self.k)
            self._expert_rows(rows_q, rows_sf, ids_recv, w_recv, w1q, w1s, w2q, w2s, res, kw)
        mark("experts")
        # partial rows return to their sources (received in place), the shared experts' rows come after them
        dist.all_to_all_single(rows_all[:n_send], res, output_split_sizes=send_counts, input_split_sizes=recv_counts,
                               group=self.group)
        mark("combine_a2a")
        if w_rows is None:
            w_rows = torch.ones(rows_all.shape[0], dtype=torch.float32, device=dev)
        if self.s:
            if side is not None:
                torch.cuda.current_stream(dev).wait_stream(side)
            mark("shared")
        if out is None:
            out = torch.empty((t, self.h), dtype=torch.bfloat16, device=dev)
        self._combine_rows(rows_all, row_of, w_rows, out)
        mark("combine")
        if marks:
            self._pending_marks = marks
        return out

    def _forward_p2p(self, ids, weights, hq, hs, w1q, w1s, w2q, w2s, out, kw):
        """One step over peer memory: no collective call, no host synchronisation, no allocation after the first step.
        plan -> dispatch kernel (rows, sizes and flags into the peers' buffers) -> [shared experts on a side stream] ->
        wait for every source -> the layer over the receive buffer, its combine pass writing into the sources' return
        buffers -> return flags -> wait for every destination -> slot-ordered combine of the returned rows."""
        from . import _lib
        from .ops import MoELayer, _stream, ep_visits
        dev = hq.device
        t = hq.shape[0]
        if t > self.t:
            raise ValueError(f"{t} tokens, the exchange buffers were sized for {self.t} per rank")
        if self._px is None:
            # every allocation of the step first, the exchange buffers last: their set-up ends with a barrier, so all ranks
            # enter their first step together and the bounded flag waits only ever cover the step itself
            seg_len = (self.t + SEGMENT_ROWS - 1) // SEGMENT_ROWS * SEGMENT_ROWS
            self._plan = CudaPlanner(self.h, self.k, self.e_local, self.world, self.t, bool(self.s), dev, message_buffer=False)
            self._routed = MoELayer(self.h, self.i, self.e_local, self.k, self.world * seg_len, sm_margin=self.sm_margin)
            self._scratch_out = torch.empty((1, self.h), dtype=torch.bfloat16, device=dev)
            if self.s:
                self._cuda_shared_layer()
            torch.cuda.synchronize(dev)
            self._px = PeerExchange(self.h, self.k, self.t, bool(self.s), self.group, dev)
            assert self._px.slots == self.world * seg_len
        px, plan, lib = self._px, self._plan, self._px.lib
        px.epoch += 1
        epoch, p = px.epoch, px.epoch & 1
        marks = []

        def mark(name):
            if self.profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        hq = hq.contiguous()
        hs8 = hs.contiguous().view(torch.uint8)
        ids, weights = ids.contiguous(), weights.contiguous()
        ret = px.ret[p]
        slots = plan.slots[:t]
        ep_visits(ids, self.e_local, self.world, slots)
        plan.layer.route_map(slots, None)
        _lib.check(lib.b200moe_ep_dispatch(plan.layer._h, hq.data_ptr(), hs8.data_ptr(), ids.data_ptr(), weights.data_ptr(), t, self.h,
                                           self.k, self.e_local, px.row_bytes, px.peers[p], epoch, int(bool(self.s)), px.shared_base,
                                           px.counter_ptr, _stream()), "b200moe_ep_dispatch")
        side = None
        if self.s:
            # The shared experts need nothing but this rank's own tokens and write fixed rows of the return buffer: they run
            # on a side stream from the moment this rank's rows are on their way, under the wait for the peers' rows. Started
            # before the dispatch their GEMM grids hold every SM and the dispatch, which all peers wait for, queues behind
            # them (8 ranks: 0.74 ms until the rows had left).
            side = self._side_stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self._shared_rows(hq, hs8, w1q, w1s, w2q, w2s, ret[px.shared_base:px.shared_base + t], kw)
        mark("plan+dispatch")
        _lib.check(lib.b200moe_ep_wait(self._routed._h, px.ctrl_ptr[p] + 4 * _lib.EP_FLAG_DISPATCH, self.world, epoch, _stream()),
                   "b200moe_ep_wait")
        mark("wait_rows")
        rows_q, rows_sf, ids_recv, w_recv = message_views(px.recv[p], self.h, self.k)
        e = self.e_local
        self._routed.run_ep(px.peers[p], px.ctrl_ptr[p], px.seg_len, ids_recv, w_recv, rows_q, rows_sf, w1q[:e], w1s[:e], w2q[:e],
                            w2s[:e], self._scratch_out, **{k: (None if v is None else v[:e]) for k, v in kw.items()})
        _lib.check(lib.b200moe_ep_post(px.peers[p], _lib.EP_FLAG_RETURN, epoch, _stream()), "b200moe_ep_post")
        mark("experts+return")
        _lib.check(lib.b200moe_ep_wait(self._routed._h, px.ctrl_ptr[p] + 4 * _lib.EP_FLAG_RETURN, self.world, epoch, _stream()),
                   "b200moe_ep_wait")
        if side is not None:
            torch.cuda.current_stream(dev).wait_stream(side)
        mark("wait_results")
        if out is None:
            out = torch.empty((t, self.h), dtype=torch.bfloat16, device=dev)
        self._combine_rows(ret, plan.ws["row_of"][:t], plan.ws["weight_of_row"], out)
        mark("combine")
        if marks:
            self._pending_marks = marks
        return out

    def _forward_pipelined(self, ids, weights, hq, hs, w1q, w1s, w2q, w2s, out, kw):
        """The same steps on two token halves, interleaved on a compute stream (the caller's) and a communication
        stream: plan(A), plan(B) | dispatch(A), dispatch(B) | experts(A) beside dispatch(B) | return(A) beside
        experts(B) | return(B) | the two final combines. Every rank issues its collectives in the same order."""
        dev = hq.device
        t = hq.shape[0]
        main = torch.cuda.current_stream(dev)
        if getattr(self, "_comm", None) is None:
            self._comm = torch.cuda.Stream(device=dev)
        comm = self._comm
        marks = []

        def mark(name):
            if self.profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        t0 = (t // 2 + SEGMENT_ROWS - 1) // SEGMENT_ROWS * SEGMENT_ROWS
        bounds = [(0, t0), (t0, t)]
        if out is None:
            out = torch.empty((t, self.h), dtype=torch.bfloat16, device=dev)
        mbs = []
        for i, (lo, hi) in enumerate(bounds):          # plans and the (tiny) size exchanges of both halves first
            planner = self._plans.get(i)
            if planner is None or planner.layer.cfg.max_tokens < hi - lo:
                planner = self._plans[i] = CudaPlanner(self.h, self.k, self.e_local, self.world, max(hi - lo, t0), bool(self.s), dev)
            msg, seg_rows_t, row_of, w_rows = planner.plan(ids[lo:hi], weights[lo:hi], hq[lo:hi], hs[lo:hi])
            seg_rows_t = seg_rows_t.to(torch.int64)
            recv_rows_t = torch.empty_like(seg_rows_t)
            dist.all_to_all_single(recv_rows_t, seg_rows_t, group=self.group)
            mbs.append(dict(lo=lo, hi=hi, msg=msg, sizes=torch.cat([seg_rows_t, recv_rows_t]), row_of=row_of, w_rows=w_rows))
        for mb in mbs:
            sizes = mb["sizes"].tolist()
            mb["send"], mb["recv"] = sizes[:self.world], sizes[self.world:]
            mb["n_send"], mb["n_recv"] = sum(mb["send"]), sum(mb["recv"])
            if mb["n_recv"] > self.recv_capacity:
                raise RuntimeError(f"rank {self.rank} received {mb['n_recv']} rows, capacity is {self.recv_capacity}")
            mb["rows_all"] = torch.empty((mb["n_send"] + (mb["hi"] - mb["lo"]) * (1 if self.s else 0), self.h), dtype=torch.bfloat16,
                                         device=dev)
        mark("plan+counts")
        side = None
        if self.s:                                        # shared experts: own tokens only, on a third stream
            side = self._side_stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for mb in mbs:
                    lo, hi = mb["lo"], mb["hi"]
                    mb["rows_all"].record_stream(side)
                    self._shared_rows(hq[lo:hi], hs[lo:hi], w1q, w1s, w2q, w2s, mb["rows_all"][mb["n_send"]:], kw)
        comm.wait_stream(main)
        with torch.cuda.stream(comm):
            for mb in mbs:
                mb["got"] = exchange(mb["msg"][:mb["n_send"]], mb["send"], mb["recv"], self.group)
                mb["got"].record_stream(main)
                mb["ev_dispatch"] = torch.cuda.Event()
                mb["ev_dispatch"].record(comm)
        for mb in mbs:
            main.wait_event(mb["ev_dispatch"])
            mb["res"] = torch.empty((mb["n_recv"], self.h), dtype=torch.bfloat16, device=dev)
            if mb["n_recv"]:
                rows_q, rows_sf, ids_recv, w_recv = message_views(mb["got"], self.h, self.k)
                self._expert_rows(rows_q, rows_sf, ids_recv, w_recv, w1q, w1s, w2q, w2s, mb["res"], kw)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev)
                mb["res"].record_stream(comm)
                mb["rows_all"].record_stream(comm)
                dist.all_to_all_single(mb["rows_all"][:mb["n_send"]], mb["res"], output_split_sizes=mb["send"],
                                       input_split_sizes=mb["recv"], group=self.group)
                mb["ev_return"] = torch.cuda.Event()
                mb["ev_return"].record(comm)
        mark("experts(+exchanges)")
        if side is not None:
            main.wait_stream(side)
        for mb in mbs:
            main.wait_event(mb["ev_return"])
            self._combine_rows(mb["rows_all"], mb["row_of"], mb["w_rows"], out[mb["lo"]:mb["hi"]])
        mark("return+combine")
        if marks:
            self._pending_marks = marks
        return out

    def stage_ms(self):
        """Durations (ms) between the profiling marks of the last forward (set `profile = True` first); synchronises."""
        marks = getattr(self, "_pending_marks", None)
        if not marks:
            return {}
        marks[-1][1].synchronize()
        return {marks[i + 1][0]: marks[i][1].elapsed_time(marks[i + 1][1]) for i in range(len(marks) - 1)}
