"""Expert-parallel wrapper: experts sharded contiguously over the ranks of one box, tokens data-parallel.

Per step and rank: bucket the (token, slot) routes by destination rank -> dispatch all-to-all of the NVFP4 rows
(payload + scale bytes + local expert id) -> grouped FC1/FC2 on the rows received (top-1 "routing" to the local
expert, weight 1, so the result rows are the per-route bf16 FC2 results of reference.py:91) -> combine all-to-all
of the bf16 rows back to the source -> routing-weighted sum in slot order on the source (b200moe_combine). The
shared expert runs on each rank's own tokens. The reference has no multi-GPU path for this operator; its result
is defined as the single-GPU result. The exchange is `torch.distributed.all_to_all_single` (NCCL over NVLink on
GPUs; the same code runs on gloo for the CPU tests, where the two compute hooks are replaced by a checker).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def build_dispatch(ids: torch.Tensor, experts_per_rank: int, world: int):
    """Index plan of one rank. ids int32 [T, K] hold global expert ids (-1 = no route).

    Returns dict: order (flat route indices sorted by destination rank, stable), send_counts [world] (int64, on
    the ids' device), local_expert (expert id relative to its owner, in send order), pos_of_route [T, K]
    (position of a route in send order, -1 if invalid).
    """
    flat = ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < experts_per_rank * world)
    dest = torch.where(valid, flat // experts_per_rank, torch.full_like(flat, world))
    order = torch.sort(dest, stable=True).indices
    n_valid = int(valid.sum())
    order = order[:n_valid]
    send_counts = torch.bincount(dest[order], minlength=world)[:world]
    local_expert = (flat[order] % experts_per_rank).to(torch.int32)
    pos = torch.full_like(flat, -1, dtype=torch.int32)
    pos[order] = torch.arange(n_valid, dtype=torch.int32, device=ids.device)
    return dict(order=order, send_counts=send_counts, local_expert=local_expert, pos_of_route=pos.view(ids.shape))


def exchange(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> torch.Tensor:
    """Uneven all-to-all of rows: send is [sum(send_counts), ...] in destination order."""
    out = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
    dist.all_to_all_single(out, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


class ExpertParallelMoE:
    """Layer instance on one rank. `expert_rows` and `combine_rows` are the two compute hooks; by default they run
    libb200moe on the current CUDA device."""

    def __init__(self, hidden, intermediate, num_experts, top_k, tokens_per_rank, num_shared_experts=0, group=None,
                 expert_rows=None, combine_rows=None, shared_rows=None, recv_capacity=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("num_experts must be a multiple of the number of ranks")
        self.h, self.i, self.k, self.s = hidden, intermediate, top_k, num_shared_experts
        self.e_local = num_experts // self.world
        self.t = tokens_per_rank
        self.recv_capacity = recv_capacity or self.world * tokens_per_rank * top_k
        self._expert_rows = expert_rows or self._cuda_expert_rows
        self._combine_rows = combine_rows or self._cuda_combine_rows
        self._shared_rows = shared_rows or self._cuda_shared_rows
        self._routed = self._shared = None
        self.profile = False
        # route map memset+3, permute, FC1, FC2, combine for the routed rows (+ the same for the shared expert) + final combine
        self.launches_per_step = 7 * (2 if num_shared_experts else 1) + 1

    # ------------------------------------------------------------------ CUDA hooks
    def _cuda_expert_rows(self, rows_q, rows_sf, local_expert, w1q, w1s, w2q, w2s, out_rows, kw):
        from .ops import MoELayer
        n = rows_q.shape[0]
        if self._routed is None or self._routed.cfg.max_tokens < n:
            if self._routed is not None:
                self._routed.close()
            self._routed = MoELayer(self.h, self.i, self.e_local, 1, max(n, self.recv_capacity))
        ones = torch.ones((n, 1), dtype=torch.float32, device=rows_q.device)
        e = self.e_local
        # top-1 "routing" of every received row to its local expert; FC2 writes the per-route rows straight into out_rows
        self._routed.run(local_expert.view(n, 1), ones, rows_q, rows_sf, w1q[:e], w1s[:e], w2q[:e], w2s[:e], out_rows,
                         direct_rows=True, **{k: (None if v is None else v[:e]) for k, v in kw.items()})

    def _cuda_shared_rows(self, hq, hs, w1q, w1s, w2q, w2s, out_rows, kw):
        from .ops import MoELayer
        if self._shared is None:
            self._shared = MoELayer(self.h, self.i, 0, 0, self.t, num_shared_experts=self.s)
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

    def status(self) -> int:
        code = 0
        for layer in (self._routed, self._shared):
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
        marks = []

        def mark(name):
            if self.profile and dev.type == "cuda":
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        plan = build_dispatch(ids, self.e_local, self.world)
        send_counts_t = plan["send_counts"]
        recv_counts_t = torch.empty_like(send_counts_t)
        dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        send_counts = send_counts_t.tolist()      # host copies: split sizes of the uneven all-to-all
        recv_counts = recv_counts_t.tolist()
        n_send, n_recv = sum(send_counts), sum(recv_counts)
        if n_recv > self.recv_capacity:
            raise RuntimeError(f"rank {self.rank} received {n_recv} rows, capacity is {self.recv_capacity}")
        mark("plan+counts")
        slots = self.k + (1 if self.s else 0)
        rows_all = torch.empty((n_send + t * (1 if self.s else 0), self.h), dtype=torch.bfloat16, device=dev)
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
        tok = plan["order"] // self.k
        rows_q = exchange(hq.index_select(0, tok), send_counts, recv_counts, self.group)
        rows_sf = exchange(hs.index_select(0, tok), send_counts, recv_counts, self.group)
        local_e = exchange(plan["local_expert"], send_counts, recv_counts, self.group)
        mark("dispatch")
        # result rows of the routed experts for the rows received, then back to their sources
        res = torch.empty((n_recv, self.h), dtype=torch.bfloat16, device=dev)
        if n_recv:
            self._expert_rows(rows_q, rows_sf, local_e, w1q, w1s, w2q, w2s, res, kw)
        mark("experts")
        # returned rows first (received in place), the shared experts' rows for the own tokens after them
        dist.all_to_all_single(rows_all[:n_send], res, output_split_sizes=send_counts, input_split_sizes=recv_counts,
                               group=self.group)
        mark("combine_a2a")
        row_of = torch.full((t, slots), -1, dtype=torch.int32, device=dev)
        row_of[:, :self.k] = plan["pos_of_route"]
        w_rows = torch.ones(rows_all.shape[0], dtype=torch.float32, device=dev)
        w_rows[:n_send] = weights.reshape(-1)[plan["order"]]
        if self.s:
            row_of[:, self.k] = n_send + torch.arange(t, dtype=torch.int32, device=dev)
            if side is not None:
                torch.cuda.current_stream(dev).wait_stream(side)
        if out is None:
            out = torch.empty((t, self.h), dtype=torch.bfloat16, device=dev)
            mark("shared")
        self._combine_rows(rows_all, row_of, w_rows, out)
        mark("combine")
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
