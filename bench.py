"""Benchmark of the NVFP4 MoE layer hot path on B200 (one JSON line on stdout, printed by rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload dsv3|qwen3|c1] [--impl reference]

A step = one pass of the whole layer over one batch of synthetic tokens: bf16 activations -> NVFP4 quantiser ->
router logits + top-k/softmax -> route map -> permute -> FC1 + SwiGLU + requantise -> FC2 -> weighted combine
-> bf16 output. `value` times it with the bf16 inputs already resident in HBM; `e2e` times the same call chain
with pinned HOST buffers (host->device copy of the tokens and device->host copy of the output inside the timed
region). With --gpus N > 1 (launched under torchrun) experts are sharded over the ranks and tokens travel by
NCCL all-to-all (weak scaling: every rank brings its own T tokens).

`--impl reference` times the CPU restatement of the reference operator's fp32 dequantise-then-matmul path
(oracle/) on the host cores, on a bounded sample of the same geometry.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: hidden, intermediate, routed experts, top-k, shared experts, tokens per rank, zipf alpha (0 = uniform)
    "dsv3": dict(h=7168, i=2048, e=256, k=8, s=1, t=8192, zipf=1.2,
                 label="deepseek_v3_moe_layer_T8192_E256_top8_shared1_zipf1.2"),
    "qwen3": dict(h=2048, i=768, e=128, k=8, s=0, t=16384, zipf=0.0, label="qwen3_30b_a3b_moe_layer_T16384_E128_top8"),
    "c1": dict(h=1024, i=512, e=8, k=2, s=0, t=256, zipf=0.0, label="small_moe_layer_T256_E8_top2"),
}
ACT_GLOBAL_SCALE = 2.0 ** -9        # static (calibrated) activation global scale: amax 6 -> 6/(6*448) ~ 2^-8.8, as a power of two
FP4_NOMINAL_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one FC1 launch, from the ncu captures summarised under profiles/
# (workload -> bytes); null for workloads that were not captured.
FC1_DRAM_TRAFFIC = {"dsv3": 4966850048 + 79877632, "qwen3": 386940416 + 49309952}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# --------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) every 5 ms while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.sm, self.power, self.reasons = [], [], set()
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = pynvml
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:   # NVML missing: report it, never fail the benchmark
            self.err = repr(exc)
            return
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.005)

    def stop(self):
        if self._thread is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["NVML unavailable: " + getattr(self, "err", "?")])
        self._stop.set()
        self._thread.join(timeout=2)
        if not self.sm:
            return dict(sm_mhz=None, sm_max_mhz=self.sm_max, reasons=["no samples"])
        return dict(sm_mhz=float(np.median(self.sm)), sm_min_mhz=float(min(self.sm)), sm_max_mhz=self.sm_max,
                    power_w_max=float(max(self.power)), samples=len(self.sm), reasons=sorted(self.reasons))


# --------------------------------------------------------------------------------------------- synthetic layer
def build_layer(wl, rank, world, device, global_scales=True):
    """Random-init weights of the named geometry, quantised on the device with per-expert global scales
    amax/(6*448); the routed experts are sharded contiguously over the ranks, the shared expert is replicated."""
    import torch
    import kernelschema_b200 as ks
    h, i, e, s = wl["h"], wl["i"], wl["e"], wl["s"]
    e_local = e // world
    etot = e_local + s
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    w1q = torch.empty((etot, 2 * i, h // 2), dtype=torch.uint8, device=device)
    w1s = torch.empty((etot, 2 * i, h // 16), dtype=torch.uint8, device=device)
    w2q = torch.empty((etot, h, i // 2), dtype=torch.uint8, device=device)
    w2s = torch.empty((etot, h, i // 16), dtype=torch.uint8, device=device)
    g1 = torch.empty(etot, dtype=torch.float32, device=device)
    g2 = torch.empty(etot, dtype=torch.float32, device=device)
    for j in range(etot):
        if j >= e_local:   # shared expert: same values on every rank
            gen_j = torch.Generator(device=device).manual_seed(7)
        else:
            gen_j = gen
        w = (torch.randn((2 * i, h), device=device, generator=gen_j) * 0.02).to(torch.bfloat16)
        g1[j] = w.float().abs().max() / (6.0 * 448.0) if global_scales else 1.0
        q, sf = ks.nvfp4_quantize(w, float(g1[j]), tiled_scales=True)
        w1q[j] = q
        w1s[j] = sf.reshape(2 * i, h // 16)
        w = (torch.randn((h, i), device=device, generator=gen_j) * 0.02).to(torch.bfloat16)
        g2[j] = w.float().abs().max() / (6.0 * 448.0) if global_scales else 1.0
        q, sf = ks.nvfp4_quantize(w, float(g2[j]), tiled_scales=True)
        w2q[j] = q
        w2s[j] = sf.reshape(h, i // 16)
    gen0 = torch.Generator(device=device).manual_seed(5)
    gate_w = (torch.randn((e, h), device=device, generator=gen0) * 0.02).to(torch.bfloat16)
    bias = None
    if wl["zipf"] > 0:
        perm = torch.randperm(e, device=device, generator=gen0)
        bias = torch.log(1.0 / (perm.float() + 1.0) ** wl["zipf"])
    return dict(w1q=w1q, w1s=w1s, w2q=w2q, w2s=w2s, scale_fc1=(g1 * ACT_GLOBAL_SCALE).contiguous(), scale_fc2=g2.contiguous(),
                gate_w=gate_w, bias=bias, e_local=e_local)


def make_step(wl, L, world, device):
    """Returns step(x_bf16_device) -> out_bf16_device, the launch count per step, and the route statistics."""
    import torch
    import kernelschema_b200 as ks
    h, i, k, s, t = wl["h"], wl["i"], wl["k"], wl["s"], wl["t"]
    if world == 1:
        layer = ks.MoELayer(h, i, L["e_local"], k, t, num_shared_experts=s, tile_n=int(os.environ.get("B200MOE_TILE_N", "0")))
        out = torch.empty((t, h), dtype=torch.bfloat16, device=device)

        def step(x, out=out):
            hq, hs = ks.nvfp4_quantize(x, ACT_GLOBAL_SCALE)
            ids, w = ks.route_topk(ks.router_logits(x, L["gate_w"]), k, L["bias"])
            layer.run(ids, w, hq, hs.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], out, scale_up=L["scale_fc1"],
                      scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
            return out, ids

        return step, layer, 10
    from kernelschema_b200.ep import ExpertParallelMoE
    ep = ExpertParallelMoE(h, i, wl["e"], k, t, num_shared_experts=s)

    def step(x, out=None):
        hq, hs = ks.nvfp4_quantize(x, ACT_GLOBAL_SCALE)
        ids, w = ks.route_topk(ks.router_logits(x, L["gate_w"]), k, L["bias"])
        out = ep.forward(ids, w, hq, hs.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], out=out,
                         scale_up=L["scale_fc1"], scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
        return out, ids

    return step, ep, ep.launches_per_step + 3


def layer_flops(wl, valid_routes, tokens):
    return 6.0 * valid_routes * wl["i"] * wl["h"] + 6.0 * tokens * wl["s"] * wl["i"] * wl["h"]


# --------------------------------------------------------------------------------------------- CPU arm
def cpu_sample_case(wl):
    """Bounded sample of the workload for the host cores: same hidden / intermediate sizes, 8 routed experts
    (+ the shared one), 256 tokens, top-2."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import make_moe_case
    e, k, t = (8, 2, 256) if wl["e"] >= 8 else (wl["e"], wl["k"], wl["t"])
    p = make_moe_case(0, t, wl["h"], wl["i"], e, k, shared=wl["s"], global_scales=True)
    valid = int((p["topk_ids"][0] >= 0).sum())
    flops = 6.0 * valid * wl["i"] * wl["h"] + 6.0 * t * wl["s"] * wl["i"] * wl["h"]
    desc = f"H={wl['h']} I={wl['i']} experts={e}+{wl['s']} shared, T={t}, top-{k}: {flops / 1e9:.1f} GFLOP per pass"
    return p, flops, t, desc


def time_cpu(wl, steps, warmup):
    from oracle import nvfp4_oracle as o
    p, flops, t, desc = cpu_sample_case(wl)
    for _ in range(warmup):
        o.moe_expected(p)
    t0 = time.perf_counter()
    for _ in range(steps):
        o.moe_expected(p)
    dt = (time.perf_counter() - t0) / steps
    return dict(tflops=flops / dt / 1e12, tokens_per_s=t / dt, seconds=dt, sample=desc, cores=os.cpu_count())


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu(wl, max(1, args.steps), max(0, min(args.warmup, 1)))
    line = dict(impl="reference", metric="nvfp4_moe_layer_tflops", value=r["tflops"], unit="TFLOP/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=r["seconds"] * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", tokens_per_s=r["tokens_per_s"],
                config=dict(workload=wl["label"], sample=r["sample"]),
                cpu_baseline=dict(value=r["tflops"], unit="TFLOP/s", cores=r["cores"], kind="port", sample=r["sample"]),
                e2e=dict(value=r["tflops"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------- GPU arm
def run_gpu(args, wl):
    import torch
    import torch.distributed as dist
    import kernelschema_b200 as ks   # noqa: F401  (fails loudly if the library is missing)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if wl["e"] % world:
        raise SystemExit("experts must divide evenly over the ranks")
    L = build_layer(wl, rank, world, device)
    step, owner, launches = make_step(wl, L, world, device)
    t, h = wl["t"], wl["h"]
    gen = torch.Generator(device=device).manual_seed(42 + rank)
    x_dev = torch.randn((t, h), device=device, generator=gen).to(torch.bfloat16)
    x_host = x_dev.cpu().pin_memory()
    out_host = torch.empty((t, h), dtype=torch.bfloat16).pin_memory()
    x_stage = torch.empty_like(x_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, finish=None, on_start=None):
        for _ in range(warmup):
            fn()
        if finish:
            finish()
        barrier()
        if on_start:
            on_start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if finish:
            finish()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    state = {}

    def resident():
        state["out"], state["ids"] = step(x_dev)

    # End to end: every step copies its tokens from pinned host memory and its bf16 output back to pinned host memory.
    # The three legs run on three streams with two buffer slots, so step i's copies overlap step i+1's compute
    # (a serving loop would do the same); the timed region ends when the last output has reached the host.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    slots = 2
    xs = [x_stage, torch.empty_like(x_dev)]
    outs = [torch.empty((t, h), dtype=torch.bfloat16, device=device) for _ in range(slots)]
    out_hosts = [out_host, torch.empty((t, h), dtype=torch.bfloat16).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(slots)]
    ev_comp = [torch.cuda.Event() for _ in range(slots)]
    ev_out = [torch.cuda.Event() for _ in range(slots)]
    counter = {"i": 0}

    def end_to_end():
        i = counter["i"]
        counter["i"] += 1
        k2 = i % slots
        cur = torch.cuda.current_stream(device)
        with torch.cuda.stream(s_in):
            if i >= slots:
                s_in.wait_event(ev_comp[k2])          # the compute that read this token buffer has finished
            xs[k2].copy_(x_host, non_blocking=True)
            ev_in[k2].record(s_in)
        cur.wait_event(ev_in[k2])
        if i >= slots:
            cur.wait_event(ev_out[k2])                # this output buffer has been copied out
        step(xs[k2], outs[k2])
        ev_comp[k2].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[k2])
            out_hosts[k2].copy_(outs[k2], non_blocking=True)
            ev_out[k2].record(s_out)

    def e2e_finish():
        cur = torch.cuda.current_stream(device)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    sampler = ClockSampler(local)
    ms = timed(resident, args.steps, args.warmup, on_start=sampler.start if rank == 0 else None)   # clocks of the timed region only
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(end_to_end, args.steps, max(1, args.warmup), finish=e2e_finish)
    # Decode sizes: the same resident step replayed from a CUDA graph (one host call per step instead of ~10 launches;
    # the programmatic-dependent-launch edges between the kernels survive the capture).
    graph_ms = None
    if world == 1 and (args.graph or t <= 2048):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(3):
                step(x_dev)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(x_dev)
        graph_ms = timed(graph.replay, args.steps, args.warmup) / args.steps
    status = owner.status()

    valid = (state["ids"] >= 0).sum().to(torch.float64)
    if world > 1:
        dist.all_reduce(valid)
    flops = layer_flops(wl, float(valid.item()), t * world)
    per_step = ms / args.steps
    tflops = flops / (per_step * 1e-3) / 1e12
    tflops_e2e = flops / (ms_e2e / args.steps * 1e-3) / 1e12

    roof = stage = None
    if world == 1:
        # stage durations with CUDA events on the launching stream (same inputs, same launches)
        hq, hs = ks.nvfp4_quantize(x_dev, ACT_GLOBAL_SCALE)
        ids, w = ks.route_topk(ks.router_logits(x_dev, L["gate_w"]), wl["k"], L["bias"])
        acc = None
        reps = max(3, min(args.steps, 10))
        for _ in range(reps):
            d = owner.run_profiled(ids, w, hq, hs.view(torch.uint8), L["w1q"], L["w1s"], L["w2q"], L["w2s"], state["out"],
                                   scale_up=L["scale_fc1"], scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
            acc = d if acc is None else {k2: acc[k2] + v for k2, v in d.items()}
        stage = {k2: v / reps for k2, v in acc.items()}
        totals = owner.workspace()["totals"].cpu().tolist()
        stage["m_tiles"] = totals[0]
        stage["tile_fill"] = totals[2] / max(1, totals[0] * 128)
        pk = peaks()
        fc1_flops = flops * 2.0 / 3.0
        rows_used = totals[1]
        fc1_bytes = (int((owner.workspace()["counts"].cpu() > 0).sum()) * 2 * wl["i"] * h * 9 / 16      # weights of the experts touched
                     + rows_used * h * 9 / 16 + rows_used * wl["i"] * 9 / 16)                           # permuted rows in, activations out
        achieved = fc1_flops / (stage["fc1"] * 1e-3) / 1e12
        peak = 4.0 * pk["bf16_sustained"]
        counts = owner.workspace()["counts"].cpu()
        touched = int((counts > 0).sum())
        weight_bytes = touched * 3 * wl["i"] * h * 9 / 16
        act_bytes = t * h * 2 * 2 + t * h * 9 / 16
        stage["experts_touched"] = touched
        stage["hbm_algorithmic_gbs"] = (weight_bytes + act_bytes) / (per_step * 1e-3) / 1e9
        stage["hbm_frac_of_measured"] = stage["hbm_algorithmic_gbs"] / pk["hbm_gbs"]
        roof = dict(bound="tensor", kernel="k_gemm_nvfp4<FC1>", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak,
                    peak_source=f"4 x bf16_tflops_sustained of {pk['source']} MEASURED_PEAKS (FP4:bf16 nominal ratio)",
                    frac_of_nominal_fp4=achieved / FP4_NOMINAL_TFLOPS,
                    traffic=FC1_DRAM_TRAFFIC.get(args.workload) if args.tokens is None and args.zipf is None else None,
                    traffic_unit="bytes of DRAM traffic per FC1 launch (ncu)",
                    algorithmic_bytes=fc1_bytes,
                    layer_frac_of_nominal_fp4=tflops / FP4_NOMINAL_TFLOPS)
    ep_stage = None
    if world > 1:
        owner.profile = True
        resident()
        ep_stage = owner.stage_ms()
        owner.profile = False
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = time_cpu(wl, 1, 0) if world == 1 else None
    line = dict(metric="nvfp4_moe_layer_tflops", value=tflops, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="nvfp4 (e2m1 x ue4m3, fp32 accumulate)",
                data="synthetic", tokens_per_s=t * world / (per_step * 1e-3),
                config=dict(workload=wl["label"], tokens_per_gpu=t, hidden=h, intermediate=wl["i"], experts=wl["e"], top_k=wl["k"],
                            shared_experts=wl["s"], parallelism=f"ep{world}",
                            l2="weights (%.2f GB per GPU) exceed the 126 MB L2; no flush needed" %
                               ((L["w1q"].numel() + L["w1s"].numel() + L["w2q"].numel() + L["w2s"].numel()) / 1e9)),
                e2e=dict(value=tflops_e2e, unit="TFLOP/s", h2d_bytes_per_step=x_host.numel() * 2, d2h_bytes_per_step=out_host.numel() * 2,
                         ms_per_step=ms_e2e / args.steps),
                gpu_launches=launches * args.steps, device_status=status, clocks=clocks)
    if graph_ms is not None:
        line["graph_replay"] = dict(ms_per_step=graph_ms, tokens_per_s=t / (graph_ms * 1e-3))
    if ep_stage:
        line["stage_ms"] = ep_stage
    if stage:
        line["stage_ms"] = stage
    if roof:
        line["roofline"] = roof
    if cpu:
        line["cpu_baseline"] = dict(value=cpu["tflops"], unit="TFLOP/s", cores=cpu["cores"], kind="port", sample=cpu["sample"],
                                    tokens_per_s=cpu["tokens_per_s"])
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_reference_gpu(args, wl):
    """A/B on identical device inputs: the reference's own Blackwell kernel (oracle/_ref, large-batch chain) against this
    library, routed experts only (the reference has no shared expert and reads no scale scalars). Not part of the
    default line; the reference arm proper (`--impl reference`) is the CPU path."""
    import torch
    import kernelschema_b200 as ks
    from oracle import ref_kernel
    if not ref_kernel.available():
        print(json.dumps(dict(impl="reference-gpu-kernel", unavailable="oracle/_ref/libnvfp4_moe_ref.so was not built (needs the reference checkout)")))
        return
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    wl = dict(wl, s=0)
    L = build_layer(wl, 0, 1, device, global_scales=False)      # the reference reads no scale scalars
    t, h, k = wl["t"], wl["h"], wl["k"]
    x = torch.randn((t, h), device=device).to(torch.bfloat16)
    hq, hs = ks.nvfp4_quantize(x)
    ids, w = ks.route_topk(ks.router_logits(x, L["gate_w"]), k, L["bias"])
    hs8 = hs.view(torch.uint8)
    alpha = torch.ones(wl["e"], device=device)
    beta = torch.zeros(wl["e"], device=device)
    out_ref = torch.zeros((t, h), dtype=torch.bfloat16, device=device)
    out_mine = torch.zeros((t, h), dtype=torch.bfloat16, device=device)
    rk = ref_kernel.ReferenceKernel()
    layer = ks.MoELayer(h, wl["i"], wl["e"], k, t)

    def run_ref():
        rk.run(ids, w, hq, hs8, L["w1q"], L["w1s"], L["w2q"], L["w2s"], alpha, beta, None, out_ref)

    def run_mine():
        layer.run(ids, w, hq, hs8, L["w1q"], L["w1s"], L["w2q"], L["w2s"], out_mine, alpha=alpha, beta=beta)

    res = {}
    for name, fn in (("reference", run_ref), ("this_library", run_mine)):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / args.steps
    flops = 6.0 * float((ids >= 0).sum()) * wl["i"] * h
    diff = (out_ref.float() - out_mine.float())
    rel_l2 = float(diff.norm() / out_ref.float().norm().clamp_min(1e-30))
    print(json.dumps(dict(impl="reference-gpu-kernel", metric="nvfp4_moe_layer_tflops", unit="TFLOP/s",
                          value=flops / (res["reference"] * 1e-3) / 1e12, ms_per_step=res["reference"], n_gpus=1,
                          steps=args.steps, warmup=args.warmup, higher_is_better=True, data="synthetic",
                          config=dict(workload=wl["label"] + "_routed_experts_only", chain="GEMM1 rung 97, GEMM2 rung 81, graph replay off"),
                          this_library_same_inputs=dict(value=flops / (res["this_library"] * 1e-3) / 1e12, ms_per_step=res["this_library"],
                                                        rel_l2_vs_reference_kernel=rel_l2, device_status=layer.status(),
                                                        output_rms=float(out_mine.float().pow(2).mean().sqrt()),
                                                        reference_output_rms=float(out_ref.float().pow(2).mean().sqrt())),
                          speedup_over_reference_kernel=res["reference"] / res["this_library"])))


def run_dense(args):
    """Single-expert dense NVFP4 GEMM (A quantised on the device, B pre-quantised): the mainloop in isolation."""
    import torch
    import kernelschema_b200 as ks
    m, n, k = (int(v) for v in args.dense.split(","))
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    bq, bsf = ks.nvfp4_quantize(b, 1.0, tiled_scales=True)
    aq, asf = ks.nvfp4_quantize(a, 1.0, tiled_scales=True)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    for _ in range(max(3, args.warmup)):
        ks.mm_nvfp4(aq, asf, bq, bsf, out=out, tile_n=args.tile_n)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ks.mm_nvfp4(aq, asf, bq, bsf, out=out, tile_n=args.tile_n)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    print(json.dumps(dict(metric="nvfp4_dense_gemm_tflops", value=tf, unit="TFLOP/s", n_gpus=1, steps=args.steps, warmup=args.warmup,
                          ms_per_step=ms, higher_is_better=True, dtype="nvfp4", data="synthetic",
                          config=dict(workload=f"dense_nvfp4_gemm_{m}x{n}x{k}", tile_n=args.tile_n,
                                      kernel_switches=os.environ.get("B200MOE_DBG", "0")),
                          frac_of_nominal_fp4=tf / FP4_NOMINAL_TFLOPS)))


def run_dense_w4a16(args):
    """Dense GEMM with bf16 activations and NVFP4 weights (A not quantised): the second catalogue operator's contract.
    Also times torch.matmul (cuBLAS bf16) on weights expanded to bf16 beforehand, as the library alternative."""
    import torch
    import kernelschema_b200 as ks
    m, n, k = (int(v) for v in args.dense.split(","))
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * k ** -0.5).to(torch.bfloat16)
    bq, bsf = ks.nvfp4_quantize(w, 1.0)
    bsf = bsf.view(torch.uint8)
    alpha = torch.ones(1, dtype=torch.float32, device="cuda")
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    ms = timed(lambda: ks.mm_bf16_nvfp4(a, bq, bsf, alpha, out=out, status=status))
    # library alternative: the same product by cuBLAS on pre-expanded bf16 weights (reads 3.6x the weight bytes)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    codes = torch.stack((bq & 15, bq >> 4), -1).long().reshape(n, k)
    w_dec = (lut[codes] * bsf.view(torch.float8_e4m3fn).float().repeat_interleave(16, -1)).to(torch.bfloat16)
    ref = torch.empty_like(out)
    ms_lib = timed(lambda: torch.matmul(a, w_dec.t(), out=ref))
    agree = float(((out.float() - ref.float()).norm() / ref.float().norm()).item())
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    pk = peaks()
    print(json.dumps(dict(metric="bf16_nvfp4_dense_gemm_tflops", value=tf, unit="TFLOP/s", n_gpus=1, steps=args.steps, warmup=args.warmup,
                          ms_per_step=ms, higher_is_better=True, dtype="bf16 x nvfp4 (weights expanded to bf16 exactly, fp32 accumulate)",
                          data="synthetic", config=dict(workload=f"dense_bf16_nvfp4_gemm_{m}x{n}x{k}"),
                          device_status=int(status.item()),
                          roofline=dict(bound="tensor", achieved=tf, peak=pk["bf16"], unit="TFLOP/s", frac=tf / pk["bf16"],
                                        peak_source=f"bf16_tflops (burst) of {pk['source']} MEASURED_PEAKS"),
                          cublas_bf16=dict(ms_per_step=ms_lib, tflops=2.0 * m * n * k / (ms_lib * 1e-3) / 1e12, rel_l2_between=agree),
                          hbm_algorithmic_gbs=(m * k * 2 + n * k * 9 / 16 + m * n * 2) / (ms * 1e-3) / 1e9)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"])
    ap.add_argument("--workload", default="dsv3", choices=sorted(WORKLOADS))
    ap.add_argument("--zipf", type=float, default=None, help="override the workload's Zipf exponent of the router bias (0 = uniform)")
    ap.add_argument("--tokens", type=int, default=None, help="override the workload's tokens per GPU (e.g. 64 or 256 for decode)")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed from a CUDA graph (always done up to 2048 tokens)")
    ap.add_argument("--dense", default=None, metavar="M,N,K", help="time the dense NVFP4 GEMM of this shape instead of the layer")
    ap.add_argument("--a-bf16", action="store_true", help="with --dense: keep A in bf16 (the bf16 x NVFP4 operator) instead of quantising it")
    ap.add_argument("--tile-n", type=int, default=0, help="GEMM tile for --dense (0 = default, 128, 256, 512 = CTA pair)")
    args = ap.parse_args()
    if args.dense:
        return run_dense_w4a16(args) if args.a_bf16 else run_dense(args)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    wl = dict(WORKLOADS[args.workload])
    if args.tokens is not None:
        wl["t"] = args.tokens
        wl["label"] = re.sub(r"_T\d+", f"_T{args.tokens}", wl["label"])
    if args.zipf is not None:
        wl["zipf"] = args.zipf
        wl["label"] += f"_zipf{args.zipf:g}_override"
    if args.impl == "reference-gpu":
        run_reference_gpu(args, wl)
    elif args.impl == "reference":
        run_reference(args, wl)
    else:
        run_gpu(args, wl)


if __name__ == "__main__":
    main()
