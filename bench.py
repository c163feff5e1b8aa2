"""Benchmark of the NVFP4 MoE layer hot path on B200 (one JSON line on stdout, printed by rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload dsv3|qwen3|c1] [--impl reference]

A step = one pass of the whole layer over one batch of synthetic tokens: bf16 activations -> NVFP4 quantiser ->
router logits + top-k/softmax -> route map -> permute -> FC1 + SwiGLU + requantise -> FC2 -> weighted combine
-> bf16 output. `value` times it with the bf16 inputs already resident in HBM; `e2e` times the same call chain
with pinned HOST buffers (host->device copy of the tokens and device->host copy of the output inside the timed
region). With --gpus N > 1 (launched under torchrun) experts are sharded over the ranks and tokens travel by
NCCL all-to-all (weak scaling: every rank brings its own T tokens).

`--impl reference` times the reference operator's own fp32 dequantise-then-matmul path (`reference.py::Model.forward`
of the staged problem files under oracle/_ref, built by oracle/build_ref.py; the numpy restatement in oracle/ when the
staging is absent) on the host cores, on a bounded sample of the same geometry.

Besides the headline workload the default run adds short sub-records (`sub`): the Qwen3-30B layer, the dense GEMM
sizes, decode batches of the headline geometry, and an A/B against the reference's own Blackwell kernel run through
its unmodified host; with N > 1 ranks: decode batches, a uniform-routing step and a parity record of the
expert-parallel result against the single-GPU layer. `--no-sub` leaves them out.
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
# static (calibrated) activation global scale amax / (6 * 448) for N(0, 1) activations whose block peaks reach ~5.7
ACT_GLOBAL_SCALE = 5.7 / (6.0 * 448.0)
FP4_NOMINAL_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one FC1 launch, from the ncu captures summarised in
# profiles/bench_dsv3_T8192_launch_list.md and profiles/layer_kernels_qwen3_T16384_ncu_full.md (workload -> bytes).
FC1_DRAM_TRAFFIC = {"dsv3": 4823125760 + 80460288, "qwen3": 386940416 + 49309952}
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


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


def make_step(wl, L, world, device, tokens=None):
    """Returns step(x_bf16_device) -> (out_bf16_device, ids), the object that owns the library state, and the launch
    count per step. Every buffer of the step is allocated here, once."""
    import torch
    import kernelschema_b200 as ks
    h, i, k, s = wl["h"], wl["i"], wl["k"], wl["s"]
    t = tokens or wl["t"]
    e = wl["e"]
    hq = torch.empty((t, h // 2), dtype=torch.uint8, device=device)
    hs = torch.empty((t, h // 16), dtype=torch.uint8, device=device)
    logits = torch.empty((t, e), dtype=torch.float32, device=device)
    ids = torch.empty((t, k), dtype=torch.int32, device=device)
    w = torch.empty((t, k), dtype=torch.float32, device=device)
    out_own = torch.empty((t, h), dtype=torch.bfloat16, device=device)

    def front(x):
        n = x.shape[0]
        ks.nvfp4_quantize(x, ACT_GLOBAL_SCALE, out=(hq[:n], hs[:n]))
        ks.route_topk(ks.router_logits(x, L["gate_w"], out=logits[:n]), k, L["bias"], out=(ids[:n], w[:n]))
        return hq[:n], hs[:n], ids[:n], w[:n]

    if world == 1:
        # one library call per step (b200moe_step: quantiser, router logits, top-k / softmax, layer), replayed from the
        # library's own CUDA graph after the second call with the same buffers
        layer = ks.MoELayer(h, i, L["e_local"], k, t, num_shared_experts=s, graph_cache=True)
        ids_view = layer.step_outputs(t)["ids"]

        def step(x, out=None):
            out = out_own[:x.shape[0]] if out is None else out
            layer.step(x, L["gate_w"], L["bias"], ACT_GLOBAL_SCALE, L["w1q"], L["w1s"], L["w2q"], L["w2s"], out,
                       scale_up=L["scale_fc1"], scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
            return out, ids_view[:x.shape[0]]

        step.front = front
        # quantiser, router logits, top-k + the layer: route map and permute are one kernel up to 8192 routes, the route map
        # alone is one kernel up to 16384 routes and three above; then FC1, FC2 and the combine
        routes = t * (k + s)
        return step, layer, 3 + (4 if routes <= 8192 else 5 if routes <= 16384 else 7)
    from kernelschema_b200.ep import ExpertParallelMoE
    ep = ExpertParallelMoE(h, i, e, k, t, num_shared_experts=s)

    def step(x, out=None):
        out = out_own[:x.shape[0]] if out is None else out
        q, sf, ids_, w_ = front(x)
        out = ep.forward(ids_, w_, q, sf, L["w1q"], L["w1s"], L["w2q"], L["w2s"], out=out,
                         scale_up=L["scale_fc1"], scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
        return out, ids_

    step.front = front
    return step, ep, ep.launches_per_step + 3


def layer_flops(wl, valid_routes, tokens):
    return 6.0 * valid_routes * wl["i"] * wl["h"] + 6.0 * tokens * wl["s"] * wl["i"] * wl["h"]


# --------------------------------------------------------------------------------------------- CPU arm
def _staged(*parts):
    return os.path.join(REF_DIR, *parts)


def reference_staged():
    return all(os.path.exists(_staged("problem", n)) for n in ("reference.py", "input.py"))


def _load_module(name, path):
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_sample_shape(wl):
    """Bounded sample of the workload for the host cores: same hidden / intermediate sizes, 8 routed experts, 256 tokens,
    top-2 (the reference has no shared expert and reads no global scales, so the sample has neither)."""
    e, k, t = (8, 2, 256) if wl["e"] >= 8 else (wl["e"], wl["k"], wl["t"])
    return dict(hidden=wl["h"], intermediate=wl["i"], local_experts=e, tokens=t, topk=k)


def time_cpu(wl, steps, warmup):
    """Times the reference's own CPU path on the sample: `reference.py::Model.forward` of the staged problem files with
    inputs from its own generator (kind "reference"); the numpy restatement on the equivalent seeded case when the
    staging is absent (kind "port")."""
    shape = cpu_sample_shape(wl)
    t = shape["tokens"]
    if reference_staged():
        import torch
        ref = _load_module("staged_reference_cpu", _staged("problem", "reference.py"))
        inp = _load_module("staged_input_cpu", _staged("problem", "input.py"))
        torch.manual_seed(0)
        kw = inp._make_inputs(**shape, device="cpu")
        model = ref.Model()
        fn = lambda: model(**kw)
        valid = int((kw["topk_ids"][0] >= 0).sum())
        kind, cores = "reference", torch.get_num_threads()
    else:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from helpers import make_moe_case
        from oracle import nvfp4_oracle as o
        p = make_moe_case(0, t, wl["h"], wl["i"], shape["local_experts"], shape["topk"])
        fn = lambda: o.moe_expected(p)
        valid = int((p["topk_ids"][0] >= 0).sum())
        kind, cores = "port", os.cpu_count()
    flops = 6.0 * valid * wl["i"] * wl["h"]
    desc = (f"H={wl['h']} I={wl['i']} experts={shape['local_experts']} T={t} top-{shape['topk']}, no shared expert: "
            f"{flops / 1e9:.1f} GFLOP per pass")
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    return dict(tflops=flops / dt / 1e12, tokens_per_s=t / dt, seconds=dt, sample=desc, cores=cores, kind=kind)


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu(wl, max(1, args.steps), max(0, min(args.warmup, 1)))
    line = dict(impl="reference", metric="nvfp4_moe_layer_tflops", value=r["tflops"], unit="TFLOP/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=r["seconds"] * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", tokens_per_s=r["tokens_per_s"],
                config=dict(workload=wl["label"], sample=r["sample"]),
                cpu_baseline=dict(value=r["tflops"], unit="TFLOP/s", cores=r["cores"], kind=r["kind"], sample=r["sample"]),
                e2e=dict(value=r["tflops"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------- GPU arm
def _timed_loop(fn, steps, warmup):
    """ms per call of `fn` with CUDA events on the current stream, after warm-up, synchronised on both sides."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def fp4_peaks(pk):
    """The three FP4 tensor denominators: 4 x the measured bf16 figures (nominal FP4 : bf16 ratio) and the nominal 9 PFLOP/s."""
    return dict(burst=4.0 * pk["bf16"], sustained=4.0 * pk["bf16_sustained"], nominal=FP4_NOMINAL_TFLOPS)


def tensor_roofline(achieved, pk, clocks, **extra):
    """`frac` uses the burst peak when the sampled SM clock stayed at >= 95 % of its maximum, the sustained one otherwise."""
    f = fp4_peaks(pk)
    sm, mx = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    which = "burst" if (sm and mx and sm >= 0.95 * mx) else "sustained"
    return dict(bound="tensor", achieved=achieved, peak=f[which], unit="TFLOP/s", frac=achieved / f[which],
                frac_burst=achieved / f["burst"], frac_sustained=achieved / f["sustained"], frac_nominal=achieved / f["nominal"],
                peak_burst=f["burst"], peak_sustained=f["sustained"], peak_nominal=f["nominal"],
                peak_source=f"4 x bf16_tflops ({which}) of {pk['source']} MEASURED_PEAKS: FP4 : bf16 nominal ratio; chosen by the sampled SM clock",
                **extra)


def sub_layer_record(name, tokens, args, device, pk, L=None, zipf=None, steps=10):
    """Short resident-input timing of another workload (or of the headline geometry at another batch) for `sub`."""
    import torch
    import kernelschema_b200 as ks
    wl = dict(WORKLOADS[name])
    if tokens:
        wl["t"] = tokens
    if zipf is not None:
        wl["zipf"] = zipf
    own_L = L is None
    if own_L:
        L = build_layer(wl, 0, 1, device)
    step, layer, _ = make_step(wl, L, 1, device)
    t, h = wl["t"], wl["h"]
    x = torch.randn((t, h), device=device, generator=torch.Generator(device=device).manual_seed(4242)).to(torch.bfloat16)
    state = {}

    def fn():
        state["out"], state["ids"] = step(x)

    ms = _timed_loop(fn, steps, 3)
    valid = float((state["ids"] >= 0).sum())
    flops = layer_flops(wl, valid, t)
    counts = layer.workspace()["counts"].cpu()
    touched = int((counts > 0).sum())
    weight_bytes = touched * 3 * wl["i"] * h * 9 / 16
    act_bytes = t * h * 2 * 2 + t * h * 9 / 16
    rec = dict(workload=wl["label"], tokens=t, ms_per_step=ms, tflops=flops / (ms * 1e-3) / 1e12, tokens_per_s=t / (ms * 1e-3),
               frac_of_nominal_fp4=flops / (ms * 1e-3) / 1e12 / FP4_NOMINAL_TFLOPS, experts_touched=touched,
               hbm_algorithmic_gbs=(weight_bytes + act_bytes) / (ms * 1e-3) / 1e9, device_status=layer.status())
    rec["hbm_frac_of_measured"] = rec["hbm_algorithmic_gbs"] / pk["hbm_gbs"]
    if t <= 2048:        # decode sizes: also the step replayed from a CUDA graph
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(3):
                step(x)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(x)
        gms = _timed_loop(graph.replay, steps, 3)
        rec["graph_replay_ms_per_step"] = gms
        rec["graph_replay_hbm_frac_of_measured"] = (weight_bytes + act_bytes) / (gms * 1e-3) / 1e9 / pk["hbm_gbs"]
    layer.close()
    return rec


def sub_dense_records(pk, steps=10):
    """The dense NVFP4 GEMM sizes of the benchmark (A quantised on the device with a global scale, B pre-quantised)."""
    import torch
    import kernelschema_b200 as ks
    out = []
    for m, n, k in ((2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (16384, 7168, 2048)):
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        b = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        gs_a, gs_b = float(a.float().abs().max()) / 2688.0, float(b.float().abs().max()) / 2688.0
        bq, bsf = ks.nvfp4_quantize(b, gs_b, tiled_scales=True)
        aq = torch.empty((m, k // 2), dtype=torch.uint8, device="cuda")
        asf = torch.zeros(((m + 127) // 128, k // 64, 32, 16), dtype=torch.uint8, device="cuda")
        y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        ms_q = _timed_loop(lambda: ks.nvfp4_quantize(a, gs_a, tiled_scales=True, out=(aq, asf)), steps, 3)
        ms = _timed_loop(lambda: ks.mm_nvfp4(aq, asf, bq, bsf, alpha=gs_a * gs_b, out=y, status=status), steps, 3)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        f = fp4_peaks(pk)
        out.append(dict(shape=[m, n, k], ms_gemm=ms, ms_quantise_a=ms_q, tflops=tf, frac_burst=tf / f["burst"],
                        frac_sustained=tf / f["sustained"], frac_nominal=tf / f["nominal"],
                        quantiser_gbs=m * k * 2.5625 / (ms_q * 1e-3) / 1e9, quantiser_hbm_frac_of_measured=m * k * 2.5625 / (ms_q * 1e-3) / 1e9 / pk["hbm_gbs"],
                        device_status=int(status[0])))
    return out


def sub_reference_kernel(steps=10):
    """The reference's own Blackwell kernel through its UNMODIFIED host (candidate/solution.py::Model: its selector, its graph
    replay), staged under oracle/_ref by oracle/build_ref.py, against this library's drop-in Model on the same device
    inputs, made by the reference's own generator: its ten fixed shapes (T = 1 ... 8192, among them an empty routing and
    all-zero activations, which its host shortcuts at graph capture and this library runs in full) and the routed part of
    the DeepSeek-V3 layer (H 7168, I 2048, E 256, top-8, T = 8192, skewed routing)."""
    import torch
    need = [_staged("candidate", "solution.py"), _staged("candidate", "nvfp4_moe.cu"), _staged("problem", "input.py"),
            _staged("problem", "shape_cases.json")]
    if not all(os.path.exists(p) for p in need):
        return dict(unavailable="oracle/_ref staging absent: python oracle/build_ref.py needs the reference checkout")
    os.environ["TORCH_EXTENSIONS_DIR"] = _staged("cache")      # where build_ref.py left the kernel prebuilt under the host's own cache name
    try:
        inp = _load_module("staged_input_gpu", _staged("problem", "input.py"))
        cand = _load_module("staged_candidate", _staged("candidate", "solution.py"))
        from kernelschema_b200.solution import Model as Mine
        with open(_staged("problem", "shape_cases.json")) as f:
            cases = json.load(f)
    except Exception as exc:
        return dict(unavailable=f"reference host does not load here: {exc!r}"[:400])
    todo = [(f"shape_{i}", cases[str(i)]["input_kwargs"]) for i in range(10) if str(i) in cases]
    todo.append(("dsv3_routed_T8192", dict(tokens=8192, hidden=7168, intermediate=2048, local_experts=256, topk=8, routing="skewed")))
    ref_model, my_model = cand.Model(), Mine()
    rows = {}
    for name, kw_shape in todo:
        try:
            torch.manual_seed(2026101501)
            kw = inp._make_inputs(**kw_shape)
            out_ref = kw["output"]
            out_mine = inp.guarded(tuple(out_ref.shape), out_ref.dtype, out_ref.device)
            kw_mine = dict(kw, output=out_mine)
            t, h = out_ref.shape
            flops = 6.0 * float((kw["topk_ids"][0] >= 0).sum()) * kw["intermediate_size"] * h
            rec = dict(tokens=t, hidden=h, intermediate=kw["intermediate_size"], experts=kw["num_experts"], gflop=flops / 1e9)
            try:
                ms_ref = _timed_loop(lambda: ref_model(**kw), steps, 4)          # its 2nd identical call captures its graph
                rec["reference_kernel_ms"] = ms_ref
            except Exception as exc:
                rec["reference_kernel_error"] = repr(exc)[:300]
                ms_ref = None
            ms_mine = _timed_loop(lambda: my_model(**kw_mine), steps, 4)
            rec["this_library_ms"] = ms_mine
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                my_model(**kw_mine)
            torch.cuda.current_stream().wait_stream(side)
            with torch.cuda.graph(g):
                my_model(**kw_mine)
            rec["this_library_graph_replay_ms"] = _timed_loop(g.replay, steps, 3)
            if ms_ref:
                rec["speedup_over_reference_kernel"] = ms_ref / ms_mine
                d = out_ref.float() - out_mine.float()
                rec["rel_l2_between"] = float(d.norm() / out_ref.float().norm().clamp_min(1e-30))
                rec["bf16_identical_fraction"] = float((d == 0).float().mean())
                rec["output_rms"] = [float(out_ref.float().pow(2).mean().sqrt()), float(out_mine.float().pow(2).mean().sqrt())]
            rows[name] = rec
            del kw, kw_mine
            torch.cuda.empty_cache()
        except Exception as exc:
            rows[name] = dict(error=repr(exc)[:300])
    return dict(host="candidate/solution.py::Model of the reference, unmodified (own selector, graph replay on)", cases=rows)


def ep_parity_record(wl, L, step, device, world, rank):
    """Expert-parallel result of this rank's tokens against the single-GPU layer holding ALL experts (gathered over the
    ranks), by the rules of the parity tests; the expert-parallel path rounds one bf16 partial row per visited rank."""
    import torch
    import torch.distributed as dist
    import kernelschema_b200 as ks
    t, h, k, s = wl["t"], wl["h"], wl["k"], wl["s"]
    e_local = L["e_local"]
    x = torch.randn((t, h), device=device, generator=torch.Generator(device=device).manual_seed(9000 + rank)).to(torch.bfloat16)
    out_ep, _ = step(x)
    out_ep = out_ep.clone()

    def gather(name, per_expert=True):
        mine = L[name][:e_local].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        return torch.cat(parts + [L[name][e_local:]], 0).contiguous()

    w1q, w1s, w2q, w2s = gather("w1q"), gather("w1s"), gather("w2q"), gather("w2s")
    sc1, sc2 = gather("scale_fc1"), gather("scale_fc2")
    layer = ks.MoELayer(h, wl["i"], wl["e"], k, t, num_shared_experts=s)
    q, sf, ids, w = step.front(x)
    ref = torch.empty((t, h), dtype=torch.bfloat16, device=device)
    layer.run(ids, w, q, sf, w1q, w1s, w2q, w2s, ref, scale_up=sc1, scale_gate=sc1, scale_out=sc2)
    torch.cuda.synchronize()
    status = layer.status()
    layer.close()
    got, exp = out_ep.float(), ref.float()
    diff = (got - exp).abs()
    rms = float(exp.pow(2).mean().sqrt())
    peak = float(exp.abs().max())
    import math
    slack = world * 2.0 ** (math.floor(math.log2(max(peak, 1e-30))) - 7)       # one bf16 step of the largest output per visited rank
    rec = dict(rel_l2=float((got - exp).norm() / exp.norm().clamp_min(1e-30)), max_abs_over_rms=float(diff.max()) / max(rms, 1e-30),
               mismatch=float((diff > 0.01 + 0.05 * got.abs()).float().mean()), single_gpu_status=status)
    ok = (rec["mismatch"] <= 1e-3 and rec["rel_l2"] <= 1e-2 and float(diff.max()) <= 2e-2 * rms + slack and status == 0
          and bool(torch.isfinite(got).all()))
    flag = torch.tensor([0 if ok else 1], device=device)
    worst = torch.tensor([rec["rel_l2"], rec["max_abs_over_rms"], rec["mismatch"]], device=device)
    dist.all_reduce(flag)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    rec = dict(rel_l2=float(worst[0]), max_abs_over_rms=float(worst[1]), mismatch=float(worst[2]), ranks_failed=int(flag.item()),
               passed=int(flag.item()) == 0, against="single-GPU layer with all experts, this rank's tokens; worst over ranks",
               rule="mismatch <= 1e-3, rel_l2 <= 1e-2, max_abs <= 2e-2 rms + world bf16 steps of the largest output")
    del w1q, w1s, w2q, w2s
    torch.cuda.empty_cache()
    return rec


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
    t_start = time.perf_counter()
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
    pk = peaks()

    roof = stage = None
    sub = {}
    if world == 1:
        # stage durations with CUDA events on the launching stream (same inputs, same launches)
        hq, hs, ids, w = step.front(x_dev)
        acc = None
        reps = max(3, min(args.steps, 10))
        for _ in range(reps):
            d = owner.run_profiled(ids, w, hq, hs, L["w1q"], L["w1s"], L["w2q"], L["w2s"], state["out"],
                                   scale_up=L["scale_fc1"], scale_gate=L["scale_fc1"], scale_out=L["scale_fc2"])
            acc = d if acc is None else {k2: acc[k2] + v for k2, v in d.items()}
        stage = {k2: v / reps for k2, v in acc.items()}
        totals = owner.workspace()["totals"].cpu().tolist()
        stage["m_tiles"] = totals[0]
        stage["tile_fill"] = totals[2] / max(1, totals[0] * 128)
        fc1_flops = flops * 2.0 / 3.0
        rows_used = totals[1]
        counts = owner.workspace()["counts"].cpu()
        touched = int((counts > 0).sum())
        fc1_bytes = (touched * 2 * wl["i"] * h * 9 / 16                                   # weights of the experts touched
                     + rows_used * h * 9 / 16 + rows_used * wl["i"] * 9 / 16)             # permuted rows in, activations out
        achieved = fc1_flops / (stage["fc1"] * 1e-3) / 1e12
        weight_bytes = touched * 3 * wl["i"] * h * 9 / 16
        act_bytes = t * h * 2 * 2 + t * h * 9 / 16
        stage["experts_touched"] = touched
        stage["hbm_algorithmic_gbs"] = (weight_bytes + act_bytes) / (per_step * 1e-3) / 1e9
        stage["hbm_frac_of_measured"] = stage["hbm_algorithmic_gbs"] / pk["hbm_gbs"]
        stage["fc2_tflops"] = flops / 3.0 / (stage["fc2"] * 1e-3) / 1e12
        roof = tensor_roofline(achieved, pk, clocks, kernel="k_gemm_nvfp4<FC1>",
                               traffic=FC1_DRAM_TRAFFIC.get(args.workload) if args.tokens is None and args.zipf is None and args.experts is None else None,
                               traffic_unit="bytes of DRAM traffic per FC1 launch (ncu capture summarised under profiles/)",
                               algorithmic_bytes=fc1_bytes, layer_frac_of_nominal_fp4=tflops / FP4_NOMINAL_TFLOPS,
                               fc1_hbm_gbs=fc1_bytes / (stage["fc1"] * 1e-3) / 1e9,
                               fc1_hbm_frac_of_measured=fc1_bytes / (stage["fc1"] * 1e-3) / 1e9 / pk["hbm_gbs"])
        if not args.no_sub and rank == 0:
            def guarded(name, fn):
                t0 = time.perf_counter()
                try:
                    sub[name] = fn()
                except Exception as exc:       # a sub-record never takes the headline line down
                    sub[name] = dict(error=repr(exc)[:300])
                if isinstance(sub[name], dict):
                    sub[name]["wall_s"] = round(time.perf_counter() - t0, 1)

            if args.workload == "dsv3" and args.tokens is None and args.experts is None:
                guarded("dsv3_decode_T64", lambda: sub_layer_record("dsv3", 64, args, device, pk, L=L))
                guarded("dsv3_decode_T256", lambda: sub_layer_record("dsv3", 256, args, device, pk, L=L))
                guarded("qwen3_T16384", lambda: sub_layer_record("qwen3", None, args, device, pk))
            guarded("dense_nvfp4_gemm", lambda: dict(sizes=sub_dense_records(pk)))
            guarded("reference_kernel", lambda: sub_reference_kernel())
    ep_stage = None
    if world > 1:
        owner.profile = True
        resident()
        ep_stage = owner.stage_ms()
        owner.profile = False
        if not args.no_sub:
            sub["parity"] = ep_parity_record(wl, L, step, device, world, rank)
            for name, tok, zipf in (("decode_T64", 64, None), ("decode_T256", 256, None), ("uniform_routing", None, 0.0)):
                try:
                    xx = x_dev[:tok] if tok else x_dev
                    L2 = L if zipf is None else dict(L, bias=None)
                    st2, own2, _ = (step, owner, None) if zipf is None else make_step(wl, L2, world, device)
                    holder = {}

                    def fn(st2=st2, xx=xx, holder=holder):
                        holder["ids"] = st2(xx)[1]

                    ms2 = timed(fn, 10, 3) / 10
                    v2 = (holder["ids"] >= 0).sum().to(torch.float64)
                    dist.all_reduce(v2)
                    tt = xx.shape[0]
                    fl2 = layer_flops(wl, float(v2.item()), tt * world)
                    sub[name] = dict(tokens_per_gpu=tt, ms_per_step=ms2, tflops=fl2 / (ms2 * 1e-3) / 1e12,
                                     tokens_per_s=tt * world / (ms2 * 1e-3), device_status=own2.status())
                    if zipf is not None:      # where rank 0's step goes when every rank holds the same load
                        own2.profile = True
                        fn()
                        torch.cuda.synchronize()
                        sub[name]["stage_ms"] = own2.stage_ms()
                        own2.profile = False
                except Exception as exc:
                    sub[name] = dict(error=repr(exc)[:300])
    if rank != 0:
        if world > 1:
            failed = bool(sub.get("parity")) and not sub["parity"]["passed"]
            dist.destroy_process_group()
            if failed:
                raise SystemExit(3)
        return
    cpu = time_cpu(wl, 1, 0) if world == 1 else None
    line = dict(metric="nvfp4_moe_layer_tflops", value=tflops, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="nvfp4 (e2m1 x ue4m3, fp32 accumulate)",
                data="synthetic", tokens_per_s=t * world / (per_step * 1e-3),
                config=dict(workload=wl["label"], tokens_per_gpu=t, hidden=h, intermediate=wl["i"], experts=wl["e"], top_k=wl["k"],
                            shared_experts=wl["s"], parallelism=f"ep{world}", activation_global_scale=ACT_GLOBAL_SCALE,
                            l2="weights (%.2f GB per GPU) exceed the 126 MB L2; no flush needed" %
                               ((L["w1q"].numel() + L["w1s"].numel() + L["w2q"].numel() + L["w2s"].numel()) / 1e9)),
                e2e=dict(value=tflops_e2e, unit="TFLOP/s", h2d_bytes_per_step=x_host.numel() * 2, d2h_bytes_per_step=out_host.numel() * 2,
                         ms_per_step=ms_e2e / args.steps),
                gpu_launches=launches * args.steps, device_status=status, clocks=clocks,
                frac_of_nominal_fp4_per_gpu=tflops / world / FP4_NOMINAL_TFLOPS)
    if graph_ms is not None:
        line["graph_replay"] = dict(ms_per_step=graph_ms, tokens_per_s=t / (graph_ms * 1e-3))
    if ep_stage:
        line["stage_ms"] = ep_stage
    if stage:
        line["stage_ms"] = stage
    if roof:
        line["roofline"] = roof
    if cpu:
        line["cpu_baseline"] = dict(value=cpu["tflops"], unit="TFLOP/s", cores=cpu["cores"], kind=cpu["kind"], sample=cpu["sample"],
                                    tokens_per_s=cpu["tokens_per_s"])
    if sub:
        line["sub"] = sub
    line["wall_s"] = round(time.perf_counter() - t_start, 1)
    print(json.dumps(line))
    failed = world > 1 and bool(sub.get("parity")) and not sub["parity"]["passed"]
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit(3)


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
                          config=dict(workload=f"dense_nvfp4_gemm_{m}x{n}x{k}", tile_n=args.tile_n),
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
    ap.add_argument("--experts", type=int, default=None, help="override the workload's number of routed experts (small profiler cases)")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed from a CUDA graph (always done up to 2048 tokens)")
    ap.add_argument("--dense", default=None, metavar="M,N,K", help="time the dense NVFP4 GEMM of this shape instead of the layer")
    ap.add_argument("--a-bf16", action="store_true", help="with --dense: keep A in bf16 (the bf16 x NVFP4 operator) instead of quantising it")
    ap.add_argument("--tile-n", type=int, default=0, help="GEMM tile for --dense (0 = default, 128, 256, 512 = CTA pair)")
    ap.add_argument("--no-sub", action="store_true", help="leave the sub-records out (headline workload only)")
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
    if args.experts is not None:
        wl["e"] = args.experts
        wl["label"] = re.sub(r"_E\d+", f"_E{args.experts}", wl["label"])
    if args.impl == "reference-gpu":
        run_reference_gpu(args, wl)
    elif args.impl == "reference":
        run_reference(args, wl)
    else:
        run_gpu(args, wl)


if __name__ == "__main__":
    main()
