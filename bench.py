"""Benchmark of the routed MXFP4 MoE layer (hidden 6144, intermediate 768, 128 experts, top-4) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference] [--no-sweep]

One "step" is one pass of the layer over one batch of T synthetic tokens (route, quantise, sort, gather, GEMM1 + SwiGLU +
requantisation, GEMM2 x routing weight, slot reduce). The workload is the same at every N: T=16384 tokens (the
expert-parallel configuration), on one GPU with all 128 experts at N=1 and split evenly over the ranks with the experts
sharded (expert parallel, dispatch and combine over NVLink) at N>1 -- fixed total work, "strong" scaling. The decode
(T=1..256) and prefill (T=2048, 8192) configurations are reported under "sweep", and the dominant decode kernel (GEMM1 at
T=256, HBM-bound) keeps its own roofline block, "roofline_decode".

Timing: every step is a CUDA-graph replay of the whole-layer C-ABI call (b200moe_forward) on one of the rotating inputs,
timed with CUDA events on the launching stream; before every step, untimed, a 512 MB buffer is overwritten and another
384 MB read, so the step starts on a cold and clean L2. "e2e" times the host-buffer C-ABI call (b200moe_forward_host):
pinned host input -> device, the layer, device -> host output, per step. "cpu_baseline" / --impl reference time the
reference's CPU path on the box's host cores on a stated sample of the workload's tokens: the reference's own torch
oracle file when a copy travels with the repository (kind "reference"), else the numpy restatement (kind "port").
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741
EXPERT_BYTES = 2 * I * (H // 2 + H // 32) + H * (I // 2 + I // 32)  # 7,520,256
W13_BYTES = 2 * I * (H // 2 + H // 32)                               # 5,013,504
FLOPS_PER_TOKEN = TOPK * (2 * H * 2 * I + 2 * I * H)                  # 113,246,208
NOMINAL_HBM_GBS, NOMINAL_FP4_TFLOPS = 8000.0, 9000.0
DECODE_SWEEP = (1, 2, 4, 8, 16, 32, 64, 128, 256)
PREFILL_SWEEP = (2048, 8192)
N_INPUTS = 8
HEADLINE_TOKENS = 16384
CPU_SAMPLE_TOKENS = 16


def ncu_traffic(tokens):
    """dram__bytes_read.sum + dram__bytes_write.sum of one GEMM1 launch from the ncu capture of this workload, as recorded
    in profiles/ncu_traffic.json by whoever made the capture (null when there is none for this token count)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get("gemm1", {}).get(str(tokens))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        ok = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in ok)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in ok), "sm_max_mhz": int(ok[0][1]), "reasons": reasons,
                "samples": len(ok)}


def cpu_reference(weights_np, x_bits, logits):
    """-> (fn, kind): one call of the reference's CPU path on a token sample (quantise, route, experts, slot rounding,
    reduce). The reference's own torch file is used when a copy sits in baseline/_ref/ (git-ignored; the build step copies
    it there where the reference checkout exists), else the numpy restatement."""
    from oracle import moe_oracle as orc
    path = os.path.join(ROOT, "baseline", "_ref", "mxfp4_moe_reference.py")
    if os.path.exists(path):
        import importlib.util
        import torch
        spec = importlib.util.spec_from_file_location("mxfp4_moe_reference", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        torch.set_num_threads(os.cpu_count())
        tw = [torch.from_numpy(a) for a in weights_np]
        x = torch.from_numpy(orc.bf16_to_f32(x_bits))
        lg = torch.from_numpy(logits)

        def call():
            xq, xs = ref.mxfp4_quant_ref(x)
            top = torch.topk(lg, 4, dim=1)
            wt = torch.softmax(top.values, dim=1)
            out = ref.w4a4_moe_ref((xq, xs), *tw, wt, top.indices.int())
            return out
        return call, "reference"
    return (lambda: orc.moe_layer(x_bits, logits, *weights_np)), "port"


def cpu_sample(weights_np, x_bits, logits, repeats):
    call, kind = cpu_reference(weights_np, x_bits[:CPU_SAMPLE_TOKENS], logits[:CPU_SAMPLE_TOKENS])
    call()  # warm
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        call()
        times.append(time.perf_counter() - t0)
    return times, kind


def reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path on the host cores (see cpu_reference), each step
    one call on a 16-token sample of the workload's tokens (all 128 experts' weights resident)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as orc
    weights_np, gen = orc.make_weights(seed=0)
    tokens = args.tokens or HEADLINE_TOKENS
    x_bits, logits = orc.make_inputs(gen, CPU_SAMPLE_TOKENS)
    call, kind = cpu_reference(weights_np, x_bits, logits)
    for _ in range(max(args.warmup, 1)):
        call()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        call()
        times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    value = CPU_SAMPLE_TOKENS / per_step
    cores = os.cpu_count()
    cfg = workload_config(tokens, args.gpus)
    cfg["cpu_sample_tokens"] = CPU_SAMPLE_TOKENS
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "mxfp4", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind,
                             "sample": f"{CPU_SAMPLE_TOKENS} of the workload's {tokens} tokens per step (tokens/s = "
                                       f"{CPU_SAMPLE_TOKENS} / step time), all 128 experts' weights resident, "
                                       + ("the reference's torch oracle, torch threads = cores" if kind == "reference"
                                          else "numpy restatement of the reference's torch oracle, BLAS threads")},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(tokens, gpus):
    return {"workload": f"mxfp4_h6144_i768_e128_top4 routed MoE layer, T={tokens}"
                        + (" (the expert-parallel configuration's token count; fits one GPU)" if tokens == HEADLINE_TOKENS else ""),
            "tokens": tokens, "hidden": H, "intermediate": I, "experts": E, "top_k": TOPK, "routing": "softmax top-4 renormalised",
            "weights": "E2M1 codes uniform, E8M0 scales 2^-7..2^-3, seed 0", "activations": "bf16 N(0,1), logits fp32 N(0,1)",
            "parallelism": "single GPU" if gpus == 1 else f"expert parallel ep{gpus}, {E // gpus} experts per GPU",
            "l2": L2_NOTE + (f"; {rotating_inputs(tokens)} rotating inputs" if gpus == 1 else "; 4 rotating inputs per rank"),
            "timing": "CUDA-graph replay of the whole-layer C-ABI call, CUDA events per step"}


def rotating_inputs(tokens):
    return N_INPUTS if tokens <= 8192 else 4


class Layer:
    """Device buffers for one token count and the graphs that replay the C-ABI call on each rotating input."""

    def __init__(self, w, tokens, lib, chain, torch, n_inputs=None, seed=1234):
        n_inputs = rotating_inputs(tokens) if n_inputs is None else n_inputs
        self.tokens, self.lib, self.torch, self.w = tokens, lib, torch, w
        dev = w.w13.device
        g = torch.Generator(device=dev).manual_seed(seed + tokens)
        self.x = [torch.randn((tokens, H), device=dev, generator=g).bfloat16() for _ in range(n_inputs)]
        self.logits = [torch.randn((tokens, E), device=dev, generator=g) for _ in range(n_inputs)]
        self.ws_bytes = int(lib.b200moe_workspace_bytes(tokens, w.num_experts))
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.slots = torch.empty((tokens, TOPK, H), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev)
        self.status = chain.status_word(dev)
        self.graphs = []

    def call(self, i, stream):
        from amd_kernels_b200 import _lib
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        _lib.check(self.lib.b200moe_forward(ctypes.byref(self.w.abi()), p(self.x[i]), p(self.logits[i]), self.tokens,
                                            p(self.workspace), self.ws_bytes, p(self.slots), p(self.out), p(self.status),
                                            ctypes.c_void_p(stream.cuda_stream)), "forward")

    def capture(self):
        torch = self.torch
        self.call(0, torch.cuda.current_stream())  # one eager call first: one-time function attributes
        torch.cuda.synchronize()
        for i in range(len(self.x)):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.call(i, torch.cuda.current_stream())
            self.graphs.append(graph)

    def active_experts(self, chain):
        n = []
        for lg in self.logits:
            _, ids = chain.topk_route(lg, None, 1.0, "softmax")
            n.append(int(ids.unique().numel()))
        return sum(n) / len(n)

    def launches_per_step(self):
        # up to 32 tokens: preparation (route + sort + quantise + gather), both GEMMs in one launch, reduce; above: routing,
        # sort (plus a count pass above 256 tokens), quantise+gather (at 128-row blocks: quantise only, GEMM1 gathers),
        # two GEMMs, reduce
        return 3 if self.tokens <= 32 else (6 if self.tokens <= 256 else 7)

    def replay(self, i):
        self.graphs[i % len(self.graphs)].replay()


class L2Flush:
    """Untimed L2 flush between steps: a 512 MB buffer is overwritten (4x the 126 MB L2), then another 384 MB buffer is
    read, so the dirty lines of the first are written back to HBM BEFORE the timed region starts. A timed step thus starts
    on a cold and clean L2, the state a profiler's cache control gives; after the write alone the step would also pay the
    write-back of ~100 MB of the flush buffer's dirty lines (measured: +12 us on a 113 us kernel)."""

    def __init__(self, torch, device="cuda"):
        self.torch = torch
        self.w = torch.empty(512 << 20, dtype=torch.uint8, device=device)
        self.r = torch.zeros(96 << 20, dtype=torch.int32, device=device)
        self.sink = torch.zeros(1, dtype=torch.int32, device=device)

    def fill_(self, i):
        self.w.fill_(i & 0xFF)
        self.sink.copy_(self.r.max().reshape(1))


L2_NOTE = "512 MB written then 384 MB read (dirty lines written back) before every timed step: cold, clean L2"


def time_steps(torch, fn, steps, warmup, flush):
    """Per-step device times (ms) of ``fn(i)``, with an untimed L2 flush before every step."""
    for i in range(warmup):
        flush.fill_(i)
        fn(i)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.fill_(i)
        starts[i].record()
        fn(warmup + i)
        stops[i].record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in zip(starts, stops)]


def with_shared_expert(torch, chain, orc, w, layer, flush, args):
    """The same workload through the package entry with the MXFP8 shared expert (its three launches on the device's side
    stream, joined before the reduce), as CUDA-graph replays; reported beside the headline, not in it."""
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import shared_expert as S
    sw = S.SharedWeights.from_row_major(*(torch.from_numpy(a).cuda() for a in orc.make_shared_weights()))
    w1 = chain.MoeWeights(None, None, w.w13, None, w.w2, None, w.routed_scaling_factor, w.routing_mode, shared_weights=sw)
    with torch.inference_mode():
        chain.mxfp4_moe(layer.x[0], w1, router_logits=layer.logits[0])
        S.shared_expert(layer.x[0], sw)
        torch.cuda.synchronize()
        graphs, alone, keep = [], [], []
        for i in range(len(layer.x)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep.append(chain.mxfp4_moe(layer.x[i], w1, router_logits=layer.logits[i]))
            graphs.append(g)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep.append(S.shared_expert(layer.x[i], sw))
            alone.append(g)
        ms = time_steps(torch, lambda i: graphs[i % len(graphs)].replay(), args.steps, args.warmup, flush)
        ms_alone = time_steps(torch, lambda i: alone[i % len(alone)].replay(), args.steps, args.warmup, flush)
    t = sum(ms) / len(ms)
    return {"us_per_step": t * 1e3, "tokens_per_s": layer.tokens / (t * 1e-3),
            "shared_expert_alone_us": sum(ms_alone) / len(ms_alone) * 1e3,
            "launches_per_step": layer.launches_per_step() + 3,
            "note": "routed layer + MXFP8 shared expert (quantise, GEMM1+SwiGLU+requantise, GEMM2) summed in the reduce"}


def roofline_times(tokens, e_active, peaks):
    byts = e_active * EXPERT_BYTES + tokens * (2 * H + 2 * H + 4 * E)
    flops = tokens * FLOPS_PER_TOKEN
    return byts, flops


def layer_report(tokens, ms, e_active, peaks):
    byts, flops = roofline_times(tokens, e_active, peaks)
    t = ms * 1e-3
    roof_meas = max(byts / (peaks["hbm_gbs"] * 1e9), flops / (4 * peaks["bf16_tflops"] * 1e12))
    roof_nom = max(byts / (NOMINAL_HBM_GBS * 1e9), flops / (NOMINAL_FP4_TFLOPS * 1e12))
    return {"tokens": tokens, "us_per_step": ms * 1e3, "tokens_per_s": tokens / t, "active_experts": e_active,
            "algorithmic_bytes": byts, "achieved_gbs": byts / t / 1e9, "achieved_tflops": flops / t / 1e12,
            "bound": "hbm" if byts / NOMINAL_HBM_GBS / 1e9 >= flops / NOMINAL_FP4_TFLOPS / 1e12 else "fp4",
            "frac_of_measured_roofline": roof_meas / t, "frac_of_nominal_roofline": roof_nom / t}


def gemm_times(torch, chain, w, layer, flush, args):
    """The two grouped GEMM launches of one layer call, each timed alone (CUDA events, cold clean L2 before every launch)."""
    wt, ids = chain.topk_route(layer.logits[0], None, 1.0, "softmax")
    sb = chain.moe_sort(ids, wt, chain.variant_for(layer.tokens))
    q = chain.mxfp4_quant(layer.x[0])
    if sb.bm == 128:  # the kernel the entry runs at this block height: it gathers its rows from the unsorted tokens
        gemm1 = lambda: chain.grouped_gemm1_gather(q[0], q[1], sb, w)
    else:
        xs, sfx = chain.dispatch_rows(q, sb)
        gemm1 = lambda: chain.grouped_gemm1(xs, sfx, sb, w)
    g1 = time_steps(torch, lambda i: gemm1(), args.steps, args.warmup, flush)
    hq, sfh = gemm1()
    g2 = time_steps(torch, lambda i: chain.grouped_gemm2(hq, sfh, sb, w, slots=layer.slots), args.steps, args.warmup, flush)
    return {"g1_ms": sum(g1) / len(g1), "g2_ms": sum(g2) / len(g2), "rows": int(sb.num_valid[0]), "bm": sb.bm,
            "rows_bound": sb.max_rows,
            "experts": int(ids.unique().numel())}


def gemm1_kernel_name(k):
    """The GEMM1 kernel the library selects for this many sorted rows."""
    if k["bm"] == 128:
        return "gemm1_wide_kernel<true> (GEMM1 gathering its token rows, 256 weight rows per MMA, + SwiGLU-OAI + MXFP4 requantisation)"
    return f"grouped_gemm_kernel<1,{k['bm']}> (GEMM1 + SwiGLU-OAI + MXFP4 requantisation)"


def gemm1_hbm_roofline(tokens, k, peaks):
    """GEMM1 against the HBM roofline: its algorithmic bytes (the active experts' W13 codes and scales once, the input
    rows' codes and scales in, the h codes and scales out) over its launch time, over the measured copy bandwidth."""
    # at 128-row blocks GEMM1 gathers its rows from the unsorted quantised tokens: one row per token is algorithmic input
    rows_in = tokens if k["bm"] == 128 else k["rows"]
    byts = k["experts"] * W13_BYTES + rows_in * (H // 2 + H // 32) + k["rows"] * (I // 2 + I // 32)
    gbs = byts / (k["g1_ms"] * 1e-3) / 1e9
    g2_bytes = k["experts"] * (EXPERT_BYTES - W13_BYTES) + k["rows"] * 408 + tokens * 4 * H * 2
    return {"kernel": gemm1_kernel_name(k), "tokens": tokens,
            "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "peak_source": peaks["source"] + " (STREAM-style copy)", "algorithmic_bytes": byts,
            "us_per_launch": k["g1_ms"] * 1e3, "traffic": ncu_traffic(tokens),
            "gemm2_us_per_launch": k["g2_ms"] * 1e3, "gemm2_achieved": g2_bytes / (k["g2_ms"] * 1e-3) / 1e9}


def gemm1_tensor_roofline(tokens, k, peaks):
    """GEMM1 against the tensor roofline: 2 * 6144 * 1536 flops for each of the 4T routed (token, slot) rows (padding rows
    are not algorithmic work) over its launch time, over 4 x the measured dense bf16 rate (the file of measured peaks has no
    FP4 figure; 4 is the nominal ratio of block-scaled FP4 to bf16 on this part)."""
    flops = 4 * tokens * 2 * H * 2 * I
    tf = flops / (k["g1_ms"] * 1e-3) / 1e12
    peak = 4 * peaks["bf16_tflops"]
    g2_tf = 4 * tokens * 2 * I * H / (k["g2_ms"] * 1e-3) / 1e12
    return {"kernel": gemm1_kernel_name(k), "tokens": tokens,
            "bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
            "peak_source": "4 x " + peaks["source"] + " dense bf16 (burst), the nominal FP4:bf16 ratio",
            "algorithmic_flops": flops, "sorted_rows_incl_padding": k["rows"], "us_per_launch": k["g1_ms"] * 1e3,
            "traffic": ncu_traffic(tokens), "gemm2_us_per_launch": k["g2_ms"] * 1e3, "gemm2_achieved": g2_tf,
            "hbm_view": {kk: v for kk, v in gemm1_hbm_roofline(tokens, k, peaks).items() if kk in ("achieved", "frac", "algorithmic_bytes")}}


def entry_with_router(torch, chain, w, flush, args, sizes=(256, 2048, 8192)):
    """The call a server makes -- mxfp4_moe(x, w) with the router inside (b200moe_forward_x) -- beside the same call fed
    with precomputed logits, as CUDA-graph replays."""
    gate = torch.randn((E, H), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) / H ** 0.5
    wg = chain.MoeWeights(gate, None, w.w13, None, w.w2, None, w.routed_scaling_factor, w.routing_mode)
    out = []
    with torch.inference_mode():
        for tokens in sizes:
            g = torch.Generator(device="cuda").manual_seed(77 + tokens)
            xs = [torch.randn((tokens, H), device="cuda", generator=g).bfloat16() for _ in range(4)]
            lgs = [(x.float() @ gate.t()).contiguous() for x in xs]
            chain.mxfp4_moe(xs[0], wg)
            torch.cuda.synchronize()
            graphs = {"x_only": [], "with_logits": []}
            keep = []
            for x, lg in zip(xs, lgs):
                for name, kw in (("x_only", {}), ("with_logits", {"router_logits": lg})):
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        keep.append(chain.mxfp4_moe(x, wg, **kw))
                    graphs[name].append(gr)
            t = {name: time_steps(torch, lambda i, L=lst: L[i % len(L)].replay(), args.steps, args.warmup, flush)
                 for name, lst in graphs.items()}
            out.append({"tokens": tokens, "x_only_us": sum(t["x_only"]) / len(t["x_only"]) * 1e3,
                        "with_logits_us": sum(t["with_logits"]) / len(t["with_logits"]) * 1e3})
            del graphs, keep, xs, lgs
    return out


def single_gpu(args):
    import torch
    from amd_kernels_b200 import _lib
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    from oracle import moe_oracle as orc
    torch.cuda.set_device(0)
    lib = _lib.load()
    peaks = measured_peaks()
    weights_np, gen = orc.make_weights(seed=0)
    x0_bits, lg0 = orc.make_inputs(gen, CPU_SAMPLE_TOKENS)
    w = chain.MoeWeights.from_row_major(None, None, *(torch.from_numpy(a).cuda() for a in weights_np),
                                        routing_mode="softmax", routed_scaling_factor=1.0)
    chain.warm_up_mxfp4_moe(w)
    flush = L2Flush(torch)
    headline_t = args.tokens or HEADLINE_TOKENS
    decode_t = 256
    sweep_ts = [headline_t] if args.no_sweep else sorted(set(DECODE_SWEEP + PREFILL_SWEEP + (headline_t,)))
    sweep, keep = [], {}
    clocks = ClockSampler(torch.cuda.current_device())
    with clocks:
        for tokens in sweep_ts:
            layer = Layer(w, tokens, lib, chain, torch)
            layer.capture()
            ms = time_steps(torch, layer.replay, args.steps, args.warmup, flush)
            rep = layer_report(tokens, sum(ms) / len(ms), layer.active_experts(chain), peaks)
            rep["us_min"] = min(ms) * 1e3
            sweep.append(rep)
            if tokens == headline_t:
                head_ms = ms
            if tokens in (headline_t, decode_t):
                keep[tokens] = gemm_times(torch, chain, w, layer, flush, args)
            if tokens == headline_t:
                head = layer
            else:
                del layer
        layer = head
        # ---- end to end through the host-buffer C-ABI call
        hx = [t.cpu().pin_memory() for t in layer.x]
        hl = [t.cpu().pin_memory() for t in layer.logits]
        hout = torch.empty((headline_t, H), dtype=torch.bfloat16).pin_memory()
        dx, dl = torch.empty_like(layer.x[0]), torch.empty_like(layer.logits[0])
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731

        def e2e_step(i):
            j = i % len(hx)
            _lib.check(lib.b200moe_forward_host(ctypes.byref(w.abi()), p(hx[j]), p(hl[j]), headline_t, p(dx), p(dl),
                                                p(layer.workspace), layer.ws_bytes, p(layer.slots), p(layer.out), p(hout),
                                                p(layer.status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                       "forward_host")
        for i in range(args.warmup):
            e2e_step(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(args.steps):
            flush.fill_(i)
            e2e_step(i)
            torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step
        e2e_wall = time.perf_counter() - t0
        e2e_ms = time_steps(torch, e2e_step, args.steps, 1, flush)
        shared_rep = None if args.no_sweep else with_shared_expert(torch, chain, orc, w, layer, flush, args)
        router_rep = None if args.no_sweep else entry_with_router(torch, chain, w, flush, args)
    status = chain.last_status()
    if status:
        raise RuntimeError(f"device status {status}: a kernel wait timed out")
    ms_per_step = sum(head_ms) / len(head_ms)
    cpu_times, cpu_kind = cpu_sample(weights_np, x0_bits, lg0, repeats=3)
    cpu_s = statistics.median(cpu_times)
    head_k = keep[headline_t]
    tensor_bound = head_k["bm"] == 128 and headline_t * FLOPS_PER_TOKEN / (NOMINAL_FP4_TFLOPS * 1e12) \
        > (128 * EXPERT_BYTES + headline_t * (4 * H + 4 * E)) / (NOMINAL_HBM_GBS * 1e9)
    roof = gemm1_tensor_roofline(headline_t, head_k, peaks) if tensor_bound else gemm1_hbm_roofline(headline_t, head_k, peaks)
    line = {"metric": "moe_layer_tokens_per_s", "value": headline_t / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "mxfp4", "data": "synthetic",
            "config": workload_config(headline_t, 1),
            "roofline": roof,
            "roofline_decode": gemm1_hbm_roofline(decode_t, keep[decode_t], peaks) if decode_t in keep and decode_t != headline_t else None,
            "layer_roofline": next(r for r in sweep if r["tokens"] == headline_t),
            "cpu_baseline": {"value": CPU_SAMPLE_TOKENS / cpu_s, "unit": "tokens/s", "cores": os.cpu_count(), "kind": cpu_kind,
                             "sample": f"{CPU_SAMPLE_TOKENS} tokens of the workload (tokens/s = {CPU_SAMPLE_TOKENS} / call time), "
                                       f"median of 3 calls, {cpu_s:.2f} s per call"},
            "e2e": {"value": headline_t / (sum(e2e_ms) / len(e2e_ms) * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": headline_t * (2 * H + 4 * E), "d2h_bytes_per_step": headline_t * 2 * H,
                    "wall_value_with_sync_per_step": headline_t * args.steps / e2e_wall},
            "with_shared_expert": shared_rep, "entry_with_router": router_rep,
            "gpu_launches": args.steps * layer.launches_per_step(),
            "clocks": clocks.summary(), "sweep": sweep}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--zipf", action="store_true", help="multi-GPU: the skewed-routing configuration (logit bias -2.2 ln rank)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return single_gpu(args)
    import ep_bench
    return ep_bench.run(args)


if __name__ == "__main__":
    main()
