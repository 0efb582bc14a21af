"""Benchmark of the routed MXFP4 MoE layer (hidden 6144, intermediate 768, 128 experts, top-4) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference] [--no-sweep]

One "step" is one pass of the layer over one batch of T synthetic tokens (route, quantise, sort, gather, GEMM1 + SwiGLU +
requantisation, GEMM2 x routing weight, slot reduce). At N=1 the headline workload is the decode configuration at its
largest size, T=256 (all 128 experts active, 963 MB of weights streamed per step); the other decode and prefill sizes are
reported under "sweep". At N>1 the 128 experts are sharded over the ranks (expert parallel, NCCL all-to-all dispatch and
combine) and the workload is T=16384 tokens split evenly over the ranks, fixed total work ("strong" scaling).

Timing: every step is a CUDA-graph replay of the whole-layer C-ABI call (b200moe_forward) on one of 8 rotating inputs,
timed with CUDA events on the launching stream; between steps a 512 MB buffer is overwritten so nothing of the previous
step survives in L2. "e2e" times the host-buffer C-ABI call (b200moe_forward_host): pinned host input -> device, the
layer, device -> host output, per step. "cpu_baseline" / --impl reference time the CPU oracle (a numpy port of the
reference's torch oracle) on the box's host cores on a 16-token sample of the same workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM1 launch at T=256, from the ncu capture summarised under
# profiles/ (None until a capture exists)
# profiles/grouped_gemm_t256_ncu_full.md: 679,282,176 read + 4,750,336 written by the layer's GEMM1 launch, which also
# asks L2 for 592 W2 tiles (30,916,608 bytes) on behalf of the GEMM2 that follows; only valid for the T=256 workload
NCU_GEMM1_TRAFFIC_BYTES = 684_032_512
NCU_GEMM1_PREFETCH_BYTES = 592 * 3 * 17408


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


def cpu_oracle_sample(weights_np, x_bits, logits, repeats=3):
    """tokens/s of the CPU oracle on a 16-token sample: quantise, route, experts, slot rounding, reduce."""
    from oracle import moe_oracle as orc
    sample = min(16, x_bits.shape[0])
    xs, lg = x_bits[:sample], logits[:sample]
    orc.moe_layer(xs, lg, *weights_np)  # warm
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.moe_layer(xs, lg, *weights_np)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return sample / med, med, sample


def reference_arm(args):
    """--impl reference: the CPU implementation of the path (the oracle port; the reference's own torch file does not
    travel to the GPU box) on the host cores, each step a 16-token sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as orc
    weights_np, gen = orc.make_weights(seed=0)
    tokens = args.tokens or (256 if args.gpus == 1 else 16384)
    x_bits, logits = orc.make_inputs(gen, 16)
    for _ in range(max(args.warmup, 1)):
        orc.moe_layer(x_bits, logits, *weights_np)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        orc.moe_layer(x_bits, logits, *weights_np)
        times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    value = 16 / per_step
    cores = os.cpu_count()
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
            "dtype": "mxfp4", "data": "synthetic",
            "config": workload_config(tokens, args.gpus),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": "16 tokens of the workload per step, all 128 experts' weights resident, numpy + BLAS threads"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(tokens, gpus):
    return {"workload": f"mxfp4_h6144_i768_e128_top4 routed MoE layer, T={tokens}"
                        + (" decode (configuration 1)" if gpus == 1 and tokens <= 256 else ""),
            "tokens": tokens, "hidden": H, "intermediate": I, "experts": E, "top_k": TOPK, "routing": "softmax top-4 renormalised",
            "weights": "E2M1 codes uniform, E8M0 scales 2^-7..2^-3, seed 0", "activations": "bf16 N(0,1), logits fp32 N(0,1)",
            "parallelism": "single GPU" if gpus == 1 else f"expert parallel ep{gpus}, {E // gpus} experts per GPU",
            "l2": L2_NOTE + ("; 8 rotating inputs" if gpus == 1 else "; 4 rotating inputs per rank"),
            "timing": "CUDA-graph replay of the whole-layer C-ABI call, CUDA events per step"}


class Layer:
    """Device buffers for one token count and the graphs that replay the C-ABI call on each rotating input."""

    def __init__(self, w, tokens, lib, chain, torch, n_inputs=N_INPUTS, seed=1234):
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
        # up to 32 tokens: route+sort, quantise+gather, both GEMMs in one launch, reduce; above: routing and sort apart
        # (plus a count pass above 256), quantise+gather, two GEMMs, reduce
        return 4 if self.tokens <= 32 else (6 if self.tokens <= 256 else 7)


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


def single_gpu(args):
    import torch
    from amd_kernels_b200 import _lib
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    from oracle import moe_oracle as orc
    torch.cuda.set_device(0)
    lib = _lib.load()
    peaks = measured_peaks()
    weights_np, gen = orc.make_weights(seed=0)
    x0_bits, lg0 = orc.make_inputs(gen, 16)
    w = chain.MoeWeights.from_row_major(None, None, *(torch.from_numpy(a).cuda() for a in weights_np),
                                        routing_mode="softmax", routed_scaling_factor=1.0)
    chain.warm_up_mxfp4_moe(w)
    flush = L2Flush(torch)
    headline_t = args.tokens or 256
    sweep_ts = [headline_t] if args.no_sweep else sorted(set(DECODE_SWEEP + PREFILL_SWEEP + (headline_t,)))
    sweep, layers = [], {}
    clocks = ClockSampler(torch.cuda.current_device())
    with clocks:
        for tokens in sweep_ts:
            layer = Layer(w, tokens, lib, chain, torch)
            layer.capture()
            ms = time_steps(torch, lambda i, L=layer: L.graphs[i % N_INPUTS].replay(), args.steps, args.warmup, flush)
            rep = layer_report(tokens, sum(ms) / len(ms), layer.active_experts(chain), peaks)
            rep["us_min"] = min(ms) * 1e3
            sweep.append(rep)
            if tokens == headline_t:
                layers[tokens] = layer
                head_ms = ms
            else:
                del layer
        layer = layers[headline_t]
        # ---- the dominant kernel alone: grouped GEMM1 (+SwiGLU + requantisation)
        wt, ids = chain.topk_route(layer.logits[0], None, 1.0, "softmax")
        sb = chain.moe_sort(ids, wt, chain.variant_for(headline_t))
        xs, sfx = chain.dispatch_rows(chain.mxfp4_quant(layer.x[0]), sb)
        g1 = time_steps(torch, lambda i: chain.grouped_gemm1(xs, sfx, sb, w), args.steps, args.warmup, flush)
        hq, sfh = chain.grouped_gemm1(xs, sfx, sb, w)
        g2 = time_steps(torch, lambda i: chain.grouped_gemm2(hq, sfh, sb, w, slots=layer.slots), args.steps, args.warmup, flush)
        rows = int(sb.num_valid[0])
        e_act = int(ids.unique().numel())
        # ---- end to end through the host-buffer C-ABI call
        hx = [t.cpu().pin_memory() for t in layer.x]
        hl = [t.cpu().pin_memory() for t in layer.logits]
        hout = torch.empty((headline_t, H), dtype=torch.bfloat16).pin_memory()
        dx, dl = torch.empty_like(layer.x[0]), torch.empty_like(layer.logits[0])
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731

        def e2e_step(i):
            j = i % N_INPUTS
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
        shared_rep = with_shared_expert(torch, chain, orc, w, layer, flush, args)
    status = chain.last_status()
    if status:
        raise RuntimeError(f"device status {status}: a kernel wait timed out")
    ms_per_step = sum(head_ms) / len(head_ms)
    g1_ms = sum(g1) / len(g1)
    g1_bytes = e_act * W13_BYTES + rows * (H // 2 + H // 32) + rows * (I // 2 + I // 32)
    cpu_value, cpu_s, cpu_sample = cpu_oracle_sample(weights_np, x0_bits, lg0)
    line = {"metric": "moe_layer_tokens_per_s", "value": headline_t / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4", "data": "synthetic",
            "config": workload_config(headline_t, 1),
            "roofline": {"kernel": "grouped_gemm_kernel<1,bm> (GEMM1 + SwiGLU-OAI + MXFP4 requantisation)", "bound": "hbm",
                         "achieved": g1_bytes / (g1_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": g1_bytes / (g1_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "algorithmic_bytes": g1_bytes, "us_per_launch": g1_ms * 1e3,
                         "traffic": NCU_GEMM1_TRAFFIC_BYTES if headline_t == 256 else None,
                         "traffic_includes_l2_prefetch_for_gemm2": NCU_GEMM1_PREFETCH_BYTES if headline_t == 256 else None,
                         "gemm2_us_per_launch": sum(g2) / len(g2) * 1e3,
                         "gemm2_achieved": (e_act * (EXPERT_BYTES - W13_BYTES) + rows * 408 + headline_t * 4 * H * 2)
                         / (sum(g2) / len(g2) * 1e-3) / 1e9},
            "layer_roofline": next(r for r in sweep if r["tokens"] == headline_t),
            "cpu_baseline": {"value": cpu_value, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": f"{cpu_sample} tokens (configuration 0), median of 3 calls, {cpu_s:.2f} s per call"},
            "e2e": {"value": headline_t / (sum(e2e_ms) / len(e2e_ms) * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": headline_t * (2 * H + 4 * E), "d2h_bytes_per_step": headline_t * 2 * H,
                    "wall_value_with_sync_per_step": headline_t * args.steps / e2e_wall},
            "with_shared_expert": shared_rep,
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
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import ep_bench
    return ep_bench.run(args)


if __name__ == "__main__":
    main()
