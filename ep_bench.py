"""The multi-GPU leg of bench.py (`python bench.py --gpus N` under torchrun lands here): the expert-parallel layer, one
process per GPU, NCCL over NVLink.

Workload: global T tokens (default 16384) split evenly over the W ranks; 128/W experts per rank; every step is one
layer call on every rank (route, quantise, all-to-all dispatch, grouped GEMMs, all-to-all combine, fixed-order reduce).
Total work is fixed as W grows ("strong" scaling; the single-GPU bench line is the same 16384 tokens on one GPU). Per-step
device time is taken with CUDA events on each rank after an untimed L2 flush (written, then evicted by a read); the job's
time is the maximum over the ranks of the summed step times. Before anything is timed every rank checks its output on its
own tokens, bit for bit, against the single-GPU layer with all 128 experts ("parity_checked" in the JSON line)."""
from __future__ import annotations

import json
import os
import time

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # peer pointers only: never bind buffers to a multicast object

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain, ep  # noqa: E402
from bench import ClockSampler, FLOPS_PER_TOKEN, L2Flush, measured_peaks, workload_config  # noqa: E402

H, E, TOPK = 6144, 128, 4
ROW_BYTES_OUT, ROW_BYTES_IN = 2 * H, H // 2 + H // 32 + 8
NVLINK_GBS_MEASURED = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool
N_INPUTS = 4


def synthetic_weights(seed=0):
    """The benchmark's checkpoint-layout weights (E2M1 codes uniform over the 16 values, E8M0 scale bytes 120..124), the
    same generator and seed the single-GPU bench and the tests use."""
    from oracle import moe_oracle as orc  # data generation only; nothing of the oracle is timed or compared against here
    return orc.make_weights(seed=seed)[0]


def build_layers(rank, world, placement, peer_pairs):
    """(this rank's expert-parallel layer, the single-GPU layer over all 128 experts used as the parity reference)."""
    raw = synthetic_weights()
    mine = ep.local_expert_ids(rank, world, placement=placement).numpy()
    w = chain.MoeWeights.from_row_major(None, None, *(torch.from_numpy(np.ascontiguousarray(a[mine])).cuda() for a in raw))
    w_all = chain.MoeWeights.from_row_major(None, None, *(torch.from_numpy(a).cuda() for a in raw), routing_mode="softmax",
                                            routed_scaling_factor=1.0)
    del raw
    layer = ep.ExpertParallelMoe(w, None, bias=None, routing_mode="softmax", scale=1.0, placement=placement,
                                 peer_pairs=peer_pairs)
    return layer, w_all


def check_parity(layer, w_all, xs, lgs):
    """Every rank: the expert-parallel output on its own tokens == the single-GPU layer on the same tokens, bit for bit.
    Returns (all ranks equal, mismatching elements summed over the ranks)."""
    bad = torch.zeros(1, dtype=torch.int64, device="cuda")
    with torch.inference_mode():
        for x, lg in zip(xs[:2], lgs[:2]):
            got = layer.forward(x, lg)
            want = chain.mxfp4_moe(x, w_all, router_logits=lg)
            bad += (got.view(torch.int16) != want.view(torch.int16)).sum()
    dist.all_reduce(bad)
    return int(bad.item()) == 0, int(bad.item())


def one_gpu_same_workload(w, flush, tokens, zipf, steps):
    """Rank 0 alone: the same global token count through the single-GPU layer (all 128 experts on this GPU), timed the
    same way, so the strong-scaling ratio can be read from one JSON line. The other ranks wait at the final barrier."""
    gen = torch.Generator(device="cuda").manual_seed(99)
    x = torch.randn((tokens, H), device="cuda", generator=gen).bfloat16()
    lg = torch.randn((tokens, E), device="cuda", generator=gen)
    if zipf:
        lg = lg - 2.2 * torch.log(torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
    with torch.inference_mode():
        for i in range(3):
            flush.fill_(i)
            chain.mxfp4_moe(x, w, router_logits=lg)
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for i in range(steps):
            flush.fill_(i)
            ev[i][0].record()
            chain.mxfp4_moe(x, w, router_logits=lg)
            ev[i][1].record()
        torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in ev) / steps
    return {"ms_per_step": ms, "value": tokens / (ms * 1e-3), "unit": "tokens/s"}


def run(args):
    """One JSON line for the configuration the arguments name; on 8 GPUs without --zipf the skewed-routing configuration
    (T=4096, Zipf-like logit bias, interleaved expert placement) is measured in the same run and reported under
    "zipf_t4096" of that line."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    zipf = bool(getattr(args, "zipf", False))
    line = measure(args, rank, world, local, args.tokens or 16384, zipf)
    if world == 8 and not zipf and not args.tokens:
        extra = measure(args, rank, world, local, 4096, True)
        if rank == 0:
            line["zipf_t4096"] = {k: extra[k] for k in ("value", "unit", "ms_per_step", "config", "roofline", "parity_checked",
                                                        "parity_mismatching_elements", "one_gpu_same_workload", "clocks")}
    if rank == 0:
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def measure(args, rank, world, local, tokens_global, zipf):
    if tokens_global % world:
        raise ValueError("the global token count must divide evenly over the ranks")
    t_loc = tokens_global // world
    placement = "interleaved" if zipf else "contiguous"
    layer, w_all = build_layers(rank, world, placement, 0 if os.environ.get("B200MOE_EP_COMBINE") == "nccl" else t_loc * TOPK)
    gen = torch.Generator(device="cuda").manual_seed(4321 + rank)
    xs = [torch.randn((t_loc, H), device="cuda", generator=gen).bfloat16() for _ in range(N_INPUTS)]
    lgs = [torch.randn((t_loc, E), device="cuda", generator=gen) for _ in range(N_INPUTS)]
    if zipf:
        skew = -2.2 * torch.log(torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
        lgs = [lg + skew for lg in lgs]
    parity_ok, parity_bad = check_parity(layer, w_all, xs, lgs)
    w_all_check = w_all
    flush = L2Flush(torch)
    hx = [t.cpu().pin_memory() for t in xs]
    hl = [t.cpu().pin_memory() for t in lgs]
    hout = torch.empty((t_loc, H), dtype=torch.bfloat16).pin_memory()

    # The step as CUDA-graph replays (one graph per rotating input, collectives included) when the fused form is in use:
    # it reads nothing on the host, so it can be captured; otherwise (NCCL form, or capture unavailable) eager calls.
    graphs, graph_outs = [], []
    want_graph = layer.peer is not None and os.environ.get("B200MOE_EP_GRAPH", "1") == "1"
    if want_graph:
        ok = torch.ones(1, device="cuda")
        try:
            with torch.inference_mode():
                layer.forward(xs[0], lgs[0])
                torch.cuda.synchronize()
                dist.barrier()
                for i in range(N_INPUTS):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        graph_outs.append(layer.forward(xs[i], lgs[i]))
                    graphs.append(g)
        except Exception:  # noqa: BLE001 - any capture failure: every rank falls back to eager calls
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if not bool(ok.item()):
            graphs = []
    if graphs:  # a replayed step must still be the single-GPU layer's bits
        graphs[0].replay()
        with torch.inference_mode():
            same = torch.equal(graph_outs[0], chain.mxfp4_moe(xs[0], w_all_check, router_logits=lgs[0])) if w_all_check is not None else True
        flag = torch.tensor([0 if same else 1], device="cuda")
        dist.all_reduce(flag)
        parity_ok = parity_ok and int(flag.item()) == 0

    def step(i):
        if graphs:
            graphs[i % N_INPUTS].replay()
            return graph_outs[i % N_INPUTS]
        return layer.forward(xs[i % N_INPUTS], lgs[i % N_INPUTS])

    def e2e_step(i):
        x = hx[i % N_INPUTS].cuda(non_blocking=True)
        lg = hl[i % N_INPUTS].cuda(non_blocking=True)
        hout.copy_(layer.forward(x, lg), non_blocking=True)

    def timed(fn, steps, warmup):
        for i in range(warmup):
            flush.fill_(i)
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        recv = []
        for i in range(steps):
            flush.fill_(i)
            ev[i][0].record()
            fn(warmup + i)
            ev[i][1].record()
            recv.append(layer._recv_rows if layer._recv_rows is not None else layer.last_recv_rows)
        torch.cuda.synchronize()
        dist.barrier()
        wall = time.perf_counter() - t0
        ms = sum(a.elapsed_time(b) for a, b in ev)
        recv = [int(r) for r in recv]  # device counts of the fused form are read only now, after the timed region
        both = torch.tensor([ms, wall * 1e3, float(max(recv)), float(sum(recv)) / steps], device="cuda", dtype=torch.float64)
        mx = both.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = both.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        return mx[0].item(), mx[1].item(), mx[2].item(), sm[3].item() / world

    if rank != 0:
        del w_all, w_all_check
    clocks = ClockSampler(local)
    with clocks:
        total_ms, wall_ms, max_rows, mean_rows = timed(step, args.steps, args.warmup)
        e2e_ms, _, _, _ = timed(e2e_step, args.steps, 1)
    status = torch.tensor([chain.last_status()], device="cuda")
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if rank == 0:
        if int(status.item()):
            raise RuntimeError("a kernel reported a device-side status on some rank")
        per_step = total_ms / args.steps
        peaks = measured_peaks()
        remote = (world - 1) / world  # share of a rank's rows that leave it under uniform routing
        link_bytes = mean_rows * remote * (ROW_BYTES_IN + ROW_BYTES_OUT)
        t_link = link_bytes / (NVLINK_GBS_MEASURED * 1e9)
        t_fp4 = tokens_global / world * FLOPS_PER_TOKEN / (4 * peaks["bf16_tflops"] * 1e12)
        one_gpu = one_gpu_same_workload(w_all, flush, tokens_global, zipf, args.steps)
        cfg = workload_config(tokens_global, world)
        cfg.update({"tokens_per_rank": t_loc, "expert_placement": placement, "routing_skew": "zipf 1.1" if zipf else "none",
                    "combine": "GEMM2 epilogue stores into the owner's slot buffer over NVLink peer mappings" if layer.peer
                    else "NCCL all-to-all of bf16 slot rows",
                    "max_rows_received_by_a_rank": max_rows, "mean_rows_received_per_rank": mean_rows,
                    "timing": ("CUDA-graph replay of the whole step (ordering points between the ranks included)" if graphs else "eager calls")
                    + ", CUDA events per step on every rank after the untimed L2 flush, max over ranks"})
        line = {"metric": "moe_layer_tokens_per_s", "value": tokens_global / (per_step * 1e-3), "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "mxfp4", "data": "synthetic",
                "config": cfg,
                "roofline": {"kernel": "expert-parallel step (dispatch all-to-all + grouped GEMMs + combine all-to-all)",
                             "bound": "nvlink" if t_link > t_fp4 else "tensor", "unit": "us",
                             "nvlink_us": t_link * 1e6, "fp4_us": t_fp4 * 1e6, "achieved": per_step * 1e3,
                             "peak": max(t_link, t_fp4) * 1e6, "frac": max(t_link, t_fp4) * 1e3 / per_step,
                             "nvlink_bytes_per_rank_per_direction": link_bytes, "nvlink_gbs_peak": NVLINK_GBS_MEASURED,
                             "traffic": None},
                "cpu_baseline": None,
                "parity_checked": parity_ok, "parity_mismatching_elements": parity_bad,
                "parity_note": "every rank, its own tokens, 2 inputs: bit-for-bit against the single-GPU layer with all 128 experts",
                "one_gpu_same_workload": one_gpu,
                "e2e": {"value": tokens_global / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": tokens_global * (2 * H + 4 * E), "d2h_bytes_per_step": tokens_global * 2 * H},
                "gpu_launches": args.steps * 8, "wall_ms_per_step": wall_ms / args.steps, "clocks": clocks.summary()}
        return line
    return None
