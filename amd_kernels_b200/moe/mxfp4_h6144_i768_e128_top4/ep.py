"""Expert-parallel form of the routed MXFP4 MoE layer: the 128 experts are sharded over W ranks (one process per GPU),
every rank routes its own tokens, sends each (token, slot) pair's quantised row to the rank that owns the expert
(all-to-all over NCCL), runs the grouped GEMMs on the rows it received and returns the bf16 slot rows (second
all-to-all); the source rank sums a token's four slots in slot order.

The reference has no expert parallelism (its multi-GPU form is tensor parallel with a sequence-parallel gather,
amd_kernels/moe/mxfp4_h6144_i768_e128_top4/prepared_input.py:116-209); what carries over is its idea of shipping the
quantised activations (3264 bytes per row) instead of bf16 (12288 bytes), and its fixed-order combine
(amd_kernels/collectives/pull_collectives_ranks4/reference.py:74-91). Because a (token, slot) row is one accumulator
column of the grouped GEMMs whatever else is in the batch, and the combine adds slots 0..3 in order, the result is
bit-identical to the single-GPU layer for every W.

The exchange bookkeeping (``plan_dispatch`` / ``scatter_combined``) is plain index arithmetic on torch tensors and runs
on CPU tensors too, which is how the world_size-2 gloo tests exercise it without a GPU.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

# Only plain peer pointers are taken from torch's symmetric memory. Its rendezvous would otherwise also bind the buffers
# to an NVLink multicast object on NVSwitch machines, and a rank that ends while its memory is bound to one can raise
# NVLink faults on the other ranks' GPUs. Must be set before the first symmetric-memory use in the process.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741


def expert_owner(ids: torch.Tensor, world: int, experts: int = E, placement: str = "contiguous"):
    """(owning rank, expert id local to that rank) of global expert ids. "contiguous": rank r owns experts
    [r*E/W, (r+1)*E/W); "interleaved": expert e lives on rank e % W (spreads a popularity ranking that follows the id)."""
    per = experts // world
    if placement == "contiguous":
        return ids // per, ids % per
    if placement == "interleaved":
        return ids % world, ids // world
    raise ValueError("placement must be 'contiguous' or 'interleaved'")


def local_expert_ids(rank: int, world: int, experts: int = E, placement: str = "contiguous") -> torch.Tensor:
    """Global ids of the experts rank ``rank`` owns, in local-id order."""
    per = experts // world
    if placement == "contiguous":
        return torch.arange(rank * per, (rank + 1) * per)
    return torch.arange(per) * world + rank


@dataclass
class DispatchPlan:
    order: torch.Tensor        # int64 [4T]: pair index q = 4*token+slot of each sent row, grouped by destination rank
    send_counts: list          # rows per destination rank
    local_expert: torch.Tensor  # int32 [4T]: the expert id on the destination rank, in send order
    weight: torch.Tensor       # fp32 [4T]: the routing weight, in send order


def plan_dispatch(topk_ids: torch.Tensor, topk_weights: torch.Tensor, world: int, experts: int = E,
                  placement: str = "contiguous") -> DispatchPlan:
    """Group the 4T pairs by destination rank, keeping pair order inside a destination."""
    dest, local = expert_owner(topk_ids.reshape(-1).long(), world, experts, placement)
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    return DispatchPlan(order, counts.tolist(), local[order].int(), topk_weights.reshape(-1)[order].float())


def exchange_counts(send_counts, group) -> list:
    """All-to-all of the per-destination row counts -> rows arriving from every source rank."""
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    send = torch.tensor(send_counts, dtype=torch.int64, device=device)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.tolist()


def all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    """Variable-size all-to-all of whole rows (dim 0)."""
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def scatter_combined(returned: torch.Tensor, plan: DispatchPlan, tokens: int) -> torch.Tensor:
    """Rows that came back in send order -> slots [T, 4, width] (row q = 4*token+slot)."""
    slots = returned.new_empty((tokens * TOPK,) + tuple(returned.shape[1:]))
    slots[plan.order] = returned
    return slots.view(tokens, TOPK, *returned.shape[1:])


class PeerBuffers:
    """Buffers of one rank that every other rank of the node can store into (torch symmetric memory: virtual-memory
    handles mapped with access for the local device; the stores themselves are plain peer stores over NVLink):
    ``slots`` bf16 [pairs, 6144] where GEMM2 on any rank deposits this rank's result rows, and the receive buffers of
    the dispatch (codes, row-major scales, meta as four column arrays) with room for every pair of every rank (the worst
    routing skew)."""

    def __init__(self, max_pairs: int, group=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_pairs, self.capacity = max_pairs, max_pairs * world
        shapes = {"slots": ((max_pairs, H), torch.bfloat16), "codes": ((self.capacity, H // 2), torch.uint8),
                  "scales": ((self.capacity, H // 32), torch.uint8), "meta": ((4, self.capacity), torch.int32),
                  # the ordering points of a step (b200moe_ep_sync): one flag per source rank, and the W x W matrix of
                  # row counts every rank deposits its row of
                  "flags": ((64,), torch.int32), "matrix": ((world, world), torch.int64)}
        self.local, self.ptrs, self._handles = {}, {}, []
        dev = torch.device("cuda", torch.cuda.current_device())
        for name, (shape, dtype) in shapes.items():
            if world == 1:  # nothing to map
                buf = torch.zeros(shape, dtype=dtype, device=dev)
                ptrs = [buf.data_ptr()]
            else:
                buf = symm_mem.empty(shape, dtype=dtype, device=dev)
                buf.zero_()
                handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
                ptrs = [int(p) for p in handle.buffer_ptrs]
                if len(ptrs) != world or ptrs[rank] != buf.data_ptr():
                    raise RuntimeError("unexpected symmetric-memory layout")
                self._handles.append(handle)
            self.local[name] = buf
            self.ptrs[name] = (ctypes.c_void_p * world)(*ptrs)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)


class ExpertParallelMoe:
    """One rank of the expert-parallel layer. ``weights`` holds this rank's experts only
    (``MoeWeights.from_row_major`` on the slice ``local_expert_ids(rank, world)`` of the checkpoint); routing parameters
    (bias over all 128 experts, mode, scale) describe the global router."""

    # Prefill sizes of the fused form: chunks the row blocks are cut into (by world size; 1 = no overlap), and the SMs GEMM2
    # of one chunk gets while GEMM1 of the next runs on the others. Measured with the 16384-token workload: at 2 ranks
    # (GEMM1 175 us, GEMM2 + combine 270 us per rank) 8 chunks with 64 SMs for GEMM2 take 0.697 ms per step against 0.745
    # without overlap (32 / 48 / 80 / 96 SMs: 0.877 / 0.759 / 0.804 / 0.837; 4 chunks: 0.718); at 4 ranks, where GEMM1 is
    # 93 us of the step, every setting measured 0.521-0.532 against 0.522: left off there and where it was not measured.
    CHUNKS_BY_WORLD, GEMM2_CTAS = {2: 8}, 64

    def __init__(self, weights, group=None, *, bias=None, routing_mode="softmax", scale=1.0, placement="contiguous",
                 experts: int = E, peer_pairs: int = 0):
        """``peer_pairs`` > 0: fuse the combine into GEMM2 — result rows are stored straight into the owning rank's slot
        buffer (room for ``peer_pairs`` = 4 x the largest local token count) instead of travelling back by all-to-all."""
        self.w, self.group = weights, group
        self.peer = None
        if peer_pairs:
            ok = torch.ones(1, device="cuda")
            try:
                self.peer = PeerBuffers(peer_pairs, group)
            except Exception:  # no peer mapping on this machine: every rank falls back to the all-to-all combine
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if not bool(ok.item()):
                self.peer = None
            self._fence = torch.zeros(1, device="cuda")
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if experts % self.world or weights.num_experts != experts // self.world:
            raise ValueError(f"needs {experts // self.world} local experts on each of {self.world} ranks")
        self.bias, self.mode, self.scale, self.placement, self.experts = bias, routing_mode, float(scale), placement, experts
        self.last_recv_rows, self._recv_rows = 0, None
        if self.peer is not None:  # the send plan lives on the device: nothing of it is read by the host
            dev = torch.device("cuda", torch.cuda.current_device())
            self._dest = torch.empty(self.peer.max_pairs, dtype=torch.int32, device=dev)
            self._counts = torch.zeros(self.world, dtype=torch.int64, device=dev)
            self._matrix = self.peer.local["matrix"]  # every rank stores its row of counts here (and in every peer's copy)
            self._epoch = torch.zeros(1, dtype=torch.int32, device=dev)
            self.chunks = int(os.environ.get("B200MOE_EP_CHUNKS", self.CHUNKS_BY_WORLD.get(self.world, 1)))
            self.gemm2_ctas = int(os.environ.get("B200MOE_EP_GEMM2_CTAS", self.GEMM2_CTAS))
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            self.gemm1_ctas_beside = max(1, sms - self.gemm2_ctas)
            self._side = torch.cuda.Stream(device=dev)
            self._chunk_done = [torch.cuda.Event() for _ in range(max(self.chunks, 1))]
            self._seg_start = torch.zeros(self.world, dtype=torch.int32, device=dev)
            self._dst_base = torch.zeros(self.world, dtype=torch.int64, device=dev)
            self._recv_pairs = torch.zeros(1, dtype=torch.int32, device=dev)

    @property
    def recv_rows(self) -> int:
        """Rows this rank received in the last call (reads the device count of the fused form: synchronises)."""
        return int(self._recv_rows.item()) if self._recv_rows is not None else self.last_recv_rows

    def experts_on_rows(self, codes, scales, local_expert, weight, n, row_rank=None, row_pair=None, live=None):
        """The grouped GEMMs on rows that arrived from any rank: row r < n -> bf16 [6144] = (h_r @ W2[e_r]^T) * weight_r.
        The buffers hold a multiple of four rows; rows beyond n carry expert id -1, or ``live`` (a device int32 scalar)
        says how many rows count: either way the sort drops the rest."""
        from . import chain
        groups = codes.shape[0] // TOPK  # rows are handed to the sort as pseudo-tokens of four pairs
        if n == 0:
            return torch.empty((0, H), dtype=torch.bfloat16, device=codes.device)
        bm = chain.variant_for(groups)
        sort = chain.moe_sort(local_expert.view(groups, TOPK), weight.view(groups, TOPK), bm, self.w.num_experts,
                              live_pairs=live)
        if bm == 128 and row_rank is not None and self.chunks > 1:
            # GEMM2 with the combine in its epilogue is bound by the link, GEMM1 by the tensor cores: the row blocks are cut
            # into chunks, and GEMM2 of a chunk runs on a second stream (on GEMM2_CTAS SMs) beside GEMM1 of the next chunk
            # (on the others). Events order a chunk's GEMM2 behind its GEMM1; the streams are joined before returning.
            main, side = torch.cuda.current_stream(), self._side
            ranges = chain.block_chunks(sort, self.chunks)
            out = None
            for c in range(self.chunks):
                out = chain.grouped_gemm1_gather(codes, scales, sort, self.w, by_pair=True, block_range=ranges[c],
                                                 max_ctas=0 if c == 0 else self.gemm1_ctas_beside, out=out)
                self._chunk_done[c].record(main)
                side.wait_event(self._chunk_done[c])
                with torch.cuda.stream(side):
                    chain.grouped_gemm2_peer(out[0], out[1], sort, self.w, row_rank, row_pair, self.peer.ptrs["slots"],
                                             self.world, self.peer.max_pairs, block_range=ranges[c],
                                             max_ctas=self.gemm2_ctas)
            main.wait_stream(side)
            return None
        if bm == 128:  # GEMM1 reads the received rows through the sorted list itself: no sorted copy
            hq, sfh = chain.grouped_gemm1_gather(codes, scales, sort, self.w, by_pair=True)
        else:
            xq, sfx = chain.dispatch_rows((codes, scales), sort, by_pair=True)
            hq, sfh = chain.grouped_gemm1(xq, sfx, sort, self.w)
        if row_rank is not None:
            chain.grouped_gemm2_peer(hq, sfh, sort, self.w, row_rank, row_pair, self.peer.ptrs["slots"], self.world,
                                     self.peer.max_pairs)
            return None
        slots = chain.grouped_gemm2(hq, sfh, sort, self.w)
        return slots.view(groups * TOPK, H)[:n]

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor, *, return_partials=False):
        """x bf16 [T_local, 6144], fp32 logits [T_local, 128] -> bf16 [T_local, 6144] (or the slots [T_local, 4, 6144])."""
        from . import chain
        tokens = x.shape[0]
        chain.variant_for(tokens)
        wt, ids = chain.topk_route(router_logits, self.bias, self.scale, self.mode)
        if self.peer is not None:
            # every rank must take the same branch (the two forms issue different collectives): the slot buffers were
            # sized at construction, so a batch that does not fit is an error here, not a silent change of path
            if tokens * TOPK > self.peer.max_pairs:
                raise ValueError(f"{tokens} tokens exceed the peer slot buffer ({self.peer.max_pairs // TOPK} tokens): "
                                 "construct ExpertParallelMoe with a larger peer_pairs")
            return self._forward_peer(x, wt, ids, return_partials)
        codes, scales = chain.mxfp4_quant(x)
        # where every pair goes; the row counts cross the ranks and reach the host in one read
        dest, local = expert_owner(ids.reshape(-1).long(), self.world, self.experts, self.placement)
        order = torch.argsort(dest, stable=True)
        counts = torch.bincount(dest, minlength=self.world)
        arrived = torch.empty_like(counts)
        dist.all_to_all_single(arrived, counts, group=self.group)
        send_counts, recv_counts = torch.stack([counts, arrived]).tolist()
        n = sum(recv_counts)
        padded = (n + TOPK - 1) // TOPK * TOPK
        self.last_recv_rows, self._recv_rows = n, None
        src_token = order // TOPK
        meta = torch.stack([local[order].int(), wt.reshape(-1)[order].view(torch.int32)], dim=1)

        def exchange(rows, width, dtype, fill=None):
            out = torch.empty((padded, width), dtype=dtype, device=x.device)
            if fill is not None and padded > n:
                out[n:] = fill
            dist.all_to_all_single(out[:n], rows.contiguous(), output_split_sizes=recv_counts,
                                   input_split_sizes=send_counts, group=self.group)
            return out

        r_codes = exchange(codes.index_select(0, src_token), H // 2, torch.uint8, 0)
        r_scales = exchange(scales.index_select(0, src_token), H // 32, torch.uint8, 0)
        r_meta = exchange(meta, 2, torch.int32, -1)
        r_expert, r_weight = r_meta[:, 0].contiguous(), r_meta[:, 1].contiguous().view(torch.float32)
        y = self.experts_on_rows(r_codes, r_scales, r_expert, r_weight, n)
        back = torch.empty((tokens * TOPK, H), dtype=torch.bfloat16, device=x.device)
        dist.all_to_all_single(back, y.contiguous(), output_split_sizes=send_counts, input_split_sizes=recv_counts,
                               group=self.group)
        # pair q sits in row where[q] of what came back (send order); the reduce reads through that index
        where = torch.empty(tokens * TOPK, dtype=torch.int32, device=x.device)
        where[order] = torch.arange(tokens * TOPK, dtype=torch.int32, device=x.device)
        if return_partials:
            return back.index_select(0, where.long()).view(tokens, TOPK, H)
        return chain.reduce_rows(back, where, tokens)

    def _sync(self, stream, counts: bool = False):
        """One ordering point between the ranks (``b200moe_ep_sync``: flags over the peer mappings, no collective call);
        ``counts``: the launch also deposits this rank's row of the send-count matrix with every rank."""
        import ctypes
        from . import chain
        from ... import _lib
        peer = self.peer
        _lib.check(_lib.load().b200moe_ep_sync(
            peer.ptrs["flags"], peer.ptrs["matrix"] if counts else None,
            ctypes.c_void_p(self._counts.data_ptr()) if counts else None, self.world, self.rank,
            ctypes.c_void_p(self._epoch.data_ptr()), ctypes.c_void_p(chain.status_word(self._epoch.device).data_ptr()),
            stream), "ep_sync")

    def _forward_peer(self, x, wt, ids, return_partials):
        """The fused form: (1) the pairs are grouped by destination rank by the routing-sort kernel; (2) one kernel
        quantises every pair's row and stores it into the destination's receive buffers; (3) the grouped GEMMs run on
        what arrived and GEMM2 stores every result row into its owner's slot buffer; (4) the owner reduces. Between the
        phases one tiny all-reduce orders the ranks. Nothing is read by the host: the W x W matrix of row counts stays on
        the device, so the step can run ahead of the CPU and be captured in a CUDA graph."""
        import ctypes
        from . import chain
        from ... import _lib
        tokens, dev, peer = x.shape[0], x.device, self.peer
        lib, st = _lib.load(), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        dest = self._dest[:tokens * TOPK]
        _lib.check(lib.b200moe_ep_dest(p(ids), tokens, self.world, self.experts // self.world,
                                       int(self.placement == "interleaved"), p(dest), p(self._counts), st), "ep_dest")
        send = chain.moe_sort(dest.view(tokens, TOPK), wt, 1, self.world)       # send order: pairs grouped by rank
        self._sync(st, counts=True)                                         # matrix[s][d]: rows from rank s to rank d
        _lib.check(lib.b200moe_ep_offsets(p(self._matrix), self.world, self.rank, p(self._seg_start), p(self._dst_base),
                                          p(self._recv_pairs), st), "ep_offsets")
        self._recv_rows = self._recv_pairs
        _lib.check(lib.b200moe_quant_push(
            p(x), p(ids), p(send.sorted_ids), p(send.sorted_weights), p(send.block_expert), tokens,
            self.world, self.rank, self.experts // self.world, int(self.placement == "interleaved"), peer.ptrs["codes"],
            peer.ptrs["scales"], peer.ptrs["meta"], p(self._dst_base), p(self._seg_start), peer.capacity,
            p(chain.status_word(dev)), st), "quant_push")
        self._sync(st)                                                        # every rank's rows have landed
        # the receive buffers are used at their full capacity: the sort takes the number of rows that arrived from the
        # device, so it never has to reach the host; meta is four column arrays: expert, weight bits, source pair, rank
        cols = peer.local["meta"]
        self.experts_on_rows(peer.local["codes"], peer.local["scales"], cols[0], cols[1].view(torch.float32),
                             peer.capacity, cols[3], cols[2], live=self._recv_pairs)
        self._sync(st)                                                        # every rank's result rows have landed
        slots = peer.local["slots"][:tokens * TOPK].view(tokens, TOPK, H)
        return slots.clone() if return_partials else chain.reduce_slots(slots)
