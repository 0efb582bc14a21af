"""World-size-2 gloo tests (CPU) of the expert-parallel exchange bookkeeping: every (token, slot) row reaches the rank
that owns its expert, comes back to its own slot, and split sizes agree on both sides — for both expert placements and
for skewed routing where one rank receives almost everything. The expert computation is replaced by a stand-in that
depends on (expert, weight, row payload), since the real one needs a GPU."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, placement, skew, errors):
    try:
        from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import ep
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(100 + rank)
        tokens, width = 5 + 3 * rank, 24
        if skew:  # everything on the experts of rank 0 (contiguous) / of one parity (interleaved)
            ids = torch.stack([torch.randperm(32, generator=g)[:4] * (1 if placement == "contiguous" else 2)
                               for _ in range(tokens)]).int()
        else:
            ids = torch.stack([torch.randperm(128, generator=g)[:4] for _ in range(tokens)]).int()
        ids[0, 1] = ids[0, 0]  # one expert twice in a token
        wts = torch.rand((tokens, 4), generator=g)
        payload = torch.randint(0, 256, (tokens, width), generator=g, dtype=torch.uint8)
        plan = ep.plan_dispatch(ids, wts, world, placement=placement)
        assert sum(plan.send_counts) == 4 * tokens
        recv_counts = ep.exchange_counts(plan.send_counts, None)
        rows = ep.all_to_all_rows(payload.index_select(0, plan.order // 4), plan.send_counts, recv_counts, None)
        meta = ep.all_to_all_rows(torch.stack([plan.local_expert, plan.weight.view(torch.int32)], 1), plan.send_counts,
                                  recv_counts, None)
        mine = ep.local_expert_ids(rank, world, placement=placement)
        assert rows.shape[0] == sum(recv_counts) and bool(((meta[:, 0] >= 0) & (meta[:, 0] < 128 // world)).all())
        global_id = mine[meta[:, 0].long()]
        # stand-in expert: depends on the expert, the routing weight and the row's bytes
        y = (global_id.float() + 1)[:, None] * meta[:, 1].contiguous().view(torch.float32)[:, None] * rows.float()
        back = ep.all_to_all_rows(y, recv_counts, plan.send_counts, None)
        slots = ep.scatter_combined(back, plan, tokens)
        expect = (ids.float() + 1)[:, :, None] * wts[:, :, None] * payload.float()[:, None, :]
        assert torch.equal(slots, expect), "a row came back to the wrong slot or from the wrong expert"
        owner, local = ep.expert_owner(ids.long(), world, placement=placement)
        assert torch.equal(ep.local_expert_ids(0, world, placement=placement)[local[owner == 0]], ids.long()[owner == 0])
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # collected, so every rank leaves the collectives the same way
        errors.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("placement", ["contiguous", "interleaved"])
@pytest.mark.parametrize("skew", [False, True])
def test_exchange_round_trip_world_2(placement, skew):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, placement, skew, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()  # exactly the processes this test started
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not alive and not msgs and all(p.exitcode == 0 for p in procs), msgs


def test_rejects_uneven_sharding():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import ep
    with pytest.raises(ValueError):
        ep.expert_owner(torch.zeros(4, dtype=torch.long), 2, placement="ring")
    assert ep.local_expert_ids(1, 4).tolist() == list(range(32, 64))
    assert ep.local_expert_ids(1, 4, placement="interleaved").tolist()[:3] == [1, 5, 9]
