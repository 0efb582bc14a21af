"""Expert parallel on 2, 4 and 8 GPUs (each skipped with fewer): both forms (NCCL all-to-all dispatch and combine; dispatch
and combine fused into the kernels over NVLink peer mappings), both expert placements. Every rank's output equals, bit for
bit, the single-GPU layer on the same tokens with all the experts. Ranks are child processes; NVLS is off and torch's
symmetric memory is kept from binding the buffers to a multicast object, so a rank that ends early cannot disturb the
others' GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, placement, experts, errors):
    try:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        import torch.distributed as dist
        from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain, ep
        from oracle import moe_oracle as orc
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        (w13, s13, w2, s2), _ = orc.make_weights(seed=5, experts=experts)
        mine = ep.local_expert_ids(rank, world, experts, placement).numpy()
        cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
        w_local = chain.MoeWeights.from_row_major(None, None, *(cu(a[mine]) for a in (w13, s13, w2, s2)))
        w_all = chain.MoeWeights.from_row_major(None, None, *(cu(a) for a in (w13, s13, w2, s2)), routing_mode="softmax",
                                                routed_scaling_factor=1.0)
        tokens = 40 + 8 * rank
        gen = torch.Generator().manual_seed(900 + rank)
        xb, lg = orc.make_inputs(gen, tokens, experts=experts)
        x = cu(xb.view(np.int16)).view(torch.bfloat16)
        logits = cu(lg)
        ref = chain.mxfp4_moe(x, w_all, router_logits=logits)
        for peer_pairs in (0, 4 * 96):  # all-to-all combine, then the combine fused into GEMM2 over peer mappings
            par = ep.ExpertParallelMoe(w_local, None, routing_mode="softmax", scale=1.0, placement=placement,
                                       experts=experts, peer_pairs=peer_pairs)
            assert peer_pairs == 0 or par.peer is not None, "peer mapping of the slot buffers failed"
            for _ in range(2):
                out = par.forward(x, logits)
                torch.cuda.synchronize()
                assert torch.equal(out, ref), f"expert-parallel output differs from the single-GPU layer ({peer_pairs})"
        assert chain.last_status() == 0
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:
        errors.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("world,experts,placement", [(2, 8, "contiguous"), (2, 8, "interleaved"), (4, 8, "contiguous"),
                                                     (4, 16, "interleaved"), (8, 16, "contiguous"), (8, 128, "interleaved")])
def test_expert_parallel_equals_single_gpu(world, experts, placement):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, placement, experts, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not alive and not msgs and all(p.exitcode == 0 for p in procs), msgs
