"""Expert parallel on 2 GPUs (skipped with fewer): NCCL all-to-all dispatch and combine, 4 experts per rank. Every rank's
output equals, bit for bit, the single-GPU layer on the same tokens with all 8 experts."""
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


def _worker(rank, world, port, placement, errors):
    try:
        import torch.distributed as dist
        from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain, ep
        from oracle import moe_oracle as orc
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        experts = 8
        (w13, s13, w2, s2), _ = orc.make_weights(seed=5, experts=experts)
        mine = ep.local_expert_ids(rank, world, experts, placement).numpy()
        cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
        w_local = chain.MoeWeights.from_row_major(None, None, *(cu(a[mine]) for a in (w13, s13, w2, s2)))
        w_all = chain.MoeWeights.from_row_major(None, None, *(cu(a) for a in (w13, s13, w2, s2)), routing_mode="softmax",
                                                routed_scaling_factor=1.0)
        tokens = 40 + 24 * rank
        gen = torch.Generator().manual_seed(900 + rank)
        xb, lg = orc.make_inputs(gen, tokens, experts=experts)
        x = cu(xb.view(np.int16)).view(torch.bfloat16)
        logits = cu(lg)
        ref = chain.mxfp4_moe(x, w_all, router_logits=logits)
        for peer_pairs in (0, 4 * 64):  # all-to-all combine, then the combine fused into GEMM2 over peer mappings
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


@pytest.mark.parametrize("placement", ["contiguous", "interleaved"])
def test_two_gpu_expert_parallel_equals_single_gpu(placement):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, placement, errors)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    assert not alive and not msgs and all(p.exitcode == 0 for p in procs), msgs
