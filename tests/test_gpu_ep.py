"""Expert parallelism on real GPUs: 2 ranks over NCCL against the single-GPU layer and the CPU oracle."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

pytestmark = pytest.mark.gpu
E, K, H, I, B, T_LOCAL = 8, 2, 512, 256, 128, 300


def _inputs(rank):
    from moe_testlib import bf16_values, make_rows_weights
    rng = np.random.default_rng(200 + rank)
    hidden = bf16_values(rng.standard_normal((T_LOCAL, H)).astype(np.float32))
    router_w = bf16_values((np.random.default_rng(3).standard_normal((H, E)) * 0.05).astype(np.float32))
    return hidden, router_w, make_rows_weights(E, H, I, seed=9)


def _worker(rank, world, port, results, backend):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import nki_library_b200 as m
        from nki_library_b200.ep import CudaOps, ExpertParallelMoE, PeerExpertParallelMoE
        hidden, router_w, w_np = _inputs(rank)
        e_l = E // world
        local = m.prepare_from_rows(*(torch.from_numpy(np.ascontiguousarray(a[rank * e_l:(rank + 1) * e_l])).cuda()
                                      for a in w_np))
        x = torch.from_numpy(hidden).to(torch.bfloat16).cuda()
        if backend == "nccl":
            layer = ExpertParallelMoE(CudaOps(torch.from_numpy(router_w).cuda(), local, E, K, B), E)
            out = layer.forward(x).clone()
            out2 = layer.forward(x).clone()
            rows = layer.last_rows_received
        else:
            layer = PeerExpertParallelMoE(torch.from_numpy(router_w).cuda(), local, E, K, B, T_LOCAL,
                                          fuse_return=backend == "peer")
            out = layer.forward(x).clone()
            out2 = layer.forward(x).clone()
            out3 = layer.forward(x).clone()
            assert not any(layer.device_status()), layer.device_status()
            assert torch.equal(out2, out3)
            rows = int((layer.row_valid >= 0).sum().item())
        torch.cuda.synchronize()
        results[rank] = (out.float().cpu().numpy(), bool(torch.equal(out, out2)), rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fuse_return", [True, False])
def test_peer_memory_exchange_single_rank(fuse_return):
    """World size 1: every 'peer' is this GPU, so the dispatch / plan / return kernels run without a second device.
    ``fuse_return``: the down contraction stores its rows into the (peer) result buffer itself, or a separate
    kernel copies them out of y_pos."""
    import nki_library_b200 as m
    from moe_testlib import bf16_values, max_rel
    from nki_library_b200.ep import PeerExpertParallelMoE
    from nki_library_b200.layer import MoELayer
    from oracle import moe, routing
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29733")
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        hidden, router_w, w_np = _inputs(0)
        full = m.prepare_from_rows(*(torch.from_numpy(a).cuda() for a in w_np))
        x = torch.from_numpy(hidden).to(torch.bfloat16).cuda()
        layer = PeerExpertParallelMoE(torch.from_numpy(router_w).cuda(), full, E, K, B, T_LOCAL,
                                      fuse_return=fuse_return)
        out = layer.forward(x).clone()
        out2 = layer.forward(x).clone()
        assert not any(layer.device_status()), layer.device_status()
        assert torch.equal(out, out2)
        assert int((layer.row_valid >= 0).sum().item()) == T_LOCAL * K
        ref_gpu = MoELayer(torch.from_numpy(router_w).cuda(), full, K, B, T_LOCAL).forward(x)
        assert max_rel(out.float().cpu().numpy(), ref_gpu.float().cpu().numpy()) <= 1e-2
        _, idx, aff = routing.router_topk(torch.from_numpy(hidden), torch.from_numpy(router_w), None, K,
                                          routing.SOFTMAX, True, True)
        ref = moe.moe_tkg_rows(hidden, aff.numpy(), idx.numpy(), *w_np)
        assert max_rel(out.float().cpu().numpy(), bf16_values(ref)) <= 2e-2
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("backend", ["nccl", "peer", "peer_unfused"])
def test_expert_parallel_two_gpus_matches_oracle_and_single_gpu(backend):
    import nki_library_b200 as m
    from moe_testlib import bf16_values, max_rel
    from nki_library_b200.layer import MoELayer
    from oracle import moe, routing
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = {"nccl": 29711, "peer": 29712, "peer_unfused": 29713}[backend]
    mp.spawn(_worker, args=(world, port, results, backend), nprocs=world, join=True)
    rows = 0
    for rank in range(world):
        hidden, router_w, w_np = _inputs(rank)
        got, deterministic, r = results[rank]
        rows += r
        assert deterministic
        # single-GPU layer with all experts on the same tokens
        full = m.prepare_from_rows(*(torch.from_numpy(a).cuda() for a in w_np))
        single = MoELayer(torch.from_numpy(router_w).cuda(), full, K, B, T_LOCAL)
        ref_gpu = single.forward(torch.from_numpy(hidden).to(torch.bfloat16).cuda()).float().cpu().numpy()
        assert max_rel(got, ref_gpu) <= 1e-2
        # CPU oracle of the whole layer
        _, idx, aff = routing.router_topk(torch.from_numpy(hidden), torch.from_numpy(router_w), None, K,
                                          routing.SOFTMAX, True, True)
        ref = moe.moe_tkg_rows(hidden, aff.numpy(), idx.numpy(), *w_np)
        assert max_rel(got, bf16_values(ref)) <= 2e-2
    assert rows == world * T_LOCAL * K
