"""Expert-parallel exchange logic on CPU: two gloo ranks, expert compute stood in by the oracle.

Checks the bookkeeping of ``nki_library_b200.ep.ExpertParallelMoE`` (pair sort, split sizes, row -> expert
reconstruction, reverse exchange, combine) against a single-process oracle of the whole layer.  The CUDA kernels
are not involved; ``OracleOps`` below exists only in this test.
"""

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

E, K, H, I, T_LOCAL = 4, 2, 64, 64, 37


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _inputs(rank):
    from moe_testlib import make_rows_weights
    rng = np.random.default_rng(100 + rank)
    hidden = _bf16(rng.standard_normal((T_LOCAL, H)).astype(np.float32))
    wr = np.random.default_rng(7)
    router_w = _bf16((wr.standard_normal((H, E)) * 0.3).astype(np.float32))
    return hidden, router_w, make_rows_weights(E, H, I, seed=5)


class OracleOps:
    def __init__(self, router_w, w_np_local):
        self.router_w, self.w = router_w, w_np_local

    def route(self, hidden):
        from oracle import routing
        _, idx, aff = routing.router_topk(hidden, torch.from_numpy(self.router_w), None, K, routing.SOFTMAX, True, True)
        return idx.to(torch.int32), aff.float()

    def sort_pairs(self, idx):
        from oracle import routing
        mask = routing.mask_from_index(idx.numpy(), E)
        T = idx.shape[0]
        tpi, b2e, _, counts = routing.group_tokens(mask, 1, T * K)
        inv = routing.inverse_map(tpi, b2e, idx.numpy(), 1)
        return torch.from_numpy(tpi), torch.from_numpy(b2e), torch.from_numpy(inv), torch.from_numpy(counts)

    def gather_rows(self, src, index):
        return src[index.to(torch.int64)].contiguous()

    def experts(self, rows, row_expert, row_aff):
        from oracle import moe
        out = np.zeros((rows.shape[0], H), dtype=np.float32)
        r = rows.float().numpy()
        for e in range(self.w[0].shape[0]):
            sel = np.flatnonzero(row_expert.numpy() == e)
            if sel.size:
                y = moe.expert_mlp_rows(r[sel], moe.ExpertWeights(*self.w, e))
                out[sel] = y * row_aff.numpy()[sel, None]
        return torch.from_numpy(out).to(torch.bfloat16)

    def combine(self, rows_back, inv):
        g = rows_back.float()[inv.to(torch.int64)]  # [T, K, H]
        return g.sum(dim=1).to(torch.bfloat16)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nki_library_b200.ep import ExpertParallelMoE
        hidden, router_w, w_np = _inputs(rank)
        e_l = E // world
        local = tuple(a[rank * e_l:(rank + 1) * e_l] for a in w_np)
        layer = ExpertParallelMoE(OracleOps(router_w, local), E)
        out = layer.forward(torch.from_numpy(hidden).to(torch.bfloat16))
        results[rank] = (out.float().numpy(), layer.last_rows_received)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_exchange_matches_single_process(world):
    from oracle import moe, routing
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29600 + world
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    total_rows = 0
    for rank in range(world):
        hidden, router_w, w_np = _inputs(rank)
        _, idx, aff = routing.router_topk(torch.from_numpy(hidden), torch.from_numpy(router_w), None, K,
                                          routing.SOFTMAX, True, True)
        ref = np.zeros((T_LOCAL, H), dtype=np.float32)
        for e in range(E):
            tok = np.flatnonzero((idx.numpy() == e).any(axis=1))
            if tok.size:
                y = moe.expert_mlp_rows(hidden[tok], moe.ExpertWeights(*w_np, e)) * aff.numpy()[tok, e][:, None]
                ref[tok] += _bf16(y)
        got, rows = results[rank]
        total_rows += rows
        assert np.abs(got - _bf16(ref)).max() <= 1e-2 * np.abs(ref).max()
    assert total_rows == world * T_LOCAL * K  # every (token, k) pair was dispatched exactly once


def test_dispatch_plan_row_order():
    from nki_library_b200.ep import dispatch_plan
    counts = torch.tensor([2, 0, 1, 3], dtype=torch.int32)            # this rank sends 2+0 rows to rank 0, 1+3 to rank 1
    recv = torch.tensor([[1, 2], [0, 3]], dtype=torch.int32)           # from rank 0: 1 row for e0, 2 for e1; rank 1: 0, 3
    ins, outs, row_e = dispatch_plan(counts, recv, 2, 2)
    assert ins == [2, 4] and outs == [3, 3]
    assert row_e.tolist() == [0, 1, 1, 1, 1, 1]
