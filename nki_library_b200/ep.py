"""Expert parallelism: one process per GPU, experts sharded, tokens data-parallel.

Rank r owns experts ``[r * E_L, (r + 1) * E_L)`` -- the reference's
``rank_id * E_L`` slice (core/moe/moe_tkg/moe_tkg.py:100-101).  A forward pass:

1. route the local tokens (``router_topk``), sort the (token, k) pairs by expert
   (stable in the token id, the grouping kernel with block size 1);
2. exchange per-expert row counts (``all_to_all_single``), then **dispatch** the
   pairs' hidden rows and their affinities to the owning ranks
   (``all_to_all_single`` with split sizes, NCCL over NVLink);
3. group the received rows by local expert into blocks and run the blockwise
   MXFP8 expert MLP (affinity applied per row);
4. **combine**: send every row's result back (reverse split sizes) and sum each
   token's K rows in fixed order.

The reference has no all-to-all of its own: its expert-parallel mode replicates
tokens or consumes an external ``all_to_all_v`` buffer
(experimental/collectives/topk_reduce.py:15,37-62).  The exchange logic here is
backend-agnostic (``ops`` object); the CUDA operations are in :class:`CudaOps`.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _lib, pipeline
from .core.moe.moe_cte.group_tokens import moe_group_tokens
from .core.moe.moe_cte.moe_cte_utils import get_n_blocks
from .core.utils.common_types import ActFnType, RouterActFnType
from .weights import ExpertWeights


def dispatch_plan(counts: torch.Tensor, recv_counts: torch.Tensor, world: int, experts_local: int):
    """Split sizes and the local-expert id of every received row.

    ``counts [E]``: rows this rank sends per global expert; ``recv_counts
    [world, E_L]``: rows each source rank sends to each of this rank's experts.
    Rows arrive source-major and, inside a source, in expert order.
    """
    both = torch.stack([counts.view(world, experts_local).sum(dim=1), recv_counts.sum(dim=1)]).tolist()  # one sync
    in_splits = [int(v) for v in both[0]]
    out_splits = [int(v) for v in both[1]]
    local_ids = torch.arange(experts_local, dtype=torch.int32, device=recv_counts.device).repeat(world)
    row_expert = torch.repeat_interleave(local_ids, recv_counts.reshape(-1).to(torch.int64),
                                         output_size=sum(out_splits))
    return in_splits, out_splits, row_expert


class CudaOps:
    """The device side of the expert-parallel layer (C-ABI kernels on the current stream)."""

    def __init__(self, router_w, weights: ExpertWeights, num_experts: int, top_k: int, block_size: int,
                 router_bias=None, router_act=RouterActFnType.SOFTMAX, router_pre_norm=True, norm_topk_prob=True,
                 act_fn=ActFnType.SiLU):
        _lib.require_cuda(router_w, router_bias)
        self.w = router_w.to(torch.bfloat16).contiguous()
        self.bias = None if router_bias is None else router_bias.reshape(-1).to(torch.bfloat16).contiguous()
        self.weights, self.E, self.K, self.B = weights, num_experts, top_k, block_size
        self.router_act, self.pre_norm, self.l1, self.act_fn = router_act, router_pre_norm, norm_topk_prob, act_fn
        self.H = weights.H
        self.launches = 0
        self.timers = None  # set to a dict to collect CUDA events around the expert kernels

    def route(self, hidden):
        T = hidden.shape[0]
        dev = hidden.device
        aff = torch.empty((T, self.E), dtype=torch.float32, device=dev)
        idx = torch.empty((T, self.K), dtype=torch.int32, device=dev)
        ws = torch.empty(_lib.load_library().b200moe_router_workspace_bytes(T, self.H, self.E), dtype=torch.uint8,
                         device=dev)
        _lib.call("b200moe_router_topk", _lib.ptr(hidden), 1, _lib.ptr(self.w), _lib.ptr(self.bias), T, self.H, self.E,
                  self.K, self.router_act.value, int(self.pre_norm), int(self.l1), None, _lib.F32, _lib.ptr(idx),
                  _lib.ptr(aff), _lib.F32, _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
        self.launches += 2
        return idx, aff

    def sort_pairs(self, idx):
        """Pairs sorted by expert, stable in the token id: block size 1 turns the grouping kernel into that sort."""
        T, K = idx.shape
        g = moe_group_tokens(idx, self.E, 1, T * K, top_k=K, skip_token=True)
        self.launches += 3
        return g["token_position_to_id"], g["block_to_expert"], g["inverse_map"], g["counts"]

    def gather_rows(self, src, index):
        """``out[p] = src[index[p]]`` (bf16 rows) with the combine kernel's one-candidate form."""
        P = index.numel()
        out = torch.empty((P, src.shape[1]), dtype=torch.bfloat16, device=src.device)
        if P:
            _lib.call("b200moe_combine", _lib.ptr(src), _lib.ptr(index), P, 1, src.shape[1], _lib.ptr(out),
                      _lib.stream_ptr())
            self.launches += 1
        return out

    def experts(self, rows, row_expert, row_aff):
        """Blockwise expert MLP over received rows; returns ``bf16(y * affinity)`` per row."""
        R = rows.shape[0]
        out = torch.empty((R, self.H), dtype=torch.bfloat16, device=rows.device)
        if R == 0:
            return out
        E_L, B = self.weights.E, self.B
        g = moe_group_tokens(row_expert.reshape(R, 1), E_L, B, get_n_blocks(R, 1, E_L, B), top_k=1, skip_token=True)
        pipeline.run_blocks(rows, R, self.weights, g["token_position_to_id"], g["block_to_expert"], g["conditions"], B,
                            row_aff, g["inverse_map"], out, self.act_fn.value, aff_per_row=True, timers=self.timers)
        self.launches += 3 + 4
        return out

    def combine(self, rows_back, inv):
        T, K = inv.shape
        out = torch.empty((T, self.H), dtype=torch.bfloat16, device=rows_back.device)
        _lib.call("b200moe_combine", _lib.ptr(rows_back), _lib.ptr(inv), T, K, self.H, _lib.ptr(out), _lib.stream_ptr())
        self.launches += 1
        return out


class ExpertParallelMoE:
    """MoE layer with experts sharded over the ranks of ``group`` (backend-agnostic exchange logic)."""

    def __init__(self, ops, num_experts: int, group: Optional[dist.ProcessGroup] = None):
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world != 0:
            raise AssertionError(_lib.ERROR_PREFIX + f"num_experts ({num_experts}) must be divisible by the number "
                                 f"of ranks ({self.world})")
        self.E = num_experts
        self.E_L = num_experts // self.world
        self.last_rows_received = 0

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        """``hidden [T_local, H]`` bf16 -> ``[T_local, H]`` bf16."""
        ops, G = self.ops, self.world
        idx, aff = ops.route(hidden)
        tpi, pos_expert, inv, counts = ops.sort_pairs(idx)
        send = ops.gather_rows(hidden, tpi)
        send_aff = aff[tpi.to(torch.int64), pos_expert.to(torch.int64)].contiguous()

        counts_mat = counts.view(G, self.E_L).contiguous()
        recv_counts = torch.empty_like(counts_mat)
        dist.all_to_all_single(recv_counts, counts_mat, group=self.group)
        in_splits, out_splits, row_expert = dispatch_plan(counts, recv_counts, G, self.E_L)  # host sync (split sizes)
        R = sum(out_splits)
        self.last_rows_received = R

        recv = torch.empty((R, hidden.shape[1]), dtype=hidden.dtype, device=hidden.device)
        recv_aff = torch.empty((R,), dtype=send_aff.dtype, device=hidden.device)
        dist.all_to_all_single(recv, send, out_splits, in_splits, group=self.group)
        dist.all_to_all_single(recv_aff, send_aff, out_splits, in_splits, group=self.group)

        y = ops.experts(recv, row_expert, recv_aff)

        back = torch.empty_like(send)
        dist.all_to_all_single(back, y, in_splits, out_splits, group=self.group)
        return ops.combine(back, inv)
