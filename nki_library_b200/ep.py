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
                  _lib.ptr(aff), _lib.F32, 0, _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
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


# --------------------------------------------------------------------------------------------------
# Peer-memory expert parallelism: the exchange is done by this library's own kernels, which store
# straight into the other GPUs' buffers over NVLink.  No collective call and no host synchronisation
# happens inside a step; torch.distributed is only used once, to hand the CUDA IPC handles around.
# --------------------------------------------------------------------------------------------------
import ctypes  # noqa: E402


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerArena:
    """One zero-initialised device allocation per rank, carved into named views and shared with every peer."""

    def __init__(self, layout: dict, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.offsets, off = {}, 0
        for name, (nbytes, _dtype) in layout.items():
            self.offsets[name] = off
            off += _align(nbytes)
        self.arena = torch.zeros(max(off, 1 << 21), dtype=torch.uint8, device=device)
        self.views = {name: self.arena[self.offsets[name]:self.offsets[name] + nbytes].view(dtype)
                      for name, (nbytes, dtype) in layout.items()}
        lib = _lib.load_library()
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_int64(0)
        _lib.call("b200moe_ipc_export", _lib.ptr(self.arena), handle, ctypes.byref(offset))
        mine = (bytes(handle.raw), int(offset.value))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self.bases = []
        for r, (h, o) in enumerate(everyone):
            if r == self.rank:
                self.bases.append(self.arena.data_ptr())
            else:
                out = ctypes.c_void_p(0)
                _lib.call("b200moe_ipc_open", ctypes.create_string_buffer(h, 64), o, ctypes.byref(out))
                self.bases.append(int(out.value))
        del lib
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def peers(self, name: str):
        """Host array of ``world`` device pointers: view ``name`` on every rank."""
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.bases[r] + self.offsets[name]
        return arr


class PeerExpertParallelMoE:
    """Expert-parallel MoE layer whose dispatch and combine are peer-memory kernels (see ``csrc/ep.cu``).

    Each rank's receive buffers hold ``capacity_factor`` times its fair share of (token, k) pairs; if the routing
    sends it more than that, ``device_status()[0]`` becomes 21 and the surplus rows are dropped.
    """

    def __init__(self, router_w, weights: ExpertWeights, num_experts: int, top_k: int, block_size: int,
                 tokens_per_rank: int, group=None, router_bias=None, capacity_factor: float = 2.5,
                 router_act=RouterActFnType.SOFTMAX, router_pre_norm=True, norm_topk_prob=True,
                 act_fn=ActFnType.SiLU, fuse_return: Optional[bool] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        # The down contraction can store its rows into the peers itself (no separate return launch).  Its epilogue
        # owns one row per thread and stores 32 bytes at a time; measured per step on B200 / NVSwitch against the
        # separate, fully coalesced copy kernel at I = 14336: 1.423 vs 1.470 ms at 2 ranks, 1.482 vs 1.546 ms at 4,
        # 1.473 vs 1.532 ms at 8.  A result row of H bf16 values costs 2*H*I flop, so with a small I the rows leave
        # faster than NVLink carries 32-byte pieces and the epilogue stalls the MMAs: at I = 1536 (32768 tokens,
        # top-8, 2 ranks) the fused form took 4.37 ms per step, the separate copy 4.17 ms.
        self.fuse_return = (weights.I >= 4096) if fuse_return is None else bool(fuse_return)
        fuse_return = self.fuse_return
        _lib.kernel_assert(num_experts % self.world == 0,
                           f"num_experts ({num_experts}) must be divisible by the number of ranks ({self.world})")
        _lib.kernel_assert(self.world <= 8, "peer-memory expert parallelism supports at most 8 ranks")
        self.ops = CudaOps(router_w, weights, num_experts, top_k, block_size, router_bias, router_act, router_pre_norm,
                           norm_topk_prob, act_fn)
        self.E, self.E_L, self.K, self.B = num_experts, num_experts // self.world, top_k, block_size
        self.T, self.H, self.I = tokens_per_rank, weights.H, weights.I
        _lib.kernel_assert(weights.E == self.E_L, "weights must hold this rank's experts only")
        dev = router_w.device
        lib = _lib.load_library()
        pairs = self.T * self.K
        self.n_blocks_cap = get_n_blocks(int(capacity_factor * pairs) + 1, 1, self.E_L, self.B)
        self.cap_rows = self.n_blocks_cap * self.B
        layout = {
            "flags": (4 * 8 * 4, torch.int32),
            "counts": (self.world * self.E * 4, torch.int32),
            "row_aff": (self.cap_rows * 4, torch.float32),
            "row_src": (self.cap_rows * 4, torch.int32),
            "sf_rows": (self.cap_rows * (self.H // 32), torch.uint8),   # scale bytes as they arrive: [row][H / 32]
            "xq": (self.cap_rows * self.H, torch.uint8),
            "back": (pairs * self.H * 2, torch.bfloat16),
        }
        self.mem = PeerArena(layout, dev, group)
        v = self.mem.views
        self.counts_all, self.row_aff, self.row_src = v["counts"], v["row_aff"], v["row_src"]
        self.xq, self.sf_rows, self.back = v["xq"], v["sf_rows"], v["back"].view(pairs, self.H)
        self.sf = torch.zeros(lib.b200moe_sf_bytes(self.cap_rows, self.H), dtype=torch.uint8, device=dev)  # atoms, local
        self.p_flags, self.p_counts = self.mem.peers("flags"), self.mem.peers("counts")
        self.p_xq, self.p_sf = self.mem.peers("xq"), self.mem.peers("sf_rows")
        self.p_aff, self.p_src, self.p_back = self.mem.peers("row_aff"), self.mem.peers("row_src"), self.mem.peers("back")
        # receiver-side plan and scratch (local)
        self.b2e = torch.zeros(self.n_blocks_cap, dtype=torch.int32, device=dev)
        self.cond = torch.zeros(self.n_blocks_cap + 2, dtype=torch.int32, device=dev)
        self.row_valid = torch.full((self.cap_rows,), -1, dtype=torch.int32, device=dev)
        self.tile_flags = torch.zeros(self.cap_rows // 128, dtype=torch.int32, device=dev)
        self.mq = torch.empty((self.cap_rows, self.I), dtype=torch.uint8, device=dev)
        self.m_sf = torch.zeros(lib.b200moe_sf_bytes(self.cap_rows, self.I), dtype=torch.uint8, device=dev)
        self.y_pos = torch.empty((self.cap_rows, self.H), dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.out = torch.empty((self.T, self.H), dtype=torch.bfloat16, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        # routing / pair-sort buffers (fixed shapes, so a step is a fixed launch sequence)
        self.aff = torch.empty((self.T, self.E), dtype=torch.float32, device=dev)
        self.idx = torch.empty((self.T, self.K), dtype=torch.int32, device=dev)
        self.rws = torch.empty(lib.b200moe_router_workspace_bytes(self.T, self.H, self.E), dtype=torch.uint8, device=dev)
        self.pair_token = torch.empty(pairs, dtype=torch.int32, device=dev)
        self.pair_expert = torch.empty(pairs, dtype=torch.int32, device=dev)
        self.pair_cond = torch.empty(pairs + 2, dtype=torch.int32, device=dev)
        self.counts = torch.empty(self.E, dtype=torch.int32, device=dev)
        self.inv = torch.empty((self.T, self.K), dtype=torch.int32, device=dev)
        self.gstatus = torch.zeros(1, dtype=torch.int32, device=dev)
        self.gws = torch.empty(lib.b200moe_group_tokens_workspace_bytes(self.T, self.E), dtype=torch.uint8, device=dev)
        self.timers = None
        # router 2, grouping 3, count exchange, dispatch (+ plan), wait, scale re-layout, contractions (CTA-pair
        # launch + left-over launch each when the block size allows pairs), return, wait, combine
        self.kernels_per_forward = (2 + 3 + 1 + 1 + 1 + 1 + (4 if self.B % 256 == 0 else 2) + (0 if fuse_return else 1)
                                    + 1 + 1)
        self._graph = None

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        """``hidden [tokens_per_rank, H]`` bf16 -> bf16 ``[tokens_per_rank, H]`` (this rank's tokens).

        Fourteen or fifteen launches of this library's kernels on the current stream, nothing else: no allocation, no
        collective call, no host synchronisation.  Every rank of the group must call it the same number of times.
        """
        _lib.kernel_assert(tuple(hidden.shape) == (self.T, self.H) and hidden.dtype == torch.bfloat16,
                           "hidden must be bf16 [tokens_per_rank, H]")
        ops, w, st = self.ops, self.ops.weights, _lib.stream_ptr()
        G, E, E_L, K, B, H, I, T = self.world, self.E, self.E_L, self.K, self.B, self.H, self.I, self.T
        status, epoch = _lib.ptr(self.status), _lib.ptr(self.epoch)
        nan = float("nan")

        def mark(name):
            if self.timers is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self.timers.setdefault(name, []).append(ev)

        _lib.call("b200moe_router_topk", _lib.ptr(hidden), 1, _lib.ptr(ops.w), _lib.ptr(ops.bias), T, H, E, K,
                  ops.router_act.value, int(ops.pre_norm), int(ops.l1), None, _lib.F32, _lib.ptr(self.idx),
                  _lib.ptr(self.aff), _lib.F32, 0, _lib.ptr(self.rws), self.rws.numel(), st)
        # block size 1 turns the grouping kernel into "sort the (token, k) pairs by expert, stable in the token id"
        _lib.call("b200moe_group_tokens", _lib.ptr(self.idx), _lib.ROUTING_INDEX, _lib.I32, T, E, K, 1, T * K, 1, 1,
                  _lib.ptr(self.pair_token), _lib.ptr(self.pair_expert), _lib.ptr(self.pair_cond), _lib.ptr(self.counts),
                  _lib.ptr(self.inv), _lib.ptr(self.gstatus), _lib.ptr(self.gws), self.gws.numel(), st)
        _lib.call("b200moe_ep_exchange_counts", _lib.ptr(self.counts), self.p_counts, self.p_flags, self.rank, G, E,
                  epoch, status, st)
        mark("t0")
        _lib.call("b200moe_ep_dispatch_quantize", _lib.ptr(hidden), _lib.ptr(self.inv), _lib.ptr(self.pair_expert),
                  _lib.ptr(self.aff), _lib.ptr(self.counts_all), T, K, H, E, B, self.rank, G, int(w.h_packed_order),
                  self.p_xq, self.p_sf, self.p_aff, self.p_src, self.cap_rows, self.n_blocks_cap,
                  _lib.ptr(self.b2e), _lib.ptr(self.cond), _lib.ptr(self.row_valid), _lib.ptr(self.tile_flags),
                  status, st)   # the receiver's plan rides in the same launch (it needs the count table only)
        _lib.call("b200moe_ep_signal_wait", self.p_flags, self.rank, G, 1, epoch, status, st)
        _lib.call("b200moe_ep_scales_to_atoms", _lib.ptr(self.sf_rows), _lib.ptr(self.tile_flags), self.cap_rows // 128,
                  H, _lib.ptr(self.sf), st)
        mark("t1")
        _lib.call("b200moe_grouped_gemm1_swiglu", _lib.ptr(self.xq), _lib.ptr(self.sf), _lib.ptr(w.w1),
                  _lib.ptr(w.w1_sf), w.w_format, _lib.ptr(w.bias_gu), _lib.ptr(self.b2e), _lib.ptr(self.cond),
                  _lib.ptr(self.tile_flags), self.n_blocks_cap, B, E_L, H, I, ops.act_fn.value, nan, nan, nan, nan,
                  _lib.ptr(self.mq), _lib.ptr(self.m_sf), _lib.ptr(self.status[1:]), 0, None, st)
        mark("t2")
        if self.fuse_return:
            # the down contraction's epilogue stores every row into the GPU its token came from
            _lib.call("b200moe_ep_gemm2_scale_return", _lib.ptr(self.mq), _lib.ptr(self.m_sf), _lib.ptr(w.w2),
                      _lib.ptr(w.w2_sf), w.w_format, _lib.ptr(w.bias_d), _lib.ptr(self.b2e), _lib.ptr(self.cond),
                      _lib.ptr(self.tile_flags), _lib.ptr(self.row_valid), self.cap_rows, self.n_blocks_cap, B, E_L,
                      H, I, _lib.ptr(self.row_aff), _lib.ptr(self.row_src), self.p_back, G, T * K,
                      _lib.ptr(self.status[2:]), 0, st)
            mark("t3")
        else:
            _lib.call("b200moe_grouped_gemm2_scale", _lib.ptr(self.mq), _lib.ptr(self.m_sf), _lib.ptr(w.w2),
                      _lib.ptr(w.w2_sf), w.w_format, _lib.ptr(w.bias_d), _lib.ptr(self.b2e), _lib.ptr(self.cond),
                      _lib.ptr(self.tile_flags), _lib.ptr(self.row_valid), self.cap_rows, self.n_blocks_cap, B, E_L,
                      H, I, _lib.ptr(self.row_aff), _lib.F32, 1, _lib.ptr(self.y_pos), _lib.ptr(self.status[2:]), 0, None, st)
            mark("t3")
            _lib.call("b200moe_ep_return_rows", _lib.ptr(self.y_pos), _lib.ptr(self.row_valid),
                      _lib.ptr(self.row_src), self.p_back, G, self.cap_rows, H, T * K, st)
        _lib.call("b200moe_ep_signal_wait", self.p_flags, self.rank, G, 2, epoch, status, st)
        _lib.call("b200moe_combine", _lib.ptr(self.back), _lib.ptr(self.inv), T, K, H, _lib.ptr(self.out), st)
        return self.out

    def capture(self, hidden: torch.Tensor) -> None:
        """Record one step on ``hidden`` (a fixed device buffer) into a CUDA graph; call after one eager step."""
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self.forward(hidden)

    def replay(self) -> torch.Tensor:
        self._graph.replay()
        return self.out

    def device_status(self) -> list:
        """[exchange / capacity, gate-up contraction, down contraction] status words (0 = fine); synchronises."""
        return self.status.cpu().tolist()[:3]
