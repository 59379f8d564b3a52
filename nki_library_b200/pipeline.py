"""Launch sequence of the blockwise expert MLP on one GPU.

gather + MXFP8 quantise -> grouped gate/up contraction (SwiGLU, re-quantise)
-> grouped down contraction (bias, affinity) -> combine.  Everything runs on
the current CUDA stream; no host synchronisation happens unless
``check_status`` is requested.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib
from .weights import ExpertWeights

NAN = float("nan")


def _clamp(v):
    return NAN if v is None else float(v)


class BlockWorkspace:
    """Device scratch for one (n_pos, H, I) shape, reused across calls."""

    def __init__(self, n_pos: int, H: int, I: int, device):
        lib = _lib.load_library()
        self.key = (n_pos, H, I, str(device))
        self.xq = torch.empty((n_pos, H), dtype=torch.uint8, device=device)
        self.x_sf = torch.zeros(lib.b200moe_sf_bytes(n_pos, H), dtype=torch.uint8, device=device)
        self.tile_flags = torch.zeros(math.ceil(n_pos / 128), dtype=torch.int32, device=device)
        self.mq = torch.empty((n_pos, I), dtype=torch.uint8, device=device)
        self.m_sf = torch.zeros(lib.b200moe_sf_bytes(n_pos, I), dtype=torch.uint8, device=device)
        self.y_pos = torch.empty((n_pos, H), dtype=torch.bfloat16, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)


_workspaces: dict = {}


def get_workspace(n_pos: int, H: int, I: int, device) -> BlockWorkspace:
    key = (n_pos, H, I, str(device))
    ws = _workspaces.get(key)
    if ws is None:
        if len(_workspaces) > 4:
            _workspaces.clear()
        ws = BlockWorkspace(n_pos, H, I, device)
        _workspaces[key] = ws
    return ws


def run_blocks(hidden: torch.Tensor, hidden_rows: int, weights: ExpertWeights, token_position_to_id: torch.Tensor,
               block_to_expert: torch.Tensor, conditions: Optional[torch.Tensor], block_size: int,
               affinities: Optional[torch.Tensor], table: torch.Tensor, out: torch.Tensor, act_fn: int = 0,
               gate_clamp=(None, None), up_clamp=(None, None), impl: int = 0, check_status: bool = False,
               workspace: Optional[BlockWorkspace] = None, aff_per_row: bool = False,
               timers: Optional[dict] = None, prequantized: bool = False) -> torch.Tensor:
    """Run the four kernels.  ``table [rows_out, n_cand]`` lists, per output row (= token), the positions that
    hold it (negative = none): the quantiser stores the token's row there and the combine sums those rows.

    ``hidden`` bf16 ``[>= hidden_rows, H]``; ids outside ``[0, hidden_rows)`` in
    ``token_position_to_id`` are pads.  ``affinities`` is the flat table addressed
    ``token * E + expert`` (fp32 or bf16), a per-row vector addressed ``token``
    when ``aff_per_row``, or None.  ``out`` bf16 ``[rows_out, H]``.  With ``prequantized`` the caller has already
    filled ``workspace.xq / x_sf / tile_flags`` for this ``table`` (the fused RMSNorm + quantise kernel) and the
    quantise launch is skipped.
    """
    E, H, I = weights.E, weights.H, weights.I
    n_blocks = block_to_expert.numel()
    n_pos = n_blocks * block_size
    _lib.kernel_assert(block_size % 128 == 0, f"block_size ({block_size}) must be a multiple of 128")
    _lib.kernel_assert(token_position_to_id.numel() == n_pos, "token_position_to_id must hold N * block_size ids")
    _lib.kernel_assert(hidden.dtype == torch.bfloat16 and hidden.shape[1] == H and hidden.is_contiguous(),
                       "hidden_states must be contiguous bf16 [rows, H]")
    ws = workspace or get_workspace(n_pos, H, I, hidden.device)
    st = _lib.stream_ptr()

    def mark(name):
        if timers is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            timers.setdefault(name, []).append(ev)

    mark("t0")
    # token-major quantise: ``table`` lists every token's positions, so a hidden row is read and quantised once
    # and stored to each of them (a position-major gather would read it once per expert the token goes to)
    if not prequantized:
        _lib.call("b200moe_scatter_quantize_mxfp8", _lib.ptr(hidden), min(hidden_rows, table.shape[0]), H, _lib.ptr(table),
                  table.shape[1], n_pos, int(weights.h_packed_order), _lib.ptr(ws.xq), _lib.ptr(ws.x_sf),
                  _lib.ptr(ws.tile_flags), st)
    mark("t1")
    _lib.call("b200moe_grouped_gemm1_swiglu", _lib.ptr(ws.xq), _lib.ptr(ws.x_sf), _lib.ptr(weights.w1),
              _lib.ptr(weights.w1_sf), weights.w_format, _lib.ptr(weights.bias_gu), _lib.ptr(block_to_expert), _lib.ptr(conditions),
              _lib.ptr(ws.tile_flags), n_blocks, block_size, E, H, I, act_fn, _clamp(gate_clamp[0]),
              _clamp(gate_clamp[1]), _clamp(up_clamp[0]), _clamp(up_clamp[1]), _lib.ptr(ws.mq), _lib.ptr(ws.m_sf),
              _lib.ptr(ws.status[1:]), impl, None, st)
    mark("t2")
    _lib.call("b200moe_grouped_gemm2_scale", _lib.ptr(ws.mq), _lib.ptr(ws.m_sf), _lib.ptr(weights.w2),
              _lib.ptr(weights.w2_sf), weights.w_format, _lib.ptr(weights.bias_d), _lib.ptr(block_to_expert), _lib.ptr(conditions),
              _lib.ptr(ws.tile_flags), _lib.ptr(token_position_to_id), hidden_rows, n_blocks, block_size, E, H, I,
              _lib.ptr(affinities), _lib.F32 if affinities is None else _lib.dtype_code(affinities),
              int(aff_per_row), _lib.ptr(ws.y_pos), _lib.ptr(ws.status[2:]), impl, None, st)
    mark("t3")
    _lib.call("b200moe_combine", _lib.ptr(ws.y_pos), _lib.ptr(table), out.shape[0], table.shape[1], H, _lib.ptr(out), st)
    if check_status:
        s = ws.status.cpu().tolist()
        _lib.kernel_assert(s[1] == 0 and s[2] == 0, f"device-side wait expired in the expert contraction (status {s})")
    return out


class DenseWorkspace:
    """Device scratch of the dense (non-MX) path for one (n_pos, H, I) shape."""

    def __init__(self, n_pos: int, H: int, I: int, device):
        self.x_pos = torch.empty((n_pos, H), dtype=torch.bfloat16, device=device)
        self.m = torch.empty((n_pos, I), dtype=torch.bfloat16, device=device)
        self.y_pos = torch.empty((n_pos, H), dtype=torch.bfloat16, device=device)
        self.tile_flags = torch.zeros(math.ceil(n_pos / 128), dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)


_dense_workspaces: dict = {}


def run_blocks_dense(hidden: torch.Tensor, hidden_rows: int, weights, token_position_to_id: torch.Tensor,
                     block_to_expert: torch.Tensor, conditions: Optional[torch.Tensor], block_size: int,
                     affinities: Optional[torch.Tensor], table: torch.Tensor, out: torch.Tensor, act_fn: int = 0,
                     gate_clamp=(None, None), up_clamp=(None, None), impl: int = 0, check_status: bool = False,
                     pre_scale: bool = False) -> torch.Tensor:
    """The four launches of the dense variants: row scatter (x affinity when ``pre_scale``) -> gate/up contraction
    + bias + clamp + act(gate) * up -> down contraction + bias (x affinity unless ``pre_scale``) -> combine.
    Arguments as :func:`run_blocks`; ``weights`` is a :class:`~nki_library_b200.weights.DenseExpertWeights`."""
    E, H, I = weights.E, weights.H, weights.I
    n_blocks = block_to_expert.numel()
    n_pos = n_blocks * block_size
    _lib.kernel_assert(block_size % 128 == 0, f"block_size ({block_size}) must be a multiple of 128")
    _lib.kernel_assert(token_position_to_id.numel() == n_pos, "token_position_to_id must hold N * block_size ids")
    _lib.kernel_assert(hidden.dtype == torch.bfloat16 and hidden.shape[1] == H and hidden.is_contiguous(),
                       "hidden_states must be contiguous bf16 [rows, H]")
    key = (n_pos, H, I, str(hidden.device))
    ws = _dense_workspaces.get(key)
    if ws is None:
        if len(_dense_workspaces) > 4:
            _dense_workspaces.clear()
        ws = _dense_workspaces[key] = DenseWorkspace(n_pos, H, I, hidden.device)
    st = _lib.stream_ptr()
    aff_code = _lib.F32 if affinities is None else _lib.dtype_code(affinities)
    _lib.call("b200moe_scatter_rows_bf16", _lib.ptr(hidden), min(hidden_rows, table.shape[0]), H, _lib.ptr(table),
              table.shape[1], n_pos, _lib.ptr(block_to_expert), block_size, E,
              _lib.ptr(affinities) if pre_scale else None, aff_code, _lib.ptr(ws.x_pos), _lib.ptr(ws.tile_flags), st)
    _lib.call("b200moe_dense_gemm1_swiglu", _lib.ptr(ws.x_pos), _lib.ptr(weights.w1), _lib.ptr(weights.scale_gu),
              _lib.ptr(weights.bias_gu), _lib.ptr(block_to_expert), _lib.ptr(conditions), _lib.ptr(ws.tile_flags),
              n_blocks, block_size, E, H, I, act_fn, _clamp(gate_clamp[0]), _clamp(gate_clamp[1]),
              _clamp(up_clamp[0]), _clamp(up_clamp[1]), _lib.ptr(ws.m), _lib.ptr(ws.status[1:]), impl, st)
    _lib.call("b200moe_dense_gemm2_scale", _lib.ptr(ws.m), _lib.ptr(weights.w2), _lib.ptr(weights.scale_d),
              _lib.ptr(weights.bias_d), _lib.ptr(block_to_expert), _lib.ptr(conditions), _lib.ptr(ws.tile_flags),
              _lib.ptr(token_position_to_id), hidden_rows, n_blocks, block_size, E, H, I,
              None if pre_scale else _lib.ptr(affinities), aff_code, 0, _lib.ptr(ws.y_pos), _lib.ptr(ws.status[2:]),
              impl, st)
    _lib.call("b200moe_combine", _lib.ptr(ws.y_pos), _lib.ptr(table), out.shape[0], table.shape[1], H, _lib.ptr(out), st)
    if check_status:
        s = ws.status.cpu().tolist()
        _lib.kernel_assert(s[1] == 0 and s[2] == 0, f"device-side wait expired in the expert contraction (status {s})")
    return out
