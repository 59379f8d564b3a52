"""CPU oracle: router top-K and token-to-block grouping (test infrastructure only).

Restates, vectorised in numpy/torch, the reference's CPU definitions:

* ``router_topk`` ............ core/router_topk/router_topk_torch.py:23-135
* ``find_nonzero_indices`` ... core/subkernels/find_nonzero_indices_torch.py:20-63
* ``cumsum`` ................. core/cumsum/cumsum.py:29-75 (inclusive, last axis)
* ``indexed_flatten`` ........ core/subkernels/indexed_flatten_torch.py:20-67
* block assignment ........... test/integration/nkilib/core/moe/moe_cte/test_moe_cte_common.py:95-98,199-264

The three torch references above import without the Trainium toolchain, so the
restatements are pinned against their outputs (fixtures under tests/golden/).
Ties in the top-K are broken towards the lowest expert index (a stable
descending sort), which is what ``torch.argsort`` of the negated logits gives
for the reference on CPU in practice and what the CUDA kernel implements.
"""

from __future__ import annotations

import math

import numpy as np
import torch

SOFTMAX = 1
SIGMOID = 0


def router_logits(x: torch.Tensor, w: torch.Tensor, w_bias=None, x_is_TH: bool = True) -> torch.Tensor:
    """fp32 logits ``[T, E] = x[T, H] @ w[H, E] (+ bias)`` (router_topk_torch.py:68-77)."""
    xf = x.float() if x_is_TH else x.float().T
    out = xf @ w.float()
    if w_bias is not None:
        out = out + w_bias.float().reshape(1, -1)
    return out


def router_from_logits(logits: torch.Tensor, k: int, act_fn: int, router_pre_norm: bool, norm_topk_prob: bool):
    """Top-K and affinities from given fp32 logits (router_topk_torch.py:79-129).

    Returns ``(expert_index int64 [T, k], expert_affinities fp32 [T, E])``.
    """
    logits = logits.float()
    T, E = logits.shape
    order = torch.argsort(-logits, dim=-1, stable=True)
    idx = order[:, :k]
    if router_pre_norm:
        full = torch.softmax(logits, dim=-1) if act_fn == SOFTMAX else torch.sigmoid(logits)
        if norm_topk_prob:
            sel = torch.zeros(T, E)
            sel.scatter_(1, idx, full.gather(1, idx))
            aff = sel / sel.sum(dim=1, keepdim=True)
        else:
            aff = full
    else:
        top = logits.gather(1, idx)
        top = torch.softmax(top, dim=-1) if act_fn == SOFTMAX else torch.sigmoid(top)
        aff = torch.zeros(T, E)
        aff.scatter_(1, idx, top)
    return idx, aff


def router_topk(x, w, w_bias, k, act_fn=SOFTMAX, router_pre_norm=True, norm_topk_prob=False, x_is_TH=True):
    logits = router_logits(x, w, w_bias, x_is_TH)
    idx, aff = router_from_logits(logits, k, act_fn, router_pre_norm, norm_topk_prob)
    return logits, idx, aff


def rms_norm(x: torch.Tensor, gamma=None, eps: float = 1e-6, hidden_actual=None) -> torch.Tensor:
    """fp32 RMSNorm (core/subkernels/rmsnorm_torch.py:22-51)."""
    x = x.float()
    if hidden_actual is not None:
        rms = (x.square().sum(dim=-1, keepdim=True) / hidden_actual + eps).sqrt()
    else:
        rms = (x.square().mean(dim=-1, keepdim=True) + eps).sqrt()
    y = x * rms.reciprocal()
    if gamma is not None:
        y = y * gamma.float().reshape(1, -1)
    return y


# --------------------------------------------------------------------------
# grouping
# --------------------------------------------------------------------------
def find_nonzero_indices(inp: np.ndarray, col_start: int = 0, n_cols: int | None = None):
    """Per column: ascending row ids of non-zero entries, -1 padded to T, and their count."""
    inp = np.asarray(inp)
    T, C = inp.shape
    n_cols = C - col_start if n_cols is None else n_cols
    indices = np.full((n_cols, T), -1, dtype=np.int32)
    counts = np.zeros(n_cols, dtype=np.int32)
    for c in range(n_cols):
        nz = np.flatnonzero(inp[:, col_start + c])
        counts[c] = nz.size
        indices[c, : nz.size] = nz
    return indices, counts


def cumsum(x: np.ndarray) -> np.ndarray:
    """Inclusive cumulative sum on the last axis, accumulated in fp32 like the kernel."""
    return np.cumsum(np.asarray(x, dtype=np.float32), axis=-1, dtype=np.float32).astype(x.dtype)


def indexed_flatten(inp: np.ndarray, f_len: int, output_len: int, row_offsets: np.ndarray,
                    row_offsets_start: int = 0, padding_val: int = -1) -> np.ndarray:
    """Write row e's ``T // f_len`` chunks at block offsets ``row_offsets[start + e] + p``.

    Later rows overwrite earlier ones where they overlap, and chunks that fall
    outside ``[0, output_len // f_len)`` are dropped (indexed_flatten_torch.py:60-66).
    """
    inp = np.asarray(inp)
    E, T = inp.shape
    parts = T // f_len
    nblk = output_len // f_len
    out = np.full(output_len, padding_val, dtype=inp.dtype)
    ob = out[: nblk * f_len].reshape(nblk, f_len)
    src = inp[:, : parts * f_len].reshape(E, parts, f_len)
    for e in range(E):
        off = int(row_offsets[row_offsets_start + e])
        for p in range(parts):
            b = off + p
            if 0 <= b < nblk:
                ob[b] = src[e, p]
    return out


def get_n_blocks(T: int, top_k: int, E: int, B: int, n_block_per_iter: int = 1) -> int:
    """Static upper bound on the number of blocks (test_moe_cte_common.py:95-98)."""
    N = math.ceil((T * top_k - (E - 1)) / B) + E - 1
    return n_block_per_iter * math.ceil(N / n_block_per_iter)


def group_tokens(mask: np.ndarray, B: int, N: int, skip_token: bool = True, mx_conditions: bool = True):
    """Block assignment from a routing mask ``[T, E]`` (non-zero = token routed to expert).

    Vectorised restatement of ``generate_token_position_to_id_and_experts``
    (test_moe_cte_common.py:218-262) for the default (non split-padding) case:
    expert e owns ``ceil(count_e / B)`` consecutive blocks in expert order,
    surplus blocks are appended to the last expert, tokens keep ascending id
    order inside an expert, the pad id is -1 (``skip_token``) or T, and
    ``conditions`` is ones followed by ``n_padding + 2`` zeros (length N + 2)
    for the MX block-parallel kernel, else ``n_padding + 1`` zeros (N + 1).

    Returns ``(token_position_to_id int32 [N*B], block_to_expert int32 [N],
    conditions int32, counts int32 [E])``.
    """
    m = np.asarray(mask) != 0
    T, E = m.shape
    counts = m.sum(axis=0).astype(np.int64)
    bpe = -(-counts // B)
    n_pad = N - int(bpe.sum())
    assert n_pad >= 0, "N is smaller than the number of occupied blocks"
    bpe_padded = bpe.copy()
    bpe_padded[E - 1] += n_pad
    block_to_expert = np.repeat(np.arange(E), bpe_padded).astype(np.int32)
    first_block = np.concatenate([[0], np.cumsum(bpe_padded)[:-1]])
    pad = -1 if skip_token else T
    tpi = np.full(N * B, pad, dtype=np.int32)
    rank = np.cumsum(m, axis=0) - 1  # 0-based arrival order inside each expert
    t_idx, e_idx = np.nonzero(m)
    tpi[first_block[e_idx] * B + rank[t_idx, e_idx]] = t_idx
    if mx_conditions:
        cond = np.ones(N + 2, dtype=np.int32)
        cond[N + 2 - (n_pad + 2):] = 0
    else:
        cond = np.ones(N + 1, dtype=np.int32)
        cond[N + 1 - (n_pad + 1):] = 0
    return tpi, block_to_expert, cond, counts.astype(np.int32)


def mask_from_index(expert_index: np.ndarray, E: int) -> np.ndarray:
    """``[T, K]`` expert ids -> ``[T, E]`` 0/1 mask."""
    idx = np.asarray(expert_index).astype(np.int64)
    T = idx.shape[0]
    m = np.zeros((T, E), dtype=np.int32)
    m[np.arange(T)[:, None], idx] = 1
    return m


def inverse_map(tpi: np.ndarray, block_to_expert: np.ndarray, expert_index: np.ndarray, B: int) -> np.ndarray:
    """``inv[t, k]`` = position p with ``tpi[p] == t`` inside a block of expert ``expert_index[t, k]``."""
    T, K = expert_index.shape
    inv = np.full((T, K), -1, dtype=np.int32)
    pos_expert = np.repeat(block_to_expert, B)
    valid = np.flatnonzero((tpi >= 0) & (tpi < T))
    look = {(int(tpi[p]), int(pos_expert[p])): int(p) for p in valid}
    for t in range(T):
        for k in range(K):
            inv[t, k] = look.get((t, int(expert_index[t, k])), -1)
    return inv
