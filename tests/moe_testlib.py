"""Seeded synthetic inputs and layout helpers shared by the MoE tests."""

from __future__ import annotations

import numpy as np
import torch

from oracle import mx, routing


def bf16_values(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 and return them as fp32."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def make_rows_weights(E, H, I, seed=0, std=0.02):
    """MXFP8 expert weights in plain rows layout (numpy): codes/scales for gate_up [E,2,I,H] and down [E,H,I]."""
    rng = np.random.default_rng(seed)
    w1 = (rng.standard_normal((E * 2 * I, H)) * std).astype(np.float32)
    w2 = (rng.standard_normal((E * H, I)) * std).astype(np.float32)
    c1, s1 = mx.quantize_mx_rows(w1)
    c2, s2 = mx.quantize_mx_rows(w2)
    return (c1.reshape(E, 2, I, H), s1.reshape(E, 2, I, H // 32), c2.reshape(E, H, I), s2.reshape(E, H, I // 32))


def make_rows_weights_fmt(E, H, I, fmt, seed=0):
    """Expert weights of element type ``fmt`` as random finite element codes (one per array element; e2m1
    codes are nibbles 0..15) with block scales 2^-9 .. 2^-6: same shapes as ``make_rows_weights``."""
    if fmt == "e4m3":
        return make_rows_weights(E, H, I, seed)
    rng = np.random.default_rng(seed)

    def codes(shape):
        if fmt == "e2m1":
            return rng.integers(0, 16, shape, dtype=np.uint8)
        sign = rng.integers(0, 2, shape, dtype=np.uint8) << 7
        return (sign | (rng.integers(9, 17, shape, dtype=np.uint8) << 2) | rng.integers(0, 4, shape, dtype=np.uint8))

    def scales(shape):
        return rng.integers(118, 122, shape, dtype=np.uint8)

    return (codes((E, 2, I, H)), scales((E, 2, I, H // 32)), codes((E, H, I)), scales((E, H, I // 32)))


def make_routing(T, H, E, K, seed=0, zipf_s=None):
    """hidden bf16 values [T,H], softmax-normalised top-K affinities [T,E] (fp32), expert_index [T,K]."""
    rng = np.random.default_rng(seed + 1000)
    hidden = bf16_values(rng.standard_normal((T, H)).astype(np.float32))
    w = bf16_values((rng.standard_normal((H, E)) * 0.02).astype(np.float32))
    bias = None
    if zipf_s is not None:
        rank = rng.permutation(E) + 1
        bias = bf16_values((-zipf_s * np.log(rank)).astype(np.float32))
    logits, idx, aff = routing.router_topk(torch.from_numpy(hidden), torch.from_numpy(w),
                                           None if bias is None else torch.from_numpy(bias), K,
                                           routing.SOFTMAX, True, True)
    return hidden, w, bias, idx.numpy().astype(np.int32), aff.numpy().astype(np.float32)


def sf_atoms_to_rows(atoms: np.ndarray, rows: int, K: int) -> np.ndarray:
    """Scale-atom buffer -> dense [rows, K/32] (inverse of the device layout)."""
    k_atoms = -(-K // 128)
    r = np.arange(rows)[:, None]
    kb = np.arange(K // 32)[None, :]
    atom = (r >> 7) * k_atoms + (kb >> 2)
    rr = r & 127
    off = atom * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (kb & 3)
    return np.asarray(atoms).reshape(-1)[off]


def gate_up_dev_rows(I: int) -> np.ndarray:
    """dev_row[s, i]: row of gate (s=0) / up (s=1) column i in the interleaved device weight."""
    i = np.arange(I)
    return np.stack([(i >> 5) * 64 + (i & 31), (i >> 5) * 64 + 32 + (i & 31)])


def max_rel(a: np.ndarray, ref: np.ndarray) -> float:
    """The build's output tolerance metric: max|a - ref| / max|ref|."""
    return float(np.abs(a.astype(np.float64) - ref.astype(np.float64)).max() / max(np.abs(ref).max(), 1e-30))
