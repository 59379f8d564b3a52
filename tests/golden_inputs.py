"""Seed-generated inputs shared by the golden-fixture generator and the tests.

They reproduce the generators of the reference's own tests so that fixtures
hold outputs only:

* router tensors: ``torch.Generator().manual_seed(0)``, uniform(-0.1, 0.1), cast
  to bf16; x, w and bias each restart from seed 0 (test_router_topk_common.py:30-49)
* sparse masks: ``np.random.seed(42)`` permutation of K*E ones (test_find_nonzero_indices.py:29-45)
* indexed_flatten: ``arange`` rows and evenly spaced row offsets (test_indexed_flatten.py:28-37,108-121)
"""

from __future__ import annotations

import math

import numpy as np
import torch

# name: (T, H, E, k, act, has_bias, router_pre_norm, norm_topk_prob) -- rows of
# test_router_topk.py:47-121 small enough to store in full, plus one larger one.
ROUTER_CASES = {
    "t4_e128_k4_bias": (4, 3072, 128, 4, "softmax", True, False, False),
    "t16_e128_k4_bias": (16, 3072, 128, 4, "softmax", True, False, False),
    "t64_e128_k4_bias": (64, 3072, 128, 4, "softmax", True, False, False),
    "t4_e128_k4_nobias": (4, 3072, 128, 4, "softmax", False, False, False),
    "t4_e256_k4_bias": (4, 3072, 256, 4, "softmax", True, False, False),
    "t48_e128_k4_bias": (48, 3072, 128, 4, "softmax", True, False, False),
    "t8_h8192_k8_sigmoid": (8, 8192, 128, 8, "sigmoid", True, False, False),
    "t8_h8192_k8_prenorm_softmax": (8, 8192, 128, 8, "softmax", True, True, False),
    "t8_h8192_k8_prenorm_sigmoid": (8, 8192, 128, 8, "sigmoid", True, True, False),
    "t8_h8192_k8_prenorm_l1_softmax": (8, 8192, 128, 8, "softmax", True, True, True),
    "t8_h8192_k8_prenorm_l1_sigmoid": (8, 8192, 128, 8, "sigmoid", True, True, True),
    "t32_e128_k4_prenorm_l1": (32, 3072, 128, 4, "softmax", True, True, True),
    "t4_k1_nobias": (4, 3072, 128, 1, "softmax", False, False, False),
    "t2_h5120_e16_k1": (2, 5120, 16, 1, "softmax", False, False, False),
    "t2_h4096_k8_prenorm": (2, 4096, 128, 8, "softmax", False, True, False),
    "t320_e128_k4_bias": (320, 3072, 128, 4, "softmax", True, False, False),
}


def _uniform_bf16(shape):
    g = torch.Generator()
    g.manual_seed(0)
    return torch.empty(shape, dtype=torch.float32).uniform_(-0.1, 0.1, generator=g).to(torch.bfloat16)


def router_inputs(T, H, E, has_bias):
    """x [T, H], w [H, E], bias [1, E] or None, all bf16."""
    return _uniform_bf16((T, H)), _uniform_bf16((H, E)), (_uniform_bf16((1, E)) if has_bias else None)


# name: (T, E, top_k, dtype, col_start, n_cols)
NONZERO_CASES = {
    "t4096_e128_k8_i32": (4096, 128, 8, "int32", None, None),
    "t4096_e128_k8_f32": (4096, 128, 8, "float32", None, None),
    "t10240_e128_k4_i32": (10240, 128, 4, "int32", None, None),
    "t10240_e128_k4_f32": (10240, 128, 4, "float32", None, None),
    "t65536_e128_k4_i32": (65536, 128, 4, "int32", None, None),
    "t4096_sub0_4_i32": (4096, 128, 8, "int32", 0, 4),
    "t10240_sub16_16_f32": (10240, 128, 4, "float32", 16, 16),
    "t65536_sub32_16_i32": (65536, 128, 4, "int32", 32, 16),
    "t10240_sub120_8_f32": (10240, 128, 4, "float32", 120, 8),
    "t256_e4_k2_i32": (256, 4, 2, "int32", None, None),
    "t384_e8_k2_f32": (384, 8, 2, "float32", None, None),
}


def sparse_input(T, E, top_k, dtype, seed=42):
    np.random.seed(seed)
    K = T * top_k // E
    flat = np.random.permutation(np.concatenate([np.ones(K * E), np.zeros((T - K) * E)]))
    x = flat.reshape(E, T).T.astype(np.int32 if dtype == "int32" else np.float32)
    if dtype == "float32":
        x[x > 0] = 0.1
    return np.ascontiguousarray(x)


# name: (T, E, f_len, n_row_offsets or None, row_offsets_start or None)
FLATTEN_CASES = {
    "t4096_e1_f128": (4096, 1, 128, None, None),
    "t4096_e2_f128": (4096, 2, 128, None, None),
    "t4096_e2_f256": (4096, 2, 256, None, None),
    "t4096_e3_f128": (4096, 3, 128, None, None),
    "t10240_e16_f128": (10240, 16, 128, None, None),
    "t10240_e17_f128": (10240, 17, 128, None, None),
    "t65536_e4_f128": (65536, 4, 128, None, None),
    "t65536_e4_f256": (65536, 4, 256, None, None),
    "t4096_e64_f128": (4096, 64, 128, None, None),
    "t4096_e128_f128": (4096, 128, 128, None, None),
    "t4096_e256_f128": (4096, 256, 128, None, None),
    "t4096_e2_f128_n4_s2": (4096, 2, 128, 4, 2),
    "t4096_e3_f128_n5_s1": (4096, 3, 128, 5, 1),
    "t10240_e8_f128_n16_s8": (10240, 8, 128, 16, 8),
}


def flatten_inputs(T, E, f_len, n_off, start):
    parts = T // f_len
    n = E if n_off is None else n_off
    out_len = ((n * T + 1024 + 127) // 128) * 128
    return {
        "input_tensor": np.arange(E * T, dtype=np.int32).reshape(E, T),
        "f_len": f_len,
        "output_len": out_len,
        "row_offsets": np.array([parts * i for i in range(n)], dtype=np.int32),
        "row_offsets_start": start,
        "padding_val": -1,
    }


# name: (T, E, K, B) -- mask -> find_nonzero_indices -> cumsum -> indexed_flatten
CHAIN_CASES = {
    "c1_t256_e4_k2_b128": (256, 4, 2, 128),
    "t384_e8_k2_b128": (384, 8, 2, 128),
    "t4096_e8_k2_b512": (4096, 8, 2, 512),
    "t8192_e256_k8_b128": (8192, 256, 8, 128),
    "t2048_e128_k8_b256": (2048, 128, 8, 256),
}


def n_blocks(T, K, E, B):
    return math.ceil((T * K - (E - 1)) / B) + E - 1


def routing_mask(T, E, K, seed=0):
    """0/1 int32 mask [T, E] with exactly K distinct experts per token (seeded)."""
    rng = np.random.default_rng(seed)
    scores = rng.random((T, E))
    idx = np.argsort(-scores, axis=1, kind="stable")[:, :K]
    m = np.zeros((T, E), dtype=np.int32)
    m[np.arange(T)[:, None], idx] = 1
    return m
