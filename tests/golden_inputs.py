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


# ---------------------------------------------------------------------------
# MX fixtures: seeded inputs for the reference's MX CPU code (quantize_to_mx,
# mx_matmul, the projection goldens, the prefill block loop and the decode
# reference).  Everything is drawn from numpy Generators, so the fixture
# generator and the tests rebuild identical arrays.
# ---------------------------------------------------------------------------
def bf16_round(a):
    """fp32 values rounded to the bf16 grid (returned as fp32)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def mx_quantize_input(P=128, F=512, seed=7):
    """``[P, F]`` fp32 with 8 x 4 blocks of very different magnitude and the awkward cases in known blocks:
    (every value is bf16-exact, so the CUDA quantiser, which takes bf16 rows, can be fed the same data)
    an all-zero block, one with a single subnormal, exact rounding ties of the e4m3 grid, block maxima whose
    scaled value exceeds 448 and must clip, negative zero, and bf16-valued gaussian data elsewhere."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((P, F)).astype(np.float32)
    mag = np.exp2(rng.integers(-24, 20, (P // 8, F // 4))).astype(np.float32)
    x = bf16_round(x * np.repeat(np.repeat(mag, 8, 0), 4, 1))
    x[0:8, 0:4] = 0.0
    x[0:8, 4:8] = 0.0
    x[3, 5] = np.float32(2.0 ** -133)                 # smallest bf16 subnormal: biased exponent 0
    x[8:16, 0:4] = np.float32(1.0625)                 # tie between 1.0 and 1.125 -> even (1.0)
    x[8:16, 4:8] = np.float32(1.1875)                 # tie between 1.125 and 1.25 -> even (1.25)
    x[8, 4] = np.float32(1.5)
    x[16:24, 0:4] = np.float32(1.96875)               # 1.96875 * 2^8 = 504 > 448: clips
    x[16:24, 4:8] = np.float32(-1.9375)               # -496: clips to -448
    x[24:32, 0:4] = np.float32(-0.0)
    x[24, 1] = np.float32(3.0)
    x[32:40, 0:4] = np.float32(2.0 ** -9) * np.arange(32, dtype=np.float32).reshape(8, 4)  # subnormal codes after scaling
    x[40:48, 0:4] = np.float32(2.0 ** 100)
    x[40:48, 4:8] = np.float32(2.0 ** -120)
    return x


def mx_matmul_input(P=64, SF=24, MF=16, seed=11):
    """Random finite e4m3 codes ``[P, 4*SF]`` / ``[P, 4*MF]`` with block scales ``[P/8, SF]`` / ``[P/8, MF]``."""
    rng = np.random.default_rng(seed)

    def codes(n):
        c = rng.integers(0, 256, (P, 4 * n), dtype=np.uint8)
        c[(c & 0x7F) == 0x7F] = 0x3C  # NaN patterns -> 1.5
        return c

    return (codes(SF), codes(MF), rng.integers(118, 132, (P // 8, SF), dtype=np.uint8),
            rng.integers(118, 132, (P // 8, MF), dtype=np.uint8))


def mx_encode_rows(values):
    """Plain block-32 MXFP8 encoding of ``[R, K]`` used to fabricate *weights* (inputs, not results):
    scale byte = block's largest biased exponent - 8, codes = value / 2^(scale-127) cast by ml_dtypes
    (a power-of-two scaling, exact in fp32).  Works through the rows in slices to bound memory."""
    import ml_dtypes

    v = np.ascontiguousarray(values, dtype=np.float32)
    R, K = v.shape
    codes = np.empty((R, K), dtype=np.uint8)
    scales = np.empty((R, K // 32), dtype=np.uint8)
    step = max(1, (1 << 24) // K)
    for r0 in range(0, R, step):
        vb = v[r0:r0 + step].reshape(-1, K // 32, 32)
        e = ((vb.view(np.uint32) >> 23) & 0xFF).astype(np.int32).max(axis=2)
        s = np.clip(e - 8, 0, 255)
        q = np.clip(np.ldexp(vb, (127 - s)[:, :, None]), -448, 448).astype(np.float32)
        codes[r0:r0 + step] = q.astype(ml_dtypes.float8_e4m3fn).view(np.uint8).reshape(-1, K)
        scales[r0:r0 + step] = s.astype(np.uint8)
    return codes, scales


# name: dict(T, H, I, E, K, B, act, bias, clamps (gate_hi, gate_lo, up_hi, up_lo), skip_token, dynamic, sample)
# ``sample`` = number of token rows of the reference output kept in the fixture (None = all rows).
MX_LAYER_CASES = {
    # BASELINE configuration 1, plain
    "c1_plain": dict(T=256, H=512, I=1024, E=4, K=2, B=128, act="silu", bias=False, clamps=(None, None, None, None),
                     skip_token=True, dynamic=False, sample=None),
    # the same layer in the style of the reference's unit vectors: bias, Swish, one-sided gate clamp, pad row T
    "c1_bias_swish_clamp": dict(T=256, H=512, I=1024, E=4, K=2, B=128, act="swish", bias=True,
                                clamps=(7.0, None, 7.0, -7.0), skip_token=False, dynamic=True, sample=None),
    # test_moe_bwmm_mx_cte.py:72 at a reduced token count (T = 10240 there): H=3072, I=384, E=128, B=256, top-4
    "ref_h3072_i384_e128_b256_k4": dict(T=1024, H=3072, I=384, E=128, K=4, B=256, act="swish", bias=True,
                                        clamps=(7.0, None, 7.0, -7.0), skip_token=True, dynamic=False, sample=48),
    # test_moe_bwmm_mx_cte.py:85 at a reduced token count (T = 4096 there): dynamic loop, n_static_blocks = 2
    "ref_h3072_i384_e2_b256_k2_dynamic": dict(T=1024, H=3072, I=384, E=2, K=2, B=256, act="silu", bias=True,
                                              clamps=(7.0, None, 7.0, -7.0), skip_token=True, dynamic=True,
                                              sample=48),
}


def _case_seed(name):
    return sum(map(ord, name))


def mx_layer_routing(name):
    """Seeded routing of a prefill case: ``expert_index [T, K]``, 0/1 ``mask [T, E]`` and bf16-valued masked
    affinities ``[rows, E]`` (rows = T, or T + 1 with a zero pad row when the case keeps the pad token)."""
    c = MX_LAYER_CASES[name]
    T, E, K = c["T"], c["E"], c["K"]
    rng = np.random.default_rng(_case_seed(name) + 2)
    idx = np.argsort(-rng.random((T, E)), axis=1, kind="stable")[:, :K].astype(np.int32)
    mask = np.zeros((T, E), dtype=np.int32)
    mask[np.arange(T)[:, None], idx] = 1
    rows = T if c["skip_token"] else T + 1
    aff = np.zeros((rows, E), dtype=np.float32)
    aff[:T] = bf16_round(rng.random((T, E)) * mask)
    return idx, mask, aff


def mx_layer_inputs(name):
    """Everything one prefill case needs, in plain rows form (the generator script converts the weights to the
    reference's storage with pure permutations).  Values the reference holds in bf16 are bf16-exact fp32."""
    c = MX_LAYER_CASES[name]
    T, H, I, E = c["T"], c["H"], c["I"], c["E"]
    rows = T if c["skip_token"] else T + 1
    hidden = bf16_round(np.random.default_rng(_case_seed(name)).standard_normal((rows, H)))
    if not c["skip_token"]:
        hidden[T] = 0
    rng = np.random.default_rng(_case_seed(name) + 1)
    c1, s1 = mx_encode_rows((rng.standard_normal((E * 2 * I, H), dtype=np.float32) * np.float32(0.02)))
    c2, s2 = mx_encode_rows((rng.standard_normal((E * H, I), dtype=np.float32) * np.float32(0.02)))
    idx, mask, aff = mx_layer_routing(name)
    out = dict(case=c, hidden=hidden, aff=aff, expert_index=idx, mask=mask,
               w1_codes=c1.reshape(E, 2, I, H), w1_scales=s1.reshape(E, 2, I, H // 32),
               w2_codes=c2.reshape(E, H, I), w2_scales=s2.reshape(E, H, I // 32), bias_gu=None, bias_d=None)
    if c["bias"]:
        rng = np.random.default_rng(_case_seed(name) + 3)
        out["bias_gu"] = bf16_round(rng.uniform(-2.0625, 0.52, (E, 2, I)))   # ranges of test_utils.py:430-433
        out["bias_d"] = bf16_round(rng.uniform(-1.632, 1.4375, (E, H)))
    return out


MX_DECODE_CASES = {
    # name: (T, H, I, E, K, act, all_expert)
    "sel_t8_h512_i256_e4_k2_swish": (8, 512, 256, 4, 2, "swish", False),
    "all_t16_h512_i256_e4_silu": (16, 512, 256, 4, 2, "silu", True),
    "sel_t8_h512_i256_e4_k2_gelu": (8, 512, 256, 4, 2, "gelu", False),
    "sel_t8_h512_i256_e4_k2_gelu_tanh": (8, 512, 256, 4, 2, "gelu_tanh", False),
    # test_moe_tkg.py "=== MXFP8" selective row at fewer experts (E = 128 there): T=2, H=3072, I=1536, top-8
    "sel_t2_h3072_i1536_e16_k8_silu": (2, 3072, 1536, 16, 8, "silu", False),
}


def mx_decode_inputs(name):
    T, H, I, E, K, act, all_expert = MX_DECODE_CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    hidden = bf16_round(rng.standard_normal((T, H)))
    w1 = (rng.standard_normal((E * 2 * I, H)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((E * H, I)) * 0.02).astype(np.float32)
    c1, s1 = mx_encode_rows(w1)
    c2, s2 = mx_encode_rows(w2)
    idx = np.argsort(-rng.random((T, E)), axis=1, kind="stable")[:, :K].astype(np.int32)
    aff = bf16_round(rng.random((T, E)))
    return dict(T=T, H=H, I=I, E=E, K=K, act=act, all_expert=all_expert, hidden=hidden, aff=aff, expert_index=idx,
                w1_codes=c1.reshape(E, 2, I, H), w1_scales=s1.reshape(E, 2, I, H // 32),
                w2_codes=c2.reshape(E, H, I), w2_scales=s2.reshape(E, H, I // 32),
                bias_gu=bf16_round(rng.uniform(-2.0625, 0.52, (E, 2, I))),
                bias_d=bf16_round(rng.uniform(-1.632, 1.4375, (E, H))),
                clamps=(7.0, None, 7.0, -7.0))


def sample_rows(name, n_rows, count):
    """The token rows of a large case whose reference outputs are kept (seeded choice, ascending)."""
    rng = np.random.default_rng(sum(map(ord, name)) + 1)
    return np.sort(rng.choice(n_rows, size=count, replace=False))


# ---------------------------------------------------------------------------
# Dense (non-MX) fixtures: inputs for moe_cte_torch_ref / moe_tkg_torch_ref.
# ---------------------------------------------------------------------------
# name: dict(T, H, I, E, K, B, weights "bf16" | "fp8row", act, bias, clamps (gate_hi, gate_lo, up_hi, up_lo),
#            scaling "post" | "pre" | "none", skip_token, hybrid)
DENSE_CTE_CASES = {
    "c1_bf16_post": dict(T=256, H=512, I=1024, E=4, K=2, B=128, weights="bf16", act="silu", bias=True,
                         clamps=(None, None, None, None), scaling="post", skip_token=True, hybrid=False),
    "c1_fp8row_pre_swish_clamp": dict(T=256, H=512, I=1024, E=4, K=2, B=128, weights="fp8row", act="swish", bias=True,
                                      clamps=(7.0, None, 7.0, -7.0), scaling="pre", skip_token=False, hybrid=False),
    "b256_bf16_hybrid_gelu": dict(T=600, H=768, I=384, E=6, K=2, B=256, weights="bf16", act="gelu", bias=False,
                                  clamps=(None, None, None, None), scaling="post", skip_token=True, hybrid=True),
}
# name: (T, H, I, E, K, weights, act, all_expert)
DENSE_TKG_CASES = {
    "sel_t8_bf16_silu": (8, 512, 256, 4, 2, "bf16", "silu", False),
    "all_t16_fp8row_swish": (16, 512, 256, 4, 2, "fp8row", "swish", True),
    "sel_t4_fp8row_gelu_tanh": (4, 768, 384, 8, 4, "fp8row", "gelu_tanh", False),
}


def _fp8_exact(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.float8_e4m3fn).float().numpy()


def _dense_weights(rng, E, H, I, kind):
    """``gate_up [E, H, 2, I]``, ``down [E, I, H]`` as fp32 values exactly representable in the storage type, and
    the fp8-row factors (None for bf16): fp8 weights hold values ~N(0, 1) and the factors carry the 0.02 magnitude."""
    if kind == "bf16":
        return (bf16_round(rng.standard_normal((E, H, 2, I)) * 0.02), bf16_round(rng.standard_normal((E, I, H)) * 0.02),
                None, None)
    gu = _fp8_exact(rng.standard_normal((E, H, 2, I)))
    dn = _fp8_exact(rng.standard_normal((E, I, H)))
    return gu, dn, (rng.uniform(0.01, 0.03, (E, 2, I))).astype(np.float32), (rng.uniform(0.01, 0.03, (E, H))).astype(np.float32)


def dense_cte_inputs(name):
    c = DENSE_CTE_CASES[name]
    T, H, I, E, K = c["T"], c["H"], c["I"], c["E"], c["K"]
    rng = np.random.default_rng(_case_seed(name))
    rows = T if c["skip_token"] else T + 1
    hidden = bf16_round(rng.standard_normal((rows, H)))
    if not c["skip_token"]:
        hidden[T] = 0
    gu, dn, gs, ds = _dense_weights(rng, E, H, I, c["weights"])
    idx = np.argsort(-rng.random((T, E)), axis=1, kind="stable")[:, :K].astype(np.int32)
    mask = np.zeros((T, E), dtype=np.int32)
    mask[np.arange(T)[:, None], idx] = 1
    aff = np.zeros((rows, E), dtype=np.float32)
    aff[:T] = bf16_round(rng.random((T, E)) * mask)
    out = dict(case=c, hidden=hidden, aff=aff, expert_index=idx, mask=mask, gate_up=gu, down=dn, gate_up_scale=gs,
               down_scale=ds, bias_gu=None, bias_d=None)
    if c["bias"]:
        out["bias_gu"] = bf16_round(rng.uniform(-2.0625, 0.52, (E, 2, I)))
        out["bias_d"] = bf16_round(rng.uniform(-1.632, 1.4375, (E, H)))
    return out


def dense_tkg_inputs(name):
    T, H, I, E, K, kind, act, all_expert = DENSE_TKG_CASES[name]
    rng = np.random.default_rng(_case_seed(name))
    hidden = bf16_round(rng.standard_normal((T, H)))
    gu, dn, gs, ds = _dense_weights(rng, E, H, I, kind)
    idx = np.argsort(-rng.random((T, E)), axis=1, kind="stable")[:, :K].astype(np.int32)
    aff = bf16_round(rng.random((T, E)))
    return dict(T=T, H=H, I=I, E=E, K=K, weights=kind, act=act, all_expert=all_expert, hidden=hidden, aff=aff,
                expert_index=idx, gate_up=gu, down=dn, gate_up_scale=gs, down_scale=ds,
                bias_gu=bf16_round(rng.uniform(-2.0625, 0.52, (E, 2, I))),
                bias_d=bf16_round(rng.uniform(-1.632, 1.4375, (E, H))), clamps=(7.0, None, 7.0, -7.0))
