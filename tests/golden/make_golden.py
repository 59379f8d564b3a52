"""Generate the golden fixtures in this directory from the reference's own CPU code.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It also runs the reference's element decoders ``unpack_float4_x4``,
``unpack_float8_e5m2_x4`` and ``unpack_float8_e4m3fn_x4``
(``core/utils/mx_torch_common.py:31-131``) over every 16-bit fp4 word and every
fp8 byte; their module imports the Trainium toolchain at the top, so the three
functions (and the lookup table they use) are compiled on their own from the
module's source.

It imports the three reference torch references that load without the Trainium
toolchain (``router_topk_torch_ref``, ``find_nonzero_indices_torch_ref``,
``indexed_flatten_torch_ref``), feeds them the seed-generated inputs of the
reference's own tests (``test_router_topk_common.py:30-49``,
``test_find_nonzero_indices.py:29-45,63-82``, ``test_indexed_flatten.py:28-70``)
and stores their outputs: small cases in full, large ones as SHA-256 digests.
The MX CPU code (``quantize_to_mx``, ``mx_matmul``, the projection goldens,
``generate_blockwise_numpy_golden``, ``_moe_tkg_mx_ref``) is run by
``make_golden_mx.py``, which this script calls last.
Inputs are not stored; ``tests/golden_inputs.py`` regenerates them from the
same seeds.  The tests then check the CPU oracle (and, on a GPU, the CUDA
path) against these files without needing the reference checkout.
"""

from __future__ import annotations

import ast
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import golden_inputs as gi  # noqa: E402


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def load_functions(path: str, names) -> dict:
    """Compile the named top-level functions / assignments of a module without running the rest of it."""
    with open(path) as f:
        tree = ast.parse(f.read())
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(getattr(t, "id", None) in names for t in node.targets):
            keep.append(node)
    ns = {"torch": torch, "np": np}
    exec(compile(ast.Module(keep, []), path, "exec"), ns)
    return ns


def element_decoders(ref_root: str) -> None:
    ns = load_functions(os.path.join(ref_root, "src", "nkilib_src", "nkilib", "core", "utils", "mx_torch_common.py"),
                        {"_FP4_LUT", "unpack_float4_x4", "unpack_float8_e5m2_x4", "unpack_float8_e4m3fn_x4"})
    words16 = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    bytes_all = np.arange(256, dtype=np.uint8).view(np.uint32).reshape(1, 64)
    np.savez_compressed(
        os.path.join(HERE, "mx_element_decode_ref.npz"),
        e2m1_x4=ns["unpack_float4_x4"](words16).numpy().astype(np.float32),          # [256, 1024]
        e5m2_x4=ns["unpack_float8_e5m2_x4"](bytes_all).numpy().astype(np.float32),   # [1, 256]
        e4m3_x4=ns["unpack_float8_e4m3fn_x4"](bytes_all).numpy().astype(np.float32))


def main(ref_root: str) -> None:
    element_decoders(ref_root)
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from nkilib_src.nkilib.core.router_topk.router_topk_torch import router_topk_torch_ref
    from nkilib_src.nkilib.core.subkernels.find_nonzero_indices_torch import find_nonzero_indices_torch_ref
    from nkilib_src.nkilib.core.subkernels.indexed_flatten_torch import indexed_flatten_torch_ref
    from nkilib_src.nkilib.core.utils.common_types import RouterActFnType

    # ---- router ---------------------------------------------------------
    router = {}
    for name, (T, H, E, k, act, has_bias, pre_norm, norm_topk) in gi.ROUTER_CASES.items():
        x, w, b = gi.router_inputs(T, H, E, has_bias)
        out = router_topk_torch_ref(
            x=x.float(), w=w.float(), w_bias=None if b is None else b.float(),
            router_logits=None, expert_affinities=None, expert_index=None,
            act_fn=RouterActFnType.SOFTMAX if act == "softmax" else RouterActFnType.SIGMOID,
            k=k, x_hbm_layout=1, x_sb_layout=0, router_pre_norm=pre_norm, norm_topk_prob=norm_topk)
        router[name + "/logits"] = out["router_logits"].numpy().astype(np.float32)
        router[name + "/index"] = out["expert_index"].numpy().astype(np.int32)
        router[name + "/aff"] = out["expert_affinities"].numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "router_topk_ref.npz"), **router)

    # ---- find_nonzero_indices / indexed_flatten -------------------------
    digests = {"find_nonzero_indices": {}, "indexed_flatten": {}, "grouping_chain": {}}
    small = {}
    for name, (T, E, top_k, dtype, col_start, n_cols) in gi.NONZERO_CASES.items():
        inp = gi.sparse_input(T, E, top_k, dtype)
        kw = {}
        if col_start is not None:
            kw = dict(col_start_id=torch.tensor([col_start], dtype=torch.int32), n_cols=n_cols)
        out = find_nonzero_indices_torch_ref(torch.from_numpy(inp), **kw)
        ind = out["indices"].numpy().astype(np.int32)
        cnt = out["nonzero_counts"].numpy().astype(np.int32)
        digests["find_nonzero_indices"][name] = {"indices": digest(ind), "counts": digest(cnt)}
        if T <= 512:
            small[name + "/indices"] = ind
            small[name + "/counts"] = cnt

    for name, (T, E, f_len, n_off, start) in gi.FLATTEN_CASES.items():
        kw = gi.flatten_inputs(T, E, f_len, n_off, start)
        out = indexed_flatten_torch_ref(
            torch.from_numpy(kw["input_tensor"]), kw["f_len"], kw["output_len"],
            torch.from_numpy(kw["row_offsets"]),
            None if kw["row_offsets_start"] is None else torch.tensor([kw["row_offsets_start"]]),
            kw["padding_val"])
        digests["indexed_flatten"][name] = digest(out["flattened_array"].numpy().astype(np.int32))

    # ---- the reference's three grouping steps chained: mask -> token_position_to_id
    for name, (T, E, K, B) in gi.CHAIN_CASES.items():
        mask = gi.routing_mask(T, E, K)
        fz = find_nonzero_indices_torch_ref(torch.from_numpy(mask))
        counts = fz["nonzero_counts"].numpy()
        bpe = -(-counts // B)
        offs = np.concatenate([[0], np.cumsum(bpe)[:-1]]).astype(np.int32)
        N = gi.n_blocks(T, K, E, B)
        Tpad = -(-T // B) * B
        ind = np.full((E, Tpad), -1, dtype=np.int32)
        ind[:, :T] = fz["indices"].numpy()
        fl = indexed_flatten_torch_ref(torch.from_numpy(ind), B, N * B, torch.from_numpy(offs))
        tpi = fl["flattened_array"].numpy().astype(np.int32)
        digests["grouping_chain"][name] = digest(tpi)
        if T <= 512:
            small[name + "/tpi"] = tpi

    np.savez_compressed(os.path.join(HERE, "grouping_ref_small.npz"), **small)
    with open(os.path.join(HERE, "grouping_ref_digests.json"), "w") as f:
        json.dump(digests, f, indent=1, sort_keys=True)
    print("wrote fixtures to", HERE)
    # MX arithmetic (quantise, block-scaled matmul, projections, prefill block loop, decode): needs the two
    # stand-in packages under tests/golden/standins, see make_golden_mx.py
    import make_golden_mx
    make_golden_mx.main(ref_root)


if __name__ == "__main__":
    main(sys.argv[1])
