"""The allocation-free grouping entry point against the regular one.

Some callers cannot allocate device memory at the point where they need the
token grouping: code running inside an allocator or memory-pool callback, a
plug-in whose host process forbids cudaMalloc once serving has started, a
latency-critical loop that must not wait on another thread's free.  For them
``b200moe_group_tokens_static`` keeps its scratch in a 1 MiB device array that
is part of the library image.  This test drives it through the C ABI twice in
a row (the second call sees whatever the first one left in the shared scratch)
and requires byte-identical results to ``b200moe_group_tokens`` with a
caller-supplied workspace.  It is collected last so a run that stops at the
first failure has already exercised everything else.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib_mod, fn_name, idx, E, B, N, extra):
    T, K = idx.shape
    dev = idx.device
    out = dict(tpi=torch.full((N * B,), 12345, dtype=torch.int32, device=dev),
               b2e=torch.full((N,), 12345, dtype=torch.int32, device=dev),
               cond=torch.full((N + 2,), 12345, dtype=torch.int32, device=dev),
               counts=torch.full((E,), 12345, dtype=torch.int32, device=dev),
               inv=torch.full((T, K), 12345, dtype=torch.int32, device=dev),
               status=torch.full((1,), 12345, dtype=torch.int32, device=dev))
    p = lib_mod.ptr
    lib_mod.call(fn_name, p(idx), lib_mod.ROUTING_INDEX, lib_mod.I32, T, E, K, B, N, 1, 1, p(out["tpi"]), p(out["b2e"]),
                 p(out["cond"]), p(out["counts"]), p(out["inv"]), p(out["status"]), *extra, lib_mod.stream_ptr())
    torch.cuda.synchronize()
    return out


def test_static_scratch_grouping_matches_workspace_grouping():
    from nki_library_b200 import _lib
    import nki_library_b200 as m
    lib = _lib.load_library()
    assert lib.b200moe_group_tokens_static_max_bytes() == 1 << 20
    rng = np.random.default_rng(9)
    # two different problems back to back: the second runs on the first one's leftovers
    for T, E, K, B in ((4096, 8, 2, 512), (8192, 256, 8, 128)):
        scores = rng.random((T, E))
        idx = torch.from_numpy(np.argsort(-scores, axis=1)[:, :K].astype(np.int32)).cuda()
        N = m.get_n_blocks(T, K, E, B)
        need = lib.b200moe_group_tokens_workspace_bytes(T, E)
        assert need <= lib.b200moe_group_tokens_static_max_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        ref = _run(_lib, "b200moe_group_tokens", idx, E, B, N, (_lib.ptr(ws), need))
        got = _run(_lib, "b200moe_group_tokens_static", idx, E, B, N, ())
        again = _run(_lib, "b200moe_group_tokens_static", idx, E, B, N, ())
        for k in ref:
            assert torch.equal(ref[k], got[k]), k
            assert torch.equal(ref[k], again[k]), k
        assert int(got["status"].item()) == 0


def test_static_scratch_grouping_rejects_oversized_problems():
    from nki_library_b200 import _lib
    lib = _lib.load_library()
    T, E = 1 << 20, 512  # 4096 chunks x 512 experts x 4 bytes = 8 MiB of counters
    assert lib.b200moe_group_tokens_workspace_bytes(T, E) > lib.b200moe_group_tokens_static_max_bytes()
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    p = _lib.ptr(dummy)
    rc = lib.b200moe_group_tokens_static(p, _lib.ROUTING_INDEX, _lib.I32, T, E, 2, 128, 4, 1, 1, p, p, p, p, None, p,
                                         _lib.stream_ptr())
    assert rc == -3
    msg = lib.b200moe_last_error().decode()
    assert "built-in scratch" in msg and "b200moe_group_tokens" in msg
