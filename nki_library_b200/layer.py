"""One MoE layer = router_topk -> token grouping -> blockwise MXFP8 expert MLP -> combine.

This is the call sequence the reference leaves to its caller for prefill
(router and grouping sub-kernels, then ``moe_cte``) and fuses for decode in
``moe_block_tkg`` (core/moe_block/moe_block_tkg.py:192-340, without the RMSNorm).
All buffers are allocated once; a forward pass launches nine to twelve kernels
(``kernels_per_forward``) on the current stream and never synchronises with the
host.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib, pipeline
from .core.moe.moe_cte.moe_cte_utils import get_n_blocks
from .core.utils.common_types import ActFnType, RouterActFnType
from .weights import ExpertWeights


class MoELayer:
    def __init__(self, router_w: torch.Tensor, weights: ExpertWeights, top_k: int, block_size: int,
                 max_tokens: int, router_bias: Optional[torch.Tensor] = None,
                 router_act: RouterActFnType = RouterActFnType.SOFTMAX, router_pre_norm: bool = True,
                 norm_topk_prob: bool = True, act_fn: ActFnType = ActFnType.SiLU, router_path: int = 0,
                 gemm_variant: int = 0):
        """``router_path`` / ``gemm_variant`` are the per-call variant words of the router and of the grouped
        contractions (0 = the library's own choice)."""
        _lib.require_cuda(router_w, router_bias)
        self.router_path, self.gemm_variant = int(router_path), int(gemm_variant)
        self.clock_probe = None  # optional int64[4] device tensor: {cycles, ns} of the gate/up and down contractions
        self.w = router_w.to(torch.bfloat16).contiguous()
        self.bias = None if router_bias is None else router_bias.reshape(-1).to(torch.bfloat16).contiguous()
        self.weights = weights
        self.E, self.H, self.I = weights.E, weights.H, weights.I
        _lib.kernel_assert(tuple(self.w.shape) == (self.H, self.E), "router weight must be [H, E]")
        self.K, self.B, self.T = top_k, block_size, max_tokens
        self.router_act, self.pre_norm, self.l1, self.act_fn = router_act, router_pre_norm, norm_topk_prob, act_fn
        dev = self.w.device
        T, E, K, B = max_tokens, self.E, top_k, block_size
        self.N = get_n_blocks(T, K, E, B)
        lib = _lib.load_library()
        self.aff = torch.empty((T, E), dtype=torch.float32, device=dev)
        self.idx = torch.empty((T, K), dtype=torch.int32, device=dev)
        self.tpi = torch.empty(self.N * B, dtype=torch.int32, device=dev)
        self.b2e = torch.empty(self.N, dtype=torch.int32, device=dev)
        self.cond = torch.empty(self.N + 2, dtype=torch.int32, device=dev)
        self.counts = torch.empty(E, dtype=torch.int32, device=dev)
        self.inv = torch.empty((T, K), dtype=torch.int32, device=dev)
        self.gstatus = torch.zeros(1, dtype=torch.int32, device=dev)
        self.rws = torch.empty(lib.b200moe_router_workspace_bytes(T, self.H, E), dtype=torch.uint8, device=dev)
        self.gws = torch.empty(lib.b200moe_group_tokens_workspace_bytes(T, E), dtype=torch.uint8, device=dev)
        self.ws = pipeline.BlockWorkspace(self.N * B, self.H, self.I, dev)
        self.out = torch.empty((T, self.H), dtype=torch.bfloat16, device=dev)
        # launches per forward pass: router (logits + ranking, or weight transpose + tcgen05 logits + ranking for
        # large T), grouping (3, or 1 up to 256 tokens), quantise, the contractions (CTA-pair launch + left-over launch each when the
        # library takes its pair path, else one each), combine -- mirrors the library's own shape rules
        tc_ok = E <= 256 and self.H % 64 == 0
        router_launches = 3 if (tc_ok and (router_path == 2 or (router_path == 0 and T >= 8192))) else 2
        pair_path = not (gemm_variant & (_lib.GEMM_NO_PAIR | _lib.GEMM_TILE_N128)) and (
            B % 256 == 0 or bool(gemm_variant & _lib.GEMM_FORCE_PAIR) or self.N * (B // 128) >= 4 * E)
        group_launches = 1 if T <= 256 else 3  # one 256-token chunk: the three grouping phases share a CTA
        self.kernels_per_forward = router_launches + group_launches + 1 + (2 if not pair_path else (2 if gemm_variant & _lib.GEMM_NO_SPLIT else 4)) + 1

    def forward(self, hidden: torch.Tensor, timers: Optional[dict] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``hidden`` bf16 ``[T, H]`` on the device; returns the bf16 ``[T, H]`` output (``out`` if given, else the
        layer's own buffer)."""
        T = hidden.shape[0]
        out = self.out if out is None else out
        _lib.kernel_assert(tuple(out.shape) == (self.T, self.H) and out.dtype == torch.bfloat16 and out.is_contiguous(),
                           "out must be a contiguous bf16 [max_tokens, H] tensor")
        _lib.kernel_assert(T == self.T and hidden.shape[1] == self.H and hidden.dtype == torch.bfloat16,
                           "hidden must be bf16 [max_tokens, H]")
        st = _lib.stream_ptr()
        E, K, B, N, H, I = self.E, self.K, self.B, self.N, self.H, self.I
        w, ws = self.weights, self.ws

        def timed(name, fn):
            if timers is None:
                fn()
                return
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            timers.setdefault(name, []).append((a, b))

        timed("router_topk", lambda: _lib.call(
            "b200moe_router_topk", _lib.ptr(hidden), 1, _lib.ptr(self.w), _lib.ptr(self.bias), T, H, E, K,
            self.router_act.value, int(self.pre_norm), int(self.l1), None, _lib.F32, _lib.ptr(self.idx),
            _lib.ptr(self.aff), _lib.F32, self.router_path, _lib.ptr(self.rws), self.rws.numel(), st))
        timed("group_tokens", lambda: _lib.call(
            "b200moe_group_tokens", _lib.ptr(self.idx), _lib.ROUTING_INDEX, _lib.I32, T, E, K, B, N, 1, 1,
            _lib.ptr(self.tpi), _lib.ptr(self.b2e), _lib.ptr(self.cond), _lib.ptr(self.counts), _lib.ptr(self.inv),
            _lib.ptr(self.gstatus), _lib.ptr(self.gws), self.gws.numel(), st))
        # token-major: each row is read and quantised once and stored to its K positions
        timed("gather_quantize", lambda: _lib.call(
            "b200moe_scatter_quantize_mxfp8", _lib.ptr(hidden), T, H, _lib.ptr(self.inv), K, N * B,
            int(w.h_packed_order), _lib.ptr(ws.xq), _lib.ptr(ws.x_sf), _lib.ptr(ws.tile_flags), st))
        nan = float("nan")
        timed("gemm1_swiglu", lambda: _lib.call(
            "b200moe_grouped_gemm1_swiglu", _lib.ptr(ws.xq), _lib.ptr(ws.x_sf), _lib.ptr(w.w1), _lib.ptr(w.w1_sf), w.w_format,
            _lib.ptr(w.bias_gu), _lib.ptr(self.b2e), _lib.ptr(self.cond), _lib.ptr(ws.tile_flags), N, B, E, H, I,
            self.act_fn.value, nan, nan, nan, nan, _lib.ptr(ws.mq), _lib.ptr(ws.m_sf), _lib.ptr(ws.status[1:]),
            self.gemm_variant, None if self.clock_probe is None else _lib.ptr(self.clock_probe[0:]), st))
        timed("gemm2_scale", lambda: _lib.call(
            "b200moe_grouped_gemm2_scale", _lib.ptr(ws.mq), _lib.ptr(ws.m_sf), _lib.ptr(w.w2), _lib.ptr(w.w2_sf), w.w_format,
            _lib.ptr(w.bias_d), _lib.ptr(self.b2e), _lib.ptr(self.cond), _lib.ptr(ws.tile_flags), _lib.ptr(self.tpi),
            T, N, B, E, H, I, _lib.ptr(self.aff), _lib.F32, 0, _lib.ptr(ws.y_pos), _lib.ptr(ws.status[2:]),
            self.gemm_variant, None if self.clock_probe is None else _lib.ptr(self.clock_probe[2:]), st))
        timed("combine", lambda: _lib.call(
            "b200moe_combine", _lib.ptr(ws.y_pos), _lib.ptr(self.inv), T, K, H, _lib.ptr(out), st))
        return out

    def capture(self, hidden: torch.Tensor) -> None:
        """Record one forward pass on ``hidden`` (a fixed device buffer) into a CUDA graph.

        Call after at least one eager ``forward`` (kernel attributes are set on first use).
        ``replay()`` then re-runs the whole launch sequence with one submission.
        """
        self._graph_input = hidden
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self.forward(hidden)

    def replay(self) -> torch.Tensor:
        self._graph.replay()
        return self.out

    def capture_slots(self, hiddens, outs) -> None:
        """One graph per (input buffer, output buffer) pair, for callers that alternate staging buffers and
        want the layer to read and write them in place.  ``replay_slot(i)`` runs pair i."""
        self._slot_graphs = []
        for h, o in zip(hiddens, outs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.forward(h, out=o)
            self._slot_graphs.append(g)

    def replay_slot(self, i: int) -> None:
        self._slot_graphs[i].replay()

    def device_status(self) -> list:
        """[grouping, gate/up contraction, down contraction, router] status words (0 = fine); synchronises."""
        return ([int(self.gstatus.item())] + self.ws.status.cpu().tolist()[1:3] +
                [int(self.rws[:4].view(torch.int32).item())])


def random_expert_weights(E: int, H: int, I: int, device, seed: int = 0, std: float = 0.02,
                          w_format: int = _lib.W_E4M3) -> ExpertWeights:
    """Synthetic MX expert weights, generated on the device directly in the feed layout.

    e4m3: bf16 values ~ N(0, std) are pushed through the library's own MXFP8
    quantiser (block-32 UE8M0 scales along the contraction axis); rows are
    i.i.d., so no relayout is needed.  e5m2 / e2m1: uniformly random finite
    element codes with block scales of 2^-9 .. 2^-6, which gives weights of the
    same order of magnitude.
    """
    lib = _lib.load_library()
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    if w_format != _lib.W_E4M3:
        per = 2 if w_format == _lib.W_E2M1 else 1

        def codes(rows, K):
            if w_format == _lib.W_E2M1:
                return torch.randint(0, 256, (E, rows, K // per), dtype=torch.uint8, device=device, generator=gen)
            sign = torch.randint(0, 2, (E, rows, K), dtype=torch.uint8, device=device, generator=gen) << 7
            expo = torch.randint(9, 17, (E, rows, K), dtype=torch.uint8, device=device, generator=gen) << 2
            return sign | expo | torch.randint(0, 4, (E, rows, K), dtype=torch.uint8, device=device, generator=gen)

        def scales(rows, K):
            return torch.randint(118, 122, (E * lib.b200moe_sf_bytes(rows, K),), dtype=torch.uint8, device=device,
                                 generator=gen)

        return ExpertWeights(E, H, I, codes(2 * I, H), scales(2 * I, H), codes(H, I), scales(H, I), None, None, False,
                             w_format)
    w1 = torch.empty((E, 2 * I, H), dtype=torch.uint8, device=device)
    w2 = torch.empty((E, H, I), dtype=torch.uint8, device=device)
    sf1_e, sf2_e = lib.b200moe_sf_bytes(2 * I, H), lib.b200moe_sf_bytes(H, I)
    w1_sf = torch.zeros(E * sf1_e, dtype=torch.uint8, device=device)
    w2_sf = torch.zeros(E * sf2_e, dtype=torch.uint8, device=device)
    st = _lib.stream_ptr()
    for e in range(E):
        a = (torch.randn((2 * I, H), device=device, generator=gen) * std).to(torch.bfloat16)
        _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(a), 2 * I, H, None, 2 * I, 0, _lib.ptr(w1[e]),
                  _lib.ptr(w1_sf[e * sf1_e:]), None, st)
        b = (torch.randn((H, I), device=device, generator=gen) * std).to(torch.bfloat16)
        _lib.call("b200moe_gather_quantize_mxfp8", _lib.ptr(b), H, I, None, H, 0, _lib.ptr(w2[e]),
                  _lib.ptr(w2_sf[e * sf2_e:]), None, st)
        torch.cuda.synchronize()
    return ExpertWeights(E, H, I, w1, w1_sf, w2, w2_sf, None, None, False)


class HostPipeline:
    """Feeds a captured layer (:class:`MoELayer` or the peer-memory expert-parallel layer) from host memory
    with copies overlapped with compute.

    ``submit(host_in, host_out)`` enqueues: pinned host -> device staging (copy stream), the layer (compute
    stream, CUDA graph), device -> pinned host (second copy stream).  Two staging buffers each way let step
    i + 1's upload and step i - 1's download run while step i computes.  A :class:`MoELayer` is captured once
    per staging pair and reads / writes the staging buffers directly, so the compute stream never queues a
    device-to-device copy behind a PCIe transfer on a copy engine.  ``drain()`` waits for everything.
    """

    def __init__(self, layer):
        dev = layer.out.device
        self.layer = layer
        # the set-up pass below runs on real-looking data: with uninitialised (or constant) input every token may
        # pick the same experts, which an expert-parallel layer reports as a receive-buffer overflow
        self.hidden = torch.randn((layer.T, layer.H), dtype=torch.float32, device=dev).to(torch.bfloat16)
        layer.forward(self.hidden)  # make sure every kernel attribute is set before capture
        torch.cuda.synchronize()
        layer.capture(self.hidden)
        self.stage_in = [torch.empty_like(self.hidden) for _ in range(2)]
        self.stage_out = [torch.empty_like(layer.out) for _ in range(2)]
        # a layer that can be captured once per staging pair works on the staging buffers in place; otherwise
        # its fixed input / output buffers are filled and drained with device-to-device copies
        self.in_place = hasattr(layer, "capture_slots")
        if self.in_place:
            layer.capture_slots(self.stage_in, self.stage_out)
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]        # upload i finished
        self.ev_in_free = [torch.cuda.Event() for _ in range(2)]   # compute consumed staging i
        self.ev_out = [torch.cuda.Event() for _ in range(2)]       # result i staged
        self.ev_out_free = [torch.cuda.Event() for _ in range(2)]  # download i finished
        self.step = 0

    def submit(self, host_in: torch.Tensor, host_out: torch.Tensor) -> None:
        i = self.step & 1
        first = self.step < 2
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if not first:
                self.s_in.wait_event(self.ev_in_free[i])
            self.stage_in[i].copy_(host_in, non_blocking=True)
            self.ev_in[i].record(self.s_in)
        cur.wait_event(self.ev_in[i])
        if self.in_place:
            if not first:
                cur.wait_event(self.ev_out_free[i])
            self.layer.replay_slot(i)
            self.ev_in_free[i].record(cur)
        else:
            self.hidden.copy_(self.stage_in[i], non_blocking=True)
            self.ev_in_free[i].record(cur)
            self.layer.replay()
            if not first:
                cur.wait_event(self.ev_out_free[i])
            self.stage_out[i].copy_(self.layer.out, non_blocking=True)
        self.ev_out[i].record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_out[i])
            host_out.copy_(self.stage_out[i], non_blocking=True)
            self.ev_out_free[i].record(self.s_out)
        self.step += 1

    def drain(self) -> None:
        self.s_in.synchronize()
        self.s_out.synchronize()
        torch.cuda.current_stream().synchronize()
