// Router: logits = x @ w (+ bias) in fp32, warp-shuffle top-K, softmax / sigmoid
// affinities, optional L1 normalisation, dense scatter.
//
// Two launches.  (1) A split-K bf16 tensor-core GEMM (mma.sync m16n8k16, fp32
// accumulate): the grid is (token tiles) x (hidden-axis splits) so that even a
// 64-token decode batch spreads over every SM; x and w slabs are staged through
// shared memory with a 2- or 3-deep cp.async ring and each split writes its own
// partial-logit slab (no atomics, so the sum order is fixed).  (2) One warp per
// token adds the partials in split order plus the bias, keeps E/32 logits per
// lane and reduces a (value, lowest index) arg-max with shuffles K times.
#include "common.cuh"

namespace b200moe {
// Large-T path (router_tc.cu): the logits GEMM on the tcgen05 tensor cores, one pass over x.
size_t router_tc_workspace_bytes(int T, int H, int E);
bool router_tc_eligible(int x_is_TH, int T, int H, int E);
int router_tc_run(const void* x, const void* w, int T, int H, int E, void* workspace, int32_t* status,
                  float** logits_out, cudaStream_t st);

namespace {

constexpr size_t kWsHeader = 256;  // workspace bytes in front of the scratch: int32 status word, then padding
constexpr int kTcMinTokens = 8192;

constexpr int kKC = 64;           // hidden slab per pipeline stage
constexpr int kXPad = 8;          // halfs of padding per smem row (bank spread)
constexpr int kMaxEPerLane = 16;  // E <= 512

struct LogitArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  int x_is_TH, T, H, E;
  int mw, nw;        // warps along tokens / experts (mw * nw == 8)
  int h_per_split;   // multiple of kKC
  int stages;        // cp.async ring depth (2 or 3)
  float* partial;    // [splits][T][E]
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// x slab in shared memory: [tok][kKC + pad] when x is [T, H]; [kKC][tok + pad] when x is [H, T].
// w slab: [kKC][EN + pad].
__global__ void __launch_bounds__(256) router_logits_kernel(LogitArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int TM = 16 * a.mw, EN = 64 * a.nw;
  const int x_stride = a.x_is_TH ? (kKC + kXPad) : (TM + kXPad);
  const int x_rows = a.x_is_TH ? TM : kKC;
  const int w_stride = EN + kXPad;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* ws = xs + a.stages * x_rows * x_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / a.nw, wn = warp % a.nw;
  const int t0 = blockIdx.x * TM;
  const int h_lo = blockIdx.y * a.h_per_split;
  const int h_hi = min(a.H, h_lo + a.h_per_split);
  const int n_chunks = (h_hi - h_lo + kKC - 1) / kKC;
  const bool x_vec = a.x_is_TH ? (a.H % 8 == 0) : (a.T % 8 == 0);
  const bool w_vec = (a.E % 8 == 0);

  auto load_chunk = [&](int chunk, int buf) {
    const int h0 = h_lo + chunk * kKC;
    __nv_bfloat16* xb = xs + buf * x_rows * x_stride;
    __nv_bfloat16* wb = ws + buf * kKC * w_stride;
    if (a.x_is_TH) {
      if (x_vec) {
        for (int i = tid; i < TM * (kKC / 8); i += 256) {
          const int r = i / (kKC / 8), c = (i - r * (kKC / 8)) * 8;
          const bool ok = (t0 + r < a.T) && (h0 + c < h_hi);
          cp_async16(xb + r * x_stride + c, a.x + (ok ? static_cast<int64_t>(t0 + r) * a.H + h0 + c : 0), ok);
        }
      } else {
        for (int i = tid; i < TM * kKC; i += 256) {
          const int r = i / kKC, c = i - r * kKC;
          const bool ok = (t0 + r < a.T) && (h0 + c < h_hi);
          xb[r * x_stride + c] = ok ? a.x[static_cast<int64_t>(t0 + r) * a.H + h0 + c] : __float2bfloat16(0.f);
        }
      }
    } else {
      if (x_vec) {
        for (int i = tid; i < kKC * (TM / 8); i += 256) {
          const int r = i / (TM / 8), c = (i - r * (TM / 8)) * 8;
          const bool ok = (h0 + r < h_hi) && (t0 + c < a.T);
          cp_async16(xb + r * x_stride + c, a.x + (ok ? static_cast<int64_t>(h0 + r) * a.T + t0 + c : 0), ok);
        }
      } else {
        for (int i = tid; i < kKC * TM; i += 256) {
          const int r = i / TM, c = i - r * TM;
          const bool ok = (h0 + r < h_hi) && (t0 + c < a.T);
          xb[r * x_stride + c] = ok ? a.x[static_cast<int64_t>(h0 + r) * a.T + t0 + c] : __float2bfloat16(0.f);
        }
      }
    }
    if (w_vec) {
      for (int i = tid; i < kKC * (EN / 8); i += 256) {
        const int r = i / (EN / 8), c = (i - r * (EN / 8)) * 8;
        const bool ok = (h0 + r < h_hi) && (c < a.E);
        cp_async16(wb + r * w_stride + c, a.w + (ok ? static_cast<int64_t>(h0 + r) * a.E + c : 0), ok);
      }
    } else {
      for (int i = tid; i < kKC * EN; i += 256) {
        const int r = i / EN, c = i - r * EN;
        const bool ok = (h0 + r < h_hi) && (c < a.E);
        wb[r * w_stride + c] = ok ? a.w[static_cast<int64_t>(h0 + r) * a.E + c] : __float2bfloat16(0.f);
      }
    }
    cp_async_commit();
  };

  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  // ring of `stages` slabs; one commit group per loop step (possibly empty) keeps the wait count fixed
  for (int c = 0; c < a.stages - 1; ++c) {
    if (c < n_chunks) load_chunk(c, c);
    else cp_async_commit();
  }
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int buf = ch % a.stages;
    const int nxt = ch + a.stages - 1;
    if (nxt < n_chunks) load_chunk(nxt, nxt % a.stages);
    else cp_async_commit();
    if (a.stages == 3) cp_async_wait<2>();
    else cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* xb = xs + buf * x_rows * x_stride;
    const __nv_bfloat16* wb = ws + buf * kKC * w_stride;
#pragma unroll
    for (int k16 = 0; k16 < kKC / 16; ++k16) {
      uint32_t af[4];
      if (a.x_is_TH) {
        // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
        ldmatrix_x4(af, xb + (wm * 16 + (lane & 15)) * x_stride + k16 * 16 + (lane >> 4) * 8);
      } else {
        const int i = lane >> 3;
        ldmatrix_x4_trans(af, xb + (k16 * 16 + (i >> 1) * 8 + (lane & 7)) * x_stride + wm * 16 + (i & 1) * 8);
      }
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, wb + (k16 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * w_stride + wn * 64 + (j + (lane >> 4)) * 8);
        mma_bf16(acc[j], af, bf[0], bf[1]);
        mma_bf16(acc[j + 1], af, bf[2], bf[3]);
      }
    }
    __syncthreads();
  }

  float* out = a.partial + static_cast<int64_t>(blockIdx.y) * a.T * a.E;
  const int r0 = t0 + wm * 16 + (lane >> 2);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = wn * 64 + j * 8 + (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = r0 + (i >> 1) * 8, ee = e + (i & 1);
      if (t < a.T && ee < a.E) out[static_cast<int64_t>(t) * a.E + ee] = acc[j][i];
    }
  }
}

struct RankArgs {
  const float* partial;
  int splits;
  const __nv_bfloat16* bias;
  int T, E, k, act, pre_norm, l1;
  void* logits_out;
  int logits_dtype;
  uint32_t* index_out;
  void* aff_out;
  int aff_dtype;
};

// NPL = experts per lane (E <= 32 * NPL); instantiated for 1, 2, 4, 8, 16 so small expert counts do not pay for 512.
template <int NPL>
__global__ void __launch_bounds__(256) router_rank_kernel(RankArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= a.T) return;
  const int E = a.E;
  const int n_per_lane = (E + 31) / 32;

  float v[NPL];
  float row_max = -INFINITY;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int e = lane + 32 * j;
    float s = -INFINITY;
    if (j < n_per_lane && e < E) {
      s = 0.f;
      for (int sp = 0; sp < a.splits; ++sp) s += a.partial[(static_cast<int64_t>(sp) * a.T + t) * E + e];
      if (a.bias != nullptr) s += __bfloat162float(a.bias[e]);
      if (a.logits_out != nullptr) store_from_float(a.logits_out, static_cast<int64_t>(t) * E + e, a.logits_dtype, s);
    }
    v[j] = s;
    row_max = fmaxf(row_max, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));

  // activation over the full row (pre-norm pipelines)
  float full[NPL];
  if (a.pre_norm) {
    if (a.act == B200MOE_ROUTER_SOFTMAX) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < NPL; ++j) {
        full[j] = (v[j] == -INFINITY) ? 0.f : expf(v[j] - row_max);
        s += full[j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float inv = 1.0f / s;
#pragma unroll
      for (int j = 0; j < NPL; ++j) full[j] *= inv;
    } else {
#pragma unroll
      for (int j = 0; j < NPL; ++j) full[j] = 1.0f / (1.0f + expf(-v[j]));
    }
  }

  // K rounds of arg-max with lowest-index tie break.  Logits become order-preserving 32-bit keys, so a
  // round is one warp-wide integer max (the winning value) and one integer min (the lowest expert holding
  // it) instead of a shuffle tree over (value, index) pairs.  Key 0 marks "nothing left in this lane".
  uint32_t key[NPL];
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    uint32_t u = __float_as_uint(v[j]);
    if (u == 0x80000000u) u = 0u;  // -0 ranks with +0
    const int e = lane + 32 * j;
    key[j] = (j < n_per_lane && e < E) ? ((u & 0x80000000u) ? ~u : (u | 0x80000000u)) : 0u;
  }
  float top_v[8];
  int top_e[8];
  float top_a[8];  // activated value of the selected expert (pre-norm)
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if (r >= a.k) break;
    uint32_t bk = 0;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < NPL; ++j)
      if (key[j] > bk) { bk = key[j]; be = lane + 32 * j; }
    const uint32_t mk = __reduce_max_sync(0xffffffffu, bk);
    const int win = static_cast<int>(__reduce_min_sync(0xffffffffu, static_cast<uint32_t>(bk == mk ? be : 0x7fffffff)));
    if ((win & 31) == lane) {
#pragma unroll
      for (int j = 0; j < NPL; ++j)
        if (j == (win >> 5)) key[j] = 0u;
    }
    top_v[r] = __uint_as_float((mk & 0x80000000u) ? (mk & 0x7fffffffu) : ~mk);
    top_e[r] = win;
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    top_a[r] = 0.f;
    if (r < a.k && a.pre_norm) {
      float mine = 0.f;
#pragma unroll
      for (int j = 0; j < NPL; ++j)
        if (j == (top_e[r] >> 5)) mine = full[j];
      top_a[r] = __shfl_sync(0xffffffffu, mine, top_e[r] & 31);
    }
  }

  if (a.index_out != nullptr && lane < a.k) {
    int e_out = 0;
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r == lane) e_out = top_e[r];
    a.index_out[static_cast<int64_t>(t) * a.k + lane] = static_cast<uint32_t>(e_out);
  }
  if (a.aff_out == nullptr) return;

  if (a.pre_norm && !a.l1) {
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
      const int e = lane + 32 * j;
      if (j < n_per_lane && e < E) store_from_float(a.aff_out, static_cast<int64_t>(t) * E + e, a.aff_dtype, full[j]);
    }
    return;
  }
  // sparse rows: values of the K winners
  float val[8];
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    val[r] = 0.f;
    if (r < a.k) {
      if (a.pre_norm) val[r] = top_a[r];
      else if (a.act == B200MOE_ROUTER_SOFTMAX) val[r] = expf(top_v[r] - top_v[0]);
      else val[r] = 1.0f / (1.0f + expf(-top_v[r]));
      s += val[r];
    }
  }
  const bool normalise = a.pre_norm || a.act == B200MOE_ROUTER_SOFTMAX;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int e = lane + 32 * j;
    if (j < n_per_lane && e < E) {
      float out = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < a.k && top_e[r] == e) out = normalise ? val[r] / s : val[r];
      store_from_float(a.aff_out, static_cast<int64_t>(t) * E + e, a.aff_dtype, out);
    }
  }
}

struct RouterPlan {
  int mw, nw, tm, splits, h_per_split, stages;
  size_t smem;
};

RouterPlan plan_router(int T, int H, int E, int x_is_TH) {
  RouterPlan p;
  p.nw = (E + 63) / 64;
  if (p.nw > 8) p.nw = 8;
  if (p.nw == 3) p.nw = 4;
  if (p.nw > 4 && p.nw < 8) p.nw = 8;
  p.mw = 8 / p.nw;
  p.tm = 16 * p.mw;
  const int token_tiles = (T + p.tm - 1) / p.tm;
  const int max_splits = (H + 4 * kKC - 1) / (4 * kKC);  // at least 128 hidden columns per split
  int want = (2 * sm_count() + token_tiles - 1) / token_tiles;
  if (want < 1) want = 1;
  p.splits = want < max_splits ? want : max_splits;
  p.h_per_split = (((H + p.splits - 1) / p.splits) + kKC - 1) / kKC * kKC;
  p.splits = (H + p.h_per_split - 1) / p.h_per_split;
  const int EN = 64 * p.nw;
  const int x_rows = x_is_TH ? p.tm : kKC;
  const int x_stride = x_is_TH ? (kKC + kXPad) : (p.tm + kXPad);
  const size_t per_stage = sizeof(__nv_bfloat16) * (static_cast<size_t>(x_rows) * x_stride + static_cast<size_t>(kKC) * (EN + kXPad));
  p.stages = 3 * per_stage <= 160 * 1024 ? 3 : 2;
  p.smem = p.stages * per_stage;
  return p;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_router_workspace_bytes(int T, int H, int E) {
  const RouterPlan p = plan_router(T, H, E, 1);
  const size_t split_k = static_cast<size_t>(p.splits) * T * E * sizeof(float);
  const size_t tc = router_tc_workspace_bytes(T, H, E);
  return kWsHeader + (split_k > tc ? split_k : tc);
}

extern "C" int b200moe_router_topk(const void* x, int x_is_TH, const void* w, const void* w_bias, int T, int H, int E,
                                   int k, int act_fn, int router_pre_norm, int norm_topk_prob, void* router_logits,
                                   int logits_dtype, uint32_t* expert_index, void* expert_affinities, int aff_dtype,
                                   int path, void* workspace, size_t workspace_bytes, b200moe_stream_t stream) {
  B200MOE_REQUIRE(path >= 0 && path <= 2, B200MOE_ERR_INVALID, "router_topk: path must be 0, 1 or 2, got %d", path);
  B200MOE_REQUIRE(x && w, B200MOE_ERR_INVALID, "router_topk: x and w must not be null");
  B200MOE_REQUIRE(T > 0 && H > 0, B200MOE_ERR_INVALID, "router_topk: T and H must be positive");
  B200MOE_REQUIRE(E >= 1 && E <= 512, B200MOE_ERR_INVALID, "router_topk: E must be in [1, 512], got %d", E);
  B200MOE_REQUIRE(k >= 1 && k <= 8 && k <= E, B200MOE_ERR_INVALID, "router_topk: k must be in [1, min(8, E)], got %d", k);
  B200MOE_REQUIRE(act_fn == B200MOE_ROUTER_SIGMOID || act_fn == B200MOE_ROUTER_SOFTMAX, B200MOE_ERR_INVALID,
                  "router_topk: unknown activation %d", act_fn);
  B200MOE_REQUIRE(!(norm_topk_prob && !router_pre_norm), B200MOE_ERR_INVALID,
                  "router_topk: norm_topk_prob requires router_pre_norm");
  B200MOE_REQUIRE((logits_dtype == B200MOE_F32 || logits_dtype == B200MOE_BF16) &&
                      (aff_dtype == B200MOE_F32 || aff_dtype == B200MOE_BF16),
                  B200MOE_ERR_INVALID, "router_topk: outputs must be fp32 or bf16");
  const RouterPlan p = plan_router(T, H, E, x_is_TH);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool use_tc = router_tc_eligible(x_is_TH, T, H, E) &&
                      (path == 2 || (path == 0 && T >= kTcMinTokens));
  const size_t need = kWsHeader + (use_tc ? router_tc_workspace_bytes(T, H, E)
                                          : static_cast<size_t>(p.splits) * T * E * sizeof(float));
  B200MOE_REQUIRE(workspace != nullptr && workspace_bytes >= need, B200MOE_ERR_WORKSPACE,
                  "router_topk: workspace of %zu bytes is smaller than the required %zu", workspace_bytes, need);
  B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, B200MOE_ERR_INVALID,
                  "router_topk: the workspace must be 256-byte aligned");
  int32_t* status = static_cast<int32_t*>(workspace);
  workspace = static_cast<uint8_t*>(workspace) + kWsHeader;
  const float* partial = static_cast<const float*>(workspace);
  int splits = p.splits;
  if (use_tc) {
    float* logits = nullptr;
    const int rc = router_tc_run(x, w, T, H, E, workspace, status, &logits, st);
    if (rc != B200MOE_OK) return rc;
    partial = logits;
    splits = 1;
  } else {
    B200MOE_CUDA_OK(cudaMemsetAsync(status, 0, 4, st));
    B200MOE_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(router_logits_kernel), 164 * 1024));
    LogitArgs la{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), x_is_TH, T, H, E,
                 p.mw, p.nw, p.h_per_split, p.stages, static_cast<float*>(workspace)};
    dim3 grid((T + p.tm - 1) / p.tm, p.splits);
    router_logits_kernel<<<grid, 256, p.smem, st>>>(la);
    B200MOE_LAUNCH_OK("router_logits_kernel");
  }
  RankArgs ra{partial, splits, static_cast<const __nv_bfloat16*>(w_bias), T, E, k,
              act_fn, router_pre_norm, norm_topk_prob, router_logits, logits_dtype, expert_index, expert_affinities,
              aff_dtype};
  const dim3 rgrid((T + 7) / 8);
  if (E <= 32) router_rank_kernel<1><<<rgrid, 256, 0, st>>>(ra);
  else if (E <= 64) router_rank_kernel<2><<<rgrid, 256, 0, st>>>(ra);
  else if (E <= 128) router_rank_kernel<4><<<rgrid, 256, 0, st>>>(ra);
  else if (E <= 256) router_rank_kernel<8><<<rgrid, 256, 0, st>>>(ra);
  else router_rank_kernel<16><<<rgrid, 256, 0, st>>>(ra);
  B200MOE_LAUNCH_OK("router_rank_kernel");
  return B200MOE_OK;
}
