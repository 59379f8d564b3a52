// Router: logits = x @ w (+ bias) in fp32, warp-shuffle top-K, softmax / sigmoid
// affinities, optional L1 normalisation, dense scatter -- one launch.
//
// A CTA owns 32 tokens and all E experts.  The H loop stages a [32 x 16] slab of
// x and a [16 x E] slab of w in shared memory as fp32 and every thread keeps a
// 4-token x (E/32)-expert register tile.  The finished [32 x E] logits tile is
// parked in shared memory and each warp then ranks 4 tokens: every lane holds
// E/32 logits, a (value, lowest index) arg-max is reduced with shuffles K times.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kTok = 32;     // tokens per CTA
constexpr int kHC = 16;      // hidden slab
constexpr int kMaxEPerLane = 16;  // E <= 512

struct RouterArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  const __nv_bfloat16* bias;
  int x_is_TH, T, H, E, k, act, pre_norm, l1;
  void* logits_out;
  int logits_dtype;
  uint32_t* index_out;
  void* aff_out;
  int aff_dtype;
};

__global__ void __launch_bounds__(256) router_topk_kernel(RouterArgs a) {
  extern __shared__ float smem[];
  const int E = a.E;
  const int Epad = (E + 31) & ~31;
  float* s_w = smem;                       // [kHC][Epad]
  float* s_x = s_w + kHC * Epad;           // [kTok][kHC + 1]
  float* s_logit = s_x + kTok * (kHC + 1); // [kTok][Epad]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.x * kTok;
  const int n_per_lane = Epad / 32;

  float acc[4][kMaxEPerLane];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < kMaxEPerLane; ++j) acc[i][j] = 0.f;

  for (int h0 = 0; h0 < a.H; h0 += kHC) {
    // stage w slab (coalesced along E)
    for (int i = tid; i < kHC * Epad; i += 256) {
      const int hh = i / Epad, e = i - hh * Epad;
      s_w[i] = (e < E && h0 + hh < a.H) ? __bfloat162float(a.w[static_cast<int64_t>(h0 + hh) * E + e]) : 0.f;
    }
    // stage x slab
    for (int i = tid; i < kTok * kHC; i += 256) {
      int tl, hh;
      if (a.x_is_TH) { tl = i / kHC; hh = i - tl * kHC; } else { hh = i / kTok; tl = i - hh * kTok; }
      const int t = t0 + tl, h = h0 + hh;
      float v = 0.f;
      if (t < a.T && h < a.H)
        v = __bfloat162float(a.x_is_TH ? a.x[static_cast<int64_t>(t) * a.H + h] : a.x[static_cast<int64_t>(h) * a.T + t]);
      s_x[tl * (kHC + 1) + hh] = v;
    }
    __syncthreads();
#pragma unroll 4
    for (int hh = 0; hh < kHC; ++hh) {
      float xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = s_x[(warp * 4 + i) * (kHC + 1) + hh];
#pragma unroll
      for (int j = 0; j < kMaxEPerLane; ++j) {
        if (j < n_per_lane) {
          const float wv = s_w[hh * Epad + lane + 32 * j];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(xv[i], wv, acc[i][j]);
        }
      }
    }
    __syncthreads();
  }

  // bias, park logits, optional store
#pragma unroll
  for (int j = 0; j < kMaxEPerLane; ++j) {
    if (j < n_per_lane) {
      const int e = lane + 32 * j;
      const float b = (a.bias != nullptr && e < E) ? __bfloat162float(a.bias[e]) : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tl = warp * 4 + i;
        const float v = acc[i][j] + b;
        s_logit[tl * Epad + e] = v;
        if (a.logits_out != nullptr && e < E && t0 + tl < a.T)
          store_from_float(a.logits_out, static_cast<int64_t>(t0 + tl) * E + e, a.logits_dtype, v);
      }
    }
  }
  __syncwarp();

  // ranking: this warp's 4 tokens
  for (int i = 0; i < 4; ++i) {
    const int tl = warp * 4 + i, t = t0 + tl;
    if (t >= a.T) break;
    float v[kMaxEPerLane];
    float row_max = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxEPerLane; ++j) {
      const int e = lane + 32 * j;
      v[j] = (j < n_per_lane && e < E) ? s_logit[tl * Epad + e] : -INFINITY;
      row_max = fmaxf(row_max, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));

    // activation over the full row (pre-norm pipelines)
    float full[kMaxEPerLane];
    if (a.pre_norm) {
      if (a.act == B200MOE_ROUTER_SOFTMAX) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxEPerLane; ++j) {
          full[j] = (v[j] == -INFINITY) ? 0.f : expf(v[j] - row_max);
          s += full[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float inv = 1.0f / s;
#pragma unroll
        for (int j = 0; j < kMaxEPerLane; ++j) full[j] *= inv;
      } else {
#pragma unroll
        for (int j = 0; j < kMaxEPerLane; ++j) full[j] = 1.0f / (1.0f + expf(-v[j]));
      }
    }

    // K rounds of arg-max with lowest-index tie break
    float top_v[8];
    int top_e[8];
    float top_a[8];  // activated value of the selected expert (pre-norm)
    uint32_t taken = 0;
    for (int r = 0; r < a.k; ++r) {
      float bv = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kMaxEPerLane; ++j) {
        const int e = lane + 32 * j;
        if (j < n_per_lane && e < E && !((taken >> j) & 1u)) {
          if (v[j] > bv || (v[j] == bv && e < be)) { bv = v[j]; be = e; }
        }
      }
      if (be == 0x7fffffff) bv = -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      float sel_a = 0.f;
      if (be != 0x7fffffff && (be & 31) == lane) {
        taken |= 1u << (be >> 5);
        if (a.pre_norm) {
#pragma unroll
          for (int j = 0; j < kMaxEPerLane; ++j)
            if (j == (be >> 5)) sel_a = full[j];
        }
      }
      sel_a = __shfl_sync(0xffffffffu, sel_a, be & 31);
      top_v[r] = bv;
      top_e[r] = be;
      top_a[r] = sel_a;
    }

    if (a.index_out != nullptr && lane < a.k) {
      int e_out = 0;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r == lane) e_out = top_e[r];
      a.index_out[static_cast<int64_t>(t) * a.k + lane] = static_cast<uint32_t>(e_out);
    }
    if (a.aff_out == nullptr) continue;

    if (a.pre_norm && !a.l1) {
      // dense activated row
#pragma unroll
      for (int j = 0; j < kMaxEPerLane; ++j) {
        const int e = lane + 32 * j;
        if (j < n_per_lane && e < E) store_from_float(a.aff_out, static_cast<int64_t>(t) * E + e, a.aff_dtype, full[j]);
      }
      continue;
    }
    // sparse rows: values of the K winners
    float val[8];
    if (a.pre_norm) {
      float s = 0.f;
      for (int r = 0; r < a.k; ++r) s += top_a[r];
      for (int r = 0; r < a.k; ++r) val[r] = top_a[r] / s;
    } else if (a.act == B200MOE_ROUTER_SOFTMAX) {
      float s = 0.f;
      for (int r = 0; r < a.k; ++r) { val[r] = expf(top_v[r] - top_v[0]); s += val[r]; }
      for (int r = 0; r < a.k; ++r) val[r] = val[r] / s;
    } else {
      for (int r = 0; r < a.k; ++r) val[r] = 1.0f / (1.0f + expf(-top_v[r]));
    }
#pragma unroll
    for (int j = 0; j < kMaxEPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < n_per_lane && e < E) {
        float out = 0.f;
        for (int r = 0; r < a.k; ++r)
          if (top_e[r] == e) out = val[r];
        store_from_float(a.aff_out, static_cast<int64_t>(t) * E + e, a.aff_dtype, out);
      }
    }
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_router_topk(const void* x, int x_is_TH, const void* w, const void* w_bias, int T, int H, int E,
                                   int k, int act_fn, int router_pre_norm, int norm_topk_prob, void* router_logits,
                                   int logits_dtype, uint32_t* expert_index, void* expert_affinities, int aff_dtype,
                                   b200moe_stream_t stream) {
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
  RouterArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
               static_cast<const __nv_bfloat16*>(w_bias), x_is_TH, T, H, E, k, act_fn, router_pre_norm, norm_topk_prob,
               router_logits, logits_dtype, expert_index, expert_affinities, aff_dtype};
  const int Epad = (E + 31) & ~31;
  const size_t smem = sizeof(float) * (static_cast<size_t>(kHC) * Epad + kTok * (kHC + 1) + static_cast<size_t>(kTok) * Epad);
  static bool attr_set = false;
  if (!attr_set) {
    B200MOE_CUDA_OK(cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
    attr_set = true;
  }
  router_topk_kernel<<<(T + kTok - 1) / kTok, 256, smem, static_cast<cudaStream_t>(stream)>>>(a);
  B200MOE_LAUNCH_OK("router_topk_kernel");
  return B200MOE_OK;
}
