// Combine: out[t, :] = sum of the rows of y_pos that belong to token t, in a
// fixed (table) order, fp32 accumulation, one bf16 rounding.  Deterministic
// replacement for the reference's per-block read-modify-write of the output.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kMaxCandidates = 8192;  // table width limit: the row list of one token lives in shared memory

__global__ void __launch_bounds__(128) combine_kernel(const __nv_bfloat16* __restrict__ y_pos,
                                                      const int32_t* __restrict__ table, int T, int n_cand, int H,
                                                      __nv_bfloat16* __restrict__ out) {
  extern __shared__ int32_t s_rows[];  // n_cand entries: every candidate may be valid (all-expert decode)
  __shared__ int s_n;
  const int t = blockIdx.x;
  if (threadIdx.x < 32) {
    int base = 0;
    for (int c0 = 0; c0 < n_cand; c0 += 32) {
      const int c = c0 + threadIdx.x;
      const int32_t p = c < n_cand ? table[static_cast<int64_t>(t) * n_cand + c] : -1;
      const unsigned m = __ballot_sync(0xffffffffu, p >= 0);
      const int slot = base + __popc(m & ((1u << threadIdx.x) - 1u));
      if (p >= 0) s_rows[slot] = p;
      base += __popc(m);
    }
    if (threadIdx.x == 0) s_n = base;
  }
  __syncthreads();
  const int n = s_n;
  for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < n; ++r) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(y_pos + static_cast<int64_t>(s_rows[r]) * H + h));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(w[i] << 16);
        acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(out + static_cast<int64_t>(t) * H + h) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_combine(const void* y_pos_bf16, const int32_t* table, int T, int n_cand, int H, void* out_bf16,
                               b200moe_stream_t stream) {
  B200MOE_REQUIRE(y_pos_bf16 && table && out_bf16, B200MOE_ERR_INVALID, "combine: null pointer argument");
  B200MOE_REQUIRE(T > 0 && n_cand > 0 && H > 0 && H % 8 == 0, B200MOE_ERR_INVALID,
                  "combine: need T, n_cand > 0 and H %% 8 == 0");
  B200MOE_REQUIRE(n_cand <= kMaxCandidates, B200MOE_ERR_INVALID, "combine: at most %d candidates per row, got %d",
                  kMaxCandidates, n_cand);
  combine_kernel<<<T, 128, static_cast<size_t>(n_cand) * sizeof(int32_t), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_pos_bf16), table, T, n_cand, H, static_cast<__nv_bfloat16*>(out_bf16));
  B200MOE_LAUNCH_OK("combine_kernel");
  return B200MOE_OK;
}
