// RMSNorm (optionally with a fused residual add) feeding the decode MoE block: one warp per token row,
// fp32 statistics, bf16 in and out.
#include "common.cuh"

namespace b200moe {
namespace {

__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ inp,
                                                      const __nv_bfloat16* __restrict__ residual,
                                                      const void* __restrict__ gamma, int gamma_dtype, int T, int H,
                                                      float inv_count, float eps, __nv_bfloat16* __restrict__ out,
                                                      __nv_bfloat16* __restrict__ residual_out) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const __nv_bfloat16* row = inp + static_cast<int64_t>(t) * H;
  const __nv_bfloat16* res = residual ? residual + static_cast<int64_t>(t) * H : nullptr;
  float ss = 0.f;
  for (int h = lane; h < H; h += 32) {
    float v = __bfloat162float(row[h]);
    if (res) {
      v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(res[h])));
      if (residual_out) residual_out[static_cast<int64_t>(t) * H + h] = __float2bfloat16_rn(v);
    }
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rinv = 1.0f / sqrtf(ss * inv_count + eps);
  for (int h = lane; h < H; h += 32) {
    float v = __bfloat162float(row[h]);
    if (res) v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(res[h])));
    v *= rinv;
    if (gamma) v *= load_as_float(gamma, h, gamma_dtype);
    out[static_cast<int64_t>(t) * H + h] = __float2bfloat16_rn(v);
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_rmsnorm(const void* inp_bf16, const void* residual_bf16, const void* gamma, int gamma_dtype,
                               int T, int H, int hidden_actual, float eps, void* out_bf16, void* residual_out_bf16,
                               b200moe_stream_t stream) {
  B200MOE_REQUIRE(inp_bf16 && out_bf16 && T > 0 && H > 0, B200MOE_ERR_INVALID, "rmsnorm: bad arguments");
  B200MOE_REQUIRE(gamma == nullptr || gamma_dtype == B200MOE_F32 || gamma_dtype == B200MOE_BF16, B200MOE_ERR_INVALID,
                  "rmsnorm: gamma must be fp32 or bf16");
  const float inv_count = 1.0f / static_cast<float>(hidden_actual > 0 ? hidden_actual : H);
  rmsnorm_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(inp_bf16), static_cast<const __nv_bfloat16*>(residual_bf16), gamma, gamma_dtype,
      T, H, inv_count, eps, static_cast<__nv_bfloat16*>(out_bf16), static_cast<__nv_bfloat16*>(residual_out_bf16));
  B200MOE_LAUNCH_OK("rmsnorm_kernel");
  return B200MOE_OK;
}
