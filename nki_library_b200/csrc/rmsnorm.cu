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

// RMSNorm (+ residual) fused with the MXFP8 activation quantisation, for callers that know where every token's
// row goes before the router has run (all-expert decode: token t sits at position e * T_pad + t of every local
// expert e).  One warp per token: pass 1 accumulates the sum of squares, pass 2 normalises 256 columns at a time,
// writes the bf16 row the router reads, and quantises the same bf16 values (32-element blocks: the four lanes
// l & ~3 .. l | 3 hold one block) to every position in the token's list -- the arithmetic and the stores of
// scatter_quantize_kernel, without the round trip of the normalised rows through HBM.
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const __nv_bfloat16* __restrict__ inp,
                                                               const __nv_bfloat16* __restrict__ residual,
                                                               const void* __restrict__ gamma, int gamma_dtype, int T,
                                                               int H, float inv_count, float eps,
                                                               __nv_bfloat16* __restrict__ out,
                                                               __nv_bfloat16* __restrict__ residual_out,
                                                               const int32_t* __restrict__ table, int K, int64_t n_pos,
                                                               int packed, uint8_t* __restrict__ codes,
                                                               uint8_t* __restrict__ sf,
                                                               int32_t* __restrict__ tile_flags) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int64_t k_atoms = (H + 127) >> 7;
  const __nv_bfloat16* row = inp + static_cast<int64_t>(t) * H;
  const __nv_bfloat16* res = residual ? residual + static_cast<int64_t>(t) * H : nullptr;
  const int32_t* my_map = table + static_cast<int64_t>(t) * K;
  if (tile_flags != nullptr)
    for (int k = lane; k < K; k += 32) {
      const int p = my_map[k];
      if (p >= 0 && p < n_pos) atomicMax(&tile_flags[p >> 7], (p & 127) + 1);
    }
  float ss = 0.f;
  for (int h = lane; h < H; h += 32) {
    float v = __bfloat162float(row[h]);
    if (res) v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(res[h])));
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rinv = 1.0f / sqrtf(ss * inv_count + eps);
  const int blk = lane >> 2, q = lane & 3;
  for (int c0 = 0; c0 < H; c0 += 256) {
    const int col = c0 + lane * 8;  // position along the contraction axis the codes are stored at
    // packed order (reference-format weights): contraction position k' = t*512 + p*4 + q holds hidden column
    // q*(H/4) + t*128 + p; lane (blk, q) reads eight consecutive p of one q and the four lanes of a block trade
    // bytes afterwards, exactly as the stand-alone quantiser does
    const int kb = (c0 >> 5) + blk;
    const int src = packed ? q * (H >> 2) + (kb >> 4) * 128 + (kb & 15) * 8 : col;
    float v[8];
    uint32_t mx = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float x = 0.f;
      if (col + j < H) {
        x = __bfloat162float(row[src + j]);
        if (res) {
          x = __bfloat162float(__float2bfloat16_rn(x + __bfloat162float(res[src + j])));
          if (residual_out) residual_out[static_cast<int64_t>(t) * H + src + j] = __float2bfloat16_rn(x);
        }
        x *= rinv;
        if (gamma) x *= load_as_float(gamma, src + j, gamma_dtype);
        const __nv_bfloat16 b = __float2bfloat16_rn(x);
        out[static_cast<int64_t>(t) * H + src + j] = b;
        x = __bfloat162float(b);  // the quantiser sees the bf16 row, as a separate quantise kernel would
      }
      v[j] = x;
      mx = max(mx, __float_as_uint(x) & 0x7fffffffu);
    }
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float f1, f2;
    mx_block_factors(mx, f1, f2);
    uint32_t w0 = pack4_e4m3(v[0] * f1 * f2, v[1] * f1 * f2, v[2] * f1 * f2, v[3] * f1 * f2);
    uint32_t w1 = pack4_e4m3(v[4] * f1 * f2, v[5] * f1 * f2, v[6] * f1 * f2, v[7] * f1 * f2);
    if (packed) {
      uint32_t o0 = 0, o1 = 0;
#pragma unroll
      for (int s2 = 0; s2 < 4; ++s2) {
        const uint32_t a0 = __shfl_sync(0xffffffffu, w0, (lane & ~3) + s2);
        const uint32_t a1 = __shfl_sync(0xffffffffu, w1, (lane & ~3) + s2);
        const uint32_t x = ((q >= 2 ? a1 : a0) >> (16 * (q & 1))) & 0xffffu;
        o0 |= (x & 0xffu) << (8 * s2);
        o1 |= (x >> 8) << (8 * s2);
      }
      w0 = o0;
      w1 = o1;
    }
    uint32_t cell = col < H ? static_cast<uint32_t>(mx_block_scale_byte(mx)) << (8 * (blk & 3)) : 0u;
    cell |= __shfl_xor_sync(0xffffffffu, cell, 4);
    cell |= __shfl_xor_sync(0xffffffffu, cell, 8);
    for (int k0 = 0; k0 < K; k0 += 8) {
      int my_pos = -1;
      if (lane < 8 && k0 + lane < K) {
        my_pos = my_map[k0 + lane];
        if (my_pos >= n_pos) my_pos = -1;
      }
      if (__ballot_sync(0xffffffffu, my_pos >= 0) == 0u) continue;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t p = __shfl_sync(0xffffffffu, my_pos, k);
        if (p < 0 || col >= H) continue;
        *reinterpret_cast<uint2*>(codes + p * H + col) = make_uint2(w0, w1);
        if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(sf + sf_atom_offset(p, col >> 5, k_atoms)) = cell;
      }
    }
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_rmsnorm_quantize_mxfp8(const void* inp_bf16, const void* residual_bf16, const void* gamma,
                                              int gamma_dtype, int T, int H, int hidden_actual, float eps,
                                              void* out_bf16, void* residual_out_bf16, const int32_t* table, int K,
                                              int64_t n_pos, int h_packed_order, uint8_t* codes, uint8_t* sf_atoms,
                                              int32_t* tile_flags, b200moe_stream_t stream) {
  B200MOE_REQUIRE(!h_packed_order || H % 512 == 0, B200MOE_ERR_INVALID,
                  "rmsnorm_quantize: the packed hidden order needs H %% 512 == 0, got %d", H);
  B200MOE_REQUIRE(inp_bf16 && out_bf16 && table && codes && sf_atoms && T > 0 && n_pos > 0 && K >= 1,
                  B200MOE_ERR_INVALID, "rmsnorm_quantize: bad arguments");
  B200MOE_REQUIRE(H > 0 && H % 128 == 0, B200MOE_ERR_INVALID,
                  "rmsnorm_quantize: H must be a positive multiple of 128, got %d", H);
  B200MOE_REQUIRE(gamma == nullptr || gamma_dtype == B200MOE_F32 || gamma_dtype == B200MOE_BF16, B200MOE_ERR_INVALID,
                  "rmsnorm_quantize: gamma must be fp32 or bf16");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tile_flags != nullptr)
    B200MOE_CUDA_OK(cudaMemsetAsync(tile_flags, 0, static_cast<size_t>(ceil_div64(n_pos, 128)) * 4, st));
  const float inv_count = 1.0f / static_cast<float>(hidden_actual > 0 ? hidden_actual : H);
  rmsnorm_quantize_kernel<<<(T + 7) / 8, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(inp_bf16), static_cast<const __nv_bfloat16*>(residual_bf16), gamma, gamma_dtype,
      T, H, inv_count, eps, static_cast<__nv_bfloat16*>(out_bf16), static_cast<__nv_bfloat16*>(residual_out_bf16), table,
      K, n_pos, h_packed_order, codes, sf_atoms, tile_flags);
  B200MOE_LAUNCH_OK("rmsnorm_quantize_kernel");
  return B200MOE_OK;
}

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
