// Shared host/device helpers for the B200 MoE hot-path library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <set>
#include <utility>

#include "../../include/b200moe.h"

namespace b200moe {

// Thread-local message returned by b200moe_last_error().
void set_error(const char* fmt, ...);

#define B200MOE_REQUIRE(cond, code, ...)      \
  do {                                        \
    if (!(cond)) {                            \
      ::b200moe::set_error(__VA_ARGS__);      \
      return (code);                          \
    }                                         \
  } while (0)

#define B200MOE_CUDA_OK(expr)                                                        \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess) {                                                         \
      ::b200moe::set_error("%s failed: %s", #expr, cudaGetErrorString(_e));          \
      return B200MOE_ERR_CUDA;                                                       \
    }                                                                                \
  } while (0)

#define B200MOE_LAUNCH_OK(name)                                                      \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess) {                                                         \
      ::b200moe::set_error("launch of %s failed: %s", name, cudaGetErrorString(_e)); \
      return B200MOE_ERR_CUDA;                                                       \
    }                                                                                \
  } while (0)

inline int sm_count() {
  static int cached[64] = {};  // per device ordinal; racing threads write the same value
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int n = cached[dev];
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cached[dev] = n;
  }
  return n;
}

// Opt a kernel in to `bytes` of dynamic shared memory, once per (device, kernel); safe to call from several
// host threads and with several devices in one process.
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({dev, kernel})) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.insert({dev, kernel});
  return e;
}

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Byte offset of the UE8M0 scale of (row, 32-block kb32) inside the
// 128-row x 4-block "scale atom" layout consumed by tcgen05 block-scaled MMA:
// atoms are 512 bytes, ordered [row / 128][kb32 / 4]; inside an atom the byte
// of (r, c) sits at (r % 32) * 16 + (r / 32) * 4 + c.
__host__ __device__ inline int64_t sf_atom_offset(int64_t row, int64_t kb32, int64_t k_atoms) {
  const int64_t atom = (row >> 7) * k_atoms + (kb32 >> 2);
  const int r = static_cast<int>(row & 127);
  return atom * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb32 & 3);
}

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
  if (dtype == B200MOE_F32) return static_cast<const float*>(p)[i];
  if (dtype == B200MOE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return static_cast<float>(static_cast<const int32_t*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dtype, float v) {
  if (dtype == B200MOE_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Activation functions of the expert MLP (ids follow ActFnType).
__device__ __forceinline__ float apply_act(float x, int kind) {
  switch (kind) {
    case B200MOE_ACT_SILU: return x / (1.0f + __expf(-x));
    case B200MOE_ACT_SWISH: return x / (1.0f + __expf(-1.702f * x));
    case B200MOE_ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    default: {  // GELU tanh approximation
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
  }
}

// One 32-element MXFP8 block: UE8M0 scale from the largest biased exponent,
// elements scaled by an exact power of two, clipped to +-448 and rounded to
// e4m3 (round-to-nearest-even).  v[] holds the 32 values; codes come back as
// eight 32-bit words (byte j of word w = element 4w + j).
__device__ __forceinline__ uint8_t mx_block_scale_byte(uint32_t max_abs_bits) {
  const int e_max = static_cast<int>((max_abs_bits >> 23) & 0xFF);
  const int s = e_max - 8;
  return static_cast<uint8_t>(s < 0 ? 0 : s);
}

__device__ __forceinline__ void mx_block_factors(uint32_t max_abs_bits, float& f1, float& f2) {
  // multiply by 2^(135 - e_max) in two exact steps so neither factor leaves fp32 range
  const int e_max = static_cast<int>((max_abs_bits >> 23) & 0xFF);
  const int n = 135 - e_max;        // in [-119, 135]
  const int a = n >> 1, b = n - a;  // each within [-60, 68]
  f1 = __uint_as_float(static_cast<uint32_t>(a + 127) << 23);
  f2 = __uint_as_float(static_cast<uint32_t>(b + 127) << 23);
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  // cvt.rn.satfinite.e4m3x2.f32 packs (hi, lo); satfinite clips to +-448
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

}  // namespace b200moe
