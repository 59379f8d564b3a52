// MXFP8 activation quantisation fused with the token gather, and the one-time
// relayout of expert weights into the tensor-core feed format.
//
// gather_quantize: one thread owns one 32-element block (64 bytes of bf16 in,
// 32 code bytes + 1 scale byte out).  In packed-order mode the 32 elements of
// block (t, g) are four 8-element runs at h = q*(H/4) + t*128 + 8g (q = 0..3),
// interleaved as p*4 + q; otherwise they are 32 consecutive columns.
#include <type_traits>

#include "common.cuh"

namespace b200moe {
namespace {

__device__ __forceinline__ void quantize_block32(const float (&v)[32], uint32_t (&codes)[8], uint8_t& scale) {
  uint32_t mx = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) mx = max(mx, __float_as_uint(v[i]) & 0x7fffffffu);
  scale = mx_block_scale_byte(mx);
  float f1, f2;
  mx_block_factors(mx, f1, f2);
#pragma unroll
  for (int w = 0; w < 8; ++w)
    codes[w] = pack4_e4m3(v[4 * w] * f1 * f2, v[4 * w + 1] * f1 * f2, v[4 * w + 2] * f1 * f2, v[4 * w + 3] * f1 * f2);
}

__device__ __forceinline__ void unpack8_bf16(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(256) gather_quantize_kernel(const __nv_bfloat16* __restrict__ hidden, int hidden_rows,
                                                              int H, const int32_t* __restrict__ tpi, int64_t n_pos,
                                                              int packed, uint8_t* __restrict__ codes,
                                                              uint8_t* __restrict__ sf,
                                                              int32_t* __restrict__ tile_flags) {
  const int blocks_per_row = H >> 5;
  const int64_t k_atoms = (H + 127) >> 7;
  const int64_t total = n_pos * blocks_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t p = i / blocks_per_row;
    const int kb = static_cast<int>(i - p * blocks_per_row);
    const int tok = tpi ? tpi[p] : static_cast<int>(p);
    uint32_t c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint8_t s = 0;
    if (tok >= 0 && tok < hidden_rows) {
      const __nv_bfloat16* row = hidden + static_cast<int64_t>(tok) * H;
      float v[32];
      if (!packed) {
        const uint4* src = reinterpret_cast<const uint4*>(row + kb * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack8_bf16(__ldg(src + j), v + 8 * j);
      } else {
        const int t = kb >> 4, g = kb & 15;
        float tmp[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(row + q * (H >> 2) + t * 128 + g * 8)), tmp);
#pragma unroll
          for (int pp = 0; pp < 8; ++pp) v[pp * 4 + q] = tmp[pp];
        }
      }
      quantize_block32(v, c, s);
      if (tile_flags != nullptr && kb == 0) atomicMax(&tile_flags[p >> 7], static_cast<int>(p & 127) + 1);
    }
    uint4* dst = reinterpret_cast<uint4*>(codes + p * H + kb * 32);
    dst[0] = make_uint4(c[0], c[1], c[2], c[3]);
    dst[1] = make_uint4(c[4], c[5], c[6], c[7]);
    sf[sf_atom_offset(p, kb, k_atoms)] = s;
  }
}

// Token-major twin of gather_quantize_kernel for callers that hold the inverse map (position of every
// (token, k) pair): one warp reads a token's row once, quantises it once and stores codes and scale cells to its
// K positions, so the hidden tensor crosses HBM once instead of K times.  Per pass of 256 columns lane l holds
// 8 bf16 (16 bytes); the four lanes l & ~3 .. l | 3 hold one 32-element block, so the block maximum is two
// shuffles away, every lane stores its 8 code bytes (256 contiguous bytes per warp and position) and lanes 0 and
// 16 store one 4-byte scale cell each.  Positions no pair maps to are not written.
__global__ void __launch_bounds__(256) scatter_quantize_kernel(const __nv_bfloat16* __restrict__ hidden, int T, int H,
                                                               const int32_t* __restrict__ inverse_map, int K,
                                                               int64_t n_pos, int packed, uint8_t* __restrict__ codes,
                                                               uint8_t* __restrict__ sf,
                                                               int32_t* __restrict__ tile_flags) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int64_t k_atoms = (H + 127) >> 7;
  const int32_t* my_map = inverse_map + static_cast<int64_t>(t) * K;
  if (tile_flags != nullptr && blockIdx.y == 0)
    for (int k = lane; k < K; k += 32) {
      const int p = my_map[k];
      if (p >= 0 && p < n_pos) atomicMax(&tile_flags[p >> 7], (p & 127) + 1);
    }
  const __nv_bfloat16* row = hidden + static_cast<int64_t>(t) * H;
  const int passes = (H + 255) >> 8;
  const int q = lane & 3, blk = lane >> 2;
  constexpr int kU = 4;  // passes per warp: blockIdx.y walks the row in chunks of 1024 columns
  {
    const int it0 = blockIdx.y * kU;
    uint4 raw[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int it = it0 + u;
      const int col = it * 256 + lane * 8;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (it < passes && col < H) {
        if (!packed) {
          raw[u] = __ldg(reinterpret_cast<const uint4*>(row + col));
        } else {
          const int kb = it * 8 + blk;
          raw[u] = __ldg(reinterpret_cast<const uint4*>(row + q * (H >> 2) + (kb >> 4) * 128 + (kb & 15) * 8));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int it = it0 + u;
      if (it >= passes) break;  // uniform across the warp
      const int col = it * 256 + lane * 8;
      float v[8];
      unpack8_bf16(raw[u], v);
      uint32_t mx = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = max(mx, __float_as_uint(v[j]) & 0x7fffffffu);
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      float f1, f2;
      mx_block_factors(mx, f1, f2);
      uint32_t w0 = pack4_e4m3(v[0] * f1 * f2, v[1] * f1 * f2, v[2] * f1 * f2, v[3] * f1 * f2);
      uint32_t w1 = pack4_e4m3(v[4] * f1 * f2, v[5] * f1 * f2, v[6] * f1 * f2, v[7] * f1 * f2);
      if (packed) {
        // lane q holds elements p*4 + q (p = 0..7) of the block; it stores bytes 8q .. 8q+7, i.e. byte pair
        // (2q, 2q+1) of every lane of its group of four
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
      // the four scale bytes of a 128-column cell sit in lanes 0, 4, 8, 12 (+16) of the warp
      uint32_t cell = col < H ? static_cast<uint32_t>(mx_block_scale_byte(mx)) << (8 * (blk & 3)) : 0u;
      cell |= __shfl_xor_sync(0xffffffffu, cell, 4);
      cell |= __shfl_xor_sync(0xffffffffu, cell, 8);
      // the token's positions, eight at a time (a top-k list is one round; a [T, E] position table has E / 8)
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
}

// Dense (non-MX) variants: the token's bf16 row is copied to its positions as it is, or multiplied by the affinity
// of the position's expert first (the reference's PRE_SCALE mode scales the hidden rows before the first
// projection, core/moe/moe_cte/moe_cte_torch.py:151-155).  One warp per token, 16-byte accesses.
__global__ void __launch_bounds__(256) scatter_rows_bf16_kernel(const __nv_bfloat16* __restrict__ hidden, int T, int H,
                                                                const int32_t* __restrict__ table, int K, int64_t n_pos,
                                                                const int32_t* __restrict__ block_to_expert, int B, int E,
                                                                const void* __restrict__ aff, int aff_dtype,
                                                                __nv_bfloat16* __restrict__ out,
                                                                int32_t* __restrict__ tile_flags) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int32_t* my_map = table + static_cast<int64_t>(t) * K;
  const uint4* src = reinterpret_cast<const uint4*>(hidden + static_cast<int64_t>(t) * H);
  const int vecs = H >> 3;
  for (int k = 0; k < K; ++k) {
    const int64_t p = my_map[k];
    if (p < 0 || p >= n_pos) continue;  // uniform across the warp
    if (tile_flags != nullptr && lane == 0) atomicMax(&tile_flags[p >> 7], static_cast<int>(p & 127) + 1);
    float a = 1.0f;
    if (aff != nullptr) {
      const int e = block_to_expert[p / B];
      a = (e >= 0 && e < E) ? load_as_float(aff, static_cast<int64_t>(t) * E + e, aff_dtype) : 0.0f;
      a = __bfloat162float(__float2bfloat16_rn(a));  // the reference casts the affinity to the hidden dtype first
    }
    uint4* dst = reinterpret_cast<uint4*>(out + p * H);
    for (int v = lane; v < vecs; v += 32) {
      uint4 raw = __ldg(src + v);
      if (aff != nullptr) {
        float f[8];
        unpack8_bf16(raw, f);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[2 * i] * a, f[2 * i + 1] * a);
          o[i] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        raw = make_uint4(o[0], o[1], o[2], o[3]);
      }
      dst[v] = raw;
    }
  }
}

// ---- weight relayout ---------------------------------------------------------
// Destination row of gate/up source row (s = 0 gate / 1 up, i): 32 gate rows then
// the matching 32 up rows.
__host__ __device__ inline int64_t gate_up_dev_row(int s, int i) { return (static_cast<int64_t>(i >> 5) << 6) + (s << 5) + (i & 31); }

// Logical -> packed intermediate position maps of the reference storage
// (tile of 512, or the whole axis when I < 512): packed j = tile*rows + p*4 + q
// holds logical column tile*rows + q*(rows/4) + p.
__device__ __forceinline__ int nki_logical_i(int j, int I) {
  const int rows = I < 512 ? I : 512;
  const int tile = j / rows, r = j - tile * rows;
  return tile * rows + (r & 3) * (rows >> 2) + (r >> 2);
}

// The relayout kernels move one 32-element block per thread: 32 bytes of 8-bit codes (x4 words of 32 bits)
// or, for e2m1 weights (FP4), 16 bytes of nibbles (x4 words of 16 bits).
template <bool FP4>
struct BlockWords {
  using Word = typename std::conditional<FP4, uint16_t, uint32_t>::type;
  static constexpr int kBytes = FP4 ? 16 : 32;
  Word c[8];
  __device__ __forceinline__ void load_contiguous(const uint8_t* src) {
    if constexpr (FP4) {
      const uint4 a = *reinterpret_cast<const uint4*>(src);
      const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { c[2 * i] = static_cast<uint16_t>(v[i] & 0xffffu); c[2 * i + 1] = static_cast<uint16_t>(v[i] >> 16); }
    } else {
      const uint4 a = reinterpret_cast<const uint4*>(src)[0], b = reinterpret_cast<const uint4*>(src)[1];
      c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
    }
  }
  __device__ __forceinline__ void store(uint8_t* dst) const {
    if constexpr (FP4) {
      *reinterpret_cast<uint4*>(dst) =
          make_uint4(c[0] | (static_cast<uint32_t>(c[1]) << 16), c[2] | (static_cast<uint32_t>(c[3]) << 16),
                     c[4] | (static_cast<uint32_t>(c[5]) << 16), c[6] | (static_cast<uint32_t>(c[7]) << 16));
    } else {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(c[0], c[1], c[2], c[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(c[4], c[5], c[6], c[7]);
    }
  }
};

template <bool FP4>
__global__ void prepare_gate_up_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ scale, int layout, int E,
                                       int H, int I, uint8_t* __restrict__ w_dev, uint8_t* __restrict__ sf_dev) {
  // one thread per (e, s, j, 32-block of H): copies the block's codes and 1 scale byte
  using BW = BlockWords<FP4>;
  const int kblocks = H >> 5;
  const int64_t k_atoms = (H + 127) >> 7;
  const int64_t sf_per_expert = ((2LL * I + 127) >> 7) * k_atoms * 512;
  const int64_t total = static_cast<int64_t>(E) * 2 * I * kblocks;
  const int nt = H >> 9;
  const int64_t row_bytes = static_cast<int64_t>(kblocks) * BW::kBytes;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int kb = static_cast<int>(idx % kblocks);
    int64_t r = idx / kblocks;
    const int j = static_cast<int>(r % I);
    r /= I;
    const int s = static_cast<int>(r & 1);
    const int e = static_cast<int>(r >> 1);
    BW blk;
    uint8_t sc;
    if (layout == B200MOE_LAYOUT_ROWS) {
      blk.load_contiguous(w + ((static_cast<int64_t>(e) * 2 + s) * I + j) * row_bytes + kb * BW::kBytes);
      sc = scale[((static_cast<int64_t>(e) * 2 + s) * I + j) * kblocks + kb];
    } else {
      // source word (e, p, s, t, i) holds q = 0..3; block kb = 16 t + g covers p in [8g, 8g+8)
      const int i = nki_logical_i(j, I);
      const int t = kb >> 4, g = kb & 15;
      const typename BW::Word* wx = reinterpret_cast<const typename BW::Word*>(w);
#pragma unroll
      for (int pp = 0; pp < 8; ++pp)
        blk.c[pp] = wx[(((static_cast<int64_t>(e) * 128 + (g * 8 + pp)) * 2 + s) * nt + t) * I + i];
      sc = scale[(((static_cast<int64_t>(e) * 16 + g) * 2 + s) * nt + t) * I + i];
    }
    const int64_t row = gate_up_dev_row(s, j);
    blk.store(w_dev + (static_cast<int64_t>(e) * 2 * I + row) * row_bytes + kb * BW::kBytes);
    sf_dev[e * sf_per_expert + sf_atom_offset(row, kb, k_atoms)] = sc;
  }
}

template <bool FP4>
__global__ void prepare_down_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ scale, int layout, int E,
                                    int H, int I, uint8_t* __restrict__ w_dev, uint8_t* __restrict__ sf_dev) {
  // one thread per (e, h, 32-block of I)
  using BW = BlockWords<FP4>;
  const int kblocks = I >> 5;
  const int64_t k_atoms = (I + 127) >> 7;
  const int64_t sf_per_expert = ((static_cast<int64_t>(H) + 127) >> 7) * k_atoms * 512;
  const int64_t total = static_cast<int64_t>(E) * H * kblocks;
  const int pI = I > 512 ? 128 : I / 4;
  const int n_tiles = I > 512 ? I / 512 : 1;
  const int64_t row_bytes = static_cast<int64_t>(kblocks) * BW::kBytes;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int kb = static_cast<int>(idx % kblocks);
    int64_t r = idx / kblocks;
    const int h = static_cast<int>(r % H);
    const int e = static_cast<int>(r / H);
    BW blk;
    uint8_t sc;
    if (layout == B200MOE_LAYOUT_ROWS) {
      blk.load_contiguous(w + (static_cast<int64_t>(e) * H + h) * row_bytes + kb * BW::kBytes);
      sc = scale[(static_cast<int64_t>(e) * H + h) * kblocks + kb];
    } else {
      // packed position j = tile*(pI*4) + p*4 + q; block kb covers p in [8g, 8g+8) of one tile
      const int blocks_per_tile = pI >> 3;
      const int tile = kb / blocks_per_tile, g = kb - tile * blocks_per_tile;
      const typename BW::Word* wx = reinterpret_cast<const typename BW::Word*>(w);
#pragma unroll
      for (int pp = 0; pp < 8; ++pp)
        blk.c[pp] = wx[((static_cast<int64_t>(e) * pI + (g * 8 + pp)) * n_tiles + tile) * H + h];
      sc = scale[((static_cast<int64_t>(e) * (pI >> 3) + g) * n_tiles + tile) * H + h];
    }
    blk.store(w_dev + (static_cast<int64_t>(e) * H + h) * row_bytes + kb * BW::kBytes);
    sf_dev[e * sf_per_expert + sf_atom_offset(h, kb, k_atoms)] = sc;
  }
}

__global__ void prepare_bias_kernel(const void* bias, int dtype, int layout, int E, int I, float* out) {
  const int64_t total = static_cast<int64_t>(E) * 2 * I;
  const int pI = I > 512 ? 128 : I / 4;
  const int n_tiles = I > 512 ? I / 512 : 1;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(idx % I);
    const int s = static_cast<int>((idx / I) & 1);
    const int e = static_cast<int>(idx / (2LL * I));
    float v;
    if (layout == B200MOE_LAYOUT_ROWS) {
      v = load_as_float(bias, idx, dtype);
    } else {
      // [E, pI, 2, n_tiles, 4] is already in packed order: j = tile*(pI*4) + p*4 + q
      const int tile = j / (pI * 4), r = j - tile * pI * 4;
      v = load_as_float(bias, (((static_cast<int64_t>(e) * pI + (r >> 2)) * 2 + s) * n_tiles + tile) * 4 + (r & 3), dtype);
    }
    out[static_cast<int64_t>(e) * 2 * I + gate_up_dev_row(s, j)] = v;
  }
}

inline int grid_for(int64_t n, int threads) {
  const int64_t g = ceil_div64(n, threads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_sf_bytes(int64_t rows, int64_t K) {
  return static_cast<size_t>(ceil_div64(rows, 128) * ceil_div64(K, 128) * 512);
}

extern "C" int b200moe_gather_quantize_mxfp8(const void* hidden_bf16, int hidden_rows, int H,
                                             const int32_t* token_position_to_id, int64_t n_pos, int h_packed_order,
                                             uint8_t* codes, uint8_t* sf_atoms, int32_t* tile_flags,
                                             b200moe_stream_t stream) {
  B200MOE_REQUIRE(hidden_bf16 && codes && sf_atoms, B200MOE_ERR_INVALID, "gather_quantize: null pointer argument");
  B200MOE_REQUIRE(H > 0 && H % 32 == 0, B200MOE_ERR_INVALID, "gather_quantize: H must be a multiple of 32, got %d", H);
  B200MOE_REQUIRE(!h_packed_order || H % 512 == 0, B200MOE_ERR_INVALID,
                  "gather_quantize: packed hidden order needs H %% 512 == 0, got %d", H);
  B200MOE_REQUIRE(n_pos > 0 && hidden_rows > 0, B200MOE_ERR_INVALID, "gather_quantize: empty input");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((n_pos % 128) != 0 || (H % 128) != 0)  // partially filled atoms must read as zero
    B200MOE_CUDA_OK(cudaMemsetAsync(sf_atoms, 0, b200moe_sf_bytes(n_pos, H), st));
  if (tile_flags != nullptr)
    B200MOE_CUDA_OK(cudaMemsetAsync(tile_flags, 0, static_cast<size_t>(ceil_div64(n_pos, 128)) * 4, st));
  gather_quantize_kernel<<<grid_for(n_pos * (H / 32), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(hidden_bf16), hidden_rows, H, token_position_to_id, n_pos, h_packed_order,
      codes, sf_atoms, tile_flags);
  B200MOE_LAUNCH_OK("gather_quantize_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_scatter_quantize_mxfp8(const void* hidden_bf16, int T, int H, const int32_t* inverse_map, int K,
                                              int64_t n_pos, int h_packed_order, uint8_t* codes, uint8_t* sf_atoms,
                                              int32_t* tile_flags, b200moe_stream_t stream) {
  B200MOE_REQUIRE(hidden_bf16 && inverse_map && codes && sf_atoms, B200MOE_ERR_INVALID,
                  "scatter_quantize: null pointer argument");
  B200MOE_REQUIRE(T > 0 && H > 0 && H % 32 == 0 && n_pos > 0, B200MOE_ERR_INVALID,
                  "scatter_quantize: T, n_pos must be positive and H a positive multiple of 32 (H = %d)", H);
  B200MOE_REQUIRE(K >= 1 && K <= 8192, B200MOE_ERR_INVALID, "scatter_quantize: K must be in [1, 8192], got %d", K);
  B200MOE_REQUIRE(!h_packed_order || H % 512 == 0, B200MOE_ERR_INVALID,
                  "scatter_quantize: the packed hidden order needs H %% 512 == 0, got %d", H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((H % 128) != 0)  // the unused quarter cells of the last 128-column atom must read as zero
    B200MOE_CUDA_OK(cudaMemsetAsync(sf_atoms, 0, b200moe_sf_bytes(n_pos, H), st));
  if (tile_flags != nullptr)
    B200MOE_CUDA_OK(cudaMemsetAsync(tile_flags, 0, static_cast<size_t>(ceil_div64(n_pos, 128)) * 4, st));
  const dim3 grid(static_cast<unsigned>((T + 7) / 8), static_cast<unsigned>((H + 1023) / 1024));
  scatter_quantize_kernel<<<grid, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(hidden_bf16), T, H, inverse_map, K, n_pos, h_packed_order, codes, sf_atoms,
      tile_flags);
  B200MOE_LAUNCH_OK("scatter_quantize_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_scatter_rows_bf16(const void* hidden_bf16, int T, int H, const int32_t* table, int K,
                                         int64_t n_pos, const int32_t* block_to_expert, int B, int E,
                                         const void* pre_scale_affinities, int aff_dtype, void* out_bf16,
                                         int32_t* tile_flags, b200moe_stream_t stream) {
  B200MOE_REQUIRE(hidden_bf16 && table && out_bf16, B200MOE_ERR_INVALID, "scatter_rows: null pointer argument");
  B200MOE_REQUIRE(T > 0 && H > 0 && H % 8 == 0 && n_pos > 0 && K >= 1, B200MOE_ERR_INVALID,
                  "scatter_rows: T, K, n_pos must be positive and H a positive multiple of 8 (H = %d)", H);
  B200MOE_REQUIRE(pre_scale_affinities == nullptr || (block_to_expert != nullptr && B > 0 && E > 0 &&
                                                      (aff_dtype == B200MOE_F32 || aff_dtype == B200MOE_BF16)),
                  B200MOE_ERR_INVALID, "scatter_rows: scaling needs block_to_expert, B, E and fp32 / bf16 affinities");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tile_flags != nullptr)
    B200MOE_CUDA_OK(cudaMemsetAsync(tile_flags, 0, static_cast<size_t>(ceil_div64(n_pos, 128)) * 4, st));
  scatter_rows_bf16_kernel<<<(T + 7) / 8, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(hidden_bf16), T, H, table, K, n_pos, block_to_expert, B, E,
      pre_scale_affinities, aff_dtype, static_cast<__nv_bfloat16*>(out_bf16), tile_flags);
  B200MOE_LAUNCH_OK("scatter_rows_bf16_kernel");
  return B200MOE_OK;
}

extern "C" int64_t b200moe_weight_bytes(int64_t rows, int64_t K, int w_format) {
  return w_format == B200MOE_W_E2M1 ? rows * K / 2 : rows * K;
}

extern "C" int b200moe_prepare_gate_up(const void* w, const uint8_t* scale, int layout, int w_format, int E, int H, int I,
                                       uint8_t* w_dev, uint8_t* sf_dev, b200moe_stream_t stream) {
  B200MOE_REQUIRE(w_format == B200MOE_W_E4M3 || w_format == B200MOE_W_E5M2 || w_format == B200MOE_W_E2M1,
                  B200MOE_ERR_INVALID, "prepare_gate_up: unknown weight format %d", w_format);
  B200MOE_REQUIRE(w_format != B200MOE_W_E2M1 || H % 128 == 0, B200MOE_ERR_INVALID,
                  "prepare_gate_up: e2m1 weights need H %% 128 == 0, got %d", H);
  B200MOE_REQUIRE(w && scale && w_dev && sf_dev, B200MOE_ERR_INVALID, "prepare_gate_up: null pointer argument");
  B200MOE_REQUIRE(layout == B200MOE_LAYOUT_ROWS || layout == B200MOE_LAYOUT_NKI_X4, B200MOE_ERR_INVALID,
                  "prepare_gate_up: unknown layout %d", layout);
  B200MOE_REQUIRE(H % 32 == 0 && I % 32 == 0, B200MOE_ERR_INVALID, "prepare_gate_up: H and I must be multiples of 32");
  if (layout == B200MOE_LAYOUT_NKI_X4)
    B200MOE_REQUIRE(H % 512 == 0 && (I % 512 == 0 || I < 512), B200MOE_ERR_INVALID,
                    "prepare_gate_up: reference storage needs H %% 512 == 0 and I %% 512 == 0 (or I < 512)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200MOE_CUDA_OK(cudaMemsetAsync(sf_dev, 0, static_cast<size_t>(E) * b200moe_sf_bytes(2LL * I, H), st));
  const int grid = grid_for(static_cast<int64_t>(E) * 2 * I * (H / 32), 256);
  if (w_format == B200MOE_W_E2M1)
    prepare_gate_up_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(w), scale, layout, E, H, I, w_dev, sf_dev);
  else
    prepare_gate_up_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(w), scale, layout, E, H, I, w_dev, sf_dev);
  B200MOE_LAUNCH_OK("prepare_gate_up_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_prepare_down(const void* w, const uint8_t* scale, int layout, int w_format, int E, int H, int I,
                                    uint8_t* w_dev, uint8_t* sf_dev, b200moe_stream_t stream) {
  B200MOE_REQUIRE(w_format == B200MOE_W_E4M3 || w_format == B200MOE_W_E5M2 || w_format == B200MOE_W_E2M1,
                  B200MOE_ERR_INVALID, "prepare_down: unknown weight format %d", w_format);
  B200MOE_REQUIRE(w_format != B200MOE_W_E2M1 || I % 128 == 0, B200MOE_ERR_INVALID,
                  "prepare_down: e2m1 weights need I %% 128 == 0, got %d", I);
  B200MOE_REQUIRE(w && scale && w_dev && sf_dev, B200MOE_ERR_INVALID, "prepare_down: null pointer argument");
  B200MOE_REQUIRE(layout == B200MOE_LAYOUT_ROWS || layout == B200MOE_LAYOUT_NKI_X4, B200MOE_ERR_INVALID,
                  "prepare_down: unknown layout %d", layout);
  B200MOE_REQUIRE(H % 32 == 0 && I % 32 == 0, B200MOE_ERR_INVALID, "prepare_down: H and I must be multiples of 32");
  if (layout == B200MOE_LAYOUT_NKI_X4)
    B200MOE_REQUIRE(I % 512 == 0 || I < 512, B200MOE_ERR_INVALID,
                    "prepare_down: reference storage needs I %% 512 == 0 (or I < 512)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200MOE_CUDA_OK(cudaMemsetAsync(sf_dev, 0, static_cast<size_t>(E) * b200moe_sf_bytes(H, I), st));
  const int grid = grid_for(static_cast<int64_t>(E) * H * (I / 32), 256);
  if (w_format == B200MOE_W_E2M1)
    prepare_down_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(w), scale, layout, E, H, I, w_dev, sf_dev);
  else
    prepare_down_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(w), scale, layout, E, H, I, w_dev, sf_dev);
  B200MOE_LAUNCH_OK("prepare_down_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_prepare_gate_up_bias(const void* bias, int dtype, int layout, int E, int I, float* bias_dev,
                                            b200moe_stream_t stream) {
  B200MOE_REQUIRE(bias && bias_dev, B200MOE_ERR_INVALID, "prepare_gate_up_bias: null pointer argument");
  B200MOE_REQUIRE(dtype == B200MOE_F32 || dtype == B200MOE_BF16, B200MOE_ERR_INVALID,
                  "prepare_gate_up_bias: bias must be fp32 or bf16");
  prepare_bias_kernel<<<grid_for(static_cast<int64_t>(E) * 2 * I, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      bias, dtype, layout, E, I, bias_dev);
  B200MOE_LAUNCH_OK("prepare_bias_kernel");
  return B200MOE_OK;
}
