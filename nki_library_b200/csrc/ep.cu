// Expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch), one process per GPU.
//
// Every rank exposes four buffers to its peers through CUDA IPC: the quantised activation rows its
// experts will consume (codes in the block layout the grouped contraction reads, scale bytes per row),
// per-row affinity and origin, a per-source count table, and the rows coming back to it.
// A step needs no host synchronisation and no collective library call:
//
//   exchange_counts   each rank stores its per-expert pair counts into every peer's table, then all
//                     ranks wait for one another (flag words written with system-scope release)
//   dispatch_quantize MXFP8-quantises each token's hidden row once and stores codes, scale bytes
//                     (row-major), affinity and origin straight into the buffers of every rank that
//                     owns one of the token's experts, at the row the receiver's block layout assigns
//                     to that (token, k) pair (computed from the count table); the same launch writes
//                     this rank's own receive plan (block_to_expert / conditions / row validity)
//   signal_wait       "my stores are done" flags, waited for before the contractions start
//   scales_to_atoms   local: the scale bytes that arrived row-major go into the 512-byte atoms the
//                     contractions read
//   return_rows       after the down contraction each result row is stored into its origin
//                     rank's return buffer (or the contraction's epilogue does so itself); a last
//                     signal_wait precedes the local combine
//
// All waits are bounded (about two seconds) and report through a status word.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxExpertsEp = 512;
constexpr long long kEpWaitCycles = 4000000000LL;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// 32-byte store; the address must be 32-byte aligned (rows are H bytes, H % 32 == 0, on a 256-byte aligned base).
__device__ __forceinline__ void st_peer_256(void* p, const uint32_t (&c)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(c[0]), "r"(c[1]), "r"(c[2]),
               "r"(c[3]), "r"(c[4]), "r"(c[5]), "r"(c[6]), "r"(c[7])
               : "memory");
}

// Thread r < world posts `epoch` into word [slot][rank] of rank r's flag table; thread s < world then waits
// for word [slot][s] of this rank's own table.  One CTA.
__device__ void post_and_wait(const PeerPtrs& flags, int rank, int world, int slot, int epoch, int32_t* status,
                              int code) {
  __threadfence_system();
  __syncthreads();
  const int t = threadIdx.x;
  if (t < world) st_release_sys(static_cast<int32_t*>(flags.p[t]) + slot * kMaxRanks + rank, epoch);
  if (t < world) {
    const int32_t* mine = static_cast<const int32_t*>(flags.p[rank]) + slot * kMaxRanks + t;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > kEpWaitCycles) {
        atomicCAS(status, 0, code);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
}

// The step counter lives in device memory (bumped here, read by the later waits of the same step) so that a
// whole step can be recorded once into a CUDA graph and replayed.
__global__ void __launch_bounds__(512) ep_exchange_counts_kernel(const int32_t* __restrict__ counts, PeerPtrs tables,
                                                                 PeerPtrs flags, int rank, int world, int E,
                                                                 int32_t* epoch_dev, int32_t* status) {
  __shared__ int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_dev + 1;
    *epoch_dev = s_epoch;
  }
  __syncthreads();
  const int epoch = s_epoch;
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    static_cast<int32_t*>(tables.p[r])[rank * E + e] = counts[e];
  }
  post_and_wait(flags, rank, world, 0, epoch, status, 11);
}

__global__ void __launch_bounds__(32) ep_signal_wait_kernel(PeerPtrs flags, int rank, int world, int slot,
                                                            const int32_t* epoch_dev, int32_t* status) {
  post_and_wait(flags, rank, world, slot, *epoch_dev, status, 12 + slot);
}

// Receiver-side layout: local expert l of rank d owns ceil(total/B) blocks, in expert order; inside an expert
// rows are ordered by source rank, then by the source's own (token-id) order.
__device__ void build_layout(const int32_t* counts_all, int world, int E, int B, int32_t* s_total, int32_t* s_first) {
  const int E_L = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += counts_all[s * E + e];
    s_total[e] = t;
  }
  __syncthreads();
  if (threadIdx.x < world) {
    int run = 0;
    for (int l = 0; l < E_L; ++l) {
      const int e = threadIdx.x * E_L + l;
      s_first[e] = run;  // first block of expert e inside its owner's buffer
      run += (s_total[e] + B - 1) / B;
    }
  }
  __syncthreads();
}

// The receiver's plan, from the count table alone: block -> local expert, the dynamic-loop conditions, which rows
// hold a token and how many leading rows of every 128-row tile do.  Rows of an expert are packed from its first
// block, so everything follows from (first block, row count) of the owning expert; nothing is scanned.  Work is
// spread over `gthreads` threads (`gtid` = this thread's index among them).
__device__ void plan_rows(const int32_t* s_total, const int32_t* s_first, int rank, int world, int E, int B,
                          int n_blocks_cap, int32_t* block_to_expert, int32_t* conditions, int32_t* row_valid,
                          int32_t* tile_flags, int32_t* status, int64_t gtid, int64_t gthreads) {
  const int E_L = E / world;
  const int e0 = rank * E_L;
  const int used_raw = s_first[e0 + E_L - 1] + (s_total[e0 + E_L - 1] + B - 1) / B;
  if (gtid == 0 && used_raw > n_blocks_cap) atomicCAS(status, 0, 21);  // more rows arrived than the buffer holds
  const int used = min(used_raw, n_blocks_cap);
  // first local expert whose block range holds b (the last expert for blocks nobody owns)
  auto owner_of = [&](int b) {
    for (int l = 0; l < E_L; ++l) {
      const int e = e0 + l;
      if (b >= s_first[e] && b < s_first[e] + (s_total[e] + B - 1) / B) return l;
    }
    return -1;
  };
  for (int64_t b = gtid; b < n_blocks_cap + 2; b += gthreads) {
    conditions[b] = b < used ? 1 : 0;
    if (b < n_blocks_cap) {
      const int l = owner_of(static_cast<int>(b));
      block_to_expert[b] = l < 0 ? E_L - 1 : l;
    }
  }
  const int tiles_per_block = B >> 7;
  const int64_t n_tiles = static_cast<int64_t>(n_blocks_cap) * tiles_per_block;
  const int lane = static_cast<int>(gtid & 31);
  for (int64_t t = gtid >> 5; t < n_tiles; t += gthreads >> 5) {  // a warp per tile (gthreads is a multiple of 32)
    const int b = static_cast<int>(t / tiles_per_block);
    const int l = b < used ? owner_of(b) : -1;
    int live = 0;  // leading rows of this tile that hold a token
    if (l >= 0) {
      const int64_t end = static_cast<int64_t>(s_first[e0 + l]) * B + s_total[e0 + l];  // one past the expert's last row
      live = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(128), end - t * 128)));
    }
    if (lane == 0) tile_flags[t] = live;
    int32_t* rv = row_valid + t * 128;
#pragma unroll
    for (int j = lane; j < 128; j += 32) rv[j] = j < live ? static_cast<int32_t>(t * 128 + j) : -1;
  }
}

__global__ void __launch_bounds__(256) ep_plan_kernel(const int32_t* __restrict__ counts_all, int rank, int world,
                                                      int E, int B, int n_blocks_cap, int32_t* block_to_expert,
                                                      int32_t* conditions, int32_t* row_valid, int32_t* tile_flags,
                                                      int32_t* status) {
  __shared__ int32_t s_total[kMaxExpertsEp];
  __shared__ int32_t s_first[kMaxExpertsEp];
  build_layout(counts_all, world, E, B, s_total, s_first);
  plan_rows(s_total, s_first, rank, world, E, B, n_blocks_cap, block_to_expert, conditions, row_valid, tile_flags,
            status, static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x,
            static_cast<int64_t>(gridDim.x) * blockDim.x);
}

// Outputs of the receiver's plan when the dispatch launch computes it as well (block_to_expert == nullptr: not).
struct PlanOut {
  int n_blocks_cap;
  int32_t* block_to_expert;
  int32_t* conditions;
  int32_t* row_valid;
  int32_t* tile_flags;
  int32_t* status;
};

__device__ __forceinline__ void unpack8_bf16_ep(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(256) ep_dispatch_quantize_kernel(
    const __nv_bfloat16* __restrict__ hidden, const int32_t* __restrict__ pair_of_token,
    const int32_t* __restrict__ pair_expert, const float* __restrict__ aff, const int32_t* __restrict__ counts_all,
    int T, int K, int H, int E, int B, int rank, int world, int packed, PeerPtrs xq, PeerPtrs sf, PeerPtrs row_aff,
    PeerPtrs row_src, int64_t cap_rows, PlanOut plan) {
  __shared__ int32_t s_total[kMaxExpertsEp];
  __shared__ int32_t s_first[kMaxExpertsEp];
  __shared__ int32_t s_base[kMaxExpertsEp];    // row of my first pair of expert e in the owner's buffer
  __shared__ int32_t s_prefix[kMaxExpertsEp];  // my pairs before expert e
  build_layout(counts_all, world, E, B, s_total, s_first);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += counts_all[s * E + e];
    s_base[e] = s_first[e] * B + before;
  }
  if (threadIdx.x < 32) {  // exclusive scan of this rank's own counts, 32 experts per round
    const int lane = threadIdx.x;
    int run = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int c = e < E ? counts_all[rank * E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (e < E) s_prefix[e] = run + incl - c;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  const int E_L = E / world;
  if (plan.block_to_expert != nullptr)
    plan_rows(s_total, s_first, rank, world, E, B, plan.n_blocks_cap, plan.block_to_expert, plan.conditions,
              plan.row_valid, plan.tile_flags, plan.status, static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x,
              static_cast<int64_t>(gridDim.x) * blockDim.x);
  // Token-major: a thread quantises one 32-element block of a token's row once and stores it to every GPU that
  // owns one of the token's experts (`pair_of_token[t, k]` = index of that (token, k) pair in the expert-sorted
  // list, or -1), so `hidden` is read and quantised once per token, not once per pair.  A token's experts are
  // spread over the ranks, so at any moment the ranks of the group store into different GPUs (walking the sorted
  // pairs instead, all ranks would write to rank 0 first, then to rank 1, ..., each time through one ingress).
  const int blocks_per_row = H >> 5;
  const int64_t n_pairs = static_cast<int64_t>(T) * K;
  const int64_t total = static_cast<int64_t>(T) * blocks_per_row;
  const int64_t total_padded = (total + 31) & ~static_cast<int64_t>(31);  // whole warps stay in the loop (shuffles)
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_padded;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const bool live = i < total;
    const int tok = live ? static_cast<int>(i / blocks_per_row) : 0;
    const int kb = live ? static_cast<int>(i - static_cast<int64_t>(tok) * blocks_per_row) : 0;
    uint32_t c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t scale = 0;
    if (live) {
      const __nv_bfloat16* src = hidden + static_cast<int64_t>(tok) * H;
      float v[32];
      if (!packed) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src + kb * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack8_bf16_ep(__ldg(s4 + j), v + 8 * j);
      } else {
        const int t = kb >> 4, g = kb & 15;
        float tmp[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          unpack8_bf16_ep(__ldg(reinterpret_cast<const uint4*>(src + q * (H >> 2) + t * 128 + g * 8)), tmp);
#pragma unroll
          for (int pp = 0; pp < 8; ++pp) v[pp * 4 + q] = tmp[pp];
        }
      }
      uint32_t mx = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) mx = max(mx, __float_as_uint(v[j]) & 0x7fffffffu);
      scale = mx_block_scale_byte(mx);
      float f1, f2;
      mx_block_factors(mx, f1, f2);
#pragma unroll
      for (int w = 0; w < 8; ++w)
        c[w] = pack4_e4m3(v[4 * w] * f1 * f2, v[4 * w + 1] * f1 * f2, v[4 * w + 2] * f1 * f2, v[4 * w + 3] * f1 * f2);
    }
    // four neighbouring lanes hold the four scale bytes of one 32-bit atom cell (H % 128 == 0)
    const int lane = threadIdx.x & 31;
    const uint32_t s1 = __shfl_sync(0xffffffffu, scale, (lane & ~3) + 1);
    const uint32_t s2 = __shfl_sync(0xffffffffu, scale, (lane & ~3) + 2);
    const uint32_t s3 = __shfl_sync(0xffffffffu, scale, (lane & ~3) + 3);
    const uint32_t cell = scale | (s1 << 8) | (s2 << 16) | (s3 << 24);
    // Scale bytes travel row-major ([row][H / 32], re-laid into 512-byte atoms by the receiver): when a warp holds 32
    // blocks of one row its 32 scale bytes leave as one 32-byte store from lane 0 -- as 4-byte cells scattered over
    // the atoms they were a third of the dispatch time (eight tiny NVLink writes per warp and destination).
    const bool warp_row = (blocks_per_row & 31) == 0;
    uint32_t cells[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cells[j] = __shfl_sync(0xffffffffu, cell, 4 * j);
    if (!live) continue;
    for (int k = 0; k < K; ++k) {
      const int64_t p = pair_of_token[static_cast<int64_t>(tok) * K + k];
      if (p < 0 || p >= n_pairs) continue;
      const int e = pair_expert[p];
      if (e < 0 || e >= E) continue;
      const int d = e / E_L;
      const int64_t row = static_cast<int64_t>(s_base[e]) + (p - s_prefix[e]);
      if (row >= cap_rows) continue;  // receive buffer too small: the receiver's plan reports it
      // one 32-byte store per thread: a warp covers 1 KB of the row with whole sectors (two 16-byte stores would
      // each touch half of every sector, which NVLink carries as twice the packets)
      st_peer_256(static_cast<uint8_t*>(xq.p[d]) + row * H + kb * 32, c);
      uint8_t* sf_row = static_cast<uint8_t*>(sf.p[d]) + row * blocks_per_row;
      if (warp_row) {
        if (lane == 0) st_peer_256(sf_row + kb, cells);
      } else if ((kb & 3) == 0) {
        *reinterpret_cast<uint32_t*>(sf_row + kb) = cell;
      }
      if (kb == 0) {
        static_cast<float*>(row_aff.p[d])[row] = aff[static_cast<int64_t>(tok) * E + e];
        static_cast<int32_t*>(row_src.p[d])[row] = (rank << 24) | static_cast<int32_t>(p);
      }
    }
  }
}

// Receiver side: scale bytes arrive row-major; the contraction's TMA reads 512-byte atoms (128 rows x one 128-wide
// K slab).  A warp builds one atom: lane l owns rows l, l+32, l+64, l+96 and writes their four cells as 16 bytes.
__global__ void __launch_bounds__(256) ep_scales_to_atoms_kernel(const uint8_t* __restrict__ sf_rows,
                                                                 const int32_t* __restrict__ tile_flags,
                                                                 int64_t n_tiles, int k_atoms, uint8_t* sf_atoms) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total = n_tiles * k_atoms;
  const int blocks_per_row = k_atoms * 4;
  for (int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
    const int64_t t = w / k_atoms;
    const int a = static_cast<int>(w - t * k_atoms);
    if (tile_flags[t] <= 0) continue;  // no row of this tile holds a token
    uint32_t c[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      c[j] = *reinterpret_cast<const uint32_t*>(sf_rows + (t * 128 + lane + 32 * j) * blocks_per_row + a * 4);
    *reinterpret_cast<uint4*>(sf_atoms + w * 512 + lane * 16) = make_uint4(c[0], c[1], c[2], c[3]);
  }
}

__global__ void __launch_bounds__(256) ep_return_rows_kernel(const __nv_bfloat16* __restrict__ y_pos,
                                                             const int32_t* __restrict__ row_valid,
                                                             const int32_t* __restrict__ row_src, PeerPtrs back,
                                                             int64_t cap_rows, int H, int64_t back_rows) {
  const int vec_per_row = H >> 3;  // 16-byte chunks
  const int64_t total = cap_rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    if (row_valid[r] < 0) continue;
    const int v = static_cast<int>(i - r * vec_per_row);
    const int32_t src = row_src[r];
    const int d = (src >> 24) & 0x7f;
    const int64_t p = src & 0xffffff;
    if (d >= kMaxRanks || p >= back_rows || back.p[d] == nullptr) continue;  // ranks past `world` hold no buffer
    const uint4 val = __ldg(reinterpret_cast<const uint4*>(y_pos + r * H) + v);
    reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(back.p[d]) + p * H)[v] = val;
  }
}

int fill_peers(PeerPtrs& out, void* const* host_array, int world) {
  B200MOE_REQUIRE(host_array != nullptr, B200MOE_ERR_INVALID, "peer pointer array must not be null");
  for (int i = 0; i < kMaxRanks; ++i) out.p[i] = i < world ? host_array[i] : nullptr;
  for (int i = 0; i < world; ++i)
    B200MOE_REQUIRE(out.p[i] != nullptr, B200MOE_ERR_INVALID, "peer pointer %d is null", i);
  return B200MOE_OK;
}

int check_world(int rank, int world, int E) {
  B200MOE_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, B200MOE_ERR_INVALID,
                  "expert parallelism supports 1..%d ranks (rank %d of %d)", kMaxRanks, rank, world);
  B200MOE_REQUIRE(E > 0 && E <= kMaxExpertsEp && E % world == 0, B200MOE_ERR_INVALID,
                  "number of experts (%d) must be a multiple of the rank count (%d) and at most %d", E, world,
                  kMaxExpertsEp);
  return B200MOE_OK;
}

inline int grid_cap(int64_t n, int threads) {
  const int64_t g = ceil_div64(n, threads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

// ---- CUDA IPC plumbing -------------------------------------------------------------------------
extern "C" int b200moe_ipc_export(const void* dev_ptr, void* handle_out_64, int64_t* offset_out) {
  B200MOE_REQUIRE(dev_ptr && handle_out_64 && offset_out, B200MOE_ERR_INVALID, "ipc_export: null argument");
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (range_fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    B200MOE_CUDA_OK(cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &q));
    B200MOE_REQUIRE(ptr != nullptr && q == cudaDriverEntryPointSuccess, B200MOE_ERR_CUDA,
                    "cuMemGetAddressRange is not available from this driver");
    range_fn = reinterpret_cast<RangeFn>(ptr);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr));
  B200MOE_REQUIRE(r == CUDA_SUCCESS, B200MOE_ERR_CUDA, "cuMemGetAddressRange failed with code %d", static_cast<int>(r));
  cudaIpcMemHandle_t h;
  B200MOE_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle_out_64, &h, 64);
  *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
  return B200MOE_OK;
}

extern "C" int b200moe_ipc_open(const void* handle_64, int64_t offset, void** dev_ptr_out) {
  B200MOE_REQUIRE(handle_64 && dev_ptr_out, B200MOE_ERR_INVALID, "ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, 64);
  void* base = nullptr;
  B200MOE_CUDA_OK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *dev_ptr_out = static_cast<char*>(base) + offset;
  return B200MOE_OK;
}

extern "C" int b200moe_ipc_close(void* dev_ptr, int64_t offset) {
  B200MOE_REQUIRE(dev_ptr != nullptr, B200MOE_ERR_INVALID, "ipc_close: null argument");
  B200MOE_CUDA_OK(cudaIpcCloseMemHandle(static_cast<char*>(dev_ptr) - offset));
  return B200MOE_OK;
}

// ---- step kernels -------------------------------------------------------------------------------
extern "C" int b200moe_ep_exchange_counts(const int32_t* counts, void* const* count_tables, void* const* flag_tables,
                                          int rank, int world, int E, int32_t* epoch_dev, int32_t* status,
                                          b200moe_stream_t stream) {
  B200MOE_REQUIRE(counts && status && epoch_dev, B200MOE_ERR_INVALID, "ep_exchange_counts: null argument");
  int rc = check_world(rank, world, E);
  if (rc != B200MOE_OK) return rc;
  PeerPtrs tables, flags;
  if ((rc = fill_peers(tables, count_tables, world)) != B200MOE_OK) return rc;
  if ((rc = fill_peers(flags, flag_tables, world)) != B200MOE_OK) return rc;
  ep_exchange_counts_kernel<<<1, 512, 0, static_cast<cudaStream_t>(stream)>>>(counts, tables, flags, rank, world, E,
                                                                              epoch_dev, status);
  B200MOE_LAUNCH_OK("ep_exchange_counts_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_signal_wait(void* const* flag_tables, int rank, int world, int slot,
                                      const int32_t* epoch_dev, int32_t* status, b200moe_stream_t stream) {
  B200MOE_REQUIRE(status != nullptr && epoch_dev != nullptr && slot >= 1 && slot <= 3, B200MOE_ERR_INVALID,
                  "ep_signal_wait: bad argument");
  B200MOE_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, B200MOE_ERR_INVALID,
                  "ep_signal_wait: bad rank %d of %d", rank, world);
  PeerPtrs flags;
  const int rc = fill_peers(flags, flag_tables, world);
  if (rc != B200MOE_OK) return rc;
  ep_signal_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, rank, world, slot, epoch_dev, status);
  B200MOE_LAUNCH_OK("ep_signal_wait_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_plan(const int32_t* counts_all, int rank, int world, int E, int B, int n_blocks_cap,
                               int32_t* block_to_expert, int32_t* conditions, int32_t* row_valid, int32_t* tile_flags,
                               int32_t* status, b200moe_stream_t stream) {
  B200MOE_REQUIRE(counts_all && block_to_expert && conditions && row_valid && tile_flags && status, B200MOE_ERR_INVALID,
                  "ep_plan: null argument");
  B200MOE_REQUIRE(B > 0 && B % 128 == 0 && n_blocks_cap > 0, B200MOE_ERR_INVALID, "ep_plan: bad block geometry");
  const int rc = check_world(rank, world, E);
  if (rc != B200MOE_OK) return rc;
  const int64_t plan_threads = (static_cast<int64_t>(n_blocks_cap) * (B / 128)) * 32;
  ep_plan_kernel<<<grid_cap(plan_threads, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, rank, world, E, B, n_blocks_cap,
                                                                   block_to_expert, conditions, row_valid, tile_flags,
                                                                   status);
  B200MOE_LAUNCH_OK("ep_plan_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_dispatch_quantize(const void* hidden_bf16, const int32_t* pair_of_token,
                                            const int32_t* pair_expert, const float* affinities,
                                            const int32_t* counts_all, int T, int K, int H, int E, int B, int rank,
                                            int world, int h_packed_order, void* const* xq_peers,
                                            void* const* sf_peers, void* const* aff_peers, void* const* src_peers,
                                            int64_t cap_rows, int n_blocks_cap, int32_t* block_to_expert,
                                            int32_t* conditions, int32_t* row_valid, int32_t* tile_flags,
                                            int32_t* status, b200moe_stream_t stream) {
  B200MOE_REQUIRE(hidden_bf16 && pair_of_token && pair_expert && affinities && counts_all, B200MOE_ERR_INVALID,
                  "ep_dispatch_quantize: null argument");
  PlanOut plan{n_blocks_cap, block_to_expert, conditions, row_valid, tile_flags, status};
  if (block_to_expert != nullptr)
    B200MOE_REQUIRE(conditions && row_valid && tile_flags && status && n_blocks_cap > 0 && B > 0 && B % 128 == 0 &&
                        static_cast<int64_t>(n_blocks_cap) * B <= cap_rows,
                    B200MOE_ERR_INVALID, "ep_dispatch_quantize: incomplete or oversized plan outputs");
  B200MOE_REQUIRE(H > 0 && H % 128 == 0, B200MOE_ERR_INVALID, "ep_dispatch_quantize: H must be a multiple of 128");
  B200MOE_REQUIRE(static_cast<int64_t>(T) * K < (1 << 24), B200MOE_ERR_INVALID,
                  "ep_dispatch_quantize: at most 2^24 (token, k) pairs per rank");
  int rc = check_world(rank, world, E);
  if (rc != B200MOE_OK) return rc;
  PeerPtrs xq, sf, ra, rs;
  if ((rc = fill_peers(xq, xq_peers, world)) != B200MOE_OK) return rc;
  if ((rc = fill_peers(sf, sf_peers, world)) != B200MOE_OK) return rc;
  if ((rc = fill_peers(ra, aff_peers, world)) != B200MOE_OK) return rc;
  if ((rc = fill_peers(rs, src_peers, world)) != B200MOE_OK) return rc;
  for (int i = 0; i < world; ++i)
    B200MOE_REQUIRE(reinterpret_cast<uintptr_t>(xq.p[i]) % 32 == 0, B200MOE_ERR_INVALID,
                    "ep_dispatch_quantize: activation buffers must be 32-byte aligned");
  for (int i = 0; i < world; ++i)
    B200MOE_REQUIRE(reinterpret_cast<uintptr_t>(sf.p[i]) % 32 == 0, B200MOE_ERR_INVALID,
                    "ep_dispatch_quantize: scale buffers must be 32-byte aligned");
  const int64_t work = static_cast<int64_t>(T) * (H / 32);
  ep_dispatch_quantize_kernel<<<grid_cap(work, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(hidden_bf16), pair_of_token, pair_expert, affinities, counts_all, T, K, H, E, B,
      rank, world, h_packed_order, xq, sf, ra, rs, cap_rows, plan);
  B200MOE_LAUNCH_OK("ep_dispatch_quantize_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_scales_to_atoms(const uint8_t* sf_rows, const int32_t* tile_flags, int64_t n_tiles, int H,
                                          uint8_t* sf_atoms, b200moe_stream_t stream) {
  B200MOE_REQUIRE(sf_rows && tile_flags && sf_atoms, B200MOE_ERR_INVALID, "ep_scales_to_atoms: null argument");
  B200MOE_REQUIRE(n_tiles > 0 && H > 0 && H % 128 == 0, B200MOE_ERR_INVALID,
                  "ep_scales_to_atoms: H must be a multiple of 128 and n_tiles positive");
  B200MOE_REQUIRE(reinterpret_cast<uintptr_t>(sf_rows) % 4 == 0 && reinterpret_cast<uintptr_t>(sf_atoms) % 16 == 0,
                  B200MOE_ERR_INVALID, "ep_scales_to_atoms: misaligned buffer");
  const int k_atoms = H / 128;
  ep_scales_to_atoms_kernel<<<grid_cap(n_tiles * k_atoms * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sf_rows, tile_flags, n_tiles, k_atoms, sf_atoms);
  B200MOE_LAUNCH_OK("ep_scales_to_atoms_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_return_rows(const void* y_pos_bf16, const int32_t* row_valid, const int32_t* row_src,
                                      void* const* back_peers, int world, int64_t cap_rows, int H, int64_t back_rows,
                                      b200moe_stream_t stream) {
  B200MOE_REQUIRE(y_pos_bf16 && row_valid && row_src, B200MOE_ERR_INVALID, "ep_return_rows: null argument");
  B200MOE_REQUIRE(H % 8 == 0 && world >= 1 && world <= kMaxRanks, B200MOE_ERR_INVALID, "ep_return_rows: bad argument");
  PeerPtrs back;
  const int rc = fill_peers(back, back_peers, world);
  if (rc != B200MOE_OK) return rc;
  ep_return_rows_kernel<<<grid_cap(cap_rows * (H / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_pos_bf16), row_valid, row_src, back, cap_rows, H, back_rows);
  B200MOE_LAUNCH_OK("ep_return_rows_kernel");
  return B200MOE_OK;
}
