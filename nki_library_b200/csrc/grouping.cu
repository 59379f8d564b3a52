// Token-to-block grouping on sm_100a: stable per-expert compaction of routed
// token ids, block offsets, padded flatten, and the bookkeeping arrays the
// blockwise expert kernels consume.  Integer-only, bit-exact by construction:
// every token's slot is (blocks before its expert) * B + (routed tokens with a
// smaller id), computed from per-chunk bitmaps with popcounts -- no atomics
// decide an ordering.
//
// Three launches (one, with block barriers in between, when all tokens fit a single chunk): (1) per 256-token chunk, build a [columns x 256-bit] bitmap in
// shared memory and emit per-chunk column counts; (2) one CTA turns the counts
// into per-chunk prefixes, per-expert block ranges, block_to_expert and
// conditions; (3) per chunk, rebuild the bitmap and scatter token ids.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kChunk = 256;           // tokens per CTA
constexpr int kWords = kChunk / 32;   // bitmap words per column
constexpr int kThreads = 256;

struct GroupArgs {
  const void* routing;
  int routing_mode;   // B200MOE_ROUTING_INDEX / _MASK
  int routing_dtype;  // mask element type
  int T, C_full, n_cols, K;
  const int32_t* col_start_dev;
};

// Fill `bits[c * kWords + w]` for this CTA's chunk.
__device__ __forceinline__ void build_bitmap(const GroupArgs& a, int chunk, uint32_t* bits) {
  const int t0 = chunk * kChunk;
  const int col_start = a.col_start_dev ? a.col_start_dev[0] : 0;
  if (a.routing_mode == B200MOE_ROUTING_INDEX) {
    for (int i = threadIdx.x; i < a.n_cols * kWords; i += blockDim.x) bits[i] = 0u;
    __syncthreads();
    const int32_t* idx = static_cast<const int32_t*>(a.routing);
    for (int i = threadIdx.x; i < kChunk * a.K; i += blockDim.x) {
      const int tl = i / a.K, t = t0 + tl;
      if (t < a.T) {
        const int e = idx[static_cast<int64_t>(t) * a.K + (i - tl * a.K)] - col_start;
        if (e >= 0 && e < a.n_cols) atomicOr(&bits[e * kWords + (tl >> 5)], 1u << (tl & 31));
      }
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c0 = 0; c0 < a.n_cols; c0 += 32) {
      const int c = c0 + lane;
      uint32_t word = 0;
      if (c < a.n_cols && warp < kWords) {  // one warp per bitmap word; extra warps of a larger CTA idle here
        for (int j = 0; j < 32; ++j) {
          const int t = t0 + warp * 32 + j;
          if (t < a.T) {
            const float v = load_as_float(a.routing, static_cast<int64_t>(t) * a.C_full + col_start + c, a.routing_dtype);
            word |= (v != 0.0f ? 1u : 0u) << j;
          }
        }
        bits[c * kWords + warp] = word;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void count_phase(const GroupArgs& a, uint32_t* bits, int32_t* chunk_counts,
                                            int32_t* fill_ptr, int64_t fill_n, int32_t fill_val) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < fill_n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    fill_ptr[i] = fill_val;
  build_bitmap(a, blockIdx.x, bits);
  for (int c = threadIdx.x; c < a.n_cols; c += blockDim.x) {
    int n = 0;
#pragma unroll
    for (int w = 0; w < kWords; ++w) n += __popc(bits[c * kWords + w]);
    chunk_counts[static_cast<int64_t>(blockIdx.x) * a.n_cols + c] = n;
  }
}

__global__ void __launch_bounds__(kThreads) group_count_kernel(GroupArgs a, int32_t* chunk_counts, int32_t* fill_ptr,
                                                               int64_t fill_n, int32_t fill_val) {
  extern __shared__ uint32_t bits[];
  count_phase(a, bits, chunk_counts, fill_ptr, fill_n, fill_val);
}

// mode 0: find_nonzero_indices (column c writes at c*T); mode 1: block grouping.
__device__ __forceinline__ void scan_phase(int32_t* chunk_counts, int n_chunks, int n_cols, int mode, int T, int B,
                                           int N, int mx_conditions, int32_t* counts, int64_t* col_base,
                                           int32_t* block_to_expert, int32_t* conditions, int32_t* status) {
  __shared__ int s_bpe[1024];
  __shared__ int s_first[1024];
  __shared__ int s_npad;
  const int c = threadIdx.x;
  int total = 0;
  if (c < n_cols) {
    for (int ch = 0; ch < n_chunks; ++ch) {
      const int v = chunk_counts[static_cast<int64_t>(ch) * n_cols + c];
      chunk_counts[static_cast<int64_t>(ch) * n_cols + c] = total;  // exclusive prefix over chunks
      total += v;
    }
    if (counts) counts[c] = total;
  }
  if (mode == 0) {
    if (c < n_cols) col_base[c] = static_cast<int64_t>(c) * T;
    return;  // (returns to the caller: the fused single-chunk kernel goes on to its scatter phase)
  }
  s_bpe[c] = (c < n_cols) ? (total + B - 1) / B : 0;
  __syncthreads();
  if (c == 0) {
    int run = 0;
    for (int e = 0; e < n_cols; ++e) {
      s_first[e] = run;
      run += s_bpe[e];
    }
    s_npad = N - run;
    if (run > N) status[0] = 1;  // N too small for this routing
  }
  __syncthreads();
  const int n_pad = s_npad < 0 ? 0 : s_npad;
  if (c < n_cols) {
    col_base[c] = static_cast<int64_t>(s_first[c]) * B;
    int nb = s_bpe[c] + (c == n_cols - 1 ? n_pad : 0);
    for (int b = 0; b < nb; ++b)
      if (s_first[c] + b < N) block_to_expert[s_first[c] + b] = c;
  }
  const int n_cond = mx_conditions ? N + 2 : N + 1;
  const int n_zero = mx_conditions ? n_pad + 2 : n_pad + 1;
  for (int i = c; i < n_cond; i += blockDim.x) conditions[i] = (i < n_cond - n_zero) ? 1 : 0;
}

__global__ void __launch_bounds__(1024) group_scan_kernel(int32_t* chunk_counts, int n_chunks, int n_cols, int mode,
                                                          int T, int B, int N, int mx_conditions, int32_t* counts,
                                                          int64_t* col_base, int32_t* block_to_expert,
                                                          int32_t* conditions, int32_t* status) {
  scan_phase(chunk_counts, n_chunks, n_cols, mode, T, B, N, mx_conditions, counts, col_base, block_to_expert,
             conditions, status);
}

__device__ __forceinline__ void scatter_phase(const GroupArgs& a, const uint32_t* bits, const int32_t* chunk_prefix,
                                              const int64_t* col_base, int64_t out_len, int32_t* out_ids,
                                              int32_t* inverse_map) {
  const int t0 = blockIdx.x * kChunk;
  for (int i = threadIdx.x; i < a.n_cols * kWords; i += blockDim.x) {
    const int c = i / kWords, w = i - c * kWords;
    uint32_t word = bits[i];
    if (!word) continue;
    int before = chunk_prefix[static_cast<int64_t>(blockIdx.x) * a.n_cols + c];
    for (int w2 = 0; w2 < w; ++w2) before += __popc(bits[c * kWords + w2]);
    const int64_t base = col_base[c] + before;
    int r = 0;
    while (word) {
      const int j = __ffs(word) - 1;
      word &= word - 1;
      const int64_t pos = base + r++;
      if (pos < out_len) out_ids[pos] = t0 + w * 32 + j;
    }
  }
  if (inverse_map != nullptr && a.routing_mode == B200MOE_ROUTING_INDEX) {
    const int32_t* idx = static_cast<const int32_t*>(a.routing);
    const int col_start = a.col_start_dev ? a.col_start_dev[0] : 0;
    for (int i = threadIdx.x; i < kChunk * a.K; i += blockDim.x) {
      const int tl = i / a.K, t = t0 + tl;
      if (t >= a.T) continue;
      const int e = idx[static_cast<int64_t>(t) * a.K + (i - tl * a.K)] - col_start;
      int32_t pos = -1;
      if (e >= 0 && e < a.n_cols) {
        const int w = tl >> 5;
        int before = chunk_prefix[static_cast<int64_t>(blockIdx.x) * a.n_cols + e];
        for (int w2 = 0; w2 < w; ++w2) before += __popc(bits[e * kWords + w2]);
        before += __popc(bits[e * kWords + w] & ((1u << (tl & 31)) - 1u));
        const int64_t p = col_base[e] + before;
        pos = p < out_len ? static_cast<int32_t>(p) : -1;
      }
      inverse_map[static_cast<int64_t>(t) * a.K + (i - tl * a.K)] = pos;
    }
  }
}

__global__ void __launch_bounds__(kThreads) group_scatter_kernel(GroupArgs a, const int32_t* chunk_prefix,
                                                                 const int64_t* col_base, int64_t out_len,
                                                                 int32_t* out_ids, int32_t* inverse_map) {
  extern __shared__ uint32_t bits[];
  build_bitmap(a, blockIdx.x, bits);
  scatter_phase(a, bits, chunk_prefix, col_base, out_len, out_ids, inverse_map);
}

// All three phases in one CTA for inputs of a single 256-token chunk (decode batches): the bitmap is built once
// and the phases are separated by block barriers instead of kernel boundaries.
__global__ void __launch_bounds__(1024) group_single_chunk_kernel(GroupArgs a, int mode, int B, int N, int mx_conditions,
                                                                  int32_t* chunk_counts, int64_t* col_base,
                                                                  int64_t out_len, int32_t fill_val, int32_t* out_ids,
                                                                  int32_t* counts, int32_t* block_to_expert,
                                                                  int32_t* conditions, int32_t* inverse_map,
                                                                  int32_t* status) {
  extern __shared__ uint32_t bits[];
  count_phase(a, bits, chunk_counts, out_ids, out_len, fill_val);
  __syncthreads();
  scan_phase(chunk_counts, 1, a.n_cols, mode, a.T, B, N, mx_conditions, counts, col_base, block_to_expert, conditions,
             status);
  __syncthreads();
  scatter_phase(a, bits, chunk_counts, col_base, out_len, out_ids, inverse_map);
}

__global__ void cumsum_kernel(const void* x, int dtype, int64_t cols, void* out) {
  // one CTA per row; thread-contiguous segments, fp32 running sum
  __shared__ float s_sum[256];
  const int64_t row = blockIdx.x;
  const int64_t seg = (cols + blockDim.x - 1) / blockDim.x;
  const int64_t lo = static_cast<int64_t>(threadIdx.x) * seg;
  const int64_t hi = lo + seg < cols ? lo + seg : cols;
  float acc = 0.f;
  for (int64_t i = lo; i < hi; ++i) acc += load_as_float(x, row * cols + i, dtype);
  s_sum[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x); ++i) {
      const float v = s_sum[i];
      s_sum[i] = run;
      run += v;
    }
  }
  __syncthreads();
  acc = s_sum[threadIdx.x];
  for (int64_t i = lo; i < hi; ++i) {
    acc += load_as_float(x, row * cols + i, dtype);
    if (dtype == B200MOE_I32) static_cast<int32_t*>(out)[row * cols + i] = static_cast<int32_t>(acc);
    else store_from_float(out, row * cols + i, dtype, acc);
  }
}

__global__ void indexed_flatten_kernel(const int32_t* input, int E, int T, int f_len, int64_t output_len,
                                       const int32_t* row_offsets, const int32_t* start_dev, int padding_val,
                                       int32_t* out) {
  const int parts = T / f_len;
  const int64_t n_blk = output_len / f_len;
  const int start = start_dev ? start_dev[0] : 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < output_len;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / f_len;
    const int j = static_cast<int>(i - b * f_len);
    int32_t v = padding_val;
    if (b < n_blk) {
      for (int e = E - 1; e >= 0; --e) {  // the last row written wins
        const int64_t off = row_offsets[start + e];
        if (b >= off && b < off + parts) {
          v = input[static_cast<int64_t>(e) * T + (b - off) * f_len + j];
          break;
        }
      }
    }
    out[i] = v;
  }
}

__global__ void position_table_kernel(const int32_t* tpi, const int32_t* block_to_expert, const int32_t* conditions,
                                      int64_t n_pos, int B, int T, int E, int32_t* table) {
  // blocks run up to the first zero condition
  __shared__ int s_n_active;
  const int n_blocks = static_cast<int>(n_pos / B);
  if (threadIdx.x == 0) s_n_active = n_blocks;
  __syncthreads();
  if (conditions != nullptr)
    for (int b = threadIdx.x; b < n_blocks; b += blockDim.x)
      if (conditions[b] == 0) atomicMin(&s_n_active, b);
  __syncthreads();
  const int n_active = s_n_active;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < n_pos;
       p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(p / B);
    if (b >= n_active) continue;
    const int t = tpi[p];
    if (t < 0 || t >= T) continue;
    const int e = block_to_expert[b];
    if (e >= 0 && e < E) table[static_cast<int64_t>(t) * E + e] = static_cast<int32_t>(p);
  }
}

size_t group_ws_bytes(int T, int n_cols) {
  const int64_t n_chunks = ceil_div64(T, kChunk);
  return static_cast<size_t>(n_chunks * n_cols * 4 + 1024 * 8 + 256);
}

int run_grouping(const GroupArgs& a, int mode, int B, int N, int mx_conditions, int64_t out_len, int32_t fill_val,
                 int32_t* out_ids, int32_t* counts, int32_t* block_to_expert, int32_t* conditions, int32_t* inverse_map,
                 int32_t* status, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  B200MOE_REQUIRE(a.T > 0 && a.n_cols > 0 && a.n_cols <= 1024, B200MOE_ERR_INVALID,
                  "grouping: need T > 0 and 0 < columns <= 1024 (got T=%d, columns=%d)", a.T, a.n_cols);
  B200MOE_REQUIRE(workspace_bytes >= group_ws_bytes(a.T, a.n_cols), B200MOE_ERR_WORKSPACE,
                  "grouping: workspace of %zu bytes is smaller than the required %zu", workspace_bytes,
                  group_ws_bytes(a.T, a.n_cols));
  const int n_chunks = static_cast<int>(ceil_div64(a.T, kChunk));
  int32_t* chunk_counts = static_cast<int32_t*>(workspace);
  int64_t* col_base = reinterpret_cast<int64_t*>(static_cast<char*>(workspace) +
                                                 ((static_cast<size_t>(n_chunks) * a.n_cols * 4 + 255) / 256) * 256);
  const size_t smem = static_cast<size_t>(a.n_cols) * kWords * 4;
  if (status) B200MOE_CUDA_OK(cudaMemsetAsync(status, 0, 4, st));
  if (n_chunks == 1) {
    group_single_chunk_kernel<<<1, 1024, smem, st>>>(a, mode, B, N, mx_conditions, chunk_counts, col_base, out_len,
                                                     fill_val, out_ids, counts, block_to_expert, conditions,
                                                     inverse_map, status);
    B200MOE_LAUNCH_OK("group_single_chunk_kernel");
    return B200MOE_OK;
  }
  group_count_kernel<<<n_chunks, kThreads, smem, st>>>(a, chunk_counts, out_ids, out_len, fill_val);
  B200MOE_LAUNCH_OK("group_count_kernel");
  group_scan_kernel<<<1, 1024, 0, st>>>(chunk_counts, n_chunks, a.n_cols, mode, a.T, B, N, mx_conditions, counts,
                                        col_base, block_to_expert, conditions, status);
  B200MOE_LAUNCH_OK("group_scan_kernel");
  group_scatter_kernel<<<n_chunks, kThreads, smem, st>>>(a, chunk_counts, col_base, out_len, out_ids, inverse_map);
  B200MOE_LAUNCH_OK("group_scatter_kernel");
  return B200MOE_OK;
}


// ---- grouping without any allocation --------------------------------------------
// Scratch of b200moe_group_tokens_static.  It lives in the library image: every
// GPU that loads the library keeps these bytes until the process exits.
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB
static __device__ __align__(256) unsigned char g_group_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_group_scratch, per device ordinal

// The array's name is only a host-side handle; kernels need the device address,
// looked up once per device while that device is current.
int static_scratch_address(void** out) {
  int dev = -1;
  B200MOE_CUDA_OK(cudaGetDevice(&dev));
  B200MOE_REQUIRE(dev >= 0 && dev < kMaxDevices, B200MOE_ERR_INVALID, "device ordinal %d is out of range", dev);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    B200MOE_CUDA_OK(cudaGetSymbolAddress(&p, g_group_scratch));
    B200MOE_REQUIRE(p != nullptr, B200MOE_ERR_CUDA, "cudaGetSymbolAddress returned a null scratch address");
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_find_nonzero_workspace_bytes(int T, int n_cols) { return group_ws_bytes(T, n_cols); }
extern "C" size_t b200moe_group_tokens_workspace_bytes(int T, int E) { return group_ws_bytes(T, E); }

extern "C" int b200moe_find_nonzero_indices(const void* input, int in_dtype, int T, int C_full,
                                            const int32_t* col_start_dev, int n_cols, int32_t* indices,
                                            int32_t* nonzero_counts, void* workspace, size_t workspace_bytes,
                                            b200moe_stream_t stream) {
  B200MOE_REQUIRE(input && indices && nonzero_counts && workspace, B200MOE_ERR_INVALID,
                  "find_nonzero_indices: null pointer argument");
  B200MOE_REQUIRE(in_dtype == B200MOE_F32 || in_dtype == B200MOE_BF16 || in_dtype == B200MOE_I32, B200MOE_ERR_INVALID,
                  "find_nonzero_indices: unsupported input dtype %d", in_dtype);
  B200MOE_REQUIRE(n_cols <= C_full, B200MOE_ERR_INVALID, "find_nonzero_indices: n_cols %d exceeds input columns %d",
                  n_cols, C_full);
  GroupArgs a{input, B200MOE_ROUTING_MASK, in_dtype, T, C_full, n_cols, 0, col_start_dev};
  return run_grouping(a, 0, 1, 0, 0, static_cast<int64_t>(n_cols) * T, -1, indices, nonzero_counts, nullptr, nullptr,
                      nullptr, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_group_tokens(const void* routing, int routing_mode, int routing_dtype, int T, int E, int K,
                                    int B, int N, int skip_token, int mx_conditions, int32_t* token_position_to_id,
                                    int32_t* block_to_expert, int32_t* conditions, int32_t* counts,
                                    int32_t* inverse_map, int32_t* status, void* workspace, size_t workspace_bytes,
                                    b200moe_stream_t stream) {
  B200MOE_REQUIRE(routing && token_position_to_id && block_to_expert && conditions && status && workspace,
                  B200MOE_ERR_INVALID, "group_tokens: null pointer argument");
  B200MOE_REQUIRE(B > 0 && N > 0, B200MOE_ERR_INVALID, "group_tokens: block size and block count must be positive");
  B200MOE_REQUIRE(routing_mode == B200MOE_ROUTING_INDEX || routing_mode == B200MOE_ROUTING_MASK, B200MOE_ERR_INVALID,
                  "group_tokens: unknown routing mode %d", routing_mode);
  if (routing_mode == B200MOE_ROUTING_INDEX)
    B200MOE_REQUIRE(K > 0 && K <= E, B200MOE_ERR_INVALID, "group_tokens: need 0 < K <= E (K=%d, E=%d)", K, E);
  B200MOE_REQUIRE(inverse_map == nullptr || routing_mode == B200MOE_ROUTING_INDEX, B200MOE_ERR_INVALID,
                  "group_tokens: inverse_map needs expert-index routing");
  GroupArgs a{routing, routing_mode, routing_dtype, T, E, E, K, nullptr};
  return run_grouping(a, 1, B, N, mx_conditions, static_cast<int64_t>(N) * B, skip_token ? -1 : T, token_position_to_id,
                      counts, block_to_expert, conditions, inverse_map, status, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_cumsum(const void* x, int dtype, int64_t rows, int64_t cols, void* out, b200moe_stream_t stream) {
  B200MOE_REQUIRE(x && out && rows > 0 && cols > 0, B200MOE_ERR_INVALID, "cumsum: bad arguments");
  B200MOE_REQUIRE(dtype == B200MOE_F32 || dtype == B200MOE_BF16 || dtype == B200MOE_I32, B200MOE_ERR_INVALID,
                  "cumsum: unsupported dtype %d", dtype);
  cumsum_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, dtype, cols, out);
  B200MOE_LAUNCH_OK("cumsum_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_indexed_flatten(const int32_t* input, int E, int T, int f_len, int64_t output_len,
                                       const int32_t* row_offsets, int n_row_offsets,
                                       const int32_t* row_offsets_start_dev, int padding_val, int32_t* out,
                                       b200moe_stream_t stream) {
  B200MOE_REQUIRE(input && row_offsets && out, B200MOE_ERR_INVALID, "indexed_flatten: null pointer argument");
  B200MOE_REQUIRE(f_len > 0 && T % f_len == 0, B200MOE_ERR_INVALID,
                  "indexed_flatten: row length %d must be a multiple of f_len %d", T, f_len);
  B200MOE_REQUIRE(n_row_offsets >= E, B200MOE_ERR_INVALID, "indexed_flatten: %d row offsets for %d rows",
                  n_row_offsets, E);
  const int grid = static_cast<int>(ceil_div64(output_len, 256) < sm_count() * 16 ? ceil_div64(output_len, 256) : sm_count() * 16);
  indexed_flatten_kernel<<<grid > 0 ? grid : 1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      input, E, T, f_len, output_len, row_offsets, row_offsets_start_dev, padding_val, out);
  B200MOE_LAUNCH_OK("indexed_flatten_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_build_position_table(const int32_t* token_position_to_id, const int32_t* block_to_expert,
                                            const int32_t* conditions, int n_blocks, int B, int T, int E,
                                            int32_t* pos_table, b200moe_stream_t stream) {
  B200MOE_REQUIRE(token_position_to_id && block_to_expert && pos_table, B200MOE_ERR_INVALID,
                  "build_position_table: null pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200MOE_CUDA_OK(cudaMemsetAsync(pos_table, 0xFF, static_cast<size_t>(T) * E * 4, st));
  const int64_t n_pos = static_cast<int64_t>(n_blocks) * B;
  const int grid = static_cast<int>(ceil_div64(n_pos, 256) < sm_count() * 8 ? ceil_div64(n_pos, 256) : sm_count() * 8);
  position_table_kernel<<<grid, 256, 0, st>>>(token_position_to_id, block_to_expert, conditions, n_pos, B, T, E,
                                              pos_table);
  B200MOE_LAUNCH_OK("position_table_kernel");
  return B200MOE_OK;
}

extern "C" size_t b200moe_group_tokens_static_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int b200moe_group_tokens_static(const void* routing, int routing_mode, int routing_dtype, int T, int E,
                                           int K, int B, int N, int skip_token, int mx_conditions,
                                           int32_t* token_position_to_id, int32_t* block_to_expert,
                                           int32_t* conditions, int32_t* counts, int32_t* inverse_map, int32_t* status,
                                           b200moe_stream_t stream) {
  const size_t need = group_ws_bytes(T, E);
  B200MOE_REQUIRE(T > 0 && E > 0 && need <= kStaticScratchBytes, B200MOE_ERR_WORKSPACE,
                  "group_tokens_static: T=%d, E=%d needs %zu scratch bytes, the built-in scratch holds %zu; "
                  "use b200moe_group_tokens with a caller workspace for larger problems",
                  T, E, need, kStaticScratchBytes);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != B200MOE_OK) return rc;
  return b200moe_group_tokens(routing, routing_mode, routing_dtype, T, E, K, B, N, skip_token, mx_conditions,
                              token_position_to_id, block_to_expert, conditions, counts, inverse_map, status, scratch,
                              kStaticScratchBytes, stream);
}
