/*
 * b200moe.h -- C ABI of the B200 (sm_100a) MoE expert hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, never
 * allocates or frees device memory, never synchronises the stream, and
 * returns 0 on success or a negative B200MOE_ERR_* code (details through
 * b200moe_last_error()).  Scratch memory is supplied by the caller; its size
 * comes from the matching *_workspace_bytes query.
 *
 * Each function names the reference interface it stands in for (paths are
 * relative to the reference project root).  The Python package in
 * nki_library_b200/ binds these with ctypes and re-exposes the reference's
 * kernel signatures.
 *
 * Device data formats
 *   "rows" fp8 operand ... uint8 e4m3fn codes [rows, K], K contiguous.
 *   "scale atoms" ........ UE8M0 bytes, one per (row, 32 consecutive K), stored as
 *                          512-byte atoms ordered [ceil(rows/128)][ceil(K/128)];
 *                          byte of (r, c) in an atom at (r%32)*16 + (r/32)*4 + c.
 *                          Size: b200moe_sf_bytes(rows, K).  Unused bytes must be 0.
 *   gate/up device weight  [E, 2I, H]: rows interleaved per 32 intermediate
 *                          columns (32 gate rows, then the matching 32 up rows).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200moe_stream_t; /* cudaStream_t */

enum {
  B200MOE_OK = 0,
  B200MOE_ERR_INVALID = -1,   /* argument validation failed */
  B200MOE_ERR_CUDA = -2,      /* a CUDA runtime/driver call failed */
  B200MOE_ERR_WORKSPACE = -3, /* workspace too small */
  B200MOE_ERR_DEVICE = -4     /* kernel reported an error through its status word */
};

/* element types of loosely typed pointers */
enum { B200MOE_F32 = 0, B200MOE_BF16 = 1, B200MOE_I32 = 2 };
/* ActFnType (core/utils/common_types.py:32-36) */
enum { B200MOE_ACT_SILU = 0, B200MOE_ACT_GELU = 1, B200MOE_ACT_GELU_TANH = 2, B200MOE_ACT_SWISH = 3 };
/* RouterActFnType (core/utils/common_types.py:39-46) */
enum { B200MOE_ROUTER_SIGMOID = 0, B200MOE_ROUTER_SOFTMAX = 1 };
/* weight source layouts accepted by the prepare functions */
enum { B200MOE_LAYOUT_ROWS = 0, B200MOE_LAYOUT_NKI_X4 = 1 };
/* element formats of expert weights (activations are always e4m3): the OCP MX element types the
 * reference's weights come in -- float8_e4m3fn_x4, float8_e5m2_x4 and float4_e2m1fn_x4
 * (core/utils/mx_torch_common.py:31-133, core/moe/moe_cte/moe_cte_mx_utils.py:58-107).  e2m1 packs two
 * elements per byte (element 2j in the low nibble), so a weight row of K elements is K/2 bytes. */
enum { B200MOE_W_E4M3 = 0, B200MOE_W_E5M2 = 1, B200MOE_W_E2M1 = 5 };
/* Variant word (`impl`) of the grouped contractions, per call.  No counterpart in the reference.
 *   B200MOE_IMPL_SIMT        CUDA-core validation kernels instead of the tensor-core path
 *   B200MOE_GEMM_TILE_N128   128 weight rows per tile instead of 256
 *   B200MOE_GEMM_NO_PAIR     never run on CTA pairs (tcgen05 cta_group::2, 256 positions x 256 weight rows)
 *   B200MOE_GEMM_FORCE_PAIR  pair an expert's 128-position tiles across its blocks whatever the block size
 *                            (default: when the block size is a multiple of 256, or experts hold four or more
 *                            tiles on average; an odd tile then ends in a half-empty pair)
 *   B200MOE_GEMM_NO_SPLIT    keep the tile an expert with an odd number of occupied tiles has left over in a
 *                            half-empty pair (default: a second, single-CTA launch takes the left-over tiles)
 *   B200MOE_GEMM_NO_OVERLAP  run that second launch strictly after the first (default: a programmatic
 *                            dependent launch that fills SMs as the first drains and finishes after it) */
enum {
  B200MOE_IMPL_SIMT = 1,
  B200MOE_GEMM_TILE_N128 = 0x100,
  B200MOE_GEMM_NO_PAIR = 0x200,
  B200MOE_GEMM_FORCE_PAIR = 0x400,
  B200MOE_GEMM_NO_SPLIT = 0x800,
  B200MOE_GEMM_NO_OVERLAP = 0x1000
};
/* routing source accepted by b200moe_group_tokens */
enum { B200MOE_ROUTING_INDEX = 0, B200MOE_ROUTING_MASK = 1 };

/* Message describing the last failure on the calling thread ("" if none).
 * Stands in for kernel_assert's exception text (core/utils/kernel_assert.py:15-16). */
const char* b200moe_last_error(void);
int b200moe_version(void);

/* Bytes of a scale-atom buffer for a [rows, K] operand. */
size_t b200moe_sf_bytes(int64_t rows, int64_t K);

/* ---- router ------------------------------------------------------------------
 * router_topk (core/router_topk/router_topk.py:55-75): logits = x @ w (+ bias) in
 * fp32, top-k (ties -> lowest expert id), affinities by one of the three pipelines
 * (router_topk.py:515-547).  x is bf16 [T,H] (x_is_TH=1) or [H,T]; w bf16 [H,E];
 * w_bias bf16 [E] or NULL.  Outputs (each may be NULL to skip): router_logits
 * [T,E], expert_index uint32 [T,k], expert_affinities [T,E] (dense, zeros outside
 * the top-k when scattered).  E <= 512, k <= 8.  workspace (256-byte aligned,
 * b200moe_router_workspace_bytes) starts with an int32 status word -- non-zero after the
 * call's kernels have run means a device-side wait ran out -- followed by scratch: split-K
 * partial logits, or the transposed router weight of the single-kernel tcgen05 path that
 * large token counts take (x [T,H], E <= 256, H % 64 == 0). */
size_t b200moe_router_workspace_bytes(int T, int H, int E);
/* path (per call, no reference counterpart): 0 = choose by shape; 1 = always the split-K path; 2 = the
 * tcgen05 path whenever the shape is eligible. */
int b200moe_router_topk(const void* x, int x_is_TH, const void* w, const void* w_bias, int T, int H, int E, int k,
                        int act_fn, int router_pre_norm, int norm_topk_prob, void* router_logits, int logits_dtype,
                        uint32_t* expert_index, void* expert_affinities, int aff_dtype, int path, void* workspace,
                        size_t workspace_bytes, b200moe_stream_t stream);

/* ---- grouping ----------------------------------------------------------------
 * find_nonzero_indices (core/subkernels/find_nonzero_indices.py:34-40): per column
 * c of input [T, C_full] (f32 / bf16 / i32), ascending row ids of non-zeros padded
 * with -1 to length T, and their count.  col_start_dev: device int32[1] or NULL. */
size_t b200moe_find_nonzero_workspace_bytes(int T, int n_cols);
int b200moe_find_nonzero_indices(const void* input, int in_dtype, int T, int C_full, const int32_t* col_start_dev,
                                 int n_cols, int32_t* indices, int32_t* nonzero_counts, void* workspace,
                                 size_t workspace_bytes, b200moe_stream_t stream);

/* cumsum (core/cumsum/cumsum.py:29): inclusive, along the last axis, fp32 accumulate. */
int b200moe_cumsum(const void* x, int dtype, int64_t rows, int64_t cols, void* out, b200moe_stream_t stream);

/* indexed_flatten (core/subkernels/indexed_flatten.py:28-35): out[(row_offsets[s+e]+p)*f_len + j]
 * = input[e, p*f_len + j]; the highest e wins where rows overlap; blocks outside
 * the output are dropped; the rest is padding_val. */
int b200moe_indexed_flatten(const int32_t* input, int E, int T, int f_len, int64_t output_len,
                            const int32_t* row_offsets, int n_row_offsets, const int32_t* row_offsets_start_dev,
                            int padding_val, int32_t* out, b200moe_stream_t stream);

/* Fused grouping = find_nonzero_indices + cumsum + indexed_flatten plus the
 * block_to_expert / conditions bookkeeping of the reference's block-assignment
 * generator (test/integration/nkilib/core/moe/moe_cte/test_moe_cte_common.py:199-264).
 * routing: uint32/int32 expert ids [T,K] (B200MOE_ROUTING_INDEX) or a [T,E] mask /
 * masked affinities of routing_dtype (B200MOE_ROUTING_MASK, K ignored).
 * Outputs: token_position_to_id [N*B] (pad -1 if skip_token else T), block_to_expert
 * [N], conditions [N+2] (mx_conditions) or [N+1], counts [E], inverse_map [T,K]
 * (position of each (t,k) pair; NULL to skip; index mode only), status[0] != 0 if N
 * was too small for the routing. */
size_t b200moe_group_tokens_workspace_bytes(int T, int E);
int b200moe_group_tokens(const void* routing, int routing_mode, int routing_dtype, int T, int E, int K, int B, int N,
                         int skip_token, int mx_conditions, int32_t* token_position_to_id, int32_t* block_to_expert,
                         int32_t* conditions, int32_t* counts, int32_t* inverse_map, int32_t* status, void* workspace,
                         size_t workspace_bytes, b200moe_stream_t stream);

/* Same grouping for callers that must not allocate device memory -- code running
 * inside a memory-pool or allocator callback, a plug-in whose host forbids
 * cudaMalloc after start-up, or a real-time serving loop where an allocation
 * could stall behind another thread's free.  No counterpart in the reference.
 * The scratch is a 1 MiB device array built into the library (held by every GPU
 * that loads it until the process exits), so the problem must satisfy
 * b200moe_group_tokens_workspace_bytes(T, E) <= b200moe_group_tokens_static_max_bytes();
 * larger problems are rejected with B200MOE_ERR_WORKSPACE.  Neither the call nor
 * anything it runs allocates or frees memory -- from the second call on a device
 * onwards.  The first call on each device looks up the array's device address (with
 * that device current), and with CUDA's lazy module loading that lookup or the first
 * launch may make the driver load the library's code, which allocates.  So make one
 * warm-up call per device at start-up: before the window in which allocation is
 * forbidden, outside any stream capture, and from one thread (the address is cached
 * per device ordinal without a lock; the library assumes the one primary context per
 * device that the CUDA runtime uses).  All calls share the one array: nothing in it needs
 * clearing between calls (each call overwrites what it reads), but two calls that
 * overlap on the GPU -- different streams without an ordering between them -- race. */
size_t b200moe_group_tokens_static_max_bytes(void);
int b200moe_group_tokens_static(const void* routing, int routing_mode, int routing_dtype, int T, int E, int K, int B,
                                int N, int skip_token, int mx_conditions, int32_t* token_position_to_id,
                                int32_t* block_to_expert, int32_t* conditions, int32_t* counts, int32_t* inverse_map,
                                int32_t* status, b200moe_stream_t stream);

/* position table for the combine when only token_position_to_id is known (moe_cte's
 * own argument list): pos_table[t*E + e] = position of token t in a block of expert e, else -1. */
int b200moe_build_position_table(const int32_t* token_position_to_id, const int32_t* block_to_expert,
                                 const int32_t* conditions, int n_blocks, int B, int T, int E, int32_t* pos_table,
                                 b200moe_stream_t stream);

/* ---- MXFP8 activation quantisation --------------------------------------------
 * load_and_quantize_hidden_states (core/moe/moe_cte/moe_cte_mx_utils.py:456-945) with
 * nisa.quantize_mx semantics as defined on CPU by quantize_to_mx
 * (core/utils/mx_torch_common.py:157-221).  Row p of the output is
 * hidden[token_position_to_id[p]] (zeros for pad ids; identity if the pointer is
 * NULL), with the H axis taken in the reference's packed order
 * k' = t*512 + p*4 + q <- h = q*(H/4) + t*128 + p when h_packed_order != 0.
 * tile_flags (int32 [ceil(n_pos/128)], may be NULL) receives, for every
 * 128-position tile, 1 + the index of its last row that holds a real token (0 = none);
 * the contractions skip empty tiles and copy only the leading rows of short ones. */
int b200moe_gather_quantize_mxfp8(const void* hidden_bf16, int hidden_rows, int H, const int32_t* token_position_to_id,
                                  int64_t n_pos, int h_packed_order, uint8_t* codes, uint8_t* sf_atoms,
                                  int32_t* tile_flags, b200moe_stream_t stream);

/* The same quantisation driven by the inverse map (inverse_map[t*K + k] = position of token t's k-th expert, or
 * negative; what b200moe_group_tokens writes): every token row is read and quantised once and stored to its K
 * positions, so hidden crosses HBM once instead of K times.  Positions that no (token, k) pair maps to are NOT
 * written -- the contractions never let such rows reach a result -- and tile_flags is filled as above.  K is
 * the width of the map, not a top-k limit: the [T, E] table of b200moe_build_position_table is accepted as well
 * (K = E, negative entries skipped), which is how moe_cte reads hidden once with only token_position_to_id given.
 * No reference counterpart (the reference gathers per block, core/moe/moe_cte/moe_cte_mx_utils.py:456-945). */
int b200moe_scatter_quantize_mxfp8(const void* hidden_bf16, int T, int H, const int32_t* inverse_map, int K,
                                   int64_t n_pos, int h_packed_order, uint8_t* codes, uint8_t* sf_atoms,
                                   int32_t* tile_flags, b200moe_stream_t stream);

/* ---- weight preparation (once per model load) ----------------------------------
 * Source B200MOE_LAYOUT_ROWS: codes [E,2,I,H] + scales [E,2,I,H/32] (gate_up) and
 * codes [E,H,I] + scales [E,H,I/32] (down).
 * Source B200MOE_LAYOUT_NKI_X4: the reference's storage
 * gate_up [E,128,2,H/512,I] x4 + scale [E,16,2,H/512,I],
 * down [E,p_I,ceil(I/512),H] x4 + scale [E,p_I/8,ceil(I/512),H]
 * (core/moe/moe_cte/bwmm_shard_on_block_mx.py:70-230).
 * w_format is one of B200MOE_W_*: 8-bit elements are one byte each (x4 = 32 bits), e2m1 elements are
 * nibbles (x4 = 16 bits, so every byte count above halves); e2m1 needs contraction lengths that are
 * multiples of 128.  The prepared arrays hold b200moe_weight_bytes(rows, K, w_format) bytes per expert.
 * Bias sources: gate_up [E,2,I] fp32 (ROWS) or [E,p_I,2,ceil(I/512),4] (NKI_X4), any of F32/BF16. */
int b200moe_prepare_gate_up(const void* w, const uint8_t* scale, int layout, int w_format, int E, int H, int I,
                            uint8_t* w_dev, uint8_t* sf_dev, b200moe_stream_t stream);
int b200moe_prepare_down(const void* w, const uint8_t* scale, int layout, int w_format, int E, int H, int I,
                         uint8_t* w_dev, uint8_t* sf_dev, b200moe_stream_t stream);
/* Bytes of `rows` prepared weight rows of K elements in the given format (no reference counterpart). */
int64_t b200moe_weight_bytes(int64_t rows, int64_t K, int w_format);
int b200moe_prepare_gate_up_bias(const void* bias, int dtype, int layout, int E, int I, float* bias_dev,
                                 b200moe_stream_t stream);

/* ---- grouped expert contractions -----------------------------------------------
 * Parameters common to both: block_to_expert [n_blocks]; conditions (NULL = all
 * blocks run; otherwise blocks run up to the first b with conditions[b] == 0, as in the
 * reference's block loop); tile_flags (NULL = all
 * tiles run; see b200moe_gather_quantize_mxfp8); token_position_to_id [n_blocks*B] and
 * hidden_rows (ids outside [0, hidden_rows) are pads, their rows are not written); status: device
 * int32[1], set non-zero if a kernel-internal wait ran out; impl: the per-call variant
 * word, 0 = tcgen05 tensor-core kernel with tile shapes chosen by the library,
 * B200MOE_IMPL_SIMT = plain CUDA-core validation kernel (slow, same results up to
 * summation order), B200MOE_GEMM_* bits = restrictions on the tile shapes (below);
 * clock_probe: NULL, or a device buffer of two 64-bit words (8-byte aligned) into which
 * CTA 0 of the contraction writes {SM cycles, nanoseconds} it ran for, which gives the SM
 * clock the kernel really saw (diagnostic, no reference counterpart).
 *
 * gemm1 = gate_up_projection_mx + clamp + act(gate)*up + quantize_mx of the result
 * (core/mlp/mlp_tkg/gate_up_projection_mx_shard_H.py:48-225,
 *  core/moe/moe_cte/bwmm_shard_on_block_mx.py:1159-1278,
 *  core/mlp/mlp_tkg/down_projection_mx_shard_H.py:73-78).  Clamp limits are
 * ignored when NaN.  Output: codes [n_blocks*B, I] + scale atoms. */
int b200moe_grouped_gemm1_swiglu(const uint8_t* x_codes, const uint8_t* x_sf, const uint8_t* w1_dev,
                                 const uint8_t* w1_sf, int w_format, const float* bias_gu_dev,
                                 const int32_t* block_to_expert,
                                 const int32_t* conditions, const int32_t* tile_flags,
                                 int n_blocks, int B, int E, int H, int I, int act_fn, float gate_lo, float gate_hi,
                                 float up_lo, float up_hi, uint8_t* m_codes, uint8_t* m_sf, int32_t* status, int impl,
                                 void* clock_probe, b200moe_stream_t stream);

/* gemm2 = down_projection_mx + bias + affinity scaling of each row
 * (core/mlp/mlp_tkg/down_projection_mx_shard_H.py:212-387,
 *  core/moe/moe_cte/bwmm_shard_on_block_mx.py:1297-1317).  affinities is the flat
 * [(rows)*E] table addressed tok*E + e (core/moe/moe_cte/moe_cte_utils.py:544-636) when
 * aff_per_row == 0, a [rows] vector addressed tok when aff_per_row != 0 (rows that arrived
 * through an expert-parallel dispatch carry their own affinity), or NULL for no scaling.  Output: bf16 y_pos [n_blocks*B, H] (pad rows untouched). */
int b200moe_grouped_gemm2_scale(const uint8_t* m_codes, const uint8_t* m_sf, const uint8_t* w2_dev,
                                const uint8_t* w2_sf, int w_format, const float* bias_d, const int32_t* block_to_expert,
                                const int32_t* conditions, const int32_t* tile_flags,
                                const int32_t* token_position_to_id, int hidden_rows,
                                int n_blocks, int B, int E, int H, int I, const void* affinities, int aff_dtype,
                                int aff_per_row, void* y_pos_bf16, int32_t* status, int impl,
                                void* clock_probe, b200moe_stream_t stream);

/* ---- dense (non-MX) expert contractions ----------------------------------------------------
 * The reference's bf16 and fp8-row expert kernels (core/moe/moe_cte/bwmm_shard_on_block.py:72,
 * core/moe/moe_cte/bwmm_shard_on_I.py:2014, core/moe/moe_tkg/all_expert_impl.py:65,
 * core/moe/moe_tkg/selective_expert_impl.py:45; CPU definition core/moe/moe_cte/moe_cte_torch.py:26-242):
 * bf16 activations x bf16 weights with fp32 accumulation on the same grouped tcgen05 kernel
 * (kind::f16 instead of the block-scaled kind).  Weights are K-major bf16 rows: gate/up
 * [E, 2I, H] with the 32 / 32 gate / up row interleave of the MX layout, down [E, H, I].
 * fp8-row weights are passed dequantised to bf16 together with their per-row factors
 * (w*_col_scale fp32 [E, 2I] in the interleaved row order / [E, H]; NULL = none), which the
 * epilogues apply to the accumulator before the bias, as the reference does.
 *
 * scatter_rows: the bf16 row of token t is copied to every position table[t*K + k] >= 0
 * (table as for b200moe_scatter_quantize_mxfp8); with pre_scale_affinities (flat [T*E] table,
 * PRE_SCALE mode) it is first multiplied by the affinity of the position's expert.
 * dense_gemm1: out m_bf16 [n_blocks*B, I] = act(gate) * up; dense_gemm2: bf16 y_pos rows. */
int b200moe_scatter_rows_bf16(const void* hidden_bf16, int T, int H, const int32_t* table, int K, int64_t n_pos,
                              const int32_t* block_to_expert, int B, int E, const void* pre_scale_affinities,
                              int aff_dtype, void* out_bf16, int32_t* tile_flags, b200moe_stream_t stream);
int b200moe_dense_gemm1_swiglu(const void* x_bf16, const void* w1_bf16, const float* w1_col_scale,
                               const float* bias_gu_dev, const int32_t* block_to_expert, const int32_t* conditions,
                               const int32_t* tile_flags, int n_blocks, int B, int E, int H, int I, int act_fn,
                               float gate_lo, float gate_hi, float up_lo, float up_hi, void* m_bf16, int32_t* status,
                               int impl, b200moe_stream_t stream);
int b200moe_dense_gemm2_scale(const void* m_bf16, const void* w2_bf16, const float* w2_col_scale, const float* bias_d,
                              const int32_t* block_to_expert, const int32_t* conditions, const int32_t* tile_flags,
                              const int32_t* token_position_to_id, int hidden_rows, int n_blocks, int B, int E, int H,
                              int I, const void* affinities, int aff_dtype, int aff_per_row, void* y_pos_bf16,
                              int32_t* status, int impl, b200moe_stream_t stream);

/* combine = the accumulate-and-scatter tail of the block loop
 * (core/moe/moe_cte/bwmm_shard_on_block_mx.py:1303-1347): out[t,:] = sum over the
 * valid entries p = table[t, j] (j ascending) of y_pos[p,:], fp32 accumulation,
 * one bf16 rounding.  table is inverse_map [T,K] or a position table [T,E]. */
int b200moe_combine(const void* y_pos_bf16, const int32_t* table, int T, int n_cand, int H, void* out_bf16,
                    b200moe_stream_t stream);

/* ---- RMSNorm in front of the decode MoE block -------------------------------------------------
 * rmsnorm_tkg as used by moe_block_tkg (core/moe_block/moe_block_tkg.py:192-232; CPU definition
 * core/subkernels/rmsnorm_torch.py:22-51): out = x / sqrt(sum(x^2) / count + eps) * gamma with fp32
 * statistics, count = hidden_actual if > 0 else H.  With a residual, x = bf16(inp + residual) and is
 * also written to residual_out (may be NULL).  gamma [H] fp32 / bf16 or NULL. */
int b200moe_rmsnorm(const void* inp_bf16, const void* residual_bf16, const void* gamma, int gamma_dtype, int T, int H,
                    int hidden_actual, float eps, void* out_bf16, void* residual_out_bf16, b200moe_stream_t stream);
/* The same RMSNorm fused with the MXFP8 activation quantisation -- rmsnorm_mx_quantize_tkg
 * (core/subkernels/rmsnorm_mx_quantize_tkg.py:29-80), which moe_block_tkg uses in MX all-expert mode
 * (core/moe_block/moe_block_tkg.py:199-218): besides the normalised bf16 rows (out, for the router) it
 * writes the rows' MXFP8 codes and scale atoms to every position table[t*K + k] >= 0 and fills
 * tile_flags, i.e. what b200moe_scatter_quantize_mxfp8 would produce from `out`.  H % 128 == 0. */
int b200moe_rmsnorm_quantize_mxfp8(const void* inp_bf16, const void* residual_bf16, const void* gamma, int gamma_dtype,
                                   int T, int H, int hidden_actual, float eps, void* out_bf16, void* residual_out_bf16,
                                   const int32_t* table, int K, int64_t n_pos, int h_packed_order, uint8_t* codes,
                                   uint8_t* sf_atoms, int32_t* tile_flags, b200moe_stream_t stream);

/* ---- expert parallelism over peer memory -------------------------------------------------------
 * One process per GPU.  The reference's expert-parallel mode slices experts by rank_id
 * (core/moe/moe_tkg/moe_tkg.py:100-101) and leaves the token exchange to an external all_to_all_v
 * (experimental/collectives/topk_reduce.py:15); these entry points are that exchange, done by kernels
 * that store straight into the peer GPUs' buffers (NVLink), with no host synchronisation.
 *
 * b200moe_ipc_export / _open / _close share a device buffer between the ranks' processes with CUDA IPC
 * (64-byte handle + byte offset inside the exported allocation).  Peer tables passed below are host
 * arrays of `world` device pointers, entry r = that buffer on rank r (own rank: the local pointer).
 * Flag tables are int32 [4][8], zero-initialised; epoch_dev is a zero-initialised device int32 that
 * exchange_counts bumps once per step (so a recorded CUDA graph of a step can be replayed).
 *
 * Step order on every rank's stream: exchange_counts -> dispatch_quantize (which also writes the receiver's
 * plan when given its outputs; b200moe_ep_plan is the same computation as a launch of its own) ->
 * signal_wait(slot 1) -> scales_to_atoms -> grouped_gemm1 / grouped_gemm2 (token_position_to_id = row_valid,
 * hidden_rows = cap_rows, per-row affinities) -> return_rows -> signal_wait(slot 2) -> combine.  A wait that
 * runs out (about two seconds) or a receive buffer that is too small sets *status non-zero.
 * dispatch_quantize walks the tokens: pair_of_token int32 [T, K] holds, for every (token, k), the index of that
 * pair in the expert-sorted list (the inverse table b200moe_group_tokens writes at block size 1; -1 = none) and
 * pair_expert [T*K] the expert of every sorted pair; a token's row is quantised once and stored to each GPU
 * that owns one of its experts (codes into xq_peers, scale bytes row-major into sf_peers = the receivers'
 * sf_rows).  Plan outputs (block_to_expert == NULL: none): block_to_expert / conditions [n_blocks_cap (+2)],
 * row_valid [n_blocks_cap * B], tile_flags [n_blocks_cap * B / 128], all in this rank's own memory; they depend
 * on the count table only. */
int b200moe_ipc_export(const void* dev_ptr, void* handle_out_64, int64_t* offset_out);
int b200moe_ipc_open(const void* handle_64, int64_t offset, void** dev_ptr_out);
int b200moe_ipc_close(void* dev_ptr, int64_t offset);
int b200moe_ep_exchange_counts(const int32_t* counts, void* const* count_tables, void* const* flag_tables, int rank,
                               int world, int E, int32_t* epoch_dev, int32_t* status, b200moe_stream_t stream);
int b200moe_ep_signal_wait(void* const* flag_tables, int rank, int world, int slot, const int32_t* epoch_dev,
                           int32_t* status, b200moe_stream_t stream);
int b200moe_ep_plan(const int32_t* counts_all, int rank, int world, int E, int B, int n_blocks_cap,
                    int32_t* block_to_expert, int32_t* conditions, int32_t* row_valid, int32_t* tile_flags,
                    int32_t* status, b200moe_stream_t stream);
/* Receiver side of the dispatch: scale bytes arrive row-major (sf_rows uint8 [cap_rows][H / 32], written by the
 * peers' dispatch_quantize); this lays the rows of every tile that holds a token (tile_flags > 0) into the 512-byte
 * atoms the contractions read.  Runs after signal_wait(slot 1). */
int b200moe_ep_scales_to_atoms(const uint8_t* sf_rows, const int32_t* tile_flags, int64_t n_tiles, int H,
                               uint8_t* sf_atoms, b200moe_stream_t stream);
int b200moe_ep_dispatch_quantize(const void* hidden_bf16, const int32_t* pair_of_token, const int32_t* pair_expert,
                                 const float* affinities, const int32_t* counts_all, int T, int K, int H, int E, int B,
                                 int rank, int world, int h_packed_order, void* const* xq_peers, void* const* sf_peers,
                                 void* const* aff_peers, void* const* src_peers, int64_t cap_rows,
                                 int n_blocks_cap, int32_t* block_to_expert, int32_t* conditions, int32_t* row_valid,
                                 int32_t* tile_flags, int32_t* status, b200moe_stream_t stream);
/* The down contraction of an expert-parallel step with the return fused into its epilogue: instead of writing
 * y_pos and copying it out afterwards (b200moe_ep_return_rows), every result row is stored straight into the
 * buffer of the GPU its token came from -- row (row_src[r] & 0xffffff) of back_peers[row_src[r] >> 24], plain
 * peer stores over NVLink -- while the tensor cores work on the next tile.  Arguments as
 * b200moe_grouped_gemm2_scale with per-row affinities (row_affinity fp32 [cap_rows]) and row_valid in the
 * place of token_position_to_id; follow it with b200moe_ep_signal_wait(slot 2) as after ep_return_rows.
 * The reference leaves this exchange to an external all_to_all_v (experimental/collectives/topk_reduce.py:31-62). */
int b200moe_ep_gemm2_scale_return(const uint8_t* m_codes, const uint8_t* m_sf, const uint8_t* w2_dev,
                                  const uint8_t* w2_sf, int w_format, const float* bias_d,
                                  const int32_t* block_to_expert, const int32_t* conditions,
                                  const int32_t* tile_flags, const int32_t* row_valid, int64_t cap_rows, int n_blocks,
                                  int B, int E_local, int H, int I, const float* row_affinity, const int32_t* row_src,
                                  void* const* back_peers, int world, int64_t back_rows, int32_t* status, int impl,
                                  b200moe_stream_t stream);
int b200moe_ep_return_rows(const void* y_pos_bf16, const int32_t* row_valid, const int32_t* row_src,
                           void* const* back_peers, int world, int64_t cap_rows, int H, int64_t back_rows,
                           b200moe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
