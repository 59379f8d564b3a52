// Router logits for large token counts on the tcgen05 tensor cores.
//
// For T in the thousands the split-K path of router_topk.cu is bound by its per-slab barriers and by re-reading
// the router weight from L2 for every 64-token tile.  Here a persistent CTA owns 128-token tiles:
//   warp 0      TMA producer: per 64-column hidden slab a [128 tokens x 128 B] tile of x and an [EN x 128 B] tile
//               of the transposed router weight (both bf16, 128B swizzle)
//   warp 1      allocates TMEM and issues four tcgen05.mma.kind::f16 (bf16 x bf16 -> fp32, M = 128, N = EN,
//               K = 16) per slab into one of two accumulator buffers
//   warps 4..7  epilogue: a thread owns one token = one TMEM lane and streams its row of fp32 logits to the
//               [T, E] scratch the ranking kernel reads (the same kernel and arithmetic as on the split-K path,
//               which it sees as a single split).
// The weight crosses L2 -> SM once per 128 tokens and x once in total.  Ranking inside this kernel's epilogue
// (one thread per row, insertion top-K) was measured slower than the warp-per-row ranking kernel: 0.14 ms
// against 0.10 ms for both launches at T = 32768, E = 128.  The transposed, zero-padded weight [EN, H] is rebuilt
// per call in the caller's workspace (H * EN * 2 bytes: noise next to T * H * 2).  Every mbarrier wait is bounded.
#include "tcgen05_ptx.cuh"

namespace b200moe {
namespace {

constexpr int kTokM = 128;   // tokens per tile = TMEM lanes
constexpr int kSlab = 64;    // bf16 hidden columns per pipeline stage (128 bytes)
constexpr int kRtThreads = 256;

struct RouterTcArgs {
  int T, H, E;
  float* logits;  // [T, E] fp32 scratch
  int32_t* status;
};

__global__ void transpose_pad_kernel(const __nv_bfloat16* __restrict__ w, int H, int E, int EN,
                                     __nv_bfloat16* __restrict__ wT) {
  // w [H, E] -> wT [EN, H], rows e >= E zero
  __shared__ __nv_bfloat16 tile[32][33];
  const int h0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int h = h0 + i, e = e0 + threadIdx.x;
    tile[i][threadIdx.x] = (h < H && e < E) ? w[static_cast<int64_t>(h) * E + e] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int e = e0 + i, h = h0 + threadIdx.x;
    if (e < EN && h < H) wT[static_cast<int64_t>(e) * H + h] = tile[threadIdx.x][i];
  }
}

template <int EN>
struct RtLayout {
  static constexpr int kStages = EN <= 128 ? 6 : 4;
  static constexpr int kA = kTokM * 128;
  static constexpr int kB = EN * 128;
  static constexpr int kOffB = kStages * kA;
  static constexpr int kOffBar = kOffB + kStages * kB;
  static constexpr int kBytes = kOffBar + 256 + 1024;
};

template <int EN>
__global__ void __launch_bounds__(kRtThreads, 1)
router_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const RouterTcArgs a) {
  using L = RtLayout<EN>;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kIdesc = make_idesc_bf16(kTokM, EN);
  constexpr uint32_t kStageBytes = L::kA + L::kB;
  constexpr int kChunks = EN / 32;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (a.T + kTokM - 1) / kTokM;
  const int k_slabs = a.H / kSlab;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < k_slabs; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, a.status, 31)) { ok = false; break; }
          mbar_expect_tx(&full[stage], kStageBytes);
          tma_load_2d(smem + stage * L::kA, &tmap_x, kb * kSlab, tile * kTokM, &full[stage]);
          tma_load_2d(smem + L::kOffB + stage * L::kB, &tmap_w, kb * kSlab, 0, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land before the CTA retires
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, a.status, 32)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * EN;
        for (int kb = 0; kb < k_slabs; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, a.status, 33)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = desc_sw128(smem_u32(smem + stage * L::kA));
          const uint64_t b_desc = desc_sw128(smem_u32(smem + L::kOffB + stage * L::kB));
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 bf16 = 32 bytes per MMA: the descriptors advance by 2 (x 16 bytes)
            tc_mma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int E = a.E;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, a.status, 34)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * EN;
      const int t = tile * kTokM + q * 32 + lane;
      float* dst = a.logits + static_cast<int64_t>(t < a.T ? t : 0) * E;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        if (c * 32 >= E) break;
        uint32_t raw[32];
        tc_ld32_nowait(taddr + c * 32, raw);
        tc_wait_ld();
        if (t < a.T) {
          if ((E & 3) == 0 && c * 32 + 32 <= E) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<uint4*>(dst + c * 32)[j] = make_uint4(raw[4 * j], raw[4 * j + 1], raw[4 * j + 2], raw[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c * 32 + j < E) dst[c * 32 + j] = __uint_as_float(raw[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

int make_bf16_map(CUtensorMap* map, const void* base, int64_t cols, int64_t rows, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  B200MOE_REQUIRE(enc != nullptr, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kSlab), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200MOE_REQUIRE(r == CUDA_SUCCESS, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled (router) failed with code %d",
                  static_cast<int>(r));
  return B200MOE_OK;
}

template <int EN>
int launch_router_tc(const CUtensorMap& mx, const CUtensorMap& mw, const RouterTcArgs& a, cudaStream_t st) {
  using L = RtLayout<EN>;
  auto kern = router_tc_kernel<EN>;
  B200MOE_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kBytes));
  const int n_tiles = (a.T + kTokM - 1) / kTokM;
  const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
  kern<<<grid, kRtThreads, L::kBytes, st>>>(mx, mw, a);
  B200MOE_LAUNCH_OK("router_tc_kernel");
  return B200MOE_OK;
}

}  // namespace

// Bytes of scratch the tensor-core path needs: the transposed, padded router weight, then the fp32 logits;
// 0 if the shape is not eligible.
size_t router_tc_weight_bytes(int H, int E) {
  const int EN = E <= 64 ? 64 : (E <= 128 ? 128 : 256);
  return (static_cast<size_t>(EN) * H * sizeof(__nv_bfloat16) + 255) & ~static_cast<size_t>(255);
}
size_t router_tc_workspace_bytes(int T, int H, int E) {
  if (E > 256 || H % kSlab != 0) return 0;
  return router_tc_weight_bytes(H, E) + static_cast<size_t>(T) * E * sizeof(float);
}

bool router_tc_eligible(int x_is_TH, int T, int H, int E) {
  return x_is_TH && E <= 256 && H % kSlab == 0 && H >= kSlab && T >= 1;
}

// x [T, H] bf16, w [H, E] bf16 -> fp32 logits [T, E] (no bias) at the returned position inside `workspace`, which
// holds at least router_tc_workspace_bytes(T, H, E); `status` is one int32.
int router_tc_run(const void* x, const void* w, int T, int H, int E, void* workspace, int32_t* status,
                  float** logits_out, cudaStream_t st) {
  const int EN = E <= 64 ? 64 : (E <= 128 ? 128 : 256);
  __nv_bfloat16* wT = static_cast<__nv_bfloat16*>(workspace);
  float* logits = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + router_tc_weight_bytes(H, E));
  B200MOE_REQUIRE((reinterpret_cast<uintptr_t>(wT) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
                  B200MOE_ERR_INVALID, "router_topk: x and the workspace must be 16-byte aligned");
  transpose_pad_kernel<<<dim3((H + 31) / 32, EN / 32), dim3(32, 8), 0, st>>>(static_cast<const __nv_bfloat16*>(w), H, E,
                                                                              EN, wT);
  B200MOE_LAUNCH_OK("transpose_pad_kernel");
  B200MOE_CUDA_OK(cudaMemsetAsync(status, 0, 4, st));
  CUtensorMap mx, mw;
  int rc = make_bf16_map(&mx, x, H, T, kTokM);
  if (rc != B200MOE_OK) return rc;
  rc = make_bf16_map(&mw, wT, H, EN, EN);
  if (rc != B200MOE_OK) return rc;
  RouterTcArgs a{T, H, E, logits, status};
  *logits_out = logits;
  if (EN == 64) return launch_router_tc<64>(mx, mw, a, st);
  if (EN == 128) return launch_router_tc<128>(mx, mw, a, st);
  return launch_router_tc<256>(mx, mw, a, st);
}

}  // namespace b200moe
